"""Pins of the CPU oracle (no GPU): the known-answer and relational tests the reference
itself holds for this path, restated against `oracle/`, plus the committed golden vectors.
"""
import os

import numpy as np
import pytest

import oracle as O
from tests_golden import GOLDEN_DIR, load_golden  # noqa: F401
from util import rng


# --- test/ParallelReverseAutoDiff.Test/PRAD/PradOpTests.cs:503-518 (TestGather): rows 2 and 0
# of a 3x2 table; upstream ones scatter back to rows 0 and 2.
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_reference_gather_known_answer(dtype):
    seed = np.array([[1, 2], [3, 4], [5, 6]], dtype)
    idx = np.array([[2], [0]], dtype)
    out = O.embedding_forward(idx, seed)
    np.testing.assert_array_equal(out.ravel(), np.array([5, 6, 1, 2], dtype))
    dW = O.embedding_backward(idx, np.ones((2, 2), dtype), 3)
    np.testing.assert_array_equal(dW.ravel(), np.array([1, 1, 0, 0, 1, 1], dtype))


# --- test/.../PRAD/TensorReverseTests.cs:101-117 (GatherReverse_Test): 3x3 table, indices 0, 2
def test_reference_gather_reverse_known_answer():
    idx = np.array([[0.0], [2.0]])
    dW = O.embedding_backward(idx, np.ones((2, 3)), 3)
    np.testing.assert_array_equal(dW.ravel(), np.array([1, 1, 1, 0, 0, 0, 1, 1, 1.0]))


def test_scatter_adds_duplicates_in_row_order():
    # float addition is not associative: ((1e16 + 1) + -1e16) != (1e16 + -1e16) + 1
    idx = np.array([[0.0], [0.0], [0.0]])
    d = np.array([[1e16], [1.0], [-1e16]])
    assert O.embedding_backward(idx, d, 1)[0, 0] == ((0.0 + 1e16) + 1.0) + -1e16


# --- test/.../LayerNormalizationTest.cs:13-80: forward-mode (dual number) derivative of the
# diagonal entry times the upstream gradient equals Backward within 1e-9.  Inputs follow the
# test: x[r,c] = (2r+1)(2c+5)*U(0,1), upstream = 10*U(0,1).
def _dual_diagonal(x, eps):
    n = x.shape[1]
    mu = x.mean(1, keepdims=True)
    sigma = np.sqrt(((x - mu) ** 2).sum(1, keepdims=True) / n)
    dsigma = (x - mu) / (n * sigma)                      # d sigma / d x_j
    return (1 - 1.0 / n) / (sigma + eps) - (x - mu) * dsigma / (sigma + eps) ** 2


@pytest.mark.parametrize("n", [22, 33, 44, 222, 333, 444])
def test_reference_layernorm_dual_number_relation(n):
    r = rng(n)
    rows = np.arange(n)[:, None] * 2.0 + 1
    cols = np.arange(n)[None, :] * 2.0 + 5
    x = rows * cols * r.random((n, n))
    up = r.random((n, n)) * 10.0
    _, mean, std = O.layernorm_forward(x)
    got = O.layernorm_backward(x, mean, std, up)
    want = _dual_diagonal(x, 1e-9) * up
    check = slice(None) if n <= 100 else slice(0, 1)      # the reference stops after row 0 above 100
    assert np.abs(got[check] - want[check]).max() < 1e-9


# --- test/.../GpuMatrixMultiplyOperationTest.cs:9-62: A 1000x1000 Xavier, B 1000x1; forward and
# both backward results of two implementations agree after Math.Round(x, 10).  Here: the
# sequential oracle against numpy's blocked float64 product.
def test_reference_matmul_relation_1e10():
    r = rng(7)
    A = (r.random((1000, 1000)) * 2 - 1) * np.sqrt(6.0 / 2000)
    B = (r.random((1000, 1)) * 2 - 1) * np.sqrt(6.0 / 1001)
    C = O.matmul_forward(A, B)
    np.testing.assert_array_equal(np.round(C, 10), np.round(A @ B, 10))
    dA, dB = O.matmul_backward(A, B, C)
    np.testing.assert_array_equal(np.round(dA, 10), np.round(C @ B.T, 10))
    np.testing.assert_array_equal(np.round(dB, 10), np.round(A.T @ C, 10))


# --- test/ParallelReverseAutoDiff.Test/SineSoftmaxTest.cs:8-24: on Xavier-initialised i x i inputs the rows of
# SineSoftmaxOperation.Forward add up to more than 0.8 on average (Matrix.InitializeXavier: uniform in
# +-sqrt(6 / (rows + cols))); a sample of the sizes 5..999 the reference walks.
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_reference_sine_softmax_rows_add_up_to_more_than_point_eight(dtype):
    r = rng(77)
    for n in (5, 6, 17, 64, 333, 999):
        lim = np.sqrt(6.0 / (2 * n))
        x = ((r.random((n, n)) * 2 - 1) * lim).astype(dtype)
        y = O.sine_softmax_forward(x)
        assert y.sum(1).mean() > 0.8
        # the definition, element by element
        e = np.exp(np.sin(x.astype(np.float64)))
        np.testing.assert_allclose(y, e / (e.sum(1, keepdims=True) + e), rtol=1e-5 if dtype == np.float32 else 1e-13)


def test_sine_softmax_backward_is_the_reference_formula():
    # SineSoftmaxOperation.cs:155-176: dx = dy * M e cos(x) / (M + e)^2, which is the derivative of e / (M + e)
    # with M held constant (not the full Jacobian)
    r = rng(3)
    x, dy = r.standard_normal((6, 120)), r.standard_normal((6, 120))
    e = np.exp(np.sin(x))
    m = e.sum(1, keepdims=True)
    np.testing.assert_allclose(O.sine_softmax_backward(x, dy), dy * m * e * np.cos(x) / (m + e) ** 2, rtol=1e-13)


def test_float_products_are_not_fused():
    # a*b+c with one rounding would give 1 + 2^-24... the managed code rounds twice
    a = np.array([[1 + 2.0 ** -12]], np.float32)
    c = O.matmul_forward(a, a)
    assert c[0, 0] == np.float32(np.float32(a[0, 0]) * np.float32(a[0, 0]))


def test_clip_reference_nan_limit_leaves_constant_tensor_alone():
    g = np.full((3, 3), 7.0)
    out = O.clip_reference(g.copy(), 4.0, 1e-16)          # sigma = 0 -> z = NaN -> Math.Min = NaN
    np.testing.assert_array_equal(out, g)


def test_gelu_derivative_is_the_reference_form_not_the_textbook_one():
    x = np.array([[0.7]])
    b = np.tanh(np.sqrt(2 / np.pi) * (x + 0.044715 * x ** 3))
    d = np.sqrt(2 / np.pi) * (0.044715 * 3 * x ** 2 + 1)
    as_written = 0.5 * x * ((1 - b ** 2) ** 2 * d + b) + 0.5 * (1 + b)
    textbook = 0.5 * (1 + b) + 0.5 * x * (1 - b ** 2) * d
    got = O.gelu_backward(x, np.ones_like(x))
    assert abs(got - as_written).max() < 1e-15
    assert abs(got - textbook).max() > 1e-3


# --- known-answer vectors of test/.../PRAD/TensorReverseTests.cs and PradOpTests.cs for the PRAD Tensor
# family (transcribed in reference_vectors.py), against the numpy restatement in oracle/__init__.py
import reference_vectors as RV


@pytest.mark.parametrize("case", RV.BINARY_REVERSE, ids=lambda c: c[0].split()[-1])
def test_reference_tensor_binary_reverse_vectors(case):
    label, op, a, b, up, want_a, want_b, places = case
    da, db = O.tensor_binary_reverse(op, np.array(a), np.array(b), np.array(up))
    RV.check(da, want_a, places, label)
    RV.check(db, want_b, places, label)


@pytest.mark.parametrize("case", RV.BINARY_FORWARD, ids=lambda c: c[0].split()[-1])
def test_reference_tensor_binary_forward_vectors(case):
    label, op, a, b, want, places = case
    RV.check(O.tensor_binary(op, np.array(a), np.array(b)), want, places, label)


@pytest.mark.parametrize("case", RV.UNARY_REVERSE, ids=lambda c: c[0].split()[-2] + c[0].split()[-1])
def test_reference_tensor_unary_reverse_vectors(case):
    label, op, x, up, want, places = case
    RV.check(O.tensor_unary_reverse(op, np.array(x), np.array(up)), want, places, label)


@pytest.mark.parametrize("case", RV.UNARY_FORWARD, ids=lambda c: c[0].split()[-1])
def test_reference_tensor_unary_forward_vectors(case):
    label, op, x, want, places = case
    RV.check(O.tensor_unary(op, np.array(x)), want, places, label)


@pytest.mark.parametrize("case", RV.GATHER, ids=lambda c: c[0].split()[-1])
def test_reference_tensor_gather_vectors(case):
    label, shape, table, idx, want, up, want_rev = case
    x = np.array(table).reshape(shape)
    RV.check(O.tensor_gather(x, np.array(idx)), want, None, label)
    RV.check(O.tensor_gather_reverse(np.array(up).reshape(len(idx), shape[1]), np.array(idx), shape), want_rev, None, label)


@pytest.mark.parametrize("case", RV.TILE_REVERSE, ids=lambda c: c[0].split()[1])
def test_reference_tensor_tile_reverse_vectors(case):
    label, shape, mult, up, want = case
    up = np.array(up).reshape(shape[0] * mult[0], shape[1] * mult[1])
    RV.check(O.tensor_tile_reverse(up, shape, mult), want, None, label)


@pytest.mark.parametrize("case", RV.TILE_FORWARD, ids=lambda c: c[0].split()[-1])
def test_reference_tensor_tile_forward_vectors(case):
    label, shape, x, mult, want = case
    RV.check(O.tensor_tile(np.array(x).reshape(shape), mult), want, None, label)


def test_reference_sum_rows_and_transpose_reverse_vectors():
    label, shape, up, want = RV.SUM_ROWS_REVERSE
    RV.check(O.row_sum_backward(np.array(up).reshape(shape[0], 1), shape[1]), want, None, label)
    for label, (depth, rows, cols), up, want in RV.TRANSPOSE_REVERSE:
        # the reverse of a transposition transposes the upstream gradient (cols x rows per slice) back
        up = np.array(up, np.float64).reshape(depth, cols, rows)
        got = np.stack([O.transpose(up[d]) for d in range(depth)])
        RV.check(got, want, None, label)


def test_tensor_matmul_shape_rule_and_reverse_relation():
    """Tensor.MatrixMultiply throws on k != other.Shape[0] (src/PRAD/Tensor.cs:582-585); the reverse is the
    NT / TN pair of TensorReverse.cs:118-156 (no known-answer test exists in the reference for it)."""
    r = rng(5)
    a, b, dc = r.standard_normal((7, 5)), r.standard_normal((5, 3)), r.standard_normal((7, 3))
    with pytest.raises(ValueError, match="Incompatible shapes"):
        O.tensor_matmul(a, r.standard_normal((4, 3)))
    np.testing.assert_allclose(O.tensor_matmul(a, b, alpha=2.0), 2.0 * (a @ b), rtol=1e-13)
    da, db = O.tensor_matmul_reverse(a, b, dc)
    np.testing.assert_allclose(da, dc @ b.T, rtol=1e-13)
    np.testing.assert_allclose(db, a.T @ dc, rtol=1e-13)


def test_tile_reverse_specialised_rows_case_is_reproduced_as_written():
    # multiples {2, 1} on a 2 x 2 tensor: the specialised routine adds upstream rows (0, 1) into row 0 and
    # (2, 3) into row 1, not rows (0, 2) and (1, 3) as the tiling layout would suggest
    up = np.arange(8.0).reshape(4, 2)
    np.testing.assert_array_equal(O.tensor_tile_reverse(up, (2, 2), (2, 1)), np.array([[2.0, 4.0], [10.0, 12.0]]))


@pytest.mark.parametrize("name", ["f32", "f64"])
def test_oracle_reproduces_committed_golden_vectors(name):
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN_DIR, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    fresh = mod.make(np.float32 if name == "f32" else np.float64)
    gold = load_golden(name)
    assert set(fresh) == set(gold.keys())
    for k in fresh:
        np.testing.assert_array_equal(fresh[k], gold[k], err_msg=k)
