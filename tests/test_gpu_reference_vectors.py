"""The reference's own known-answer vectors (reference_vectors.py) through the CUDA entry points of the
PRAD Tensor family: prad_tensor_unary/binary(+reverse), prad_tensor_gather(+reverse),
prad_tensor_tile(+reverse), prad_row_sum_backward (SumRowsReverse), prad_transpose (TransposeReverse),
prad_tensor_matmul(+reverse); plus randomised comparisons with the CPU oracle for the new entry points."""
import numpy as np
import pytest

import oracle as O
import reference_vectors as RV
from parallelreverseautodiff_b200 import _lib
from util import assert_close, rng

pytestmark = pytest.mark.gpu


def _up(engine, a, dtype=np.float64, shape=None):
    a = np.asarray(a, dtype)
    return engine.upload(a.reshape(shape) if shape is not None else a.reshape(1, -1))


@pytest.mark.parametrize("case", RV.BINARY_REVERSE, ids=lambda c: c[0].split()[-1])
def test_binary_reverse_vectors(engine, case):
    label, op, a, b, up, want_a, want_b, places = case
    da, db = engine.tensor_binary_reverse(op, _up(engine, a), _up(engine, b), _up(engine, up))
    RV.check(da.numpy(), want_a, places, label)
    RV.check(db.numpy(), want_b, places, label)


@pytest.mark.parametrize("case", RV.BINARY_FORWARD, ids=lambda c: c[0].split()[-1])
def test_binary_forward_vectors(engine, case):
    label, op, a, b, want, places = case
    RV.check(engine.tensor_binary(op, _up(engine, a), _up(engine, b)).numpy(), want, places, label)


@pytest.mark.parametrize("case", RV.UNARY_REVERSE, ids=lambda c: c[0].split()[-2] + c[0].split()[-1])
def test_unary_reverse_vectors(engine, case):
    label, op, x, up, want, places = case
    RV.check(engine.tensor_unary_reverse(op, _up(engine, x), _up(engine, up)).numpy(), want, places, label)


@pytest.mark.parametrize("case", RV.UNARY_FORWARD, ids=lambda c: c[0].split()[-1])
def test_unary_forward_vectors(engine, case):
    label, op, x, want, places = case
    RV.check(engine.tensor_unary(op, _up(engine, x)).numpy(), want, places, label)


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("case", RV.GATHER, ids=lambda c: c[0].split()[-1])
def test_gather_vectors(engine, case, dtype):
    label, shape, table, idx, want, up, want_rev = case
    x = _up(engine, table, dtype, shape)
    i = _up(engine, idx, dtype, (len(idx),))
    RV.check(engine.tensor_gather(x, i).numpy(), want, None, label)
    u = _up(engine, up, dtype, (len(idx), shape[1]))
    RV.check(engine.tensor_gather_reverse(u, i, shape).numpy(), want_rev, None, label)


@pytest.mark.parametrize("case", RV.TILE_REVERSE, ids=lambda c: c[0].split()[1])
def test_tile_reverse_vectors(engine, case):
    label, shape, mult, up, want = case
    u = _up(engine, up, np.float64, (shape[0] * mult[0], shape[1] * mult[1]))
    RV.check(engine.tensor_tile_reverse(u, shape, mult).numpy(), want, None, label)


@pytest.mark.parametrize("case", RV.TILE_FORWARD, ids=lambda c: c[0].split()[-1])
def test_tile_forward_vectors(engine, case):
    label, shape, x, mult, want = case
    RV.check(engine.tensor_tile(_up(engine, x, np.float64, shape), mult).numpy(), want, None, label)


def test_sum_rows_and_transpose_reverse_vectors(engine):
    label, shape, up, want = RV.SUM_ROWS_REVERSE
    RV.check(engine.row_sum_backward(_up(engine, up, np.float64, (shape[0], 1)), shape[1]).numpy(), want, None, label)
    for label, (depth, rows, cols), up, want in RV.TRANSPOSE_REVERSE:
        u = _up(engine, up, np.float64, (depth, cols, rows) if depth > 1 else (cols, rows))
        RV.check(engine.transpose(u).numpy(), want, None, label)


# ---------------------------------------------------------------- against the oracle on random data
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_tensor_matmul_and_reverse(engine, dtype):
    r = rng(11)
    for (m, k, n) in [(7, 5, 3), (64, 96, 48), (1, 33, 1)]:
        a = r.standard_normal((m, k)).astype(dtype)
        b = r.standard_normal((k, n)).astype(dtype)
        dc = r.standard_normal((m, n)).astype(dtype)
        A, B, dC = engine.upload(a), engine.upload(b), engine.upload(dc)
        # the default path for small products is the sequential-order kernel: identical bits to the oracle's loops
        np.testing.assert_array_equal(engine.tensor_matmul(A, B).numpy(), O.tensor_matmul(a, b))
        assert_close(engine.tensor_matmul(A, B, alpha=0.5).numpy(), O.tensor_matmul(a, b, alpha=0.5),
                     np.abs(a) @ np.abs(b), "Tensor.MatrixMultiply alpha")
        da, db = engine.tensor_matmul_reverse(A, B, dC)
        ra, rb = O.tensor_matmul_reverse(a, b, dc)
        np.testing.assert_array_equal(da.numpy(), ra)
        np.testing.assert_array_equal(db.numpy(), rb)
    with pytest.raises(_lib.PradError) as e:
        engine.tensor_matmul(engine.upload(np.zeros((3, 4), dtype)), engine.upload(np.zeros((5, 2), dtype)))
    assert e.value.status == _lib.ERR_SHAPE and "Incompatible shapes" in str(e.value)


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("shape,axis,count", [((50, 7), 0, 33), ((6, 40, 5), 1, 64), ((4, 9), 1, 9), ((3000, 16), 0, 5000)])
def test_tensor_gather_and_ordered_reverse(engine, dtype, shape, axis, count):
    r = rng(count)
    x = r.standard_normal(shape).astype(dtype)
    n = shape[axis]
    idx = r.integers(-n, n, count).astype(dtype)          # negative indices count from the end; duplicates abound
    X, I = engine.upload(x), engine.upload(idx.reshape(1, -1))
    y = engine.tensor_gather(X, I.view((count,)), axis)
    ref = O.tensor_gather(x, idx, axis)
    np.testing.assert_array_equal(y.numpy(), ref)
    up = (r.standard_normal(ref.shape) * 1e3).astype(dtype)   # large spread: the order of the additions shows
    dx = engine.tensor_gather_reverse(engine.upload(up), I.view((count,)), shape, axis)
    np.testing.assert_array_equal(dx.numpy(), O.tensor_gather_reverse(up, idx, shape, axis))


def test_tensor_gather_rejects_an_index_outside_the_axis(engine):
    X = engine.upload(np.zeros((4, 3)))
    I = engine.upload(np.array([[0.0, 4.0]])).view((2,))
    with pytest.raises(_lib.PradError) as e:
        engine.tensor_gather(X, I, 0)
    assert e.value.status == _lib.ERR_INVALID and "out of bounds" in str(e.value)


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("shape,mult", [((5, 7), (3, 2)), ((4, 6), (5, 1)), ((6, 3), (1, 4)), ((1, 9), (2, 1)), ((3, 3), (1, 1))])
def test_tensor_tile_and_reverse(engine, dtype, shape, mult):
    r = rng(3)
    x = r.standard_normal(shape).astype(dtype)
    np.testing.assert_array_equal(engine.tensor_tile(engine.upload(x), mult).numpy(), O.tensor_tile(x, mult))
    up = (r.standard_normal((shape[0] * mult[0], shape[1] * mult[1])) * 1e3).astype(dtype)
    np.testing.assert_array_equal(engine.tensor_tile_reverse(engine.upload(up), shape, mult).numpy(),
                                  O.tensor_tile_reverse(up, shape, mult))
