"""Size-independent properties of the backward GEMMs at the benchmark's full layer size
(65536 x 4096 activations, 4096 x 4096 weights, float32, tensor-core path), where the CPU
oracle's naive loops would take minutes:

  * column sums:   1^T dA = (1^T dC) W^T         (dA = dC W^T)
  * probe vector:  dW v  = A^T (dC v)            (dW = A^T dC)
  * linearity:     backward(2 dC) = 2 backward(dC), exactly (power-of-two scaling)
  * determinism:   two runs give identical bits
  * the Adam / clip step is idempotent where it must be (global-norm clip of an already
    clipped set changes nothing beyond rounding)
"""
import numpy as np
import pytest

from parallelreverseautodiff_b200 import engine as E

pytestmark = pytest.mark.gpu

ROWS, WIDTH = 65536, 4096


@pytest.fixture(scope="module")
def layer(engine):
    f = np.float32
    r = np.random.default_rng(42)
    A = engine.empty((ROWS, WIDTH), f)
    dC = engine.empty((ROWS, WIDTH), f)
    blk = 8192
    for r0 in range(0, ROWS, blk):
        engine.upload(r.standard_normal((blk, WIDTH), dtype=f), out=A.view((blk, WIDTH), r0 * WIDTH))
        engine.upload(r.standard_normal((blk, WIDTH), dtype=f), out=dC.view((blk, WIDTH), r0 * WIDTH))
    Wh = (r.standard_normal((WIDTH, WIDTH)) * np.sqrt(2.0 / WIDTH)).astype(f)
    W = engine.upload(Wh)
    dA = engine.empty((ROWS, WIDTH), f)
    dW = engine.empty((WIDTH, WIDTH), f)
    n0 = engine.launch_count()
    engine.matmul_backward(A, W, dC, dA=dA, dB=dW)
    # tensor-core path: 2 x (2 operand splits + GEMM) (+ split-K combine); the FP16 scheme adds a
    # column-maximum pass before each of the two transposing splits of the dW product
    assert engine.launch_count() - n0 in (6, 7, 8, 9)
    engine.sync()
    return dict(A=A, dC=dC, W=W, Wh=Wh, dA=dA, dW=dW)


def test_column_sums_of_dA(engine, layer):
    cs_dC = engine.add_broadcast_backward(layer["dC"]).numpy().astype(np.float64)      # 1^T dC
    cs_dA = engine.add_broadcast_backward(layer["dA"]).numpy().astype(np.float64)      # 1^T dA
    want = cs_dC @ layer["Wh"].astype(np.float64).T
    # each entry of 1^T dA sums 65536 * 4096 products of size ~0.02: rounding of the float
    # results enters as ~1e-6 of sqrt(count) * typical magnitude
    scale = np.abs(cs_dC) @ np.abs(layer["Wh"].astype(np.float64)).T
    assert np.abs(cs_dA - want).max() <= 1e-5 * scale.max()
    assert np.abs(cs_dA - want).max() <= 2e-4 * np.abs(want).max()


def test_probe_vector_through_dW(engine, layer):
    f = np.float32
    v = engine.upload(np.random.default_rng(7).standard_normal((WIDTH, 1)).astype(f))
    engine.set_option("gemm_f32", "simt")       # small products: bit-exact FP32 kernels
    try:
        dCv = engine.empty((ROWS, 1), f)
        engine.gemm(layer["dC"], v, dCv)                                # dC v
        rhs = engine.empty((WIDTH, 1), f)
        engine.gemm(layer["A"], dCv, rhs, transA=True)                  # A^T (dC v)
        lhs = engine.empty((WIDTH, 1), f)
        engine.gemm(layer["dW"], v, lhs)                                # dW v
    finally:
        engine.set_option("gemm_f32", "auto")
    a, b = lhs.numpy().astype(np.float64), rhs.numpy().astype(np.float64)
    assert np.abs(a - b).max() <= 1e-5 * np.abs(b).max() * 10           # 10 = sum|terms| / |sum| headroom


def test_linearity_and_determinism(engine, layer):
    f = np.float32
    rows = 8192                                                          # a 128 MiB slice is enough
    A = layer["A"].view((rows, WIDTH))
    dC = layer["dC"].view((rows, WIDTH))
    dA1 = engine.empty((rows, WIDTH), f)
    dW1 = engine.empty((WIDTH, WIDTH), f)
    engine.matmul_backward(A, layer["W"], dC, dA=dA1, dB=dW1)
    dA2 = engine.empty((rows, WIDTH), f)
    dW2 = engine.empty((WIDTH, WIDTH), f)
    engine.matmul_backward(A, layer["W"], dC, dA=dA2, dB=dW2)
    a1, w1 = dA1.numpy(), dW1.numpy()
    np.testing.assert_array_equal(a1, dA2.numpy())
    np.testing.assert_array_equal(w1, dW2.numpy())
    dC2 = engine.scale(dC, 2.0)
    engine.matmul_backward(A, layer["W"], dC2, dA=dA2, dB=dW2)
    np.testing.assert_array_equal(dA2.numpy(), a1 * f(2))                # scaling by 2 is exact everywhere
    np.testing.assert_array_equal(dW2.numpy(), w1 * f(2))


def test_global_norm_clip_is_idempotent(engine, layer):
    g = [engine.clone(layer["dW"])]
    n1 = engine.clip_global_norm(g, 4.0)
    once = g[0].numpy()
    n2 = engine.clip_global_norm(g, 4.0)
    assert n1 > 4.0 and n2 <= 4.0 * (1 + 1e-6)
    # the second pass sees a norm of 4 up to rounding: it may rescale by 1 +- 1e-7 at most
    np.testing.assert_allclose(g[0].numpy(), once, rtol=1e-6, atol=0)
