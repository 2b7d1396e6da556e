"""The FP64 tensor-core GEMM (DMMA, mma.sync m8n8k4) against the CPU oracle: every transpose
form, ragged shapes, strided batches and the fused epilogues, within 1e-12 relative plus
1e-14 times the magnitude of the summed terms."""
import numpy as np
import pytest

import oracle as O
from parallelreverseautodiff_b200 import engine as E
from util import assert_close, normal, rng, uniform

pytestmark = pytest.mark.gpu


@pytest.fixture()
def dmma_engine(engine):
    engine.set_option("gemm_f64", "dmma")
    yield engine
    engine.set_option("gemm_f64", "auto")


@pytest.mark.parametrize("shape", [(1, 1, 1), (7, 5, 3), (64, 64, 64), (65, 17, 63), (130, 257, 100),
                                   (512, 784, 256), (300, 1, 17)])
def test_dmma_matmul_forward_backward(dmma_engine, shape):
    eng = dmma_engine
    M, K, N = shape
    r = rng(sum(shape))
    A = uniform(r, (M, K), -1, 1, np.float64)
    B = normal(r, (K, N), np.sqrt(2.0 / K), np.float64)
    dC = normal(r, (M, N), 1.0, np.float64)
    a, b, dc = eng.upload(A), eng.upload(B), eng.upload(dC)
    assert_close(eng.matmul_forward(a, b).numpy(), O.matmul_forward(A, B), np.abs(A) @ np.abs(B), "C")
    dA, dB = eng.matmul_backward(a, b, dc)
    dA_ref, dB_ref = O.matmul_backward(A, B, dC)
    assert_close(dA.numpy(), dA_ref, np.abs(dC) @ np.abs(B.T), "dA")
    assert_close(dB.numpy(), dB_ref, np.abs(A.T) @ np.abs(dC), "dB")


def test_dmma_batched_and_epilogue(dmma_engine):
    eng = dmma_engine
    r = rng(5)
    depth, M, K, N = 9, 49, 32, 49
    A, B, dC = normal(r, (depth, M, K), 1, np.float64), normal(r, (depth, K, N), 1, np.float64), normal(r, (depth, M, N), 1, np.float64)
    a, b, dc = eng.upload(A), eng.upload(B), eng.upload(dC)
    assert_close(eng.batch_matmul_forward(a, b).numpy(), O.batch_matmul_forward(A, B), 40.0, "bmm")
    dA, dB, _ = eng.batch_matmul_backward(a, b, dc)
    dA_ref, dB_ref = O.batch_matmul_backward(A, B, dC)
    assert_close(dA.numpy(), dA_ref, 60.0, "bmm dA")
    assert_close(dB.numpy(), dB_ref, 60.0, "bmm dB")
    Zb = normal(r, (77, 130), 1.0, np.float64)
    Aa = O.tanh_forward(Zb)
    W = normal(r, (130, 64), 0.1, np.float64)
    d = normal(r, (77, 64), 1.0, np.float64)
    dA_ref, _ = O.matmul_backward(Aa, W, d, need_dB=False)
    dZ, _ = eng.matmul_backward(eng.upload(Aa), eng.upload(W), eng.upload(d), need_dB=False,
                                act_below=E.ACT_TANH, saved_below=eng.upload(Aa))
    assert_close(dZ.numpy(), O.tanh_backward(Aa, dA_ref), np.abs(d) @ np.abs(W.T), "dA * tanh'")


@pytest.mark.parametrize("shape", [(1536, 300, 1664), (1540, 131, 1667), (2048, 16, 1280), (1664, 1030, 1537)])
def test_dmma_large_tiles_with_the_asynchronous_ring(dmma_engine, shape):
    """Shapes with at least one 128 x 128 tile per SM take the cp.async kernel: ragged edges, odd pitches
    (8-byte copies), k shorter than the ring, all three transpose forms of forward and backward."""
    eng = dmma_engine
    M, K, N = shape
    r = rng(sum(shape))
    A = uniform(r, (M, K), -1, 1, np.float64)
    B = normal(r, (K, N), np.sqrt(2.0 / K), np.float64)
    dC = normal(r, (M, N), 1.0, np.float64)
    a, b, dc = eng.upload(A), eng.upload(B), eng.upload(dC)
    n0 = eng.launch_count()
    assert_close(eng.matmul_forward(a, b).numpy(), O.matmul_forward(A, B), np.abs(A) @ np.abs(B), "C (async dmma)")
    assert eng.launch_count() == n0 + 1
    dA, dB = eng.matmul_backward(a, b, dc)
    dA_ref, dB_ref = O.matmul_backward(A, B, dC)
    assert_close(dA.numpy(), dA_ref, np.abs(dC) @ np.abs(B.T), "dA (async dmma)")
    if K >= 128:      # dB is K x N: it takes the large tiles only when K fills one
        assert_close(dB.numpy(), dB_ref, np.abs(A.T) @ np.abs(dC), "dB (async dmma)")
    # bias + pre-activation copy + activation in the epilogue, and beta
    bias = normal(r, (1, N), 1.0, np.float64)
    z = O.add_broadcast_forward(O.matmul_forward(A, B), bias)
    Z = eng.empty((M, N), np.float64)
    Y = eng.matmul_forward(a, b, bias=eng.upload(bias), Z_out=Z, act=E.ACT_TANH)
    assert_close(Z.numpy(), z, np.abs(A) @ np.abs(B) + 1.0, "Z (async dmma)")
    assert_close(Y.numpy(), O.tanh_forward(z), np.abs(A) @ np.abs(B) + 1.0, "tanh Z (async dmma)")
