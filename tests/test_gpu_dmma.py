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


@pytest.mark.parametrize("case", [(100, 2048, 130, 1), (128, 2048, 256, 4), (64, 3000, 66, 3), (33, 1024, 17, 2)])
def test_dmma_few_tiles_over_a_long_k_are_cut_into_slices(dmma_engine, case):
    """Outputs of a few tiles over k >= 1024 (the time-batched weight gradients of an LSTM) run as k slices
    into scratch plus an ordered sum: one launch more, the same values, alpha and beta applied once, batches with
    their own strides and a shared right operand."""
    eng = dmma_engine
    M, K, N, batch = case
    r = rng(sum(case))
    At = normal(r, (batch, K, M), 1.0, np.float64)          # A^T per batch: the product is At^T B
    B = normal(r, (K, N), 1.0, np.float64)                  # shared by every batch (stride 0)
    C0 = normal(r, (batch, M, N), 1.0, np.float64)
    a, b, c = eng.upload(At), eng.upload(B), eng.upload(C0)
    n0 = eng.launch_count()
    eng.gemm(a, b, c, transA=True, alpha=0.25, beta=1.0, M=M, N=N, K=K, lda=M, ldb=N, ldc=N, batch=batch,
             strideA=K * M, strideB=0, strideC=M * N)
    assert eng.launch_count() == n0 + 2
    ref = np.stack([C0[i] + 0.25 * (At[i].T @ B) for i in range(batch)])
    mag = np.stack([np.abs(C0[i]) + 0.25 * (np.abs(At[i].T) @ np.abs(B)) for i in range(batch)])
    assert_close(c.numpy(), ref, mag, "sliced At^T B")
    # the other transpose forms through the public forward / backward of one product
    A = uniform(r, (M, K), -1, 1, np.float64)
    W = normal(r, (K, N), np.sqrt(2.0 / K), np.float64)
    assert_close(eng.matmul_forward(eng.upload(A), eng.upload(W)).numpy(), O.matmul_forward(A, W),
                 np.abs(A) @ np.abs(W), "sliced A W")
    d = normal(r, (N, K), 1.0, np.float64)
    X = normal(r, (M, K), 1.0, np.float64)
    out = eng.empty((M, N), np.float64)
    eng.gemm(eng.upload(X), eng.upload(d), out, transB=True, M=M, N=N, K=K, lda=K, ldb=K, ldc=N)
    assert_close(out.numpy(), X @ d.T, np.abs(X) @ np.abs(d.T), "sliced X d^T")
