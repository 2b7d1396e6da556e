"""The tensor-core FP32 GEMM (3xTF32 on tcgen05) against the CPU oracle, forced on for shapes
of every raggedness, for all transpose forms and the fused epilogues."""
import numpy as np
import pytest

import oracle as O
from parallelreverseautodiff_b200 import engine as E
from util import assert_close, normal, rng, uniform

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["tf32x3", "tf32b16", "bf16x3", "fp16x3"])
def tc_engine(engine, request):
    """Every split scheme: three TF32 products; one TF32 product + two BF16 corrections; six
    BF16 products of three-piece operands; three FP16 products of row-scaled two-piece operands."""
    engine.set_option("gemm_f32", request.param)
    yield engine
    engine.set_option("gemm_f32", "auto")


SHAPES = [(128, 32, 256), (128, 64, 256), (256, 96, 512), (200, 70, 300), (129, 33, 257),
          (1, 5, 3), (384, 1000, 130), (512, 784, 256), (8200, 300, 260)]


@pytest.mark.parametrize("shape", SHAPES)
def test_tf32x3_matmul_forward_backward(tc_engine, shape):
    eng = tc_engine
    M, K, N = shape
    r = rng(sum(shape))
    A = uniform(r, (M, K), -1, 1, np.float32)
    B = normal(r, (K, N), np.sqrt(2.0 / K), np.float32)
    dC = normal(r, (M, N), 1.0, np.float32)
    a, b, dc = eng.upload(A), eng.upload(B), eng.upload(dC)
    n0 = eng.launch_count()
    C = eng.matmul_forward(a, b).numpy()
    dA, dB = eng.matmul_backward(a, b, dc)
    # 3 products x (2 operand passes + 1 GEMM) (+ split-K combine); the FP16 scheme packs ragged
    # operands with one launch for the interior tiles, one for a partly filled last column tile and
    # one for what is left at the edges
    assert 9 <= eng.launch_count() - n0 <= 24
    assert_close(C, O.matmul_forward(A, B), np.abs(A).astype(np.float64) @ np.abs(B), "C")
    dA_ref, dB_ref = O.matmul_backward(A, B, dC)
    assert_close(dA.numpy(), dA_ref, np.abs(dC).astype(np.float64) @ np.abs(B.T), "dA")
    assert_close(dB.numpy(), dB_ref, np.abs(A.T).astype(np.float64) @ np.abs(dC), "dB")


def test_tf32x3_is_as_accurate_as_fp32_fma(tc_engine):
    """Error against an exact (float64) product is of FP32 size, not of TF32 size."""
    eng = tc_engine
    r = rng(1)
    M, K, N = 256, 2048, 256
    A, B = normal(r, (M, K), 1, np.float32), normal(r, (K, N), 1, np.float32)
    exact = A.astype(np.float64) @ B.astype(np.float64)
    got = eng.matmul_forward(eng.upload(A), eng.upload(B)).numpy().astype(np.float64)
    rel = np.abs(got - exact).max() / np.abs(exact).max()
    assert rel < 5e-6, rel          # plain TF32 would be ~1e-3


def test_tf32x3_epilogues(tc_engine):
    eng = tc_engine
    r = rng(2)
    M, K, N = 256, 160, 384
    Zb = normal(r, (M, K), 1.0, np.float32)
    A = O.gelu_forward(Zb)
    B = normal(r, (K, N), 0.1, np.float32)
    dC = normal(r, (M, N), 1.0, np.float32)
    dA_ref, dB_ref = O.matmul_backward(A, B, dC)
    dZ, _ = eng.matmul_backward(eng.upload(A), eng.upload(B), eng.upload(dC), need_dB=False,
                                act_below=E.ACT_GELU, saved_below=eng.upload(Zb))
    bound = (np.abs(dC).astype(np.float64) @ np.abs(B.T)) * 1.2
    assert_close(dZ.numpy(), O.gelu_backward(Zb, dA_ref), bound, "dA * gelu'")
    dest = normal(r, (K, N), 1, np.float32)
    d = eng.upload(dest)
    eng.matmul_backward(eng.upload(A), eng.upload(B), eng.upload(dC), dB=d, need_dA=False,
                        accumulate_dB=True, dB_scale=0.5)
    assert_close(d.numpy(), (dest + dB_ref * np.float32(0.5)).astype(np.float32),
                 np.abs(A.T).astype(np.float64) @ np.abs(dC) + np.abs(dest), "dB accumulate")
    bias = normal(r, (1, N), 1, np.float32)
    Zf = eng.empty((M, N), np.float32)
    Y = eng.matmul_forward(eng.upload(A), eng.upload(B), bias=eng.upload(bias), Z_out=Zf,
                           act=E.ACT_LEAKY_RELU, act_alpha=0.01)
    z_ref = O.add_broadcast_forward(O.matmul_forward(A, B), bias)
    bound = np.abs(A).astype(np.float64) @ np.abs(B) + 1.0
    assert_close(Zf.numpy(), z_ref, bound, "Z")
    assert_close(Y.numpy(), O.leaky_relu_forward(z_ref, 0.01), bound, "Y")


def test_tf32x3_deterministic(tc_engine):
    eng = tc_engine
    r = rng(3)
    A, B = normal(r, (300, 200), 1, np.float32), normal(r, (200, 280), 1, np.float32)
    a, b = eng.upload(A), eng.upload(B)
    np.testing.assert_array_equal(eng.matmul_forward(a, b).numpy(), eng.matmul_forward(a, b).numpy())


def _fp16x3_bound(P, Q):
    """Error scale of P @ Q under the FP16 scheme: the usual sum |p||q| of a float product plus
    what the narrow FP16 exponent adds -- an element more than ~8 decades below the largest of
    its row (along k) keeps fewer than 22 bits, at worst an absolute 2^-39 of that largest
    magnitude; times the other operand's largest magnitude and sqrt(k) for the sum.  (The 1e-5
    of the float tolerance is applied on top, hence 2^-39 / 1e-5 ~ 2e-7.)"""
    P, Q = np.abs(P).astype(np.float64), np.abs(Q).astype(np.float64)
    return P @ Q + 2e-7 * np.sqrt(P.shape[1]) * np.outer(P.max(axis=1), Q.max(axis=0))


@pytest.mark.parametrize("shape", [(256, 512, 256), (130, 333, 257)])
def test_fp16x3_row_scaling_over_the_float_range(engine, shape):
    """Rows of A and columns of B spread over 40 decades: the power-of-two row scaling keeps
    every output element at FP32 accuracy relative to its own |A||B| bound, up to the stated
    range term where one k carries a huge factor in one operand and a tiny one in the other."""
    engine.set_option("gemm_f32", "fp16x3")
    try:
        M, K, N = shape
        r = rng(11)
        A = (normal(r, (M, K), 1, np.float64) * 10.0 ** r.uniform(-12, 12, (M, 1))).astype(np.float32)
        A[5] = normal(r, (K,), 1, np.float64) * 1e29      # a row near the top of the float range ...
        A[6] = normal(r, (K,), 1, np.float64) * 1e-28     # ... and one near the bottom (products stay normal floats)
        B = (normal(r, (K, N), 1, np.float64) * 10.0 ** r.uniform(-7, 7, (1, N))).astype(np.float32)
        A[3] = 0                     # an all-zero row stays zero
        dC = (normal(r, (M, N), 1, np.float64) * 10.0 ** r.uniform(-5, 5, (M, 1))).astype(np.float32)
        a, b, dc = engine.upload(A), engine.upload(B), engine.upload(dC)
        C = engine.matmul_forward(a, b).numpy()
        assert not C[3].any()
        # forward: the spread is across rows of A and columns of B only, never along k
        assert_close(C, O.matmul_forward(A, B), np.abs(A).astype(np.float64) @ np.abs(B), "C")
        dA, dB = engine.matmul_backward(a, b, dc)
        dA_ref, dB_ref = O.matmul_backward(A, B, dC)
        assert_close(dA.numpy(), dA_ref, _fp16x3_bound(dC, B.T), "dA")
        assert_close(dB.numpy(), dB_ref, _fp16x3_bound(A.T, dC), "dB")
        # the TF32 + BF16 scheme has the full float exponent in every piece: plain bound
        engine.set_option("gemm_f32", "tf32b16")
        dA, dB = engine.matmul_backward(a, b, dc)
        assert_close(dA.numpy(), dA_ref, np.abs(dC).astype(np.float64) @ np.abs(B.T), "dA (tf32b16)")
        assert_close(dB.numpy(), dB_ref, np.abs(A.T).astype(np.float64) @ np.abs(dC), "dB (tf32b16)")
    finally:
        engine.set_option("gemm_f32", "auto")
