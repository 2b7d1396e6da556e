"""GPU parity: every kernel family of libprad_cuda against the CPU oracle, through the C ABI.

Inputs are seeded; sizes are small enough for the oracle to finish in seconds and include
the ragged shapes (1, 7, 8, 9, 63, 64, 65, ...) that exercise tile edges.
"""
import numpy as np
import pytest

import oracle as O
from parallelreverseautodiff_b200 import engine as E
from util import assert_close, normal, rms, rng, uniform

pytestmark = pytest.mark.gpu

DTYPES = [np.float64, np.float32]
ACTS = {
    "leaky": (E.ACT_LEAKY_RELU, 0.01),
    "sigmoid": (E.ACT_SIGMOID, 0.0),
    "tanh": (E.ACT_TANH, 0.0),
    "gelu": (E.ACT_GELU, 0.0),
    "relu": (E.ACT_RELU, 0.0),
    "ampsig": (E.ACT_AMPLIFIED_SIGMOID, 0.0),
}


def _act_oracle(name, x, alpha):
    fwd = {"leaky": lambda v: O.leaky_relu_forward(v, alpha), "sigmoid": O.sigmoid_forward,
           "tanh": O.tanh_forward, "gelu": O.gelu_forward, "relu": O.relu_forward,
           "ampsig": O.amplified_sigmoid_forward}[name]
    return fwd(x)


def _act_oracle_bwd(name, x, y, dy, alpha):
    if name == "leaky":
        return O.leaky_relu_backward(x, dy, alpha)
    if name == "sigmoid":
        return O.sigmoid_backward(y, dy)
    if name == "tanh":
        return O.tanh_backward(y, dy)
    if name == "relu":
        return O.relu_backward(x, dy)
    if name == "ampsig":
        return O.amplified_sigmoid_backward(x, dy)
    return O.gelu_backward(x, dy)


GEMM_SHAPES = [(1, 1, 1), (7, 5, 3), (8, 9, 63), (64, 65, 33), (65, 64, 129), (130, 257, 100),
               (512, 784, 256), (256, 512, 10), (300, 1, 17), (1, 300, 1)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", GEMM_SHAPES)
def test_matmul_forward_backward(engine, dtype, shape):
    M, K, N = shape
    r = rng(hash(shape) % 1000)
    A = uniform(r, (M, K), -1, 1, dtype)
    B = normal(r, (K, N), np.sqrt(2.0 / K), dtype)
    dC = normal(r, (M, N), 1.0, dtype)
    dA_ref, dB_ref = O.matmul_backward(A, B, dC)
    C_ref = O.matmul_forward(A, B)
    dA_, dB_, dC_ = engine.upload(A), engine.upload(B), engine.upload(dC)
    Cg = engine.matmul_forward(dA_, dB_).numpy()
    gA, gB = engine.matmul_backward(dA_, dB_, dC_)
    # default SIMT path: products and sums rounded separately in k order == the C# loop, bit for bit
    np.testing.assert_array_equal(Cg, C_ref)
    np.testing.assert_array_equal(gA.numpy(), dA_ref)
    np.testing.assert_array_equal(gB.numpy(), dB_ref)
    # the FMA variant of the same kernel agrees within the tolerance
    engine.set_option("gemm_f32", "simt_fma")
    engine.set_option("gemm_f64", "simt_fma")
    try:
        fA, fB = engine.matmul_backward(dA_, dB_, dC_)
        assert_close(fA.numpy(), dA_ref, np.abs(dC).astype(np.float64) @ np.abs(B.T), "dA (fma)")
        assert_close(fB.numpy(), dB_ref, np.abs(A.T).astype(np.float64) @ np.abs(dC), "dB (fma)")
    finally:
        engine.set_option("gemm_f32", "auto")
        engine.set_option("gemm_f64", "auto")


@pytest.mark.parametrize("dtype", DTYPES)
def test_matmul_backward_accumulate_and_scale(engine, dtype):
    r = rng(5)
    M, K, N = 96, 70, 45
    A, B, dC = normal(r, (M, K), 1, dtype), normal(r, (K, N), 1, dtype), normal(r, (M, N), 1, dtype)
    dest = normal(r, (K, N), 1, dtype)
    _, dB_ref = O.matmul_backward(A, B, dC, need_dA=False)
    expect = (dest + dB_ref * dtype(0.25)).astype(dtype)
    d = engine.upload(dest)
    engine.matmul_backward(engine.upload(A), engine.upload(B), engine.upload(dC), dB=d,
                           need_dA=False, accumulate_dB=True, dB_scale=0.25)
    assert_close(d.numpy(), expect, np.abs(A.T).astype(np.float64) @ np.abs(dC) + np.abs(dest), "dB+=")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", list(ACTS))
def test_matmul_act_backward_node(engine, dtype, act):
    """MatMul -> activation node: dPre, dA, dB (benchmark config 1 is the leaky/float64 case)."""
    code, alpha = ACTS[act]
    r = rng(42)
    M, K, N = 128, 200, 72
    A = uniform(r, (M, K), -1, 1, dtype)
    B = normal(r, (K, N), np.sqrt(2.0 / K), dtype)
    dOut = normal(r, (M, N), 1.0, dtype)
    pre = O.matmul_forward(A, B)
    y = _act_oracle(act, pre, alpha)
    saved = y if act in ("sigmoid", "tanh") else pre
    dPre_ref = _act_oracle_bwd(act, pre, y, dOut, alpha)
    dA_ref, dB_ref = O.matmul_backward(A, B, dPre_ref)
    dPre, dA, dB = engine.matmul_act_backward(engine.upload(A), engine.upload(B), engine.upload(dOut),
                                              code, engine.upload(saved), alpha)
    assert_close(dPre.numpy(), dPre_ref, rms(dPre_ref), "dPre")
    if act in ("leaky", "sigmoid", "relu"):     # dPre is bit-exact for these, and so are the products
        np.testing.assert_array_equal(dA.numpy(), dA_ref)
        np.testing.assert_array_equal(dB.numpy(), dB_ref)
    else:
        assert_close(dA.numpy(), dA_ref, np.abs(dPre_ref).astype(np.float64) @ np.abs(B.T), "dA")
        assert_close(dB.numpy(), dB_ref, np.abs(A.T).astype(np.float64) @ np.abs(dPre_ref), "dB")
    # the host-buffer form of the same node
    hPre, hA, hB = engine.matmul_act_backward_host(A, B, dOut, code, saved, alpha)
    np.testing.assert_array_equal(hPre, dPre.numpy())
    np.testing.assert_array_equal(hA, dA.numpy())
    np.testing.assert_array_equal(hB, dB.numpy())


@pytest.mark.parametrize("dtype", DTYPES)
def test_matmul_backward_fused_activation_below(engine, dtype):
    """dA epilogue multiplies by the derivative of the activation that produced A."""
    r = rng(9)
    M, K, N = 77, 130, 64
    Zb = normal(r, (M, K), 1.0, dtype)          # pre-activation of the layer below
    A = O.gelu_forward(Zb)
    B = normal(r, (K, N), 0.1, dtype)
    dC = normal(r, (M, N), 1.0, dtype)
    dA_ref, _ = O.matmul_backward(A, B, dC, need_dB=False)
    dZ_ref = O.gelu_backward(Zb, dA_ref)
    dZ, _ = engine.matmul_backward(engine.upload(A), engine.upload(B), engine.upload(dC),
                                   need_dB=False, act_below=E.ACT_GELU, saved_below=engine.upload(Zb))
    bound = (np.abs(dC).astype(np.float64) @ np.abs(B.T)) * 1.2
    assert_close(dZ.numpy(), dZ_ref, bound, "dZ")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shared", [False, True])
def test_batch_matmul(engine, dtype, shared):
    r = rng(3)
    depth, M, K, N = 13, 49, 32, 49
    A = normal(r, (depth, M, K), 1, dtype)
    B = normal(r, (K, N) if shared else (depth, K, N), 1, dtype)
    dC = normal(r, (depth, M, N), 1, dtype)
    C_ref = O.batch_matmul_forward(A, B)
    dA_ref, dB_ref = O.batch_matmul_backward(A, B, dC)
    a, b, dc = engine.upload(A), engine.upload(B), engine.upload(dC)
    np.testing.assert_array_equal(engine.batch_matmul_forward(a, b).numpy(), C_ref)
    dA, dB, dBm = engine.batch_matmul_backward(a, b, dc, per_slice_dB=True, mean_dB=shared)
    np.testing.assert_array_equal(dA.numpy(), dA_ref)
    np.testing.assert_array_equal(dB.numpy(), dB_ref)
    if shared:
        mean_ref = O.batch_mean([dB_ref[d] for d in range(depth)])
        assert_close(dBm.numpy(), mean_ref, 60.0, "dB mean")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(49, 32, 49), (49, 49, 32), (64, 64, 64), (5, 150, 7), (1, 1, 1), (33, 70, 64)])
def test_many_small_products_take_one_cta_each(engine, dtype, shape):
    """Strided batches of at least one product per SM with outputs of at most 64 x 64 (the attention products per
    window and head) run on one CTA per product: bit-identical to the oracle's sequential sums and to the tiled
    kernel, in every transpose form, with alpha and beta, addressing slices of wider matrices in place."""
    M, K, N = shape
    r = rng(sum(shape))
    depth = 300
    A = normal(r, (depth, M, K), 1, dtype)
    B = normal(r, (depth, K, N), 1, dtype)
    dC = normal(r, (depth, M, N), 1, dtype)
    a, b, dc = engine.upload(A), engine.upload(B), engine.upload(dC)
    wide_a = np.zeros((depth, M, K + 5), dtype)
    wide_a[:, :, 3:3 + K] = A
    wide_c0 = normal(r, (depth, M, N + 2), 1, dtype)
    results = {}
    for small in ("0", "1"):
        engine.set_option("gemm_small", small)
        try:
            C = engine.batch_matmul_forward(a, b)
            dA, dB, _ = engine.batch_matmul_backward(a, b, dc, per_slice_dB=True)
            # in place: the product of batch i reads columns 3..3+K of a wide A and accumulates into columns 1..1+N of a wide C
            wa, wc = engine.upload(wide_a), engine.upload(wide_c0)
            engine.gemm(wa.view((1, 1), 3), b.view((1, 1), 0), wc.view((1, 1), 1), alpha=0.5, beta=1.0, M=M, N=N, K=K,
                        lda=K + 5, ldb=N, ldc=N + 2, batch=depth, strideA=M * (K + 5), strideB=K * N, strideC=M * (N + 2))
            results[small] = (C.numpy(), dA.numpy(), dB.numpy(), wc.numpy())
        finally:
            engine.set_option("gemm_small", "1")
    C_ref = O.batch_matmul_forward(A, B)
    dA_ref, dB_ref = O.batch_matmul_backward(A, B, dC)
    for small in ("0", "1"):
        C, dA, dB, wc = results[small]
        wc0 = wide_c0
        np.testing.assert_array_equal(C, C_ref)
        np.testing.assert_array_equal(dA, dA_ref)
        np.testing.assert_array_equal(dB, dB_ref)
        half = (np.asarray(0.5, dtype) * C_ref).astype(dtype)
        np.testing.assert_array_equal(wc[:, :, 1:1 + N], wc0[:, :, 1:1 + N] + half)
        np.testing.assert_array_equal(wc[:, :, 0], wc0[:, :, 0])
        np.testing.assert_array_equal(wc[:, :, N + 1], wc0[:, :, N + 1])


@pytest.mark.parametrize("dtype", DTYPES)
def test_matmul_and_sum(engine, dtype):
    r = rng(4)
    n, P = 24, 5
    A = normal(r, (n, n), 1, dtype)
    B = normal(r, (P, n, n), 1, dtype)
    dOut = normal(r, (1, P), 1, dtype)
    out_ref = O.matmul_and_sum_forward(A, B)
    dA_ref, dB_ref = O.matmul_and_sum_backward(A, B, dOut)
    a, b = engine.upload(A), engine.upload(B)
    assert_close(engine.matmul_and_sum_forward(a, b).numpy(), out_ref, 600.0, "out")
    dA, dB = engine.matmul_and_sum_backward(a, b, engine.upload(dOut))
    np.testing.assert_array_equal(dB.numpy(), dB_ref)   # one product per element: exact
    assert_close(dA.numpy(), dA_ref, 5.0, "dA")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", list(ACTS))
@pytest.mark.parametrize("n", [1, 5, 1023, 4096 + 3, 300001])
def test_activation_forward_backward(engine, dtype, act, n):
    code, alpha = ACTS[act]
    r = rng(n)
    x = normal(r, (1, n), 2.0, dtype)
    dy = normal(r, (1, n), 1.0, dtype)
    y_ref = _act_oracle(act, x, alpha)
    dx_ref = _act_oracle_bwd(act, x, y_ref, dy, alpha)
    xd = engine.upload(x)
    y = engine.act_forward(code, xd, alpha)
    assert_close(y.numpy(), y_ref, rms(y_ref), f"{act} forward")
    saved = engine.upload(y_ref) if act in ("sigmoid", "tanh") else xd
    dx = engine.act_backward(code, saved, engine.upload(dy), alpha)
    if act == "relu":
        np.testing.assert_array_equal(y.numpy(), y_ref)
    if act in ("leaky", "sigmoid", "relu"):
        np.testing.assert_array_equal(dx.numpy(), dx_ref)   # same roundings: bit-exact
    else:
        assert_close(dx.numpy(), dx_ref, rms(dx_ref), f"{act} backward")


@pytest.mark.parametrize("dtype", DTYPES)
def test_hadamard_add_scale_transpose(engine, dtype):
    r = rng(11)
    a, b, c, dy = (normal(r, (37, 53), 1, dtype) for _ in range(4))
    A, B, Cc, DY = (engine.upload(v) for v in (a, b, c, dy))
    np.testing.assert_array_equal(engine.hadamard_forward(A, B).numpy(), O.hadamard_forward(a, b))
    da, db = engine.hadamard_backward(A, B, DY)
    da_ref, db_ref = O.hadamard_backward(a, b, dy)
    np.testing.assert_array_equal(da.numpy(), da_ref)
    np.testing.assert_array_equal(db.numpy(), db_ref)
    np.testing.assert_array_equal(engine.add_forward(A, B).numpy(), O.add_forward(a, b))
    np.testing.assert_array_equal(engine.add_forward(A, B, Cc).numpy(), O.add3_forward(a, b, c))
    np.testing.assert_array_equal(engine.scale(A, 1 / np.sqrt(32)).numpy(),
                                  O.scale(a, dtype(1 / np.sqrt(32))))
    np.testing.assert_array_equal(engine.transpose(A).numpy(), O.transpose(a))
    deep = normal(r, (5, 49, 32), 1, dtype)
    np.testing.assert_array_equal(engine.transpose(engine.upload(deep)).numpy(),
                                  np.stack([O.transpose(deep[d]) for d in range(5)]))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 1), (256, 10), (333, 96), (4097, 33), (64, 4096), (20001, 96), (700, 4096), (9000, 130)])
def test_add_broadcast(engine, dtype, shape):
    r = rng(shape[1])
    x, dy = normal(r, shape, 1, dtype), normal(r, shape, 1, dtype)
    bias = normal(r, (1, shape[1]), 1, dtype)
    np.testing.assert_array_equal(
        engine.add_broadcast_forward(engine.upload(x), engine.upload(bias)).numpy(),
        O.add_broadcast_forward(x, bias))
    _, db_ref = O.add_broadcast_backward(dy)
    db = engine.add_broadcast_backward(engine.upload(dy))
    assert_close(db.numpy(), db_ref, np.abs(dy).astype(np.float64).sum(0, keepdims=True), "dBias")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 1), (6, 120), (300, 17), (5, 1000), (2, 4099)])
def test_sine_softmax(engine, dtype, shape):
    """SineSoftmaxOperation: y = e / (sum e + e), e = exp(sin x); Backward reads the input."""
    r = rng(shape[1])
    x, dy = normal(r, shape, 2.0, dtype), normal(r, shape, 1.0, dtype)
    y_ref = O.sine_softmax_forward(x)
    y = engine.sine_softmax_forward(engine.upload(x))
    assert_close(y.numpy(), y_ref, 0.0, "sine softmax")
    dx = engine.sine_softmax_backward(engine.upload(x), engine.upload(dy))
    assert_close(dx.numpy(), O.sine_softmax_backward(x, dy), 0.0, "sine softmax backward")
    assert engine.sine_softmax_forward(engine.empty((0, 5), dtype)).shape == (0, 5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 1), (256, 10), (49 * 12, 49), (7, 1000), (3, 4097)])
def test_softmax(engine, dtype, shape):
    r = rng(shape[0])
    x, dy = normal(r, shape, 2.0, dtype), normal(r, shape, 1.0, dtype)
    y_ref = O.softmax_forward(x)
    dx_ref = O.softmax_backward(y_ref, dy)
    y = engine.softmax_forward(engine.upload(x))
    assert_close(y.numpy(), y_ref, 1.0 / shape[1], "softmax")
    dx = engine.softmax_backward(engine.upload(y_ref), engine.upload(dy))
    # row scale of the Jacobian product: sum_k |dy_k| y_k y_j
    bound = np.abs(y_ref) * (np.abs(dy) + (np.abs(dy) * y_ref).sum(1, keepdims=True))
    assert_close(dx.numpy(), dx_ref, bound.astype(np.float64) + 1e-300, "softmax backward")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 2), (22, 22), (333, 96), (5, 4097), (1001, 49), (7, 300)])
def test_layernorm(engine, dtype, shape):
    r = rng(shape[1])
    x, dy = normal(r, shape, 3.0, dtype) + dtype(0.5), normal(r, shape, 1.0, dtype)
    y_ref, mean_ref, std_ref = O.layernorm_forward(x)
    dx_ref = O.layernorm_backward(x, mean_ref, std_ref, dy)
    y, mean, std = engine.layernorm_forward(engine.upload(x))
    assert_close(mean.numpy(), mean_ref, rms(x), "mean")
    assert_close(std.numpy(), std_ref, rms(x), "std")
    assert_close(y.numpy(), y_ref, 1.0, "layernorm")
    dx = engine.layernorm_backward(engine.upload(x), engine.upload(mean_ref), engine.upload(std_ref),
                                   engine.upload(dy))
    # the two terms of the derivative cancel (completely for 2 columns), so the error scale is
    # the size of the terms, dy/(sigma+eps), not of the result
    assert_close(dx.numpy(), dx_ref, rms(dy / (std_ref[:, None] + 1e-9)), "layernorm backward")


@pytest.mark.parametrize("dtype", DTYPES)
def test_losses(engine, dtype):
    r = rng(21)
    out = normal(r, (256, 10), 1, dtype)
    tgt = normal(r, (256, 10), 1, dtype)
    o, t = engine.upload(out), engine.upload(tgt)
    assert_close(engine.mse_forward(o, t).numpy().reshape(()), np.asarray(O.mse_forward(out, tgt), dtype), 1.0, "mse")
    np.testing.assert_array_equal(engine.mse_backward(o, t).numpy(), O.mse_backward(out, tgt))
    np.testing.assert_array_equal(engine.mse_backward(o, t, rows_total=1024).numpy(),
                                  O.mse_backward(out, tgt, rows_total=1024))
    probs = O.softmax_forward(out)
    onehot = np.eye(10, dtype=dtype)[r.integers(0, 10, 256)]
    p, h = engine.upload(probs), engine.upload(onehot)
    assert_close(engine.cce_forward(p, h).numpy().reshape(()), np.asarray(O.cce_forward(probs, onehot), dtype), 1.0, "cce")
    np.testing.assert_array_equal(engine.cce_backward(p, h).numpy(), O.cce_backward(probs, onehot))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", [(2, 3, 2, "unique"), (1000, 50, 96, "dups"), (5000, 7, 33, "heavy"),
                                  (300, 2000, 8, "sparse"), (9000, 3, 12, "more hits per row than a CTA lists")])
def test_embedding_bit_exact(engine, dtype, case):
    n, vocab, dim, _ = case
    r = rng(n)
    W = normal(r, (vocab, dim), 1, dtype)
    idx = r.integers(0, vocab, n)
    if case[3] == "unique":
        idx = np.array([2, 0])
    col = idx.astype(dtype).reshape(-1, 1)
    dOut = normal(r, (n, dim), 1, dtype)
    icol = engine.upload(col)
    np.testing.assert_array_equal(engine.embedding_forward(icol, engine.upload(W)).numpy(),
                                  O.embedding_forward(col, W))
    np.testing.assert_array_equal(engine.embedding_backward(icol, engine.upload(dOut), vocab).numpy(),
                                  O.embedding_backward(col, dOut, vocab))


def test_embedding_rejects_bad_index(engine):
    from parallelreverseautodiff_b200._lib import PradError
    col = engine.upload(np.array([[0.0], [5.0]], np.float32))
    with pytest.raises(PradError):
        engine.embedding_forward(col, engine.upload(np.zeros((3, 4), np.float32)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("count", [1, 2, 5, 20])
def test_segmented_sum_accumulate_batch_mean(engine, dtype, count):
    r = rng(count)
    gs = [normal(r, (64, 33), 1, dtype) for _ in range(count)]
    dev = [engine.upload(g) for g in gs]
    got = engine.segmented_sum(dev).numpy()
    if count <= 8 or dtype == np.float64:
        np.testing.assert_array_equal(got, O.accumulate_gradients(gs))
    else:
        assert_close(got, O.accumulate_gradients(gs), count, "segmented sum")
    np.testing.assert_array_equal(engine.batch_mean(dev).numpy(), O.batch_mean(gs))
    dest = normal(r, (64, 33), 1, dtype)
    d = engine.upload(dest)
    engine.accumulate(d, dev[0])
    np.testing.assert_array_equal(d.numpy(), O.accumulate_into(dest.copy(), gs[0]))


@pytest.mark.parametrize("dtype", DTYPES)
def test_clip_reference(engine, dtype):
    r = rng(77)
    shapes = [(784, 64), (1, 64), (33, 7), (1, 1), (300, 300)]
    gs = [normal(r, s, 3.0, dtype) for s in shapes]
    gs[2][0, :3] = [1e-20, -1e-20, 0.0]          # minimum-threshold branch
    gs[3][0, 0] = 2.5                            # one element: sigma = 0 -> NaN limit, unchanged
    minv = 1e-16 if dtype == np.float64 else 1e-8
    ref = [O.clip_reference(g.copy(), 4.0, minv) for g in gs]
    dev = [engine.upload(g) for g in gs]
    engine.clip_reference(dev, 4.0, minv)
    for d, e, g in zip(dev, ref, gs):
        got = d.numpy()
        # clamped values are (1+|z|): sensitive to mean/sigma rounding, hence a tolerance
        assert_close(got, e, 1.0, "clip")
        assert (np.abs(got) <= np.abs(g) + minv).all()


@pytest.mark.parametrize("dtype", DTYPES)
def test_clip_global_norm(engine, dtype):
    r = rng(78)
    gs = [normal(r, s, 1.0, dtype) for s in [(100, 50), (1, 50), (50, 10)]]
    ref = [g.copy() for g in gs]
    norm_ref = O.clip_global_norm(ref, 4.0)
    dev = [engine.upload(g) for g in gs]
    norm = engine.clip_global_norm(dev, 4.0)
    assert abs(norm - norm_ref) <= 1e-12 * norm_ref
    for d, e in zip(dev, ref):
        assert_close(d.numpy(), e, rms(e), "global-norm clip")
    small = [engine.upload(g * dtype(1e-3)) for g in gs]
    engine.clip_global_norm(small, 4.0)
    np.testing.assert_array_equal(small[0].numpy(), gs[0] * dtype(1e-3))   # below the limit: untouched


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("form", ["rmad", "prad"])
def test_adam(engine, dtype, form):
    r = rng(79)
    shapes = [(784, 32), (1, 32), (9000,)]
    w = [normal(r, s, 1, dtype) for s in shapes]
    g = [normal(r, s, 0.1, dtype) for s in shapes]
    m = [normal(r, s, 0.01, dtype) for s in shapes]
    v = [np.abs(normal(r, s, 0.01, dtype)) for s in shapes]
    W, G, M_, V = ([engine.upload(a) for a in arrs] for arrs in (w, g, m, v))
    for it in (1, 2, 3):
        for k in range(len(shapes)):
            if form == "rmad":
                O.adam_rmad(w[k], m[k], v[k], g[k], 1e-3, 0.9, 0.999, 1e-8, float(it))
            else:
                O.adam_prad(w[k], m[k], v[k], g[k], 1e-3, 0.9, 0.999, 1e-8, it)
        engine.adam(W, G, M_, V, 1e-3, 0.9, 0.999, 1e-8, float(it),
                    form=E.ADAM_RMAD if form == "rmad" else E.ADAM_PRAD)
    for k in range(len(shapes)):
        # same operations in the same order with IEEE sqrt/div: bit-exact
        np.testing.assert_array_equal(W[k].numpy(), w[k])
        np.testing.assert_array_equal(M_[k].numpy(), m[k])
        np.testing.assert_array_equal(V[k].numpy(), v[k])


@pytest.mark.parametrize("dtype", DTYPES)
def test_clip_adam_fused_equals_separate(engine, dtype):
    r = rng(80)
    shapes = [(300, 40), (1, 40)]
    w0 = [normal(r, s, 1, dtype) for s in shapes]
    g0 = [normal(r, s, 2.0, dtype) for s in shapes]
    zeros = [np.zeros(s, dtype) for s in shapes]
    minv = 1e-16 if dtype == np.float64 else 1e-8
    for mode in (E.CLIP_REFERENCE, E.CLIP_GLOBAL_NORM):
        W1, G1, M1, V1 = ([engine.upload(a) for a in arrs] for arrs in (w0, g0, zeros, zeros))
        if mode == E.CLIP_REFERENCE:
            engine.clip_reference(G1, 4.0, minv)
        else:
            engine.clip_global_norm(G1, 4.0)
        engine.adam(W1, G1, M1, V1, 1e-3, 0.9, 0.999, 1e-8, 1.0)
        W2, G2, M2, V2 = ([engine.upload(a) for a in arrs] for arrs in (w0, g0, zeros, zeros))
        engine.clip_adam(W2, G2, M2, V2, mode, 4.0, minv, 1e-3, 0.9, 0.999, 1e-8, 1.0, zero_grad=True)
        for k in range(len(shapes)):
            np.testing.assert_array_equal(W2[k].numpy(), W1[k].numpy())
            np.testing.assert_array_equal(M2[k].numpy(), M1[k].numpy())
            np.testing.assert_array_equal(V2[k].numpy(), V1[k].numpy())
            assert not G2[k].numpy().any()


def test_jagged_rows_roundtrip(engine):
    r = rng(1)
    rows = [r.standard_normal(17) for _ in range(9)]
    m = engine.upload_rows(rows)
    np.testing.assert_array_equal(m.numpy(), np.stack(rows))
    back = engine.download_rows(m)
    for a, b in zip(rows, back):
        np.testing.assert_array_equal(a, b)


def test_errors_are_status_codes(engine):
    from parallelreverseautodiff_b200._lib import PradError, ERR_SHAPE
    a = engine.upload(np.zeros((4, 5)))
    b = engine.upload(np.zeros((6, 3)))
    with pytest.raises(PradError) as ei:
        engine.matmul_forward(a, b)
    assert ei.value.status == ERR_SHAPE
    with pytest.raises(PradError):
        engine.set_option("gemm_f32", "bogus")


def test_determinism_run_twice(engine):
    r = rng(2)
    A, B, dC = (normal(r, s, 1, np.float32) for s in [(300, 200), (200, 150), (300, 150)])
    a, b, dc = engine.upload(A), engine.upload(B), engine.upload(dC)
    x1 = [t.numpy() for t in engine.matmul_backward(a, b, dc)]
    x2 = [t.numpy() for t in engine.matmul_backward(a, b, dc)]
    for p, q in zip(x1, x2):
        np.testing.assert_array_equal(p, q)
    db1 = engine.add_broadcast_backward(dc).numpy()
    db2 = engine.add_broadcast_backward(dc).numpy()
    np.testing.assert_array_equal(db1, db2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 1), (7, 3), (64, 96), (33, 257), (500, 1000), (3, 4099)])
def test_scale_and_shift(engine, dtype, shape):
    """ScaleAndShiftOperation: per-row beta and gamma; the row sums of the backward accumulate in
    double on the device and sequentially in T in the managed loop (tolerance-level)."""
    r = rng(shape[0] + shape[1])
    x, dy = normal(r, shape, 1, dtype), normal(r, shape, 1, dtype)
    beta, gamma = normal(r, (shape[0], 1), 1, dtype), normal(r, (shape[0], 1), 1, dtype)
    X, B, G, DY = (engine.upload(v) for v in (x, beta, gamma, dy))
    np.testing.assert_array_equal(engine.scale_shift_forward(X, B, G).numpy(), O.scale_shift_forward(x, beta, gamma))
    dx, db, dg = engine.scale_shift_backward(X, B, DY)
    dx_ref, db_ref, dg_ref = O.scale_shift_backward(x, beta, dy)
    np.testing.assert_array_equal(dx.numpy(), dx_ref)
    sc = np.sqrt(shape[1])
    assert_close(db.numpy().reshape(-1), db_ref, sc, "dbeta")
    assert_close(dg.numpy().reshape(-1), dg_ref, sc, "dgamma")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 1), (7, 3), (64, 96), (33, 257), (500, 1000), (3, 4099)])
def test_rmsnorm(engine, dtype, shape):
    """RMSNormOperation with its diagonal-form backward."""
    r = rng(shape[0] * 3 + shape[1])
    x, dy, g = normal(r, shape, 1, dtype), normal(r, shape, 1, dtype), normal(r, shape, 1, dtype)
    X, Gm, DY = (engine.upload(v) for v in (x, g, dy))
    y_ref = O.rmsnorm_forward(x, g)
    assert_close(engine.rmsnorm_forward(X, Gm).numpy(), y_ref, np.abs(y_ref) + 1e-30, "y")
    dx, dg = engine.rmsnorm_backward(X, Gm, DY)
    dx_ref, dg_ref = O.rmsnorm_backward(x, g, dy)
    # dx is a difference of two terms of the size of |dy g / rms|
    rmsv = np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True))
    assert_close(dx.numpy(), dx_ref, np.abs(dy * g) / rmsv * (1 + (x / rmsv) ** 2 / shape[1]) + 1e-30, "dx")
    assert_close(dg.numpy(), dg_ref, np.abs(dg_ref) + 1e-30, "dg")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [1, 77, 5000, 200003])
def test_swish(engine, dtype, n):
    r = rng(n)
    x, dy = normal(r, (1, n), 2.0, dtype), normal(r, (1, n), 1.0, dtype)
    beta = dtype(1.3)
    X, DY, B = engine.upload(x), engine.upload(dy), engine.upload(np.full((1, 1), beta, dtype))
    y_ref = O.swish_forward(x, beta)
    assert_close(engine.swish_forward(X, B).numpy(), y_ref, np.abs(y_ref) + 1e-30, "swish")
    dx, db = engine.swish_backward(X, B, DY)
    dx_ref, db_ref = O.swish_backward(x, beta, dy)
    assert_close(dx.numpy(), dx_ref, np.abs(dx_ref) + 1e-30, "swish dx")
    # the managed loop adds n terms of size ~1 into a T cell one by one; the device sums in double
    assert_close(db.numpy().reshape(()), np.asarray(db_ref, dtype), 3.0 * np.sqrt(n) * (50 if dtype == np.float32 else 1), "dbeta")
    dx2, db2 = engine.swish_backward(X, B, DY, out=(dx, db), accumulate=True)
    assert_close(db2.numpy().reshape(()), np.asarray(2 * db_ref, dtype), 6.0 * np.sqrt(n) * (50 if dtype == np.float32 else 1), "dbeta +=")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 1), (9, 5), (300, 96), (4100, 130), (17, 1000)])
def test_swiglu(engine, dtype, shape):
    r = rng(shape[0] + 7 * shape[1])
    x, dy = normal(r, shape, 1.5, dtype), normal(r, shape, 1.0, dtype)
    w, v, b, c = (normal(r, (shape[1], 1), 1.0, dtype) for _ in range(4))
    beta = 1.1
    X, DY, W, V, B, Cc = (engine.upload(t) for t in (x, dy, w, v, b, c))
    y_ref = O.swiglu_forward(x, w, v, b, c, beta)
    assert_close(engine.swiglu_forward(X, W, V, B, Cc, beta).numpy(), y_ref, np.abs(y_ref) + 1e-30, "swiglu")
    got = engine.swiglu_backward(X, W, V, B, Cc, beta, DY)
    ref = O.swiglu_backward(x, w, v, b, c, beta, dy)
    assert_close(got[0].numpy(), ref[0], np.abs(ref[0]) + 1e-30, "dx")
    # column sums over the rows: double accumulators on both sides, different grouping
    f = x.astype(np.float64) * w.reshape(1, -1) + b.reshape(1, -1)
    lin = np.abs(x.astype(np.float64) * v.reshape(1, -1) + c.reshape(1, -1))
    bound = (np.abs(dy) * (1 + np.abs(f)) * (1 + np.abs(x)) * (1 + lin)).sum(axis=0)
    for k, name in enumerate(("dw", "dv", "db", "dc"), start=1):
        assert_close(got[k].numpy().reshape(-1), ref[k], bound, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 1), (5, 3), (64, 96), (33, 4099)])
def test_row_sum_average_broadcast_concatenate(engine, dtype, shape):
    r = rng(shape[0] * 5 + shape[1])
    x = normal(r, shape, 1, dtype)
    X = engine.upload(x)
    for avg in (False, True):
        y = engine.row_sum_forward(X, avg).numpy().reshape(-1)
        assert_close(y, O.row_sum_forward(x, avg), np.sqrt(shape[1]) if not avg else 1.0, "row sum")
        dyv = normal(r, (shape[0], 1), 1, dtype)
        np.testing.assert_array_equal(engine.row_sum_backward(engine.upload(dyv), shape[1], avg).numpy(),
                                      O.row_sum_backward(dyv, shape[1], avg))
    R, Cc = 2 * shape[0] + 1, 3 * shape[1] + 2
    if R * Cc < 3_000_000:
        np.testing.assert_array_equal(engine.broadcast_forward(X, R, Cc).numpy(), O.broadcast_forward(x, R, Cc))
        dy = normal(r, (R, Cc), 1, dtype)
        np.testing.assert_array_equal(engine.broadcast_backward(engine.upload(dy), *shape).numpy(),
                                      O.broadcast_backward(dy, *shape))          # same order of additions: exact
    other = normal(r, (shape[0], 7), 1, dtype)
    cat = engine.concatenate_forward([X, engine.upload(other), X])
    np.testing.assert_array_equal(cat.numpy(), np.concatenate([x, other, x], axis=1))
    parts = engine.concatenate_backward(cat, [shape[1], 7, shape[1]])
    for got, want in zip(parts, (x, other, x)):
        np.testing.assert_array_equal(got.numpy(), want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 1), (5, 7), (64, 96), (300, 1000)])
def test_batchnorm_as_written(engine, dtype, shape):
    r = rng(shape[0] + 11 * shape[1])
    x, dy = normal(r, shape, 1.0, dtype) + dtype(0.3), normal(r, shape, 1.0, dtype)
    X, DY = engine.upload(x), engine.upload(dy)
    y_ref, st_ref = O.batchnorm_forward(x)
    y, st = engine.batchnorm_forward(X)
    n = shape[0] * shape[1]
    assert_close(st.numpy().reshape(-1)[:2], st_ref, np.array([np.sqrt(n) / n * 4, max(st_ref[1], 1.0)]), "mean, var")
    assert_close(y.numpy(), y_ref, np.abs(y_ref) + 1e-3, "y")
    dx = engine.batchnorm_backward(X, st, DY)
    assert_close(dx.numpy(), O.batchnorm_backward(x, st_ref, dy), np.abs(dy) * 2 + 1e-30, "dx")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("op", ["exp", "ln", "log", "abs", "square", "sqrt", "sin", "cos", "reciprocal", "negate"])
def test_tensor_unary_family(engine, dtype, op):
    """PRAD Tensor / TensorReverse elementwise operations (MKL VML in the reference)."""
    r = rng(len(op) * 7 + 1)
    x = normal(r, (33, 77), 1.5, dtype)
    if op in ("ln", "log", "sqrt"):
        x = np.abs(x) + dtype(0.05)
        x[0, :3] = 0 if op == "sqrt" else x[0, :3]          # sqrt(0): the reverse clamps the divisor to 1e-10
    if op == "reciprocal":
        x = x + np.sign(x) * dtype(0.1)
    dy = normal(r, x.shape, 1.0, dtype)
    X, DY = engine.upload(x), engine.upload(dy)
    y_ref = O.tensor_unary(op, x)
    y = engine.tensor_unary(op, X)
    exact_fwd = op in ("abs", "square", "sqrt", "reciprocal", "negate")
    if exact_fwd:
        np.testing.assert_array_equal(y.numpy(), y_ref)
    else:
        assert_close(y.numpy(), y_ref, np.abs(y_ref) + 1e-30, op)
    saved_h = y_ref if op == "reciprocal" else x
    dx_ref = O.tensor_unary_reverse(op, saved_h, dy)
    dx = engine.tensor_unary_reverse(op, engine.upload(saved_h), DY)
    if op in ("ln", "log", "abs", "square", "sqrt", "reciprocal", "negate"):
        np.testing.assert_array_equal(dx.numpy(), dx_ref)       # IEEE operations only: same bits
    else:
        assert_close(dx.numpy(), dx_ref, np.abs(dy) * (np.abs(y_ref) + 1) + 1e-30, op + " reverse")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
def test_tensor_binary_family(engine, dtype, op):
    r = rng(len(op) + 40)
    a, b, dy = normal(r, (50, 41), 1, dtype), normal(r, (50, 41), 1, dtype), normal(r, (50, 41), 1, dtype)
    b = b + np.sign(b) * dtype(0.2)
    A, B, DY = engine.upload(a), engine.upload(b), engine.upload(dy)
    np.testing.assert_array_equal(engine.tensor_binary(op, A, B).numpy(), O.tensor_binary(op, a, b))
    da, db = engine.tensor_binary_reverse(op, A, B, DY)
    da_ref, db_ref = O.tensor_binary_reverse(op, a, b, dy)
    np.testing.assert_array_equal(da.numpy(), da_ref)
    np.testing.assert_array_equal(db.numpy(), db_ref)


def test_new_row_ops_reject_bad_arguments(engine):
    from parallelreverseautodiff_b200._lib import ERR_INVALID, PradError
    x = engine.zeros((4, 4), np.float32)
    with pytest.raises(PradError) as ei:
        E.check(engine.lib.prad_rmsnorm_forward(engine.ctx, E.F32, x.ptr, None, x.ptr, 4, 4))
    assert ei.value.status == ERR_INVALID
    E.check(engine.lib.prad_rmsnorm_forward(engine.ctx, E.F32, None, None, None, 0, 4))     # empty: nothing to do
    E.check(engine.lib.prad_scale_shift_forward(engine.ctx, E.F32, None, None, None, None, 0, 0))
