"""The five benchmark configurations end to end: the CUDA path (through the C ABI and the
host drivers in networks.py) against the same graph composed from CPU-oracle operations on
identical seeded inputs.  C1-C3 run at their full sizes; C4 and C5 at reduced batch (the
oracle's naive loops would take minutes at full size), C5's full size being covered by
size-independent properties in test_gpu_properties.py.
"""
import numpy as np
import pytest

import oracle as O
from oracle.configs import lstm_oracle as _lstm_oracle, mlp_oracle as _mlp_oracle, swin_oracle as _swin_oracle
from parallelreverseautodiff_b200 import engine as E
from parallelreverseautodiff_b200.networks import FeedForwardNetwork, LstmNetwork, SwinBlock
from util import assert_close, rms

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------ C1
def test_c1_matmul_leakyrelu_node_double(engine):
    """A[512x784]~U(-1,1), B[784x256]~N(0,2/784), dOut~N(0,1), seed 42: dPre, dA, dB."""
    r = np.random.default_rng(42)
    A = r.uniform(-1, 1, (512, 784))
    B = r.standard_normal((784, 256)) * np.sqrt(2.0 / 784)
    dOut = r.standard_normal((512, 256))
    pre = O.matmul_forward(A, B)
    dPre_ref = O.leaky_relu_backward(pre, dOut, 0.01)
    dA_ref, dB_ref = O.matmul_backward(A, B, dPre_ref)
    a, b = engine.upload(A), engine.upload(B)
    pre_dev = engine.matmul_forward(a, b)
    dPre, dA, dB = engine.matmul_act_backward(a, b, engine.upload(dOut), E.ACT_LEAKY_RELU, pre_dev, 0.01)
    # every operation on this path rounds exactly as the C# loops do: identical bits
    np.testing.assert_array_equal(pre_dev.numpy(), pre)
    np.testing.assert_array_equal(dPre.numpy(), dPre_ref)
    np.testing.assert_array_equal(dA.numpy(), dA_ref)
    np.testing.assert_array_equal(dB.numpy(), dB_ref)
    # the tensor-core variant of the double GEMM stays within 1e-12 relative / 1e-14 absolute
    # of it, the absolute part scaled by the size of the summed terms
    engine.set_option("gemm_f64", "dmma")
    try:
        _, dA2, dB2 = engine.matmul_act_backward(a, b, engine.upload(dOut), E.ACT_LEAKY_RELU, pre_dev, 0.01)
        assert_close(dA2.numpy(), dA_ref, np.abs(dPre_ref) @ np.abs(B.T), "dA (dmma)")
        assert_close(dB2.numpy(), dB_ref, np.abs(A.T) @ np.abs(dPre_ref), "dB (dmma)")
    finally:
        engine.set_option("gemm_f64", "auto")


# ------------------------------------------------------------------ C2
@pytest.mark.parametrize("clip", ["reference", "global_norm"])
def test_c2_mlp_float_backward_clip_adam(engine, clip):
    """784->512->512->10, LeakyReLU, softmax + CCE, batch 256; clip + one Adam step."""
    r = np.random.default_rng(42)
    sizes = [784, 512, 512, 10]
    x = r.uniform(0, 1, (256, 784)).astype(np.float32)
    onehot = np.eye(10, dtype=np.float32)[r.integers(0, 10, 256)]
    Ws = [(r.standard_normal((sizes[i], sizes[i + 1])) * np.sqrt(2.0 / sizes[i])).astype(np.float32) for i in range(3)]
    bs = [np.zeros((1, sizes[i + 1]), np.float32) for i in range(3)]
    probs_ref, dW_ref, db_ref, dx_ref = _mlp_oracle(x, onehot, Ws, bs, np.float32(0.01))
    mode = E.CLIP_REFERENCE if clip == "reference" else E.CLIP_GLOBAL_NORM
    net = FeedForwardNetwork(engine, np.float32, sizes, hidden_act=E.ACT_LEAKY_RELU, softmax_output=True,
                             loss="cce", use_bias=True, clip_mode=mode)
    net.set_weights(Ws, bs)
    net._ensure_buffers(256)
    engine.upload(x, out=net.A[0])
    engine.upload(onehot, out=net.target)
    probs = net.forward()
    assert_close(probs.numpy(), probs_ref, 0.1, "probabilities")
    net.backward()
    for l in range(3):
        scale = np.abs(dW_ref[l]).max()
        assert_close(net.dW[l].numpy(), dW_ref[l], scale, f"dW{l}")
        assert_close(net.db[l].numpy(), db_ref[l], np.abs(db_ref[l]).max(), f"db{l}")
    assert_close(net.dX.numpy(), dx_ref, np.abs(dx_ref).max(), "dX")
    # clip + Adam on the oracle's gradients vs the device step on the device's gradients
    grads_ref = [g.copy() for g in dW_ref + db_ref]
    if clip == "reference":
        for g in grads_ref:
            O.clip_reference(g, np.float32(4.0), np.float32(1e-8))
    else:
        O.clip_global_norm(grads_ref, 4.0)
    w_ref = [w.copy() for w in Ws + bs]
    for w, g in zip(w_ref, grads_ref):
        O.adam_rmad(w, np.zeros_like(w), np.zeros_like(w), g, 1e-3, 0.9, 0.999, 1e-8, 1.0)
    net.clip_and_optimize(zero_grad=True)
    for k, (p, w) in enumerate(zip(net.params, w_ref)):
        # first Adam step moves every weight by ~lr*sign(g): compare the update, not the weight
        upd = p.numpy() - (Ws + bs)[k]
        upd_ref = w - (Ws + bs)[k]
        big = np.abs(grads_ref[k]) > 1e-6           # where g ~ 0 the direction is rounding noise
        assert_close(upd[big], upd_ref[big], 1e-3, f"Adam update {k}")
    assert not net.grads[0].numpy().any()


# ------------------------------------------------------------------ C3
@pytest.mark.parametrize("shape", [(5, 3, 12, 16), (64, 32, 128, 256)])
def test_c3_lstm_double_bptt(engine, shape):
    """Input 128, hidden 256, 64 steps, batch 32 (and a tiny case): full BPTT."""
    T, B, n_in, nh = shape
    r = np.random.default_rng(42)
    x = r.standard_normal((T, B, n_in))
    y = r.standard_normal((T, B, nh))
    G = ("i", "f", "g", "o")
    W = {g: r.uniform(-1, 1, (nh, n_in)) * np.sqrt(6.0 / (nh + n_in)) for g in G}
    U = {g: r.uniform(-1, 1, (nh, nh)) * np.sqrt(6.0 / (nh + nh)) for g in G}
    b = {g: r.standard_normal(nh) * 0.1 for g in G}
    H_ref, dW_ref, dU_ref, db_ref, dX_ref = _lstm_oracle(x, y, W, U, b)
    net = LstmNetwork(engine, np.float64, n_in, nh, T, B)
    net.set_parameters(W, U, b)
    H = net.forward(x, y)
    assert_close(H.numpy().reshape(T, B, nh), H_ref, 1.0, "h")
    net.backward()
    for g in G:
        assert_close(net.dW[g].numpy(), dW_ref[g], 1.0, f"dW_{g}")
        assert_close(net.dU[g].numpy(), dU_ref[g], 1.0, f"dU_{g}")
        assert_close(net.db[g].numpy().ravel(), db_ref[g], 1.0, f"db_{g}")
    assert_close(net.dX.numpy().reshape(T, B, n_in), dX_ref, 1.0, "dX")


def test_c3_fused_cell_backward_is_bit_identical_to_the_operation_chain(engine):
    """prad_lstm_cell_backward (one launch per time step) against the same step as eleven library calls."""
    T, B, n_in, nh = 7, 5, 12, 16
    r = np.random.default_rng(1)
    x = r.standard_normal((T, B, n_in))
    y = r.standard_normal((T, B, nh))
    G = ("i", "f", "g", "o")
    W = {g: r.uniform(-1, 1, (nh, n_in)) * 0.4 for g in G}
    U = {g: r.uniform(-1, 1, (nh, nh)) * 0.4 for g in G}
    b = {g: r.standard_normal(nh) * 0.1 for g in G}
    nets = []
    for fused in (True, False):
        net = LstmNetwork(engine, np.float64, n_in, nh, T, B, fused_cell=fused)
        net.set_parameters(W, U, b)
        net.forward(x, y)
        n0 = engine.launch_count()
        net.backward()
        nets.append((net, engine.launch_count() - n0))
    (a, la), (c, lc) = nets
    assert la < lc / 3
    for g in G:
        np.testing.assert_array_equal(a.dW[g].numpy(), c.dW[g].numpy())
        np.testing.assert_array_equal(a.dU[g].numpy(), c.dU[g].numpy())
        np.testing.assert_array_equal(a.db[g].numpy(), c.db[g].numpy())
        np.testing.assert_array_equal(a.dpre[g].numpy(), c.dpre[g].numpy())
    np.testing.assert_array_equal(a.dX.numpy(), c.dX.numpy())


# ------------------------------------------------------------------ C4
@pytest.mark.parametrize("images", [1, 64])
def test_c4_swin_block_float(engine, images):
    """dim 96, 3 heads, 7x7 windows over a 56x56 token map (one image = 64 windows); 64 images is
    the configured batch."""
    d, heads, ws, hidden = 96, 3, 49, 384
    T = images * 3136
    r = np.random.default_rng(42)
    f = np.float32
    x = r.standard_normal((T, d)).astype(f)
    d_out = r.standard_normal((T, d)).astype(f)
    p = {"Wqkv": (r.standard_normal((d, 3 * d)) * np.sqrt(2.0 / d)).astype(f), "bqkv": (r.standard_normal((1, 3 * d)) * 0.1).astype(f),
         "Wproj": (r.standard_normal((d, d)) * np.sqrt(2.0 / d)).astype(f), "bproj": (r.standard_normal((1, d)) * 0.1).astype(f),
         "W1": (r.standard_normal((d, hidden)) * np.sqrt(2.0 / d)).astype(f), "b1": (r.standard_normal((1, hidden)) * 0.1).astype(f),
         "W2": (r.standard_normal((hidden, d)) * np.sqrt(2.0 / hidden)).astype(f), "b2": (r.standard_normal((1, d)) * 0.1).astype(f)}
    out_ref, g_ref, dx_ref, mid = _swin_oracle(x, d_out, p, heads, ws)
    blk = SwinBlock(engine, f, d, heads, ws, hidden // d)
    blk.set_parameters(p)
    out = blk.forward(engine.upload(x))
    assert_close(out.numpy(), out_ref, 2 * rms(out_ref), "block output")
    nw = T // ws
    assert_close(blk.P.numpy().reshape(nw * heads, ws, ws), mid["P"], 1.0, "attention probabilities")
    dx = blk.backward(engine.upload(d_out))
    assert_close(blk.d_qkv.numpy(), mid["d_qkv"], 5 * rms(mid["d_qkv"]), f"C4[{images}] d_qkv")
    for k in g_ref:
        # weight gradients sum over all T tokens: the error scale is sum |terms| ~ T * typical product
        assert_close(blk.g[k].numpy(), g_ref[k], 16 * rms(g_ref[k]), f"grad {k}")
    assert_close(dx.numpy(), dx_ref, 3 * rms(dx_ref), "d_x")


# ------------------------------------------------------------------ C5 (reduced rows)
@pytest.mark.parametrize("gemm", ["simt", "auto"])
def test_c5_wide_mlp_float_reduced(engine, gemm):
    """Same graph as the benchmark (width x width GELU layers, MSE) at 3 x 1024 wide, 384 rows."""
    engine.set_option("gemm_f32", gemm)
    try:
        r = np.random.default_rng(42)
        width, L, rows = 1024, 3, 384
        f = np.float32
        x = r.standard_normal((rows, width)).astype(f)
        t = r.standard_normal((rows, width)).astype(f)
        Ws = [(r.standard_normal((width, width)) * np.sqrt(2.0 / width)).astype(f) for _ in range(L)]
        acts, pres = [x], []
        for W in Ws:
            z = O.matmul_forward(acts[-1], W)
            pres.append(z)
            acts.append(O.gelu_forward(z))
        d = O.mse_backward(acts[-1], t)
        dW_ref = [None] * L
        for l in range(L - 1, -1, -1):
            d = O.gelu_backward(pres[l], d)
            dA, dW_ref[l] = O.matmul_backward(acts[l], Ws[l], d)
            d = dA
        net = FeedForwardNetwork(engine, f, [width] * (L + 1), hidden_act=E.ACT_GELU, output_act=E.ACT_GELU,
                                 loss="mse", use_bias=False)
        net.set_weights(Ws)
        net._ensure_buffers(rows)
        engine.upload(x, out=net.A[0])
        engine.upload(t, out=net.target)
        net.forward()
        assert_close(net.A[L].numpy(), acts[-1], 3 * rms(acts[-1]), "output")
        net.backward()
        for l in range(L):
            assert_close(net.dW[l].numpy(), dW_ref[l], 10 * rms(dW_ref[l]), f"C5 reduced [{gemm}] dW{l}")
        assert_close(net.dX.numpy(), d, 5 * rms(d), f"C5 reduced [{gemm}] dX")
    finally:
        engine.set_option("gemm_f32", "auto")


# ------------------------------------------------------------------ C5 at its real width
@pytest.mark.parametrize("scheme", ["auto", "tf32b16"])
def test_c5_layer_at_full_width_elementwise(engine, scheme):
    """One 4096 x 4096 GELU layer of the benchmark network on 512 batch rows, every output element
    against the oracle: forward product and GELU, then GELU', dW = A^T dZ and dA = dZ W^T through
    the path `auto` takes at this size (the tensor-core kernel), and through the tf32b16 option."""
    if scheme != "auto":
        engine.set_option("tc_auto", scheme)
    try:
        r = np.random.default_rng(42)
        width, rows = 4096, 512
        f = np.float32
        x = r.standard_normal((rows, width)).astype(f)
        t = r.standard_normal((rows, width)).astype(f)
        W = (r.standard_normal((width, width)) * np.sqrt(2.0 / width)).astype(f)
        z = O.matmul_forward(x, W)
        a = O.gelu_forward(z)
        d = O.gelu_backward(z, O.mse_backward(a, t))
        dA_ref, dW_ref = O.matmul_backward(x, W, d)
        net = FeedForwardNetwork(engine, f, [width, width], hidden_act=E.ACT_GELU, output_act=E.ACT_GELU,
                                 loss="mse", use_bias=False)
        net.set_weights([W])
        net._ensure_buffers(rows)
        engine.upload(x, out=net.A[0])
        engine.upload(t, out=net.target)
        n0 = engine.launch_count()
        net.forward()
        # error of a dot product is proportional to sum_k |a_k||b_k|: that is the absolute scale
        assert_close(net.Z[1].numpy(), z, np.abs(x) @ np.abs(W), f"C5 full width [{scheme}] Z")
        assert_close(net.A[1].numpy(), a, np.abs(x) @ np.abs(W), f"C5 full width [{scheme}] A")
        net.backward()
        assert engine.launch_count() > n0
        assert_close(net.dW[0].numpy(), dW_ref, np.abs(x.T) @ np.abs(d), f"C5 full width [{scheme}] dW")
        assert_close(net.dX.numpy(), dA_ref, np.abs(d) @ np.abs(W.T), f"C5 full width [{scheme}] dX")
    finally:
        engine.set_option("tc_auto", "fp16x3")


def test_overlapped_host_steps_equal_plain_host_steps(engine):
    """train_steps_host (upload of batch i+1 overlapped with step i) == train_step_host, bit for bit."""
    f = np.float32
    r = np.random.default_rng(3)
    sizes = [64, 96, 32]
    Ws = [(r.standard_normal((sizes[i], sizes[i + 1])) * 0.2).astype(f) for i in range(2)]
    batches = []
    for _ in range(4):
        x, t = engine.pinned_empty((50, 64), f), engine.pinned_empty((50, 32), f)
        x[:] = r.standard_normal((50, 64))
        t[:] = r.standard_normal((50, 32))
        batches.append((x, t))

    def make():
        net = FeedForwardNetwork(engine, f, sizes, hidden_act=E.ACT_GELU, output_act=E.ACT_NONE, loss="mse")
        net.set_weights(Ws)
        return net

    a, b = make(), make()
    plain = [a.train_step_host(x, t) for x, t in batches]
    overlapped = list(b.train_steps_host(batches))
    assert plain == overlapped
    for p, q in zip(a.params, b.params):
        np.testing.assert_array_equal(p.numpy(), q.numpy())
