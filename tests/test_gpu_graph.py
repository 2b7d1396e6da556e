"""Graph mode (prad_graph_*): the static-schedule backward against the visitor's semantics
restated with CPU-oracle operations -- every consumer's gradient delivered once, summed in
consumer registration order (GradientUtils.AccumulateGradients), weight gradients added into
their destinations (OperationBase.AccumulateGradient), shared weights accumulating over uses."""
import numpy as np
import pytest

import oracle as O
from parallelreverseautodiff_b200._lib import ERR_SHAPE, PradError
from parallelreverseautodiff_b200.graph import Graph
from util import assert_close, rms

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_fan_out_and_shared_weight(engine, dtype):
    """x -> MatMul(W) -> Tanh = h ; h feeds three consumers (fan-out 3); W is used twice."""
    r = np.random.default_rng(42)
    B, n = 24, 40
    x = r.standard_normal((B, n)).astype(dtype)
    W = (r.standard_normal((n, n)) * 0.2).astype(dtype)
    bias = (r.standard_normal((1, n)) * 0.1).astype(dtype)
    d_out = r.standard_normal((B, n)).astype(dtype)
    # ---- oracle, visitor semantics
    z = O.add_broadcast_forward(O.matmul_forward(x, W), bias)
    h = O.tanh_forward(z)
    u = O.matmul_forward(h, W)                 # consumer 1 of h (W shared)
    s = O.sigmoid_forward(h)                   # consumer 2 of h
    p = O.hadamard_forward(u, s)
    q = O.add_forward(p, h)                    # consumer 3 of h
    y = O.gelu_forward(q)
    d_q = O.gelu_backward(q, d_out)
    d_p, d_h3 = d_q, d_q                       # MatrixAdd: both inputs receive dOut
    d_u, d_s = O.hadamard_backward(u, s, d_p)
    d_h2 = O.sigmoid_backward(s, d_s)
    d_h1, dW_b = O.matmul_backward(h, W, d_u)
    d_h = O.accumulate_gradients([d_h1, d_h2, d_h3])            # consumer order
    d_z = O.tanh_backward(h, d_h)
    _, d_bias = O.add_broadcast_backward(d_z)
    d_x, dW_a = O.matmul_backward(x, W, d_z)
    dW = np.zeros_like(W)
    O.accumulate_into(dW, dW_b)                # backward order: the later use delivers first
    O.accumulate_into(dW, dW_a)
    # ---- graph mode
    g = Graph(engine, dtype)
    gW, gb = engine.zeros(W.shape, dtype), engine.zeros(bias.shape, dtype)
    vx = g.input(engine.upload(x))
    vW = g.weight(engine.upload(W), gW)
    vb = g.weight(engine.upload(bias), gb)
    vz = g.node("MatrixAddBroadcastingOperation", [g.node("MatrixMultiplyOperation", [vx, vW]), vb])
    vh = g.node("TanhOperation", [vz])
    vu = g.node("MatrixMultiplyOperation", [vh, vW])
    vs = g.node("SigmoidOperation", [vh])
    vp = g.node("HadamardProductOperation", [vu, vs])
    vq = g.node("MatrixAddOperation", [vp, vh])
    vy = g.node("GELUOperation", [vq])
    g.forward()
    assert_close(g.data(vy).numpy(), y, rms(y), "forward")
    g.backward(vy, engine.upload(d_out))
    assert g.consumers(vh) == 3 and g.consumers(vW) == 2 and g.consumers(vx) == 1
    scale = 30 * max(rms(dW), 1e-30)
    assert_close(g.gradient(vh).numpy(), d_h, 10 * rms(d_h), "fan-in at h")
    assert_close(g.gradient(vx).numpy(), d_x, 10 * rms(d_x), "dX")
    assert_close(gW.numpy(), dW, scale, "shared weight gradient")
    assert_close(gb.numpy(), d_bias, 30 * rms(d_bias), "bias gradient")
    # a second backward adds into the destinations again (`+=`), and is deterministic
    first = gW.numpy()
    g.backward(vy, engine.upload(d_out))
    assert_close(gW.numpy(), (first + first).astype(dtype), 2 * scale, "destination accumulates")
    g.close()


def test_lstm_cell_steps_through_graph_mode(engine):
    """Three LSTM steps with weights shared across time, double precision."""
    r = np.random.default_rng(7)
    B, n_in, nh, T = 8, 12, 16, 3
    dt = np.float64
    xs = [r.standard_normal((B, n_in)) for _ in range(T)]
    Wg = {k: r.standard_normal((n_in, nh)) * 0.3 for k in "ifgo"}
    Ug = {k: r.standard_normal((nh, nh)) * 0.3 for k in "ifgo"}
    d_last = r.standard_normal((B, nh))
    act = {"i": (O.sigmoid_forward, O.sigmoid_backward), "f": (O.sigmoid_forward, O.sigmoid_backward),
           "g": (O.tanh_forward, O.tanh_backward), "o": (O.sigmoid_forward, O.sigmoid_backward)}
    # ---- oracle
    h, c, tape = np.zeros((B, nh)), np.zeros((B, nh)), []
    for t in range(T):
        gate = {k: act[k][0](O.add_forward(O.matmul_forward(xs[t], Wg[k]), O.matmul_forward(h, Ug[k]))) for k in "ifgo"}
        c_new = O.add_forward(O.hadamard_forward(gate["f"], c), O.hadamard_forward(gate["i"], gate["g"]))
        tc = O.tanh_forward(c_new)
        h_new = O.hadamard_forward(gate["o"], tc)
        tape.append((h, c, gate, tc))
        h, c = h_new, c_new
    dW = {k: np.zeros_like(Wg[k]) for k in "ifgo"}
    dU = {k: np.zeros_like(Ug[k]) for k in "ifgo"}
    dh, dc_next = d_last, None
    for t in range(T - 1, -1, -1):
        hp, cp, gate, tc = tape[t]
        d_o, d_tc = O.hadamard_backward(gate["o"], tc, dh)
        dc_a = O.tanh_backward(tc, d_tc)
        # consumers of c_t in registration order: tanh (step t), then the f-Hadamard of step t+1
        dc = dc_a if dc_next is None else O.accumulate_gradients([dc_a, dc_next])
        d_f, dc_next = O.hadamard_backward(gate["f"], cp, dc)
        d_i, d_g = O.hadamard_backward(gate["i"], gate["g"], dc)
        dz = {"i": act["i"][1](gate["i"], d_i), "f": act["f"][1](gate["f"], d_f),
              "g": act["g"][1](gate["g"], d_g), "o": act["o"][1](gate["o"], d_o)}
        parts = []
        for k in "ifgo":                         # gate nodes were registered in this order
            _, dWk = O.matmul_backward(xs[t], Wg[k], dz[k])
            dhk, dUk = O.matmul_backward(hp, Ug[k], dz[k])
            parts.append(dhk)
            O.accumulate_into(dW[k], dWk)
            O.accumulate_into(dU[k], dUk)
        dh = O.accumulate_gradients(parts)
    # ---- graph mode
    g = Graph(engine, dt)
    gW = {k: engine.zeros(Wg[k].shape, dt) for k in "ifgo"}
    gU = {k: engine.zeros(Ug[k].shape, dt) for k in "ifgo"}
    vW = {k: g.weight(engine.upload(Wg[k]), gW[k]) for k in "ifgo"}
    vU = {k: g.weight(engine.upload(Ug[k]), gU[k]) for k in "ifgo"}
    vh = g.input(engine.zeros((B, nh), dt))
    vc = g.input(engine.zeros((B, nh), dt))
    opname = {"i": "SigmoidOperation", "f": "SigmoidOperation", "g": "TanhOperation", "o": "SigmoidOperation"}
    for t in range(T):
        vx = g.input(engine.upload(xs[t]))
        gate = {}
        for k in "ifgo":
            pre = g.node("MatrixAddOperation", [g.node("MatrixMultiplyOperation", [vx, vW[k]]),
                                                g.node("MatrixMultiplyOperation", [vh, vU[k]])])
            gate[k] = g.node(opname[k], [pre])
        vc = g.node("MatrixAddOperation", [g.node("HadamardProductOperation", [gate["f"], vc]),
                                           g.node("HadamardProductOperation", [gate["i"], gate["g"]])])
        vtc = g.node("TanhOperation", [vc])
        vh = g.node("HadamardProductOperation", [gate["o"], vtc])
    g.forward()
    assert_close(g.data(vh).numpy(), h, 1.0, "h after three steps")
    g.backward(vh, engine.upload(d_last))
    for k in "ifgo":
        assert_close(gW[k].numpy(), dW[k], 10.0, f"dW_{k}")
        assert_close(gU[k].numpy(), dU[k], 10.0, f"dU_{k}")
    g.close()


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_relu_and_amplified_sigmoid_nodes(engine, dtype):
    """x -> ReLU -> r ; x -> AmplifiedSigmoid -> s ; y = r (.) s : two consumers of x."""
    r = np.random.default_rng(3)
    x = r.standard_normal((17, 29)).astype(dtype)
    d_out = r.standard_normal((17, 29)).astype(dtype)
    rl, sg = O.relu_forward(x), O.amplified_sigmoid_forward(x)
    d_r, d_s = O.hadamard_backward(rl, sg, d_out)
    d_x = O.accumulate_gradients([O.relu_backward(x, d_r), O.amplified_sigmoid_backward(x, d_s)])
    g = Graph(engine, dtype)
    vx = g.input(engine.upload(x))
    vy = g.node("HadamardProductOperation", [g.node("ReLUOperation", [vx]), g.node("AmplifiedSigmoidOperation", [vx])])
    g.forward()
    assert_close(g.data(vy).numpy(), O.hadamard_forward(rl, sg), 1.0, "forward")
    g.backward(vy, engine.upload(d_out))
    assert g.consumers(vx) == 2
    assert_close(g.gradient(vx).numpy(), d_x, rms(d_x), "dX")
    g.close()


def test_graph_errors_are_status_codes(engine):
    g = Graph(engine, np.float32)
    a = g.input(engine.zeros((4, 5), np.float32))
    b = g.input(engine.zeros((6, 3), np.float32))
    with pytest.raises(PradError) as ei:
        g.node("MatrixMultiplyOperation", [a, b], out_shape=(4, 3))
    assert ei.value.status == ERR_SHAPE
    with pytest.raises(PradError):
        g.backward(99, engine.zeros((1, 1), np.float32))
    g.close()
