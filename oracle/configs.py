"""TEST INFRASTRUCTURE -- not part of the product path.

The benchmark configurations composed from CPU-oracle operations (`oracle/__init__.py`), in the
reference's graph spelling: what the CUDA path is compared with in tests/test_gpu_configs.py and
what `bench.py --workload c1..c4` times as the CPU baseline.  Only tests and the benchmark's
CPU-baseline leg import this module.
"""
import numpy as np

import oracle as O


def c1_oracle(A, B, dOut, alpha=0.01):
    """MatMul -> LeakyReLU node (config 1): returns pre-activation, dPre, dA, dB."""
    pre = O.matmul_forward(A, B)
    dPre = O.leaky_relu_backward(pre, dOut, alpha)
    dA, dB = O.matmul_backward(A, B, dPre)
    return pre, dPre, dA, dB


def mlp_oracle(x, onehot, Ws, bs, alpha):
    acts, pres = [x], []
    for l, (W, b) in enumerate(zip(Ws, bs)):
        z = O.add_broadcast_forward(O.matmul_forward(acts[-1], W), b)
        pres.append(z)
        acts.append(O.leaky_relu_forward(z, alpha) if l < len(Ws) - 1 else z)
    probs = O.softmax_forward(acts[-1])
    d = O.softmax_backward(probs, O.cce_backward(probs, onehot))
    dW, db = [None] * len(Ws), [None] * len(Ws)
    for l in range(len(Ws) - 1, -1, -1):
        if l < len(Ws) - 1:
            d = O.leaky_relu_backward(pres[l], d, alpha)
        db[l] = O.add_broadcast_backward(d)[1]
        dA, dW[l] = O.matmul_backward(acts[l], Ws[l], d)
        d = dA
    return probs, dW, db, d


def lstm_oracle(x, y, W, U, b):
    """Column-vector spelling of the reference: per sample columns, weights [hidden x in];
    per-step weight gradients are the left-fold batch mean, summed over steps last to first."""
    T, B, n_in = x.shape
    nh = y.shape[2]
    sig, tanh = O.sigmoid_forward, O.tanh_forward
    G = ("i", "f", "g", "o")
    act = {"i": sig, "f": sig, "g": tanh, "o": sig}
    h = np.zeros((nh, B))
    c = np.zeros((nh, B))
    st = []
    for t in range(T):
        xt = np.ascontiguousarray(x[t].T)                       # [in x B]: one column per sample
        gate = {}
        for g in G:
            wx = O.matmul_forward(W[g], xt)
            if t > 0:
                wx = O.add_forward(wx, O.matmul_forward(U[g], h))
            pre = O.add_forward(wx, np.repeat(b[g].reshape(-1, 1), B, 1))
            gate[g] = act[g](pre)
        ig = O.hadamard_forward(gate["i"], gate["g"])
        fc = O.hadamard_forward(gate["f"], c) if t > 0 else np.zeros_like(c)
        c_new = O.add_forward(fc, ig)
        tc = tanh(c_new)
        h_new = O.hadamard_forward(gate["o"], tc)
        st.append(dict(x=xt, hprev=h, cprev=c, gate=gate, tc=tc, h=h_new, c=c_new))
        h, c = h_new, c_new
    dW = {g: np.zeros_like(W[g]) for g in G}
    dU = {g: np.zeros_like(U[g]) for g in G}
    db = {g: np.zeros(nh) for g in G}
    dX = np.zeros((T, B, n_in))
    dh_rec, dc_next = None, None
    inv = 1.0 / B
    for t in range(T - 1, -1, -1):
        s = st[t]
        yt = np.ascontiguousarray(y[t].T)
        dloss = (2.0 / nh) * (s["h"] - yt)                       # per-sample MSE on a [hidden x 1] column
        dh = dloss if dh_rec is None else O.accumulate_gradients([dloss] + dh_rec)
        d_o, d_tc = O.hadamard_backward(s["gate"]["o"], s["tc"], dh)
        dc_a = O.tanh_backward(s["tc"], d_tc)
        dc = dc_a if dc_next is None else O.accumulate_gradients([dc_a, dc_next])
        d_i, d_g = O.hadamard_backward(s["gate"]["i"], s["gate"]["g"], dc)
        if t > 0:
            d_f, dc_next = O.hadamard_backward(s["gate"]["f"], s["cprev"], dc)
        else:
            d_f = np.zeros_like(dc)
        dz = {"i": O.sigmoid_backward(s["gate"]["i"], d_i), "f": O.sigmoid_backward(s["gate"]["f"], d_f),
              "g": O.tanh_backward(s["gate"]["g"], d_g), "o": O.sigmoid_backward(s["gate"]["o"], d_o)}
        dx_parts, dh_rec = [], []
        for g in G:
            # batch mean of the per-sample outer products == sequential sum over samples * (1/B)
            O.accumulate_into(dW[g], O.matmul_forward(dz[g], np.ascontiguousarray(s["x"].T)) * inv)
            if t > 0:
                O.accumulate_into(dU[g], O.matmul_forward(dz[g], np.ascontiguousarray(s["hprev"].T)) * inv)
                dh_rec.append(O.matmul_forward(np.ascontiguousarray(U[g].T), dz[g]))
            db[g] = db[g] + dz[g].sum(1) * inv
            dx_parts.append(O.matmul_forward(np.ascontiguousarray(W[g].T), dz[g]))
        dX[t] = O.accumulate_gradients(dx_parts).T
        if t == 0:
            dh_rec = None
    H = np.stack([s["h"].T for s in st])
    return H, dW, dU, db, dX


def swin_oracle(x, d_out, p, heads, ws):
    T, d = x.shape
    hd = d // heads
    nw = T // ws
    scale = np.float32(1.0 / np.sqrt(hd))
    ln1, mu1, sd1 = O.layernorm_forward(x)
    qkv = O.add_broadcast_forward(O.matmul_forward(ln1, p["Wqkv"]), p["bqkv"])

    def heads_of(m, off):       # [T x 3d] -> DeepMatrix [nw*heads, ws, hd] (window-major, then head)
        return np.ascontiguousarray(m[:, off:off + d].reshape(nw, ws, heads, hd).transpose(0, 2, 1, 3)
                                    .reshape(nw * heads, ws, hd))

    def merge(m):               # inverse of heads_of for one d-wide block
        return np.ascontiguousarray(m.reshape(nw, heads, ws, hd).transpose(0, 2, 1, 3).reshape(T, d))

    Q, K, V = heads_of(qkv, 0), heads_of(qkv, d), heads_of(qkv, 2 * d)
    Kt = np.ascontiguousarray(K.transpose(0, 2, 1))
    S = O.scale(O.batch_matmul_forward(Q, Kt), scale)
    P = O.softmax_forward(S.reshape(-1, ws)).reshape(S.shape)
    attn = merge(O.batch_matmul_forward(P, V))
    proj = O.add_broadcast_forward(O.matmul_forward(attn, p["Wproj"]), p["bproj"])
    r1 = O.add_forward(x, proj)
    ln2, mu2, sd2 = O.layernorm_forward(r1)
    z1 = O.add_broadcast_forward(O.matmul_forward(ln2, p["W1"]), p["b1"])
    a1 = O.gelu_forward(z1)
    m2 = O.add_broadcast_forward(O.matmul_forward(a1, p["W2"]), p["b2"])
    out = O.add_forward(r1, m2)
    g = {}
    g["b2"] = O.add_broadcast_backward(d_out)[1]
    d_a1, g["W2"] = O.matmul_backward(a1, p["W2"], d_out)
    d_z1 = O.gelu_backward(z1, d_a1)
    g["b1"] = O.add_broadcast_backward(d_z1)[1]
    d_ln2, g["W1"] = O.matmul_backward(ln2, p["W1"], d_z1)
    d_r1 = O.accumulate_gradients([d_out, O.layernorm_backward(r1, mu2, sd2, d_ln2)])
    g["bproj"] = O.add_broadcast_backward(d_r1)[1]
    d_attn, g["Wproj"] = O.matmul_backward(attn, p["Wproj"], d_r1)
    dO = heads_of(np.concatenate([d_attn, d_attn, d_attn], 1), 0)
    dP, dV = O.batch_matmul_backward(P, V, dO)
    dS = O.softmax_backward(P.reshape(-1, ws), dP.reshape(-1, ws)).reshape(S.shape)
    dSs = O.scale(dS, scale)
    dQ, dKt = O.batch_matmul_backward(Q, Kt, dSs)
    dK = np.ascontiguousarray(dKt.transpose(0, 2, 1))
    d_qkv = np.concatenate([merge(dQ), merge(dK), merge(dV)], 1)
    g["bqkv"] = O.add_broadcast_backward(d_qkv)[1]
    d_ln1, g["Wqkv"] = O.matmul_backward(ln1, p["Wqkv"], d_qkv)
    d_x = O.accumulate_gradients([d_r1, O.layernorm_backward(x, mu1, sd1, d_ln1)])
    return out, g, d_x, dict(P=P, d_qkv=d_qkv, dS=dS)
