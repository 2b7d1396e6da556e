"""Generates tests/golden/ops_f32.npz and ops_f64.npz: seeded inputs and the CPU oracle's
outputs for every operation of the path, small enough to commit.

    python tests/golden/make_golden.py

The reference itself (C#) cannot run where this repository is built, so these vectors pin
the ORACLE (a regression fixture for it and the expected values for the CUDA kernels); the
reference's own known-answer vectors are transcribed in tests/test_oracle_pins.py.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle as O  # noqa: E402


def make(dtype):
    r = np.random.default_rng(42)
    n = lambda *s, std=1.0: (r.standard_normal(s) * std).astype(dtype)  # noqa: E731
    g = {}
    M, K, N = 33, 47, 21
    A = (r.random((M, K)) * 2 - 1).astype(dtype)
    B = n(K, N, std=np.sqrt(2.0 / K))
    dC = n(M, N)
    g["mm_A"], g["mm_B"], g["mm_dC"] = A, B, dC
    g["mm_C"] = O.matmul_forward(A, B)
    g["mm_dA"], g["mm_dB"] = O.matmul_backward(A, B, dC)
    pre = g["mm_C"]
    g["node_dPre"] = O.leaky_relu_backward(pre, dC, 0.01)
    g["node_dA"], g["node_dB"] = O.matmul_backward(A, B, g["node_dPre"])
    bA, bB, bdC = n(5, 9, 8), n(5, 8, 9), n(5, 9, 9)
    g["bmm_A"], g["bmm_B"], g["bmm_dC"] = bA, bB, bdC
    g["bmm_C"] = O.batch_matmul_forward(bA, bB)
    g["bmm_dA"], g["bmm_dB"] = O.batch_matmul_backward(bA, bB, bdC)
    x, dy = n(19, 23, std=2.0), n(19, 23)
    g["x"], g["dy"] = x, dy
    g["leaky_y"], g["leaky_dx"] = O.leaky_relu_forward(x, 0.01), O.leaky_relu_backward(x, dy, 0.01)
    g["sigmoid_y"] = O.sigmoid_forward(x)
    g["sigmoid_dx"] = O.sigmoid_backward(g["sigmoid_y"], dy)
    g["tanh_y"] = O.tanh_forward(x)
    g["tanh_dx"] = O.tanh_backward(g["tanh_y"], dy)
    g["gelu_y"], g["gelu_dx"] = O.gelu_forward(x), O.gelu_backward(x, dy)
    g["had_da"], g["had_db"] = O.hadamard_backward(x, dy, dy)
    g["bias_db"] = O.add_broadcast_backward(dy)[1]
    g["softmax_y"] = O.softmax_forward(x)
    g["softmax_dx"] = O.softmax_backward(g["softmax_y"], dy)
    g["ln_y"], g["ln_mean"], g["ln_std"] = O.layernorm_forward(x)
    g["ln_dx"] = O.layernorm_backward(x, g["ln_mean"], g["ln_std"], dy)
    g["mse_grad"] = O.mse_backward(x, dy)
    g["mse_loss"] = np.asarray(O.mse_forward(x, dy), dtype)
    onehot = np.eye(23, dtype=dtype)[r.integers(0, 23, 19)]
    g["onehot"] = onehot
    g["cce_grad"] = O.cce_backward(g["softmax_y"], onehot)
    g["cce_loss"] = np.asarray(O.cce_forward(g["softmax_y"], onehot), dtype)
    idx = r.integers(0, 7, 40).astype(dtype).reshape(-1, 1)
    Wemb, dE = n(7, 6), n(40, 6)
    g["emb_idx"], g["emb_W"], g["emb_dOut"] = idx, Wemb, dE
    g["emb_out"] = O.embedding_forward(idx, Wemb)
    g["emb_dW"] = O.embedding_backward(idx, dE, 7)
    gs = [n(11, 13) for _ in range(4)]
    g["acc_srcs"] = np.stack(gs)
    g["acc_sum"] = O.accumulate_gradients(gs)
    g["acc_mean"] = O.batch_mean(gs)
    grad = n(40, 30, std=3.0)
    g["clip_in"] = grad
    minv = 1e-8 if dtype == np.float32 else 1e-16
    g["clip_out"] = O.clip_reference(grad.copy(), 4.0, minv)
    w, m, v = n(40, 30), n(40, 30, std=0.01), np.abs(n(40, 30, std=0.01))
    g["adam_w0"], g["adam_m0"], g["adam_v0"] = w.copy(), m.copy(), v.copy()
    O.adam_rmad(w, m, v, g["clip_out"], 1e-3, 0.9, 0.999, 1e-8, 3.0)
    g["adam_w1"], g["adam_m1"], g["adam_v1"] = w, m, v
    # operations added after the first release of these files: appended, so that the draws above
    # (and with them every earlier vector) stay what they were
    g["relu_y"], g["relu_dx"] = O.relu_forward(x), O.relu_backward(x, dy)
    g["ampsig_y"], g["ampsig_dx"] = O.amplified_sigmoid_forward(x), O.amplified_sigmoid_backward(x, dy)
    beta, gamma = n(19, 1), n(19, 1)
    g["ss_beta"], g["ss_gamma"] = beta, gamma
    g["ss_y"] = O.scale_shift_forward(x, beta, gamma)
    g["ss_dx"], g["ss_dbeta"], g["ss_dgamma"] = O.scale_shift_backward(x, beta, dy)
    gain = n(19, 23)
    g["rms_g"] = gain
    g["rms_y"] = O.rmsnorm_forward(x, gain)
    g["rms_dx"], g["rms_dg"] = O.rmsnorm_backward(x, gain, dy)
    return g


if __name__ == "__main__":
    for dt, name in ((np.float32, "f32"), (np.float64, "f64")):
        np.savez_compressed(os.path.join(HERE, f"ops_{name}.npz"), **make(dt))
        print("wrote", f"ops_{name}.npz")
