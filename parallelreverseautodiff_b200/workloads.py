"""The small benchmark configurations (C1-C4) as device-resident backward steps.

Each `make_*` returns seeded synthetic inputs (numpy, seed 42) of the configuration's shapes and
value distributions; each `*Runner` uploads them once, runs the forward once, and exposes
`backward()` -- the timed hot path -- plus `samples`, the backward GEMM flop count and the
outputs to compare.  No arithmetic happens here: everything goes through the C ABI.
"""
from __future__ import annotations

import numpy as np

from . import engine as E
from .networks import FeedForwardNetwork, LstmNetwork, SwinBlock


def make_c1(seed=42):
    r = np.random.default_rng(seed)
    return dict(A=r.uniform(-1, 1, (512, 784)), B=r.standard_normal((784, 256)) * np.sqrt(2.0 / 784),
                dOut=r.standard_normal((512, 256)))


def make_c2(seed=42):
    r = np.random.default_rng(seed)
    f = np.float32
    sizes = [784, 512, 512, 10]
    return dict(sizes=sizes, x=r.uniform(0, 1, (256, 784)).astype(f),
                onehot=np.eye(10, dtype=f)[r.integers(0, 10, 256)],
                Ws=[(r.standard_normal((sizes[i], sizes[i + 1])) * np.sqrt(2.0 / sizes[i])).astype(f) for i in range(3)],
                bs=[np.zeros((1, sizes[i + 1]), f) for i in range(3)])


def make_c3(seed=42, T=64, B=32, n_in=128, nh=256):
    r = np.random.default_rng(seed)
    G = ("i", "f", "g", "o")
    return dict(x=r.standard_normal((T, B, n_in)), y=r.standard_normal((T, B, nh)),
                W={g: r.uniform(-1, 1, (nh, n_in)) * np.sqrt(6.0 / (nh + n_in)) for g in G},
                U={g: r.uniform(-1, 1, (nh, nh)) * np.sqrt(6.0 / (nh + nh)) for g in G},
                b={g: r.standard_normal(nh) * 0.1 for g in G})


def make_c4(seed=42, images=64, d=96, heads=3, ws=49, hidden=384):
    r = np.random.default_rng(seed)
    f = np.float32
    T = images * 3136
    he = lambda a, b: (r.standard_normal((a, b)) * np.sqrt(2.0 / a)).astype(f)  # noqa: E731
    bias = lambda n: (r.standard_normal((1, n)) * 0.1).astype(f)  # noqa: E731
    p = {"Wqkv": he(d, 3 * d), "bqkv": bias(3 * d), "Wproj": he(d, d), "bproj": bias(d),
         "W1": he(d, hidden), "b1": bias(hidden), "W2": he(hidden, d), "b2": bias(d)}
    x = np.empty((T, d), f)
    d_out = np.empty((T, d), f)
    for r0 in range(0, T, 3136):        # image by image keeps the generator's temporaries small
        x[r0:r0 + 3136] = r.standard_normal((3136, d))
        d_out[r0:r0 + 3136] = r.standard_normal((3136, d))
    return dict(x=x, d_out=d_out, p=p, heads=heads, ws=ws, d=d, hidden=hidden, images=images)


class C1Runner:
    """MatMul -> LeakyReLU(0.01) node, PRAD double: dPre, dA, dB."""
    name, dtype, samples = "C1 MatMul->LeakyReLU node 512x784x256 (double)", "f64", 512
    flops = 4.0 * 512 * 784 * 256
    # algorithmic bytes of one step: A, B, dOut, saved pre-activation read; dPre, dA, dB written
    bytes = 8.0 * (2 * 512 * 784 + 2 * 784 * 256 + 3 * 512 * 256)

    def __init__(self, eng, inp):
        self.eng = eng
        self.A, self.B, self.dOut = eng.upload(inp["A"]), eng.upload(inp["B"]), eng.upload(inp["dOut"])
        self.pre = eng.matmul_forward(self.A, self.B)
        self.out = [eng.empty((512, 256), np.float64), eng.empty((512, 784), np.float64), eng.empty((784, 256), np.float64)]

    def backward(self):
        e = self.eng
        E.check(e.lib.prad_matmul_act_backward(e.ctx, E.F64, self.A.ptr, self.B.ptr, self.dOut.ptr, E.ACT_LEAKY_RELU,
                                               self.pre.ptr, 0.01, self.out[0].ptr, self.out[1].ptr, self.out[2].ptr,
                                               512, 784, 256))


class C2Runner:
    """MLP 784-512-512-10, PRADLite float, batch 256: backward + clip + Adam."""
    name, dtype, samples = "C2 MLP 784-512-512-10 batch 256 (float) + clip + Adam", "f32", 256
    flops = 4.0 * 256 * (784 * 512 + 512 * 512 + 512 * 10)
    # per layer: A, W, dZ read, dA, dW written, three activation-backward streams; then 11 streams of
    # 4 bytes per parameter for clip + Adam + clear
    bytes = 4.0 * sum(2 * 256 * k + 2 * k * n + 4 * 256 * n for k, n in ((784, 512), (512, 512), (512, 10))) + 44.0 * 669706

    def __init__(self, eng, inp, clip_mode=E.CLIP_REFERENCE):
        net = FeedForwardNetwork(eng, np.float32, inp["sizes"], hidden_act=E.ACT_LEAKY_RELU, softmax_output=True,
                                 loss="cce", use_bias=True, clip_mode=clip_mode)
        net.set_weights(inp["Ws"], inp["bs"])
        net._ensure_buffers(256)
        eng.upload(inp["x"], out=net.A[0])
        eng.upload(inp["onehot"], out=net.target)
        net.forward()
        self.net = net

    def backward(self):
        self.net.backward()
        self.net.clip_and_optimize()


class C3Runner:
    """Single-layer LSTM 128 -> 256, 64 steps, batch 32, PRAD double: full BPTT."""
    name, dtype, samples = "C3 LSTM in 128 hidden 256 T 64 batch 32 (double), BPTT", "f64", 32
    flops = 64 * 4.0 * 32 * 1024 * (128 + 256)
    # per time step: the gate tensors (about twenty streams of 32 x 256 doubles) and the 32 x (128 + 256)
    # inputs of the gate products; once per step of the optimiser: the 394 240 weights read and their
    # gradients written
    bytes = 64 * 8.0 * (20 * 32 * 256 + 2 * 32 * (128 + 256)) + 2 * 8.0 * 4 * (256 * 128 + 256 * 256 + 256)

    def __init__(self, eng, inp):
        T, B, n_in = inp["x"].shape
        nh = inp["y"].shape[2]
        self.net = LstmNetwork(eng, np.float64, n_in, nh, T, B)
        self.net.set_parameters(inp["W"], inp["U"], inp["b"])
        self.net.forward(inp["x"], inp["y"])

    def backward(self):
        self.net.backward()


class C4Runner:
    """Swin-style windowed attention block, PRADLite float: full backward."""
    dtype = "f32"

    def __init__(self, eng, inp):
        self.samples = inp["images"]
        self.name = f"C4 Swin block dim 96, 3 heads, 7x7 windows, {inp['images']} images (float)"
        self.flops = 96.3e9 * inp["images"] / 64.0
        # tokens x (LayerNorm backward 2 x 3 x 96, GELU backward 3 x 384, product operands and results of the
        # five projections read and written once, attention scores 3 x 3 x 49 per token and head set) x 4 bytes
        t = inp["images"] * 3136
        self.bytes = 4.0 * t * (6 * 96 + 3 * 384 + 2 * (96 + 288) + 2 * (96 + 96) + 2 * (96 + 384) + 2 * (384 + 96) + 9 * 49 * 3)
        self.blk = SwinBlock(eng, np.float32, inp["d"], inp["heads"], inp["ws"], inp["hidden"] // inp["d"])
        self.blk.set_parameters(inp["p"])
        self.d_out = eng.upload(inp["d_out"])
        self.blk.forward(eng.upload(inp["x"]))

    def backward(self):
        self.blk.backward(self.d_out)
