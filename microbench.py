"""Per-kernel micro-benchmarks of libprad_cuda (CUDA-event timing on the context's stream).

    python microbench.py                 # every HBM-bound kernel
    python microbench.py --only gelu     # names containing "gelu"
    python microbench.py --gemm          # float GEMM variants at the C5 layer shape
    python microbench.py --packed        # packing kernels and products of packed operands (C5 layer shape)
    python microbench.py --f64           # double GEMM variants and the FP64 FMA rate of the device

HBM kernels are reported as algorithmic bytes / time against the measured copy bandwidth in
MEASURED_PEAKS.json (6546 GB/s if that file is absent), GEMMs as 2*M*N*K / time.  Operands are
1 GiB (larger than L2), so no cache flush is needed between iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from parallelreverseautodiff_b200 import engine as E  # noqa: E402


def _peak_gbs() -> float:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f).get("hbm_gbs", 6546.2))
    return 6546.2


class _Timer:
    def __init__(self, eng):
        import torch

        self.torch, self.eng = torch, eng
        self.stream = torch.cuda.ExternalStream(eng.stream())

    def __call__(self, fn, iters=10, warm=3):
        for _ in range(warm):
            fn()
        self.eng.sync()
        e0, e1 = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
        e0.record(self.stream)
        for _ in range(iters):
            fn()
        e1.record(self.stream)
        self.eng.sync()
        return e0.elapsed_time(e1) / iters


def hbm_kernels(eng, only=None, rows=65536, cols=4096):
    f = np.float32
    peak = _peak_gbs()
    t = _Timer(eng)
    n = rows * cols
    x, dy, out, out2 = (eng.zeros((rows, cols), f) for _ in range(4))
    eng.upload(np.random.default_rng(0).standard_normal((min(rows, 4096), cols), dtype=f), out=x.view((min(rows, 4096), cols)))
    db = eng.empty((1, cols), f)
    idx = eng.upload(np.random.default_rng(1).integers(0, 50000, (rows, 1)).astype(f))
    table = eng.empty((50000, cols), f)
    srows = n // 49
    S, dS, oS = x.view((srows, 49)), dy.view((srows, 49)), out.view((srows, 49))
    lrows = n // 96
    Lx, dL, oL = x.view((lrows, 96)), dy.view((lrows, 96)), out.view((lrows, 96))
    mu, sd = eng.zeros((lrows,), f), eng.zeros((lrows,), f)
    eng.layernorm_forward(Lx, out=(oL, mu, sd))
    P = [[eng.zeros((4096, 4096), f) for _ in range(8)] for _ in range(4)]
    npar = 8 * 4096 * 4096
    cases = [
        ("gelu_backward", 3 * n * 4, lambda: eng.act_backward(E.ACT_GELU, x, dy, out=out)),
        ("leaky_relu_backward", 3 * n * 4, lambda: eng.act_backward(E.ACT_LEAKY_RELU, x, dy, 0.01, out=out)),
        ("sigmoid_backward", 3 * n * 4, lambda: eng.act_backward(E.ACT_SIGMOID, x, dy, out=out)),
        ("tanh_backward", 3 * n * 4, lambda: eng.act_backward(E.ACT_TANH, x, dy, out=out)),
        ("hadamard_backward", 5 * n * 4, lambda: eng.hadamard_backward(x, dy, out2, out=(out, out2.view(out2.shape)))),
        ("mse_backward", 3 * n * 4, lambda: eng.mse_backward(x, dy, grad=out)),
        ("bias_colsum", n * 4, lambda: eng.add_broadcast_backward(x, dbias=db)),
        ("bias_colsum_96", lrows * 96 * 4, lambda: eng.add_broadcast_backward(Lx, dbias=db.view((1, 96)))),
        ("accumulate", 3 * n * 4, lambda: eng.accumulate(out, x)),
        ("segmented_sum_3", 4 * n * 4, lambda: eng.segmented_sum([x, dy, out2], out=out)),
        ("segmented_sum_2", 3 * n * 4, lambda: eng.segmented_sum([x, dy], out=out)),
        # reads dOut and the indices, writes the whole 50000-row table (rows nobody hit are zeroed)
        ("embedding_scatter_ordered", n * 4 + rows * 4 + 50000 * cols * 4, lambda: eng.embedding_backward(idx, x, 50000, out=table)),
        ("softmax_backward_49", 3 * srows * 49 * 4, lambda: eng.softmax_backward(S, dS, out=oS)),
        ("layernorm_backward_96", 3 * lrows * 96 * 4, lambda: eng.layernorm_backward(Lx, mu, sd, dL, out=oL)),
        ("adam", 7 * npar * 4, lambda: eng.adam(P[0], P[1], P[2], P[3], 1e-3, .9, .999, 1e-8, 1.0)),
        ("clip_reference_adam_zero", 11 * npar * 4,
         lambda: eng.clip_adam(P[0], P[1], P[2], P[3], 1, 4.0, 1e-8, 1e-3, .9, .999, 1e-8, 1.0, zero_grad=True)),
        ("clip_global_norm_adam_zero", 9 * npar * 4,
         lambda: eng.clip_adam(P[0], P[1], P[2], P[3], 2, 4.0, 1e-8, 1e-3, .9, .999, 1e-8, 1.0, zero_grad=True)),
    ]
    res = []
    for name, nbytes, fn in cases:
        if only and only not in name:
            continue
        ms = t(fn)
        gbs = nbytes / ms / 1e6
        res.append({"kernel": name, "ms": ms, "GB/s": gbs, "frac_of_measured_copy": gbs / peak})
        print(f"{name:30s} {ms:8.3f} ms {gbs:8.0f} GB/s  {gbs / peak:5.2f} of measured copy peak", flush=True)
    return res


def gemm_variants(eng, rows=16384, width=4096, modes=("simt_fma", "tf32x3", "tf32b16", "bf16x3", "fp16x3")):
    f = np.float32
    t = _Timer(eng)
    A, C_ = eng.zeros((rows, width), f), eng.zeros((rows, width), f)
    W, D = eng.zeros((width, width), f), eng.empty((width, width), f)
    h = np.random.default_rng(0).standard_normal((width, width), dtype=f)
    eng.upload(h, out=W)
    for r0 in range(0, rows, width):
        eng.upload(h, out=A.view((width, width), r0 * width))
        eng.upload(h, out=C_.view((width, width), r0 * width))
    fl = 2.0 * rows * width * width
    for mode in modes:
        eng.set_option("gemm_f32", mode)
        for name, fn in (("dA = dC W^T (NT)", lambda: eng.matmul_backward(None, W, C_, dA=A, need_dB=False)),
                         ("dW = A^T dC (TN)", lambda: eng.matmul_backward(A, None, C_, dB=D, need_dA=False)),
                         ("Y = A W    (NN)", lambda: eng.matmul_forward(A, W, Y=C_))):
            ms = t(fn, iters=5, warm=2)
            print(f"{mode:9s} {name:18s} {ms:8.3f} ms {fl / ms / 1e9:7.1f} TFLOP/s", flush=True)
    eng.set_option("gemm_f32", "auto")


def packed_operands(eng, rows=16384, width=4096, block_cols=0):
    """Packing kernels (HBM-bound: bytes read + written / time) and the three products of one layer on
    packed operands (2 * M * N * K / time, kernel only)."""
    f = np.float32
    peak = _peak_gbs()
    t = _Timer(eng)
    n = rows * width
    z, dy, out = (eng.zeros((rows, width), f) for _ in range(3))
    h = np.random.default_rng(0).standard_normal((min(rows, 4096), width), dtype=f)
    for r0 in range(0, rows, h.shape[0]):
        eng.upload(h, out=z.view(h.shape, r0 * width))
        eng.upload(h * f(1e-3), out=dy.view(h.shape, r0 * width))
    W = eng.upload(np.random.default_rng(1).standard_normal((width, width), dtype=f) * f(0.02))
    both = E.PACK_ROWS | E.PACK_COLS
    PA = eng.packed(rows, width, both, 0, block_cols)
    PD = eng.packed(rows, width, both, 0, block_cols)
    PR = eng.packed(rows, width, E.PACK_ROWS)
    PC = eng.packed(rows, width, E.PACK_COLS)
    PW = eng.packed(width, width, both, PD.blocks()[0], PA.blocks()[0])
    piece = 4          # two FP16 pieces per element and form
    cases = [
        ("pack by rows", n * (4 + piece), lambda: PR.pack(z)),
        ("pack by columns", n * (4 + piece), lambda: PC.pack(z)),
        ("pack both forms", n * (4 + 2 * piece), lambda: PA.pack(z)),
        ("gelu forward -> both forms", n * (4 + 2 * piece), lambda: PA.act_forward(E.ACT_GELU, z, None)),
        ("gelu backward -> both forms", n * (8 + 2 * piece), lambda: PD.act_backward(E.ACT_GELU, z, dy, None)),
        ("gelu backward -> both forms + fp32", n * (12 + 2 * piece), lambda: PD.act_backward(E.ACT_GELU, z, dy, out)),
        ("pack weights both forms", width * width * (4 + 2 * piece), lambda: PW.pack(W)),
    ]
    print(f"blocks: activations by rows {PA.blocks()[0]}, by columns {PA.blocks()[1]}")
    for name, nbytes, fn in cases:
        ms = t(fn)
        gbs = nbytes / ms / 1e6
        print(f"{name:38s} {ms:8.3f} ms {gbs:8.0f} GB/s  {gbs / peak:5.2f} of measured copy peak", flush=True)
    PA.act_forward(E.ACT_GELU, z, None)
    PD.act_backward(E.ACT_GELU, z, dy, None)
    PW.pack(W)
    dW = eng.empty((width, width), f)
    fl = 2.0 * rows * width * width
    for name, fn in (("dA = dZ W^T", lambda: eng.gemm_packed(PD, E.PACK_ROWS, PW, E.PACK_ROWS, out)),
                     ("dW = A^T dZ", lambda: eng.gemm_packed(PA, E.PACK_COLS, PD, E.PACK_COLS, dW)),
                     ("Z = A W", lambda: eng.gemm_packed(PA, E.PACK_ROWS, PW, E.PACK_COLS, out))):
        ms = t(fn, iters=5, warm=2)
        print(f"packed {name:14s} {ms:8.3f} ms {fl / ms / 1e9:7.1f} TFLOP/s", flush=True)


def short_k_products(eng, rows=200704):
    """Products of packed operands with a short k and few columns (the input-gradient products of a narrow
    network: rows x 96 over k = 96 or 384, rows x 384 over k = 96): what they take is their tile stores."""
    f = np.float32
    t = _Timer(eng)
    r = np.random.default_rng(0)
    for K, N in ((96, 96), (384, 96), (96, 384)):
        PA = eng.packed(rows, K, E.PACK_ROWS, 128, 128).pack(eng.upload(r.standard_normal((rows, K), dtype=f)))
        PW = eng.packed(N, K, E.PACK_ROWS, 128, 128).pack(eng.upload(r.standard_normal((N, K), dtype=f)))
        out = eng.empty((rows, N), f)
        ms = t(lambda: eng.gemm_packed(PA, E.PACK_ROWS, PW, E.PACK_ROWS, out), iters=5, warm=2)
        nbytes = rows * (2 * K + 64) * 2 + rows * N * 4
        print(f"{rows} x {N} over k = {K}: {ms * 1e3:8.1f} us {nbytes / ms / 1e6:7.0f} GB/s (pieces read + output written)", flush=True)


def small_products(eng, batch=4096):
    """Strided batches of per-window attention products (49 x 49 over k = 32, 49 x 32 over k = 49): time per launch
    and bytes moved (operands read once, output written once) against the copy bandwidth."""
    f = np.float32
    peak = _peak_gbs()
    t = _Timer(eng)
    r = np.random.default_rng(0)
    for name, (M, K, N), ta, tb in (("S = Q K^T", (49, 32, 49), False, True), ("O = P V", (49, 49, 32), False, False),
                                    ("dV = P^T dO", (49, 49, 32), True, False)):
        a_shape = (batch, K, M) if ta else (batch, M, K)
        b_shape = (batch, N, K) if tb else (batch, K, N)
        a, b = eng.upload(r.standard_normal(a_shape, dtype=f)), eng.upload(r.standard_normal(b_shape, dtype=f))
        c = eng.empty((batch, M, N), f)
        for small in ("1", "0"):
            eng.set_option("gemm_small", small)
            ms = t(lambda: eng.gemm(a, b, c, transA=ta, transB=tb, M=M, N=N, K=K, lda=a_shape[2], ldb=b_shape[2], ldc=N,
                                    batch=batch, strideA=M * K, strideB=K * N, strideC=M * N), iters=10, warm=3)
            nbytes = 4.0 * batch * (M * K + K * N + M * N)
            kern = "one CTA per product" if small == "1" else "64 x 64 tiles"
            print(f"{name:12s} {kern:20s} {ms * 1e3:7.1f} us {nbytes / ms / 1e6:6.0f} GB/s {nbytes / ms / 1e6 / peak:5.2f} of measured copy peak",
                  flush=True)
        eng.set_option("gemm_small", "1")


def f64_variants(eng, n=4096):
    """Double-precision GEMM variants at n^3 and the device's FP64 multiply-add rate (a register-resident
    chain of independent FMAs per thread, every SM full), the denominator for the FP64 kernels."""
    t = _Timer(eng)
    d = np.float64
    A = eng.upload(np.random.default_rng(0).standard_normal((n, n)))
    B = eng.upload(np.random.default_rng(1).standard_normal((n, n)))
    Cm = eng.empty((n, n), d)
    fl = 2.0 * n ** 3
    peak = eng.pipe_rate(0)
    mma = eng.pipe_rate(1)
    print(f"FP64 FMA rate (register-resident chains): {peak:.1f} TFLOP/s; FP64 MMA (m8n8k4): {mma:.1f} TFLOP/s; "
          f"FP32 FMA: {eng.pipe_rate(2):.1f} TFLOP/s", flush=True)
    peak = max(peak, mma)
    for mode in ("simt", "simt_fma", "dmma"):
        eng.set_option("gemm_f64", mode)
        for name, ta, tb in (("NN", False, False), ("NT", False, True), ("TN", True, False)):
            ms = t(lambda: eng.gemm(A, B, Cm, transA=ta, transB=tb), iters=5, warm=2)
            print(f"{mode:9s} {name} {ms:8.3f} ms {fl / ms / 1e9:7.1f} TFLOP/s  {fl / ms / 1e9 / peak:5.2f} of the faster FP64 pipe", flush=True)
    eng.set_option("gemm_f64", "auto")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--gemm", action="store_true")
    ap.add_argument("--packed", action="store_true")
    ap.add_argument("--f64", action="store_true")
    ap.add_argument("--short-k", action="store_true", help="packed products with k of 96 .. 384")
    ap.add_argument("--small-products", action="store_true", help="strided batches of 49 x 49 x 32 products")
    ap.add_argument("--block-cols", type=int, default=0, help="--packed: block length of the by-columns forms (0, 128, 256)")
    ap.add_argument("--rows", type=int, default=None)
    ap.add_argument("--opt", action="append", default=[], metavar="KEY=VALUE", help="prad_set_option before running")
    ap.add_argument("--modes", default="simt_fma,tf32x3,tf32b16,bf16x3,fp16x3")
    args = ap.parse_args()
    with E.Engine(0) as eng:
        for kv in args.opt:
            eng.set_option(*kv.split("=", 1))
        if args.packed:
            packed_operands(eng, rows=args.rows or 16384, block_cols=args.block_cols)
        elif args.small_products:
            small_products(eng, batch=args.rows or 4096)
        elif args.short_k:
            short_k_products(eng, rows=args.rows or 200704)
        elif args.f64:
            f64_variants(eng, n=args.rows or 4096)
        elif args.gemm:
            gemm_variants(eng, rows=args.rows or 16384, modes=tuple(args.modes.split(",")))
        else:
            hbm_kernels(eng, only=args.only, rows=args.rows or 65536)


if __name__ == "__main__":
    main()
