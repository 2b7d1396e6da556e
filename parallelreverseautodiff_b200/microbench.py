"""Per-kernel micro-benchmarks of libprad_cuda (CUDA-event timing on the context's stream).

    python -m parallelreverseautodiff_b200.microbench                 # every HBM-bound kernel
    python -m parallelreverseautodiff_b200.microbench --only gelu     # names containing "gelu"
    python -m parallelreverseautodiff_b200.microbench --gemm          # GEMM variants at the C5 layer shape

HBM kernels are reported as algorithmic bytes / time against the measured copy bandwidth in
MEASURED_PEAKS.json (6546 GB/s if that file is absent), GEMMs as 2*M*N*K / time.  Operands are
1 GiB (larger than L2), so no cache flush is needed between iterations.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np

from . import engine as E


def _peak_gbs() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
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
        ("accumulate", 3 * n * 4, lambda: eng.accumulate(out, x)),
        ("segmented_sum_3", 4 * n * 4, lambda: eng.segmented_sum([x, dy, out2], out=out)),
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--gemm", action="store_true")
    ap.add_argument("--rows", type=int, default=None)
    ap.add_argument("--opt", action="append", default=[], metavar="KEY=VALUE", help="prad_set_option before running")
    ap.add_argument("--modes", default="simt_fma,tf32x3,tf32b16,bf16x3,fp16x3")
    args = ap.parse_args()
    with E.Engine(0) as eng:
        for kv in args.opt:
            eng.set_option(*kv.split("=", 1))
        if args.gemm:
            gemm_variants(eng, rows=args.rows or 16384, modes=tuple(args.modes.split(",")))
        else:
            hbm_kernels(eng, only=args.only, rows=args.rows or 65536)


if __name__ == "__main__":
    main()
