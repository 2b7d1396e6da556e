#!/usr/bin/env python
"""Benchmark of the backward hot path on the large data-parallel MLP (PRADLite float32):
8 layers of 4096x4096 with GELU, MSE loss, global batch 65536 rows sharded over N GPUs,
weight-gradient all-reduce overlapped with the backward, then clip + Adam.

    python bench.py --gpus N --steps K --warmup W            # this library (one JSON line)
    python bench.py --impl reference --steps K --warmup W    # CPU restatement of the C# loops

A step of the device-resident measurement (`value`) is one backward pass of the whole
network (loss gradient, per layer dW and dA GEMMs with the GELU derivative fused in, the
all-reduces) followed by gradient clip + Adam, on activations that already sit in HBM.
`e2e` is the same metric through the host-buffer API: each step uploads the batch and the
targets from page-locked host memory, runs forward, loss, backward, clip + Adam and reads
the loss back.  Data is synthetic (seeded N(0,1) inputs and targets, He-initialised weights).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WIDTH, LAYERS, GLOBAL_BATCH = 4096, 8, 65536
METRIC, UNIT = "backward_samples_per_s", "samples/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="c5", choices=["c1", "c2", "c3", "c4", "c5"],
                    help="benchmark configuration (c5, the large data-parallel MLP, is the headline)")
    ap.add_argument("--images", type=int, default=64, help="c4: images per batch")
    ap.add_argument("--batch", type=int, default=GLOBAL_BATCH, help="global batch rows")
    ap.add_argument("--width", type=int, default=WIDTH)
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--clip", default="reference", choices=["reference", "global_norm", "none"])
    ap.add_argument("--dp-mode", default="sharded", choices=["sharded", "overlap", "end"],
                    help="N > 1: sharded = each weight gradient is reduced to the rank that owns the tensor, beside the "
                         "backward; the owner alone clips and updates it and broadcasts the new weights beside the next "
                         "step's first product.  overlap = all-reduce each weight gradient beside the backward, every rank "
                         "runs the whole optimiser.  end = one all-reduce of all gradients after the backward")
    ap.add_argument("--no-sequence", action="store_true",
                    help="c1..c4: call the entry points every step instead of replaying a recorded launch sequence")
    ap.add_argument("--opt", action="append", default=[], metavar="KEY=VALUE",
                    help="library option set with prad_set_option before the run (repeatable)")
    ap.add_argument("--gemm", default="auto", choices=["auto", "simt", "simt_fma", "tf32x3", "tf32b16", "bf16x3", "fp16x3"])
    ap.add_argument("--tc-pipeline", default=None, choices=[None, "16x4", "32x2", "8x8"])
    ap.add_argument("--lr", type=float, default=1e-5,
                    help="Adam learning rate (1e-3, the reference default, makes this 8-layer GELU net "
                         "diverge within ten steps on random targets; the arithmetic per step is the same)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--pack-block-cols", type=int, default=0, choices=[0, 128, 256],
                    help="block length of the by-columns packed forms (0 = the library's default)")
    return ap.parse_args()


def backward_flops(batch, width, layers):
    # MatrixMultiplyOperation.Backward: two products of 2*M*N*K each, per layer
    return 4.0 * batch * width * width * layers


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples nvidia-smi (read-only) while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()  # the exact child we started
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # samples under load: the upper half of the observed clocks
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------ CPU baseline (oracle)
CPU_SLICE_ROWS = 64   # batch rows of the bounded CPU sample; the same for every leg that times the CPU path


def host_threads() -> int:
    """Host threads the CPU legs use: every core this process may run on.  Launchers such as
    torch.distributed.run export OMP_NUM_THREADS=1 to their workers; the CPU path stands for the
    reference's Parallel.For loops, which use all cores, so that setting is overridden."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def c5_config(args, world):
    """The `config` object of the C5 workload -- identical for the native and the reference arm."""
    rows = args.batch // max(world, 1)
    return {"workload": f"C5 data-parallel MLP {args.layers}x({args.width}x{args.width}, GELU), "
                        f"MSE, global batch {args.batch}, clip={args.clip} + Adam",
            "global_batch": args.batch, "rows_per_gpu": rows, "parallelism": f"dp{world}",
            "dp_mode": args.dp_mode if world > 1 else None, "gemm": args.gemm, "lr": args.lr,
            "l2": f"inputs larger than L2: a step streams {args.layers * rows * args.width * 16 / 2**30:.1f} GiB of "
                  f"activations, gradients and packed operands per GPU between two uses of the same line"}


class CpuStep:
    """The same step the device arm times, restated on the CPU (oracle) for a bounded sample:
    MSE gradient, then per layer GELU' + dB + dA (MatrixMultiplyOperation.Backward), all
    `layers` layers on CPU_SLICE_ROWS batch rows; then the z-score clip and Adam on ONE of the
    `layers` weight tensors.  The row part is linear in the rows (measured here on a slice that
    fits the caches better than the full batch would, which favours the CPU) and the optimiser
    part is linear in the tensors, so one full step costs
        t_rows * (batch / CPU_SLICE_ROWS) + t_opt * layers."""

    def __init__(self, args, seed=42):
        import oracle as O

        self.O = O
        self.threads = host_threads()
        O.set_num_threads(self.threads)
        self.args = args
        w, L, S = args.width, args.layers, CPU_SLICE_ROWS
        r = np.random.default_rng(seed)
        f = np.float32
        self.W = [(r.standard_normal((w, w)) * np.sqrt(2.0 / w)).astype(f) for _ in range(L)]
        self.A = [r.standard_normal((S, w)).astype(f) for _ in range(L + 1)]
        self.Z = [r.standard_normal((S, w)).astype(f) for _ in range(L)]
        self.T = r.standard_normal((S, w)).astype(f)
        self.m = np.zeros((w, w), f)
        self.v = np.zeros((w, w), f)

    def step(self):
        """Returns (t_rows, t_opt) in seconds."""
        O, a = self.O, self.args
        L = a.layers
        t0 = time.perf_counter()
        d = O.mse_backward(self.A[L], self.T, rows_total=a.batch)
        dW = None
        for l in range(L - 1, -1, -1):
            d = O.gelu_backward(self.Z[l], d)
            d, dW = O.matmul_backward(self.A[l], self.W[l], d)
        t1 = time.perf_counter()
        if a.clip == "reference":
            O.clip_reference(dW, np.float32(4.0), np.float32(1e-8))
        elif a.clip == "global_norm":
            O.clip_global_norm([dW], 4.0)
        w = self.W[0].copy()
        O.adam_rmad(w, self.m, self.v, dW, a.lr, 0.9, 0.999, 1e-8, 1.0)
        t2 = time.perf_counter()
        return t1 - t0, t2 - t1

    def full_step_seconds(self, t_rows, t_opt):
        a = self.args
        return t_rows * (a.batch / CPU_SLICE_ROWS) + t_opt * a.layers

    def describe(self, t_rows, t_opt):
        a = self.args
        return (f"MSE gradient + {a.layers} layers of GELU' + dA + dB on {CPU_SLICE_ROWS} rows ({t_rows:.2f} s), "
                f"clip={a.clip} + Adam on one {a.width}x{a.width} tensor ({t_opt:.2f} s); full step = "
                f"rows part x {a.batch // CPU_SLICE_ROWS} + optimiser part x {a.layers}; "
                f"C++ restatement of the C# loops with OpenMP, not the .NET runtime")


def cpu_baseline_c5(args, repeats=2):
    """cpu_baseline of the native arm: `repeats` timed sample steps after one untimed."""
    cs = CpuStep(args)
    cs.step()
    ts = [cs.step() for _ in range(repeats)]
    t_rows = min(t[0] for t in ts)
    t_opt = min(t[1] for t in ts)
    sps = args.batch / cs.full_step_seconds(t_rows, t_opt)
    return {"value": sps, "unit": UNIT, "cores": cs.threads, "kind": "port",
            "sample": cs.describe(t_rows, t_opt)}


def run_reference(args, rank):
    """--impl reference: the reference's CPU path (restated in C++, OpenMP over the index the
    C# code gives Parallel.For) on the box's host cores.  Rank 0 only; a step is one bounded
    sample of the workload (see CpuStep)."""
    if rank != 0:
        return
    cs = CpuStep(args)
    ts = []
    for i in range(args.warmup + args.steps):
        t = cs.step()
        if i >= args.warmup:
            ts.append(t)
    t_rows = statistics.mean(t[0] for t in ts)
    t_opt = statistics.mean(t[1] for t in ts)
    full = cs.full_step_seconds(t_rows, t_opt)
    sps = args.batch / full
    line = {
        "impl": "reference", "metric": METRIC, "value": sps, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        # one timed step of this arm is the bounded sample, not the extrapolated full step
        "ms_per_step": 1e3 * (t_rows + t_opt), "full_step_ms_extrapolated": 1e3 * full,
        "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": c5_config(args, args.gpus),
        "tflops": backward_flops(1, args.width, args.layers) * sps / 1e12,
        "cpu_baseline": {"value": sps, "unit": UNIT, "cores": cs.threads, "kind": "port",
                         "sample": cs.describe(t_rows, t_opt)},
        "e2e": {"value": sps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ native arm
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p.get("hbm_gbs"), "tensor_tflops": p.get("bf16_tflops_sustained") or p.get("bf16_tflops"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tensor_tflops": 1400.0, "source": "fallback"}


def gemm_traffic_bytes(rows, width, gemm):
    """DRAM bytes of one backward GEMM launch of the default kernel (CTA pairs): one ncu capture of a
    16384-row launch on packed operands (0.814 GB read + 0.250 GB written; algorithmic 0.604 GB --
    the row operand streams once per column panel), scaled linearly in the rows: the traffic is
    dominated by the row-proportional operand and result.  None for other kernels or widths."""
    if gemm != "auto" or width != 4096:
        return None
    return 1.0635e9 * rows / 16384.0


def run_native(args, rank, world, local_rank):
    import torch

    from parallelreverseautodiff_b200 import engine as E
    from parallelreverseautodiff_b200.networks import FeedForwardNetwork

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    assert args.batch % world == 0, "global batch must divide over the ranks"
    rows = args.batch // world

    eng = E.Engine(local_rank)
    eng.set_option("gemm_f32", args.gemm)
    for kv in args.opt:
        eng.set_option(*kv.split("=", 1))
    if args.tc_pipeline:
        eng.set_option("tc_pipeline", args.tc_pipeline)
    if world > 1:
        ids = [E.Engine.dp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        eng.dp_init(ids[0], rank, world)

    clip = {"reference": E.CLIP_REFERENCE, "global_norm": E.CLIP_GLOBAL_NORM, "none": E.CLIP_NONE}[args.clip]
    sizes = [args.width] * (args.layers + 1)
    net = FeedForwardNetwork(eng, np.float32, sizes, hidden_act=E.ACT_GELU, output_act=E.ACT_GELU,
                             loss="mse", use_bias=False, clip_mode=clip, rank=rank, world=world,
                             dp_overlap=args.dp_mode != "end",
                             dp_sharded=args.dp_mode == "sharded" and clip != E.CLIP_GLOBAL_NORM,
                             pack_block_cols=args.pack_block_cols)
    net.Parameters.LearningRate = args.lr
    wr = np.random.default_rng(42)  # identical weights on every rank
    net.set_weights([(wr.standard_normal((args.width, args.width), dtype=np.float32)
                      * np.float32(np.sqrt(2.0 / args.width))) for _ in range(args.layers)])
    dr = np.random.default_rng(1000 + rank)  # this rank's rows of the batch
    x_host = eng.pinned_empty((rows, args.width), np.float32)
    t_host = eng.pinned_empty((rows, args.width), np.float32)
    chunk = 4096
    for r0 in range(0, rows, chunk):
        r1 = min(rows, r0 + chunk)
        x_host[r0:r1] = dr.standard_normal((r1 - r0, args.width), dtype=np.float32)
        t_host[r0:r1] = dr.standard_normal((r1 - r0, args.width), dtype=np.float32)

    stream = torch.cuda.ExternalStream(eng.stream(), device=torch.device("cuda", local_rank))

    def barrier():
        eng.sync()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        eng.sync()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if not dist:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # warm-up: full end-to-end steps (they also leave valid activations in HBM)
    loss = None
    for _ in range(max(args.warmup, 1)):
        loss = net.train_step_host(x_host, t_host, rows_total=args.batch)

    # ---- (A) device-resident hot path: backward + clip + Adam ---------------------------
    net.forward_follows = False     # a backward follows each optimiser step here: owners publish W_L-1 first
    marks = {"gemm": [], "join": [], "opt": [], "pack": []}

    def probe(kind, begin):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(stream)
        marks[kind].append(ev)

    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    launches0 = eng.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        net.backward(rows_total=args.batch, probe=probe)
        probe("opt", True)
        net.clip_and_optimize()
        probe("opt", False)
    net._join_broadcasts()      # sharded optimiser: the last step's weight broadcasts belong to the timed region
    ev1.record(stream)
    barrier()
    launches = eng.launch_count() - launches0
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    ms_step = ms_total / args.steps
    def bracket_ms(kind):
        evs = marks[kind]
        return sum(evs[i].elapsed_time(evs[i + 1]) for i in range(0, len(evs), 2))

    gemm_ms = bracket_ms("gemm")
    n_gemm = len(marks["gemm"]) // 2
    # where this rank's step went (device time per step): products with their operand passes, the join
    # with the communication stream at the end of the backward, clip + Adam; the rest is the loss
    # gradient, activation derivatives and whatever the stream waited for
    mine = {"rank": rank, "step_ms": ev0.elapsed_time(ev1) / args.steps, "gemm_ms": gemm_ms / args.steps,
            "pack_ms": bracket_ms("pack") / args.steps, "join_ms": bracket_ms("join") / args.steps,
            "optimizer_ms": bracket_ms("opt") / args.steps}
    per_rank = [mine]
    if dist:
        per_rank = [None] * world
        dist.all_gather_object(per_rank, mine)

    # ---- (B) end to end through the host-buffer API -------------------------------------
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    # every step copies its batch from page-locked host memory and reads its loss back; the copy
    # of step i+1 overlaps with the compute of step i (FeedForwardNetwork.train_steps_host)
    for loss in net.train_steps_host([(x_host, t_host)] * args.steps, rows_total=args.batch):
        pass
    e1.record(stream)
    barrier()
    clocks = sampler.stop()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps

    flops_step = backward_flops(args.batch, args.width, args.layers)
    value = args.batch / (ms_step * 1e-3)
    peaks = measured_peaks()
    flops_per_gemm = 2.0 * rows * args.width * args.width
    achieved_tflops = flops_per_gemm * n_gemm / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cpu = cpu_baseline_c5(args)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 1), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": c5_config(args, world),
            "tflops": flops_step / (ms_step * 1e-3) / 1e12,
            "roofline": {"bound": "tensor", "achieved": achieved_tflops, "peak": peaks["tensor_tflops"],
                         "unit": "TFLOP/s",
                         "frac": (achieved_tflops / peaks["tensor_tflops"]) if achieved_tflops else None,
                         # an FP32-faithful product costs three FP16 tensor-core products (two-piece operands):
                         # the tensor pipe's own share of the measured dense peak is three times `frac`
                         "tensor_products_per_flop": 3 if args.gemm in ("auto", "fp16x3") else None,
                         "tensor_pipe_frac": (3 * achieved_tflops / peaks["tensor_tflops"])
                         if achieved_tflops and args.gemm in ("auto", "fp16x3") else None,
                         "traffic": gemm_traffic_bytes(rows, args.width, args.gemm),
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one "
                                           "16384 x 4096 x 4096 launch of the default kernel (CTA pairs) on packed operands (1.0635 GB), scaled by rows",
                         "kernel": "backward GEMMs (dW = A^T dZ, dA = dZ W^T)",
                         "peak_source": peaks["source"] + " dense bf16, sustained",
                         "launches_timed": n_gemm},
            "cpu_baseline": cpu,
            "e2e": {"value": args.batch / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": int(x_host.nbytes + t_host.nbytes) * world,
                    "d2h_bytes_per_step": 4 * world, "ms_per_step": e2e_ms, "loss": loss},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "per_rank": [{k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()} for r in per_rank],
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        eng.dp_shutdown()
    eng.close()
    if dist:
        dist.destroy_process_group()


# ------------------------------------------------------------------ small configurations
def cpu_small(workload, inp):
    """CPU restatement of one whole forward + backward of the configuration (forward needed to
    produce what the backward reads; only the backward part is timed where separable)."""
    import oracle as O
    from oracle import configs as OC

    t0 = time.perf_counter()
    if workload == "c1":
        pre = O.matmul_forward(inp["A"], inp["B"])
        t0 = time.perf_counter()
        dPre = O.leaky_relu_backward(pre, inp["dOut"], 0.01)
        O.matmul_backward(inp["A"], inp["B"], dPre)
        return time.perf_counter() - t0, "backward only, full size", 1.0
    if workload == "c2":
        OC.mlp_oracle(inp["x"], inp["onehot"], inp["Ws"], inp["bs"], np.float32(0.01))
        return time.perf_counter() - t0, "forward + backward, full size (backward is 2/3 of the flops)", 2.0 / 3.0
    if workload == "c3":
        OC.lstm_oracle(inp["x"], inp["y"], inp["W"], inp["U"], inp["b"])
        return time.perf_counter() - t0, "forward + backward, full size (backward is 2/3 of the flops)", 2.0 / 3.0
    imgs = min(2, inp["images"])
    T = imgs * 3136
    OC.swin_oracle(inp["x"][:T], inp["d_out"][:T], inp["p"], inp["heads"], inp["ws"])
    scale = inp["images"] / imgs
    return (time.perf_counter() - t0) * scale, f"forward + backward on {imgs} images, scaled linearly to {inp['images']}", 2.0 / 3.0


def run_small(args, rank, world, local_rank):
    """C1-C4: too small to shard, so N GPUs run N independent replicas (weak scaling)."""
    import torch

    from parallelreverseautodiff_b200 import engine as E
    from parallelreverseautodiff_b200 import workloads as WL

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    eng = E.Engine(local_rank)
    make = {"c1": WL.make_c1, "c2": WL.make_c2, "c3": WL.make_c3, "c4": lambda: WL.make_c4(images=args.images)}[args.workload]
    inp = make()
    runner = {"c1": WL.C1Runner, "c2": WL.C2Runner, "c3": WL.C3Runner, "c4": WL.C4Runner}[args.workload](eng, inp)
    stream = torch.cuda.ExternalStream(eng.stream(), device=torch.device("cuda", local_rank))
    flush = eng.empty((64 * 1024 * 1024,), np.float32)     # 256 MiB > L2: written between timed steps

    def barrier():
        eng.sync()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()

    for _ in range(max(args.warmup, 3)):
        runner.backward()
    # the step as a recorded launch sequence (one submission per step) unless --no-sequence
    seq = None if args.no_sequence else eng.record(runner.backward)
    step = seq.launch if seq else runner.backward
    step()
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    n0 = eng.launch_count()
    total_ms = 0.0
    for _ in range(args.steps):
        eng.zero_(flush)                                   # L2 flush, outside the timed bracket
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        step()
        e1.record(stream)
        eng.sync()
        total_ms += e0.elapsed_time(e1)
    launches = eng.launch_count() - n0
    barrier()
    clocks = sampler.stop()
    ms = total_ms / args.steps
    if dist:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    # end to end for C1: the host-buffer entry point (numpy in, numpy out)
    e2e = None
    if args.workload == "c1":
        pre = runner.pre.numpy()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            eng.matmul_act_backward_host(inp["A"], inp["B"], inp["dOut"], E.ACT_LEAKY_RELU, pre, 0.01)
        dt = (time.perf_counter() - t0) / args.steps
        nbytes = sum(inp[k].nbytes for k in ("A", "B", "dOut")) + pre.nbytes
        e2e = {"value": world * runner.samples / dt, "unit": UNIT, "h2d_bytes_per_step": int(nbytes),
               "d2h_bytes_per_step": int(inp["A"].nbytes + inp["B"].nbytes + pre.nbytes), "ms_per_step": dt * 1e3,
               "note": "prad_matmul_act_backward_host, pageable host arrays, wall clock"}
    if rank == 0:
        cpu = None
        if not args.no_cpu_baseline:
            import oracle as O

            secs, what, bwd_frac = cpu_small(args.workload, inp)
            cpu = {"value": runner.samples / (secs * bwd_frac), "unit": UNIT, "cores": O.num_threads(), "kind": "port",
                   "sample": what + "; C++ restatement of the C# loops with OpenMP, not the .NET runtime"}
        peaks = measured_peaks()
        tflops = runner.flops / (ms * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": world * runner.samples / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": runner.dtype, "data": "synthetic",
            "config": {"workload": runner.name, "parallelism": f"replicas x{world}",
                       "submission": "direct calls" if seq is None else "recorded launch sequence (prad_sequence_launch)",
                       "l2": "256 MiB buffer written between timed steps (L2 flush)"},
            "tflops": tflops * world,
            # these steps are hundreds of small dependent kernels: nothing saturates a pipe.  The honest yardstick
            # is the memory system: algorithmic bytes of the step over its time against the measured copy bandwidth,
            # with the launch count beside it (ms_per_step / launches = time per kernel)
            "roofline": {"bound": "hbm", "achieved": runner.bytes / (ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": runner.bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "traffic": None,
                         "kernel": "whole backward step (launch-latency-bound at this size)",
                         "launches_per_step": int(launches // max(args.steps, 1)),
                         "us_per_launch": 1e3 * ms / max(1, launches // max(args.steps, 1)),
                         "tensor_frac_for_context": tflops / peaks["tensor_tflops"],
                         "peak_source": peaks["source"] + " copy bandwidth"},
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    eng.close()
    if dist:
        dist.destroy_process_group()


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if args.workload != "c5":
            if rank == 0:
                from parallelreverseautodiff_b200 import workloads as WL
                import oracle as O

                make = {"c1": WL.make_c1, "c2": WL.make_c2, "c3": WL.make_c3,
                        "c4": lambda: WL.make_c4(images=args.images)}[args.workload]
                inp = make()
                samples = {"c1": 512, "c2": 256, "c3": 32, "c4": args.images}[args.workload]
                secs, what, frac = cpu_small(args.workload, inp)
                v = samples / (secs * frac)
                print(json.dumps({"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
                                  "steps": 1, "warmup": 0, "ms_per_step": secs * frac * 1e3, "higher_is_better": True,
                                  "scaling": "weak", "vs_baseline": None, "data": "synthetic",
                                  "config": {"workload": args.workload, "parallelism": "cpu"},
                                  "cpu_baseline": {"value": v, "unit": UNIT, "cores": O.num_threads(), "kind": "port", "sample": what},
                                  "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                                  "gpu_launches": 0}), flush=True)
            return
        run_reference(args, rank)
        return
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    if args.workload != "c5":
        run_small(args, rank, world, local_rank)
        return
    run_native(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
