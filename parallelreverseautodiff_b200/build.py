"""Builds ``libprad_cuda.so`` for sm_100a with nvcc (in-tree, next to this file).

``python -m parallelreverseautodiff_b200.build`` compiles every ``csrc/*.cu`` file into an
object and links the shared library.  Objects are rebuilt only when their source (or any
header) is newer.  The elementwise / row / optimiser files are compiled with ``-fmad=false``
so that products and sums round separately, as the managed reference code does; the GEMM
files keep FMA contraction.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libprad_cuda.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
          "-Xcompiler", "-fno-strict-aliasing"]
# files whose kernels must not contract a*b+c into an FMA
NO_FMAD = {"elementwise.cu", "rowops.cu", "loss_embedding.cu", "optimizer.cu", "matmul.cu", "tensor_ops.cu", "pack_fp16.cu", "lstm_cell.cu"}


def nvcc() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found: libprad_cuda cannot be built")
    return path


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_header() -> float:
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdrs.append(os.path.join(HERE, "..", "include", "prad_cuda.h"))
    return max(os.path.getmtime(h) for h in hdrs)


def _compile(src: str, verbose: bool, ptxas_v: bool) -> str:
    obj = os.path.join(OBJ, src[:-3] + ".o")
    cmd = [nvcc(), *ARCH, *COMMON, "-c", os.path.join(CSRC, src), "-o", obj]
    if src in NO_FMAD:
        cmd.insert(1, "-fmad=false")
    if ptxas_v:
        cmd += ["-Xptxas", "-v"]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    if ptxas_v:
        sys.stderr.write(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False, ptxas_v: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdr_time = _newest_header()
    todo, objs = [], []
    for src in _sources():
        obj = os.path.join(OBJ, src[:-3] + ".o")
        objs.append(obj)
        stale = (force or not os.path.exists(obj)
                 or os.path.getmtime(obj) < max(os.path.getmtime(os.path.join(CSRC, src)), hdr_time))
        if stale:
            todo.append(src)
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            list(ex.map(lambda s: _compile(s, verbose, ptxas_v), todo))
    if todo or not os.path.exists(LIB):
        # link beside the target and rename: whoever loads or copies the library never sees half of it
        tmp = LIB + ".linking"
        cmd = [nvcc(), *ARCH, "-shared", "-o", tmp, *objs, "-lcudart", "-ldl"]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_v="--ptxas-v" in sys.argv))
