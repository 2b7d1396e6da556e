"""TEST INFRASTRUCTURE -- not part of the product path.

numpy front end of the CPU oracle (``prad_oracle.cpp``): the restatement of the
reference's C# backward loops that the CUDA library is checked against and that the
benchmark times as its CPU baseline.  Only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import this package.

Parity status: pinned by the known-answer and relational tests the reference itself holds
for this path (the Tensor / TensorReverse vectors for the elementwise family, gather, tile,
sum-rows, transpose and matrix-multiply reverses; the LayerNorm dual-number relation; the
matmul GPU == CPU relation; the SineSoftmax row-sum property) -- tests/test_oracle_pins.py.
Values no reference test holds (activations, softmax, losses, clip, Adam) follow the cited
lines only: "parity unpinned", because the C# reference cannot be executed where this is built.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libprad_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with its Makefile (g++ only, no CUDA)."""
    if force or not os.path.exists(_LIB_PATH) or (
        os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "prad_oracle.cpp"))
    ):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
    return _lib


_SUF = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64"}
_CT = {np.dtype(np.float32): C.c_float, np.dtype(np.float64): C.c_double}


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _c(a, dt=None):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


def _fn(name, dt, restype=None):
    f = getattr(lib(), f"oracle_{name}_{_SUF[np.dtype(dt)]}")
    f.restype = restype
    return f


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(int(n))


# ---------------------------------------------------------------- matmul family
def matmul_forward(A, B):
    A, B = _c(A), _c(B, A.dtype)
    M, K = A.shape
    N = B.shape[1]
    Cm = np.empty((M, N), A.dtype)
    _fn("matmul_forward", A.dtype)(_p(A), _p(B), _p(Cm), M, K, N)
    return Cm


def matmul_backward(A, B, dC, need_dA=True, need_dB=True):
    A, B, dC = _c(A), _c(B, A.dtype), _c(dC, A.dtype)
    M, K = A.shape
    N = B.shape[1]
    dA = np.empty((M, K), A.dtype) if need_dA else None
    dB = np.empty((K, N), A.dtype) if need_dB else None
    _fn("matmul_backward", A.dtype)(_p(A), _p(B), _p(dC), _p(dA), _p(dB), M, K, N)
    return dA, dB


def batch_matmul_forward(A, B):
    """A: [depth,M,K]; B: [depth,K,N] or [K,N] (the (DeepMatrix, Matrix) overload)."""
    A = _c(A)
    B = _c(B, A.dtype)
    depth, M, K = A.shape
    shared = int(B.ndim == 2)
    N = B.shape[-1]
    out = np.empty((depth, M, N), A.dtype)
    _fn("batch_matmul_forward", A.dtype)(_p(A), _p(B), _p(out), depth, M, K, N, shared)
    return out


def batch_matmul_backward(A, B, dC):
    """Returns per-slice (dA [depth,M,K], dB [depth,K,N])."""
    A = _c(A)
    B, dC = _c(B, A.dtype), _c(dC, A.dtype)
    depth, M, K = A.shape
    shared = int(B.ndim == 2)
    N = B.shape[-1]
    dA = np.empty((depth, M, K), A.dtype)
    dB = np.empty((depth, K, N), A.dtype)
    _fn("batch_matmul_backward", A.dtype)(_p(A), _p(B), _p(dC), _p(dA), _p(dB), depth, M, K, N,
                                          shared)
    return dA, dB


def matmul_and_sum_forward(A, B):
    A = _c(A)
    B = _c(B, A.dtype)
    R, Cc = A.shape
    P, _, N = B.shape
    out = np.empty((1, P), A.dtype)
    _fn("matmul_and_sum_forward", A.dtype)(_p(A), _p(B), _p(out), R, Cc, N, P)
    return out


def matmul_and_sum_backward(A, B, dOut):
    A = _c(A)
    B, dOut = _c(B, A.dtype), _c(dOut, A.dtype)
    R, Cc = A.shape
    P, _, N = B.shape
    dA = np.empty((N, Cc), A.dtype)
    dB = np.empty((P, Cc, R), A.dtype)
    _fn("matmul_and_sum_backward", A.dtype)(_p(A), _p(B), _p(dOut), _p(dA), _p(dB), R, Cc, N, P)
    return dA, dB


# ---------------------------------------------------------------- elementwise
def _unary(name, x, *extra):
    x = _c(x)
    y = np.empty_like(x)
    ct = _CT[x.dtype]
    _fn(name, x.dtype)(_p(x), _p(y), C.c_longlong(x.size), *[ct(e) for e in extra])
    return y


def _binary_bwd(name, s, dy, *extra):
    s = _c(s)
    dy = _c(dy, s.dtype)
    dx = np.empty_like(s)
    ct = _CT[s.dtype]
    _fn(name, s.dtype)(_p(s), _p(dy), _p(dx), C.c_longlong(s.size), *[ct(e) for e in extra])
    return dx


def leaky_relu_forward(x, alpha):
    return _unary("leaky_relu_forward", x, alpha)


def leaky_relu_backward(x, dy, alpha):
    return _binary_bwd("leaky_relu_backward", x, dy, alpha)


def sigmoid_forward(x):
    return _unary("sigmoid_forward", x)


def sigmoid_backward(y, dy):
    return _binary_bwd("sigmoid_backward", y, dy)


def tanh_forward(x):
    return _unary("tanh_forward", x)


def tanh_backward(y, dy):
    return _binary_bwd("tanh_backward", y, dy)


def relu_forward(x):
    return _unary("relu_forward", x)


def relu_backward(x, dy):
    return _binary_bwd("relu_backward", x, dy)


def amplified_sigmoid_forward(x):
    return _unary("amplified_sigmoid_forward", x)


def amplified_sigmoid_backward(x, dy):
    return _binary_bwd("amplified_sigmoid_backward", x, dy)


def scale_shift_forward(x, beta, gamma):
    """beta, gamma: one value per row (ScaleAndShiftOperation's [rows x 1] matrices)."""
    x = _c(x)
    beta, gamma = _c(np.reshape(beta, -1), x.dtype), _c(np.reshape(gamma, -1), x.dtype)
    y = np.empty_like(x)
    _fn("scale_shift_forward", x.dtype)(_p(x), _p(beta), _p(gamma), _p(y), x.shape[0], x.shape[1])
    return y


def scale_shift_backward(x, beta, dy):
    """Returns (dx, dbeta[rows], dgamma[rows])."""
    x = _c(x)
    beta, dy = _c(np.reshape(beta, -1), x.dtype), _c(dy, x.dtype)
    dx = np.empty_like(x)
    db, dg = np.empty(x.shape[0], x.dtype), np.empty(x.shape[0], x.dtype)
    _fn("scale_shift_backward", x.dtype)(_p(x), _p(beta), _p(dy), _p(dx), _p(db), _p(dg), x.shape[0], x.shape[1])
    return dx, db, dg


def rmsnorm_forward(x, g):
    x = _c(x)
    g = _c(g, x.dtype)
    y = np.empty_like(x)
    _fn("rmsnorm_forward", x.dtype)(_p(x), _p(g), _p(y), x.shape[0], x.shape[1])
    return y


def rmsnorm_backward(x, g, dy):
    """Returns (dx, dg)."""
    x = _c(x)
    g, dy = _c(g, x.dtype), _c(dy, x.dtype)
    dx, dg = np.empty_like(x), np.empty_like(x)
    _fn("rmsnorm_backward", x.dtype)(_p(x), _p(g), _p(dy), _p(dx), _p(dg), x.shape[0], x.shape[1])
    return dx, dg


def swish_forward(x, beta):
    return _unary("swish_forward", x, beta)


def swish_backward(x, beta, dy):
    """Returns (dx, dbeta) with dbeta a scalar of x's dtype."""
    x = _c(x)
    dy = _c(dy, x.dtype)
    dx = np.empty_like(x)
    db = np.zeros(1, x.dtype)
    _fn("swish_backward", x.dtype)(_p(x), _p(dy), _p(dx), C.c_longlong(x.size), _CT[x.dtype](beta), _p(db))
    return dx, db[0]


def swiglu_forward(x, w, v, b, c, beta):
    """w, v, b, c: one value per column (SwigLUOperation's [cols x 1] matrices)."""
    x = _c(x)
    w, v, b, c = (_c(np.reshape(t, -1), x.dtype) for t in (w, v, b, c))
    y = np.empty_like(x)
    _fn("swiglu_forward", x.dtype)(_p(x), _p(w), _p(v), _p(b), _p(c), C.c_double(beta), _p(y), x.shape[0], x.shape[1])
    return y


def swiglu_backward(x, w, v, b, c, beta, dy):
    """Returns (dx, dw, dv, db, dc)."""
    x = _c(x)
    w, v, b, c = (_c(np.reshape(t, -1), x.dtype) for t in (w, v, b, c))
    dy = _c(dy, x.dtype)
    dx = np.empty_like(x)
    outs = [np.empty(x.shape[1], x.dtype) for _ in range(4)]
    _fn("swiglu_backward", x.dtype)(_p(x), _p(w), _p(v), _p(b), _p(c), C.c_double(beta), _p(dy), _p(dx),
                                    *[_p(o) for o in outs], x.shape[0], x.shape[1])
    return (dx, *outs)


def row_sum_forward(x, average=False):
    """MatrixSumOperation / MatrixAverageOperation: one value per row."""
    x = _c(x)
    y = np.empty(x.shape[0], x.dtype)
    _fn("row_sum_forward", x.dtype)(_p(x), _p(y), x.shape[0], x.shape[1], int(average))
    return y


def row_sum_backward(dy, cols, average=False):
    dy = _c(np.reshape(dy, -1))
    dx = np.empty((dy.shape[0], cols), dy.dtype)
    _fn("row_sum_backward", dy.dtype)(_p(dy), _p(dx), dy.shape[0], cols, int(average))
    return dx


def broadcast_forward(x, rows, cols):
    x = _c(x)
    y = np.empty((rows, cols), x.dtype)
    _fn("broadcast_forward", x.dtype)(_p(x), x.shape[0], x.shape[1], _p(y), rows, cols)
    return y


def broadcast_backward(dy, in_rows, in_cols):
    dy = _c(dy)
    dx = np.empty((in_rows, in_cols), dy.dtype)
    _fn("broadcast_backward", dy.dtype)(_p(dy), dy.shape[0], dy.shape[1], _p(dx), in_rows, in_cols)
    return dx


def batchnorm_forward(x):
    """BatchNormalizationOperation as written.  Returns (y, stats) with stats = [this.mean, this.var] (float64)."""
    x = _c(x)
    y = np.empty_like(x)
    stats = np.zeros(2, np.float64)
    _fn("batchnorm_forward", x.dtype)(_p(x), _p(y), _p(stats), x.shape[0], x.shape[1])
    return y, stats


def batchnorm_backward(x, stats, dy):
    x = _c(x)
    dy = _c(dy, x.dtype)
    stats = np.ascontiguousarray(stats, np.float64)
    dx = np.empty_like(x)
    _fn("batchnorm_backward", x.dtype)(_p(x), _p(stats), _p(dy), _p(dx), x.shape[0], x.shape[1])
    return dx


def gelu_forward(x):
    return _unary("gelu_forward", x)


def gelu_backward(x, dy):
    return _binary_bwd("gelu_backward", x, dy)


def hadamard_forward(a, b):
    a = _c(a)
    b = _c(b, a.dtype)
    y = np.empty_like(a)
    _fn("hadamard_forward", a.dtype)(_p(a), _p(b), _p(y), C.c_longlong(a.size))
    return y


def hadamard_backward(a, b, dy):
    a = _c(a)
    b, dy = _c(b, a.dtype), _c(dy, a.dtype)
    da, db = np.empty_like(a), np.empty_like(a)
    _fn("hadamard_backward", a.dtype)(_p(a), _p(b), _p(dy), _p(da), _p(db), C.c_longlong(a.size))
    return da, db


def add_forward(a, b):
    a = _c(a)
    b = _c(b, a.dtype)
    y = np.empty_like(a)
    _fn("add_forward", a.dtype)(_p(a), _p(b), _p(y), C.c_longlong(a.size))
    return y


def add3_forward(a, b, c):
    a = _c(a)
    b, c = _c(b, a.dtype), _c(c, a.dtype)
    y = np.empty_like(a)
    _fn("add3_forward", a.dtype)(_p(a), _p(b), _p(c), _p(y), C.c_longlong(a.size))
    return y


def add_backward(dy, n_inputs=2):
    dy = _c(dy)
    outs = [np.empty_like(dy) for _ in range(n_inputs)]
    ptrs = [_p(o) for o in outs] + [None] * (3 - n_inputs)
    _fn("add_backward", dy.dtype)(_p(dy), *ptrs, C.c_longlong(dy.size))
    return outs


def add_broadcast_forward(x, bias):
    x = _c(x)
    bias = _c(bias, x.dtype).reshape(-1)
    y = np.empty_like(x)
    _fn("add_broadcast_forward", x.dtype)(_p(x), _p(bias), _p(y), x.shape[0], x.shape[1])
    return y


def add_broadcast_backward(dy):
    """Returns (dInput -- dOut itself, dBias [1,C])."""
    dy = _c(dy)
    db = np.empty((1, dy.shape[1]), dy.dtype)
    _fn("add_broadcast_backward", dy.dtype)(_p(dy), _p(db), dy.shape[0], dy.shape[1])
    return dy, db


def scale(x, s):
    return _unary("scale", x, s)


def transpose(x):
    x = _c(x)
    y = np.empty((x.shape[1], x.shape[0]), x.dtype)
    _fn("transpose", x.dtype)(_p(x), _p(y), x.shape[0], x.shape[1])
    return y


# ---------------------------------------------------------------- row ops
def softmax_forward(x):
    x = _c(x)
    y = np.empty_like(x)
    _fn("softmax_forward", x.dtype)(_p(x), _p(y), x.shape[0], x.shape[1])
    return y


def softmax_backward(y, dy):
    y = _c(y)
    dy = _c(dy, y.dtype)
    dx = np.empty_like(y)
    _fn("softmax_backward", y.dtype)(_p(y), _p(dy), _p(dx), y.shape[0], y.shape[1])
    return dx


def sine_softmax_forward(x):
    x = _c(x)
    y = np.empty_like(x)
    _fn("sine_softmax_forward", x.dtype)(_p(x), _p(y), x.shape[0], x.shape[1])
    return y


def sine_softmax_backward(x, dy):
    x = _c(x)
    dy = _c(dy, x.dtype)
    dx = np.empty_like(x)
    _fn("sine_softmax_backward", x.dtype)(_p(x), _p(dy), _p(dx), x.shape[0], x.shape[1])
    return dx


def layernorm_forward(x):
    """Returns (y, mean[R], std[R])."""
    x = _c(x)
    y = np.empty_like(x)
    mean = np.empty(x.shape[0], x.dtype)
    std = np.empty(x.shape[0], x.dtype)
    _fn("layernorm_forward", x.dtype)(_p(x), _p(y), _p(mean), _p(std), x.shape[0], x.shape[1])
    return y, mean, std


def layernorm_backward(x, mean, std, dy):
    x = _c(x)
    mean, std, dy = _c(mean, x.dtype), _c(std, x.dtype), _c(dy, x.dtype)
    dx = np.empty_like(x)
    _fn("layernorm_backward", x.dtype)(_p(x), _p(mean), _p(std), _p(dy), _p(dx), x.shape[0],
                                       x.shape[1])
    return dx


# ---------------------------------------------------------------- losses
def mse_forward(out, target):
    out = _c(out)
    target = _c(target, out.dtype)
    return _fn("mse_forward", out.dtype, _CT[out.dtype])(_p(out), _p(target), out.shape[0],
                                                          out.shape[1])


def mse_backward(out, target, rows_total=None):
    out = _c(out)
    target = _c(target, out.dtype)
    g = np.empty_like(out)
    rt = out.shape[0] if rows_total is None else rows_total
    _fn("mse_backward", out.dtype)(_p(out), _p(target), _p(g), out.shape[0], out.shape[1],
                                   C.c_longlong(rt))
    return g


def cce_forward(out, target):
    out = _c(out)
    target = _c(target, out.dtype)
    return _fn("cce_forward", out.dtype, _CT[out.dtype])(_p(out), _p(target), out.shape[0],
                                                          out.shape[1])


def cce_backward(out, target, rows_total=None):
    out = _c(out)
    target = _c(target, out.dtype)
    g = np.empty_like(out)
    rt = out.shape[0] if rows_total is None else rows_total
    _fn("cce_backward", out.dtype)(_p(out), _p(target), _p(g), out.shape[0], out.shape[1],
                                   C.c_longlong(rt))
    return g


# ---------------------------------------------------------------- embedding
def embedding_forward(index_col, W):
    W = _c(W)
    idx = _c(index_col, W.dtype).reshape(-1)
    out = np.empty((idx.size, W.shape[1]), W.dtype)
    _fn("embedding_forward", W.dtype)(_p(idx), _p(W), _p(out), idx.size, W.shape[1])
    return out


def embedding_backward(index_col, dOut, vocab):
    dOut = _c(dOut)
    idx = _c(index_col, dOut.dtype).reshape(-1)
    dW = np.empty((vocab, dOut.shape[1]), dOut.dtype)
    _fn("embedding_backward", dOut.dtype)(_p(idx), _p(dOut), _p(dW), idx.size, vocab,
                                          dOut.shape[1])
    return dW


# ---------------------------------------------------------------- accumulation
def _ptr_array(arrs):
    return (C.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])


def accumulate_gradients(grads):
    grads = [_c(g) for g in grads]
    out = np.empty_like(grads[0])
    _fn("accumulate_gradients", out.dtype)(_ptr_array(grads), len(grads), _p(out),
                                           C.c_longlong(out.size))
    return out


def accumulate_into(dest, src):
    assert dest.flags.c_contiguous
    src = _c(src, dest.dtype)
    _fn("accumulate_into", dest.dtype)(_p(dest), _p(src), C.c_longlong(dest.size))
    return dest


def batch_mean(grads):
    grads = [_c(g) for g in grads]
    out = np.empty_like(grads[0])
    _fn("batch_mean", out.dtype)(_ptr_array(grads), len(grads), _p(out), C.c_longlong(out.size))
    return out


# ---------------------------------------------------------------- clip + Adam
def clip_reference(g, clip, minv):
    """In place, like GradientClipper.ClipGradients(Matrix)."""
    assert g.flags.c_contiguous
    ct = _CT[g.dtype]
    _fn("clip_reference", g.dtype)(_p(g), C.c_longlong(g.size), ct(clip), ct(minv))
    return g


def clip_prad(g, clip):
    g = _c(g)
    out = np.empty_like(g)
    _fn("clip_prad", g.dtype)(_p(g), _p(out), C.c_longlong(g.size), _CT[g.dtype](clip))
    return out


def clip_global_norm(grads, max_norm):
    """In place over a list of arrays; returns the norm before clipping."""
    for g in grads:
        assert g.flags.c_contiguous
    sizes = (C.c_longlong * len(grads))(*[g.size for g in grads])
    return _fn("clip_global_norm", grads[0].dtype, C.c_double)(_ptr_array(grads), sizes,
                                                               len(grads), C.c_double(max_norm))


def adam_rmad(w, m, v, g, lr, b1, b2, eps, iteration):
    for a in (w, m, v):
        assert a.flags.c_contiguous
    g = _c(g, w.dtype)
    ct = _CT[w.dtype]
    _fn("adam_rmad", w.dtype)(_p(w), _p(m), _p(v), _p(g), C.c_longlong(w.size), ct(lr), ct(b1),
                              ct(b2), ct(eps), ct(iteration))


def adam_prad(w, m, v, g, lr, b1, b2, eps, t):
    for a in (w, m, v):
        assert a.flags.c_contiguous
    g = _c(g, w.dtype)
    ct = _CT[w.dtype]
    _fn("adam_prad", w.dtype)(_p(w), _p(m), _p(v), _p(g), C.c_longlong(w.size), ct(lr), ct(b1),
                              ct(b2), ct(eps), int(t))


# ---------------------------------------------------------------- PRAD Tensor elementwise family
# src/PRAD/Tensor.Common.cs / TensorReverse.Common.cs evaluate these with one MKL VML call per step
# over flat arrays; numpy's elementwise operations in the storage dtype restate that (one rounding
# per step).  Line references are in include/prad_cuda.h next to prad_tensor_op.
def tensor_unary(op, x):
    x = _c(x)
    t = x.dtype.type
    with np.errstate(all="ignore"):
        return {"exp": np.exp, "ln": np.log, "log": np.log10, "abs": np.abs, "square": lambda v: v * v,
                "sqrt": np.sqrt, "sin": np.sin, "cos": np.cos, "reciprocal": lambda v: t(1) / v,
                "negate": lambda v: v * t(-1)}[op](x).astype(x.dtype)


def tensor_unary_reverse(op, saved, dy):
    """`saved` is the input x, except for "reciprocal" where it is the forward result."""
    s = _c(saved)
    dy = _c(dy, s.dtype)
    t = s.dtype.type
    with np.errstate(all="ignore"):
        if op == "exp":
            return (np.exp(s).astype(s.dtype) * dy).astype(s.dtype)
        if op in ("ln", "log"):                      # LogReverse multiplies by 1/x as well
            return ((t(1) / s).astype(s.dtype) * dy).astype(s.dtype)
        if op == "abs":
            return np.where(s >= 0, dy, -dy).astype(s.dtype)
        if op == "square":
            return (t(2) * (dy * s).astype(s.dtype)).astype(s.dtype)
        if op == "sqrt":
            r = np.sqrt(s).astype(s.dtype)
            m = np.where(np.abs(r) >= np.abs(t(1e-10)), r, t(1e-10)).astype(s.dtype)      # Vml.MaxMag
            return (t(0.5) * (dy / m).astype(s.dtype)).astype(s.dtype)
        if op == "sin":
            return (dy * np.cos(s).astype(s.dtype)).astype(s.dtype)
        if op == "cos":
            return (t(-1) * (dy * np.sin(s).astype(s.dtype)).astype(s.dtype)).astype(s.dtype)
        if op == "reciprocal":
            return ((dy * (s * s).astype(s.dtype)).astype(s.dtype) * t(-1)).astype(s.dtype)
        if op == "negate":
            return (dy * t(-1)).astype(s.dtype)
    raise KeyError(op)


def tensor_binary(op, a, b):
    a = _c(a)
    b = _c(b, a.dtype)
    with np.errstate(all="ignore"):
        return {"add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide}[op](a, b).astype(a.dtype)


def tensor_binary_reverse(op, a, b, dy):
    a = _c(a)
    b, dy = _c(b, a.dtype), _c(dy, a.dtype)
    t = a.dtype.type
    with np.errstate(all="ignore"):
        if op == "add":
            return dy.copy(), dy.copy()
        if op == "sub":
            return dy.copy(), (t(-1) * dy).astype(a.dtype)
        if op == "mul":
            return (dy * b).astype(a.dtype), (dy * a).astype(a.dtype)
        if op == "div":
            return (dy / b).astype(a.dtype), (t(-1) * ((dy * a).astype(a.dtype) / (b * b).astype(a.dtype)).astype(a.dtype)).astype(a.dtype)
    raise KeyError(op)


# ---------------------------------------------------------------- PRAD Tensor matmul / gather / tile
def tensor_matmul(a, b, alpha=1.0, beta=0.0, c=None):
    """Tensor.MatrixMultiply (src/PRAD/Tensor.cs:572-613): 2-D only, ArgumentException on a shape
    mismatch; the product itself is MKL's (third party, summation order unknown) -- restated with the
    sequential loops of matmul_forward."""
    a, b = _c(a), _c(b)
    if a.ndim != 2 or b.ndim != 2:
        raise ValueError("Matrix multiplication is only supported for 2D tensors.")
    if a.shape[1] != b.shape[0]:
        raise ValueError("Incompatible shapes for matrix multiplication.")
    t = a.dtype.type
    prod = matmul_forward(a, b)
    out = (t(alpha) * prod).astype(a.dtype)
    if beta != 0.0:
        out = (out + (t(beta) * _c(c, a.dtype)).astype(a.dtype)).astype(a.dtype)
    return out


def tensor_matmul_reverse(a, b, dc):
    """TensorReverse.MatrixMultiplyReverse (src/PRAD/TensorReverse.cs:94-160): dA = dC B^T, dB = A^T dC."""
    return matmul_backward(a, b, dc)


def tensor_gather(x, indices, axis=0):
    """Tensor.Gather (src/PRAD/Tensor.Common.cs:959-1090): negative indices count from the end;
    result shape = x.shape[:axis] + indices.shape + x.shape[axis+1:]."""
    x = _c(x)
    idx = np.asarray(indices)
    n = x.shape[axis]
    w = np.where(idx < 0, n + idx.astype(np.int64), idx.astype(np.int64))
    if ((w < 0) | (w >= n)).any():
        raise ValueError("Index out of bounds.")
    return np.ascontiguousarray(np.take(x, w, axis=axis))


def tensor_gather_reverse(upstream, indices, input_shape, axis=0):
    """TensorReverse.GatherReverse (src/PRAD/TensorReverse.Common.cs:2358-2426) with the contributions of
    repeated indices added in the order of the upstream gradient's flat index (a sequential loop)."""
    up = _c(upstream)
    idx = np.asarray(indices)
    n = input_shape[axis]
    w = np.where(idx < 0, n + idx.astype(np.int64), idx.astype(np.int64)).ravel()
    if ((w < 0) | (w >= n)).any():
        raise ValueError("Index out of bounds.")
    outer = int(np.prod(input_shape[:axis], dtype=np.int64))
    inner = int(np.prod(input_shape[axis + 1:], dtype=np.int64))
    up3 = up.reshape(outer, w.size, inner)
    dx = np.zeros((outer, n, inner), up.dtype)
    for c, v in enumerate(w):                       # ascending c == ascending flat index per element
        dx[:, v, :] = (dx[:, v, :] + up3[:, c, :]).astype(up.dtype)
    return dx.reshape(input_shape)


def tensor_tile(x, multiples):
    """Tensor.Tile (src/PRAD/Tensor.Common.cs:1096-1230), 2-D."""
    return np.ascontiguousarray(np.tile(_c(x), tuple(multiples)))


def tensor_tile_reverse(upstream, input_shape, multiples):
    """TensorReverse.TileReverse (src/PRAD/TensorReverse.Common.cs:2713-2785; specialised cases
    :3278-3370), 2-D, as written: multiples {m, 1} read rows i*m .. i*m+m-1 for input row i."""
    up = _c(upstream)
    rows, cols = input_shape
    mr, mc = multiples
    dx = np.zeros((rows, cols), up.dtype)
    if mc == 1:
        for m in range(mr):
            dx = (dx + up.reshape(rows, mr, cols)[:, m, :]).astype(up.dtype)
        return dx
    for tr in range(mr):
        for tc in range(mc):
            dx = (dx + up[tr * rows:(tr + 1) * rows, tc * cols:(tc + 1) * cols]).astype(up.dtype)
    return dx
