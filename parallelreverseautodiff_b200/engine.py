"""Thin object layer over the C ABI: a context (``Engine``) and device-resident matrices.

Nothing here computes: every method forwards to one ``prad_*`` entry point of
``libprad_cuda.so``.  numpy arrays only appear at the upload / download boundary.
"""
from __future__ import annotations

import ctypes as C
from typing import Iterable, List, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import check

F32, F64 = 0, 1
ACT_NONE, ACT_LEAKY_RELU, ACT_SIGMOID, ACT_TANH, ACT_GELU, ACT_RELU, ACT_AMPLIFIED_SIGMOID = range(7)
ADAM_RMAD, ADAM_PRAD = 0, 1
CLIP_NONE, CLIP_REFERENCE, CLIP_GLOBAL_NORM = 0, 1, 2
DP_MARKS = 256          # PRAD_DP_MARKS: slots of prad_dp_mark
PACK_ROWS, PACK_COLS = 1, 2

_DT = {np.dtype(np.float32): F32, np.dtype(np.float64): F64}


def dtype_code(dtype) -> int:
    try:
        return _DT[np.dtype(dtype)]
    except KeyError:
        raise TypeError(f"only float32 (PRADLite) and float64 (PRAD) are supported, got {dtype}")


class DeviceMatrix:
    """A dense row-major device buffer: Matrix (2-D) or DeepMatrix (3-D, depth first)."""

    __slots__ = ("engine", "ptr", "shape", "dtype", "_owned")

    def __init__(self, engine: "Engine", ptr: int, shape: Sequence[int], dtype, owned=True):
        self.engine = engine
        self.ptr = ptr
        self.shape = tuple(int(s) for s in shape)
        self.dtype = np.dtype(dtype)
        self._owned = owned

    @property
    def size(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def nbytes(self) -> int:
        return self.size * self.dtype.itemsize

    @property
    def Rows(self) -> int:
        return self.shape[-2]

    @property
    def Cols(self) -> int:
        return self.shape[-1]

    @property
    def Depth(self) -> int:
        return self.shape[0] if len(self.shape) == 3 else 1

    def numpy(self) -> np.ndarray:
        return self.engine.download(self)

    def view(self, shape: Sequence[int], offset_elems: int = 0) -> "DeviceMatrix":
        """A non-owning alias of (part of) this buffer with another shape."""
        return DeviceMatrix(self.engine, self.ptr + offset_elems * self.dtype.itemsize, shape,
                            self.dtype, owned=False)

    def slice(self, d: int) -> "DeviceMatrix":
        """Slice d of a DeepMatrix as a Matrix (alias)."""
        per = self.shape[-2] * self.shape[-1]
        return self.view(self.shape[-2:], d * per)

    def free(self) -> None:
        if self._owned and self.ptr and self.engine is not None and self.engine.ctx:
            self.engine._free(self.ptr)
        self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class PackedOperand:
    """A float matrix in the packed FP16-piece form of the tensor-core GEMM (prad_packed): by rows
    (the matrix as an operand with k = its columns), by columns (its transpose), or both."""

    def __init__(self, engine: "Engine", rows: int, cols: int, forms: int, block_rows=0, block_cols=0):
        self.engine, self.rows, self.cols, self.forms = engine, int(rows), int(cols), int(forms)
        h = C.c_void_p()
        check(engine.lib.prad_packed_create(engine.ctx, self.rows, self.cols, self.forms, block_rows, block_cols,
                                            C.byref(h)))
        self.handle = h

    def blocks(self):
        br, bc = C.c_int(), C.c_int()
        check(self.engine.lib.prad_packed_shape(self.handle, None, None, None, C.byref(br), C.byref(bc)))
        return br.value, bc.value

    def pack(self, x: "DeviceMatrix", ld: Optional[int] = None) -> "PackedOperand":
        check(self.engine.lib.prad_pack(self.handle, x.ptr, ld or self.cols))
        return self

    def act_forward(self, act: int, x: "DeviceMatrix", y: Optional["DeviceMatrix"] = None, alpha=0.0):
        check(self.engine.lib.prad_act_forward_pack(self.handle, act, x.ptr, y.ptr if y is not None else None, alpha))
        return self

    def act_backward(self, act: int, saved, dy: "DeviceMatrix", dx: Optional["DeviceMatrix"] = None, alpha=0.0):
        check(self.engine.lib.prad_act_backward_pack(self.handle, act, saved.ptr if saved is not None else None, dy.ptr,
                                                     dx.ptr if dx is not None else None, alpha))
        return self

    def mse_act_backward(self, act: int, saved, output: "DeviceMatrix", target: "DeviceMatrix", rows_total: int,
                         dx: Optional["DeviceMatrix"] = None, alpha=0.0):
        """MSE gradient times the output activation's derivative, packed (prad_mse_act_backward_pack)."""
        check(self.engine.lib.prad_mse_act_backward_pack(self.handle, act, saved.ptr if saved is not None else None,
                                                         output.ptr, target.ptr, rows_total,
                                                         dx.ptr if dx is not None else None, alpha))
        return self

    def free(self) -> None:
        if self.handle and self.engine is not None and self.engine.ctx:
            self.engine.lib.prad_packed_destroy(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Sequence:
    """A recorded launch sequence of one Engine (prad_sequence)."""

    def __init__(self, eng, handle, keep=()):
        self.eng, self.handle, self._keep = eng, handle, list(keep)
        n = C.c_int64()
        check(eng.lib.prad_sequence_launch_count(handle, C.byref(n)))
        self.launches = n.value

    def launch(self) -> None:
        check(self.eng.lib.prad_sequence_launch(self.eng.ctx, self.handle))

    def close(self) -> None:
        if self.handle is not None:
            check(self.eng.lib.prad_sequence_destroy(self.eng.ctx, self.handle))
            self.handle = None
            self._keep = []


class Engine:
    """One libprad_cuda context on one GPU (CudaBlas.Instance of the reference, per device)."""

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        ctx = C.c_void_p()
        check(self.lib.prad_init(int(device), C.byref(ctx)))
        self.ctx = ctx
        self.device = device
        self.options = {}          # what set_option was given (the library has no getter)

    # ------------------------------------------------------------ lifecycle
    def close(self) -> None:
        if self.ctx:
            check(self.lib.prad_shutdown(self.ctx))
            self.ctx = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def sync(self) -> None:
        check(self.lib.prad_sync(self.ctx))

    def set_option(self, key: str, value: str) -> None:
        check(self.lib.prad_set_option(self.ctx, key.encode(), value.encode()))
        self.options[key] = value

    def packs_large_float_products(self) -> bool:
        """True while large float products take the packed FP16 tensor-core path (the defaults)."""
        return (self.options.get("gemm_f32", "auto") in ("auto", "fp16x3")
                and self.options.get("tc_auto", "fp16x3") == "fp16x3")

    def launch_count(self) -> int:
        n = C.c_int64()
        check(self.lib.prad_launch_count(self.ctx, C.byref(n)))
        return n.value

    def record(self, fn) -> "Sequence":
        """Runs `fn()` with the context recording (prad_capture_begin/end): its launches are not
        executed but kept as a sequence that `Sequence.launch()` replays in one submission.  Run
        `fn()` once unrecorded first so that library scratch has its final size."""
        check(self.lib.prad_capture_begin(self.ctx))
        self._record_keep = keep = []
        self._deferred_free = []
        try:
            fn()
        except BaseException:
            self._record_keep = None
            h = C.c_void_p()
            self.lib.prad_capture_end(self.ctx, C.byref(h))      # close the recording; drop the result
            if h.value:
                self.lib.prad_sequence_destroy(self.ctx, h)
            self._flush_deferred_free()
            raise
        self._record_keep = None
        h = C.c_void_p()
        check(self.lib.prad_capture_end(self.ctx, C.byref(h)))
        self._flush_deferred_free()
        return Sequence(self, h, keep)

    def stream(self) -> int:
        s = C.c_void_p()
        check(self.lib.prad_stream(self.ctx, C.byref(s)))
        return s.value or 0

    def use_stream(self, stream: int) -> None:
        check(self.lib.prad_use_stream(self.ctx, C.c_void_p(stream)))

    # ------------------------------------------------------------ memory
    def empty(self, shape, dtype) -> DeviceMatrix:
        dtype = np.dtype(dtype)
        dtype_code(dtype)
        shape = (shape,) if isinstance(shape, int) else tuple(shape)
        n = 1
        for s in shape:
            n *= int(s)
        p = C.c_void_p()
        check(self.lib.prad_alloc(self.ctx, n * dtype.itemsize, C.byref(p)))
        m = DeviceMatrix(self, p.value, shape, dtype)
        keep = getattr(self, "_record_keep", None)
        if keep is not None:       # a buffer born inside a recording lives as long as the sequence
            keep.append(m)
        return m

    def zeros(self, shape, dtype) -> DeviceMatrix:
        m = self.empty(shape, dtype)
        check(self.lib.prad_zero(self.ctx, m.ptr, m.nbytes))
        return m

    def zero_(self, m: DeviceMatrix) -> None:
        check(self.lib.prad_zero(self.ctx, m.ptr, m.nbytes))

    def _free(self, ptr: int) -> None:
        if getattr(self, "_record_keep", None) is not None:    # prad_free cannot be recorded: do it afterwards
            self._deferred_free.append(ptr)
            return
        check(self.lib.prad_free(self.ctx, C.c_void_p(ptr)))

    def _flush_deferred_free(self) -> None:
        pending, self._deferred_free = self._deferred_free, []
        for ptr in pending:
            check(self.lib.prad_free(self.ctx, C.c_void_p(ptr)))

    def upload(self, a: np.ndarray, out: Optional[DeviceMatrix] = None) -> DeviceMatrix:
        a = np.ascontiguousarray(a)
        if out is None:
            out = self.empty(a.shape, a.dtype)
        assert out.nbytes == a.nbytes
        check(self.lib.prad_upload(self.ctx, out.ptr, a.ctypes.data, a.nbytes))
        # pageable host memory: the copy has consumed `a` when the call returns
        return out

    def upload_rows(self, rows: Sequence[np.ndarray]) -> DeviceMatrix:
        """Jagged upload: one host array per matrix row (the reference's T[rows][cols])."""
        rows = [np.ascontiguousarray(r) for r in rows]
        out = self.empty((len(rows), rows[0].size), rows[0].dtype)
        ptrs = (C.c_void_p * len(rows))(*[r.ctypes.data for r in rows])
        check(self.lib.prad_upload_rows(self.ctx, out.ptr, ptrs, len(rows), rows[0].nbytes))
        self.sync()
        return out

    def download(self, m: DeviceMatrix) -> np.ndarray:
        out = np.empty(m.shape, m.dtype)
        check(self.lib.prad_download(self.ctx, out.ctypes.data, m.ptr, m.nbytes))
        return out

    def download_rows(self, m: DeviceMatrix):
        rows = [np.empty(m.shape[1], m.dtype) for _ in range(m.shape[0])]
        ptrs = (C.c_void_p * len(rows))(*[r.ctypes.data for r in rows])
        check(self.lib.prad_download_rows(self.ctx, ptrs, m.ptr, len(rows), rows[0].nbytes))
        return rows

    def pinned_empty(self, shape, dtype) -> np.ndarray:
        """numpy array over page-locked host memory (freed with the engine's process)."""
        dtype = np.dtype(dtype)
        shape = (shape,) if isinstance(shape, int) else tuple(shape)
        n = int(np.prod(shape, dtype=np.int64))
        p = C.c_void_p()
        check(self.lib.prad_alloc_host(self.ctx, n * dtype.itemsize, C.byref(p)))
        buf = (C.c_char * (n * dtype.itemsize)).from_address(p.value)
        return np.frombuffer(buf, dtype=dtype, count=n).reshape(shape)

    def upload_async(self, a: np.ndarray, out: DeviceMatrix) -> None:
        """Enqueue a host->device copy; `a` must stay untouched until the stream reaches it
        (page-locked memory from pinned_empty makes the copy truly asynchronous)."""
        assert a.flags.c_contiguous and out.nbytes == a.nbytes
        check(self.lib.prad_upload(self.ctx, out.ptr, a.ctypes.data, a.nbytes))

    def upload_prefetch(self, a: np.ndarray, out: DeviceMatrix) -> None:
        """Host->device copy on the copy stream (overlaps with compute); `a` must be page-locked."""
        assert a.flags.c_contiguous and out.nbytes == a.nbytes
        check(self.lib.prad_upload_prefetch(self.ctx, out.ptr, a.ctypes.data, a.nbytes))

    def upload_join(self) -> None:
        check(self.lib.prad_upload_join(self.ctx))

    def copy(self, dst: DeviceMatrix, src: DeviceMatrix) -> None:
        assert dst.nbytes == src.nbytes
        check(self.lib.prad_copy(self.ctx, dst.ptr, src.ptr, src.nbytes))

    def clone(self, src: DeviceMatrix) -> DeviceMatrix:
        out = self.empty(src.shape, src.dtype)
        self.copy(out, src)
        return out

    # ------------------------------------------------------------ helpers
    @staticmethod
    def _p(m: Optional[DeviceMatrix]):
        return C.c_void_p(m.ptr) if m is not None else None

    @staticmethod
    def _ptr_list(ms: Iterable[DeviceMatrix]):
        ms = list(ms)
        return (C.c_void_p * len(ms))(*[m.ptr for m in ms])

    @staticmethod
    def _size_list(ms: Iterable[DeviceMatrix]):
        ms = list(ms)
        return (C.c_int64 * len(ms))(*[m.size for m in ms])

    # ------------------------------------------------------------ GEMM family
    def gemm(self, A, B, Cm, transA=False, transB=False, alpha=1.0, beta=0.0, M=None, N=None,
             K=None, lda=None, ldb=None, ldc=None, batch=1, strideA=0, strideB=0, strideC=0):
        dt = dtype_code(A.dtype)
        if M is None:
            M = A.shape[-1] if transA else A.shape[-2]
            K = A.shape[-2] if transA else A.shape[-1]
            N = B.shape[-2] if transB else B.shape[-1]
        lda = lda or A.shape[-1]
        ldb = ldb or B.shape[-1]
        ldc = ldc or Cm.shape[-1]
        check(self.lib.prad_gemm(self.ctx, dt, int(transA), int(transB), M, N, K, alpha, A.ptr, lda,
                                 B.ptr, ldb, beta, Cm.ptr, ldc, batch, strideA, strideB, strideC))

    def packed(self, rows, cols, forms, block_rows=0, block_cols=0) -> PackedOperand:
        return PackedOperand(self, rows, cols, forms, block_rows, block_cols)

    def gemm_packed(self, A: PackedOperand, form_a: int, B: PackedOperand, form_b: int, out: DeviceMatrix,
                    alpha=1.0, beta=0.0, bias=None, ldc=None):
        """out (M x N) = alpha * opA * opB^T + beta * out (+ bias row); prad_gemm_packed."""
        n = B.rows if form_b == PACK_ROWS else B.cols
        check(self.lib.prad_gemm_packed(self.ctx, A.handle, form_a, B.handle, form_b, alpha, beta, out.ptr,
                                        ldc or n, self._p(bias)))
        return out

    def matmul_forward(self, A, B, Y=None, bias=None, Z_out=None, act=ACT_NONE, act_alpha=0.0):
        M, K = A.shape
        K2, N = B.shape
        if K != K2:
            raise _lib.PradError(_lib.ERR_SHAPE, "Input 1 columns do not match Input 2 rows")
        Y = Y or self.empty((M, N), A.dtype)
        check(self.lib.prad_matmul_forward(self.ctx, dtype_code(A.dtype), A.ptr, B.ptr, Y.ptr, M, K,
                                           N, self._p(bias), self._p(Z_out), act, act_alpha))
        return Y

    def matmul_backward(self, A, B, dC, dA=None, dB=None, need_dA=True, need_dB=True,
                        accumulate_dB=False, dB_scale=1.0, act_below=ACT_NONE, saved_below=None,
                        act_alpha=0.0):
        M, N = dC.shape
        K = B.shape[0] if B is not None else A.shape[1]
        if need_dA and dA is None:
            dA = self.empty((M, K), dC.dtype)
        if need_dB and dB is None:
            dB = self.empty((K, N), dC.dtype)
        check(self.lib.prad_matmul_backward(
            self.ctx, dtype_code(dC.dtype), self._p(A), self._p(B), dC.ptr,
            self._p(dA if need_dA else None), self._p(dB if need_dB else None), M, K, N,
            int(accumulate_dB), dB_scale, act_below, self._p(saved_below), act_alpha))
        return dA, dB

    def matmul_act_backward(self, A, B, dOut, act, saved, act_alpha=0.0):
        M, K = A.shape
        N = B.shape[1]
        dPre = self.empty((M, N), A.dtype)
        dA = self.empty((M, K), A.dtype)
        dB = self.empty((K, N), A.dtype)
        check(self.lib.prad_matmul_act_backward(self.ctx, dtype_code(A.dtype), A.ptr, B.ptr, dOut.ptr,
                                                act, self._p(saved), act_alpha, dPre.ptr, dA.ptr,
                                                dB.ptr, M, K, N))
        return dPre, dA, dB

    def matmul_act_backward_host(self, A, B, dOut, act, saved, act_alpha=0.0, out=None):
        """numpy in, numpy out: uploads, computes, downloads inside the one C call."""
        A = np.ascontiguousarray(A)
        M, K = A.shape
        N = B.shape[1]
        if out is None:
            out = (np.empty((M, N), A.dtype), np.empty((M, K), A.dtype), np.empty((K, N), A.dtype))
        dPre, dA, dB = out
        check(self.lib.prad_matmul_act_backward_host(
            self.ctx, dtype_code(A.dtype), A.ctypes.data, B.ctypes.data, dOut.ctypes.data, act,
            saved.ctypes.data if saved is not None else None, act_alpha, dPre.ctypes.data,
            dA.ctypes.data, dB.ctypes.data, M, K, N))
        return dPre, dA, dB

    def batch_matmul_forward(self, A, B, Cm=None):
        depth, M, K = A.shape
        shared = len(B.shape) == 2
        N = B.shape[-1]
        Cm = Cm or self.empty((depth, M, N), A.dtype)
        check(self.lib.prad_batch_matmul_forward(self.ctx, dtype_code(A.dtype), A.ptr, B.ptr, Cm.ptr,
                                                 depth, M, K, N, int(shared)))
        return Cm

    def batch_matmul_backward(self, A, B, dC, per_slice_dB=True, mean_dB=False):
        depth, M, K = A.shape
        shared = len(B.shape) == 2
        N = B.shape[-1]
        dA = self.empty((depth, M, K), A.dtype)
        dB = self.empty((depth, K, N), A.dtype) if per_slice_dB else None
        dBm = self.empty((K, N), A.dtype) if mean_dB else None
        check(self.lib.prad_batch_matmul_backward(self.ctx, dtype_code(A.dtype), A.ptr, B.ptr, dC.ptr,
                                                  dA.ptr, self._p(dB), self._p(dBm), depth, M, K,
                                                  N, int(shared)))
        return dA, dB, dBm

    def matmul_and_sum_forward(self, A, B):
        R, Cc = A.shape
        P, _, N = B.shape
        out = self.empty((1, P), A.dtype)
        check(self.lib.prad_matmul_and_sum_forward(self.ctx, dtype_code(A.dtype), A.ptr, B.ptr,
                                                   out.ptr, R, Cc, N, P))
        return out

    def matmul_and_sum_backward(self, A, B, dOut):
        R, Cc = A.shape
        P, _, N = B.shape
        dA = self.empty((N, Cc), A.dtype)
        dB = self.empty((P, Cc, R), A.dtype)
        check(self.lib.prad_matmul_and_sum_backward(self.ctx, dtype_code(A.dtype), A.ptr, B.ptr,
                                                    dOut.ptr, dA.ptr, dB.ptr, R, Cc, N, P))
        return dA, dB

    # ------------------------------------------------------------ elementwise
    def act_forward(self, act, x, alpha=0.0, out=None):
        out = out or self.empty(x.shape, x.dtype)
        check(self.lib.prad_act_forward(self.ctx, dtype_code(x.dtype), act, x.ptr, out.ptr, x.size,
                                        alpha))
        return out

    def act_backward(self, act, saved, dy, alpha=0.0, out=None):
        out = out or self.empty(dy.shape, dy.dtype)
        check(self.lib.prad_act_backward(self.ctx, dtype_code(dy.dtype), act, saved.ptr, dy.ptr,
                                         out.ptr, dy.size, alpha))
        return out

    def hadamard_forward(self, a, b, out=None):
        out = out or self.empty(a.shape, a.dtype)
        check(self.lib.prad_hadamard_forward(self.ctx, dtype_code(a.dtype), a.ptr, b.ptr, out.ptr,
                                             a.size))
        return out

    def hadamard_backward(self, a, b, dy, out=None):
        da, db = out if out is not None else (self.empty(a.shape, a.dtype), self.empty(a.shape, a.dtype))
        check(self.lib.prad_hadamard_backward(self.ctx, dtype_code(a.dtype), a.ptr, b.ptr, dy.ptr,
                                              da.ptr, db.ptr, a.size))
        return da, db

    def lstm_cell_backward(self, h, target, loss_scale, dh_contrib, dc_next, gates_ifgo, tanh_c, c_prev, dpre_ifgo,
                           dc_prev):
        """One time step of BPTT in one launch (prad_lstm_cell_backward)."""
        n = tanh_c.size
        contrib = (C.c_void_p * max(1, len(dh_contrib)))(*[m.ptr for m in dh_contrib])
        gates = (C.c_void_p * 4)(*[m.ptr for m in gates_ifgo])
        dpre = (C.c_void_p * 4)(*[m.ptr for m in dpre_ifgo])
        check(self.lib.prad_lstm_cell_backward(self.ctx, dtype_code(tanh_c.dtype), n, self._p(h), self._p(target),
                                               loss_scale, contrib, len(dh_contrib), self._p(dc_next), gates, tanh_c.ptr,
                                               self._p(c_prev), dpre, self._p(dc_prev)))

    def add_forward(self, a, b, c=None, out=None):
        out = out or self.empty(a.shape, a.dtype)
        check(self.lib.prad_add_forward(self.ctx, dtype_code(a.dtype), a.ptr, b.ptr, self._p(c),
                                        out.ptr, a.size))
        return out

    def add_broadcast_forward(self, x, bias, out=None):
        out = out or self.empty(x.shape, x.dtype)
        check(self.lib.prad_add_broadcast_forward(self.ctx, dtype_code(x.dtype), x.ptr, bias.ptr,
                                                  out.ptr, x.shape[0], x.shape[1]))
        return out

    def add_broadcast_backward(self, dy, dbias=None, accumulate=False):
        dbias = dbias or self.empty((1, dy.shape[1]), dy.dtype)
        check(self.lib.prad_add_broadcast_backward(self.ctx, dtype_code(dy.dtype), dy.ptr, dbias.ptr,
                                                   dy.shape[0], dy.shape[1], int(accumulate)))
        return dbias

    def scale(self, x, s, out=None):
        out = out or self.empty(x.shape, x.dtype)
        check(self.lib.prad_scale(self.ctx, dtype_code(x.dtype), x.ptr, out.ptr, x.size, s))
        return out

    def transpose(self, x, out=None):
        depth = x.shape[0] if len(x.shape) == 3 else 1
        r, c = x.shape[-2:]
        shape = (depth, c, r) if len(x.shape) == 3 else (c, r)
        out = out or self.empty(shape, x.dtype)
        check(self.lib.prad_transpose(self.ctx, dtype_code(x.dtype), x.ptr, out.ptr, r, c, depth))
        return out

    # ------------------------------------------------------------ row operations
    def softmax_forward(self, x, out=None):
        out = out or self.empty(x.shape, x.dtype)
        check(self.lib.prad_softmax_forward(self.ctx, dtype_code(x.dtype), x.ptr, out.ptr,
                                            x.size // x.shape[-1], x.shape[-1]))
        return out

    def softmax_backward(self, y, dy, out=None):
        out = out or self.empty(y.shape, y.dtype)
        check(self.lib.prad_softmax_backward(self.ctx, dtype_code(y.dtype), y.ptr, dy.ptr, out.ptr,
                                             y.size // y.shape[-1], y.shape[-1]))
        return out

    def sine_softmax_forward(self, x, out=None):
        """SineSoftmaxOperation.Forward: e / (sum e + e) with e = exp(sin x), row by row."""
        out = out or self.empty(x.shape, x.dtype)
        check(self.lib.prad_sine_softmax_forward(self.ctx, dtype_code(x.dtype), x.ptr, out.ptr,
                                                 x.size // x.shape[-1], x.shape[-1]))
        return out

    def sine_softmax_backward(self, x, dy, out=None):
        """SineSoftmaxOperation.Backward; `x` is the operation's input."""
        out = out or self.empty(x.shape, x.dtype)
        check(self.lib.prad_sine_softmax_backward(self.ctx, dtype_code(x.dtype), x.ptr, dy.ptr, out.ptr,
                                                  x.size // x.shape[-1], x.shape[-1]))
        return out

    def layernorm_forward(self, x, out=None):
        rows = x.size // x.shape[-1]
        if out is not None:
            y, mean, std = out
        else:
            y = self.empty(x.shape, x.dtype)
            mean = self.empty((rows,), x.dtype)
            std = self.empty((rows,), x.dtype)
        check(self.lib.prad_layernorm_forward(self.ctx, dtype_code(x.dtype), x.ptr, y.ptr, mean.ptr,
                                              std.ptr, rows, x.shape[-1]))
        return y, mean, std

    def layernorm_backward(self, x, mean, std, dy, out=None):
        out = out or self.empty(x.shape, x.dtype)
        check(self.lib.prad_layernorm_backward(self.ctx, dtype_code(x.dtype), x.ptr, mean.ptr,
                                               std.ptr, dy.ptr, out.ptr, x.size // x.shape[-1],
                                               x.shape[-1]))
        return out

    def swish_forward(self, x, beta, out=None):
        """SwishOperation: beta is a [1 x 1] device matrix."""
        out = out or self.empty(x.shape, x.dtype)
        check(self.lib.prad_swish_forward(self.ctx, dtype_code(x.dtype), x.ptr, beta.ptr, out.ptr, x.size))
        return out

    def swish_backward(self, x, beta, dy, out=None, accumulate=False):
        """Returns (dx, dbeta[1 x 1])."""
        dx, db = out or (self.empty(x.shape, x.dtype), self.zeros((1, 1), x.dtype))
        check(self.lib.prad_swish_backward(self.ctx, dtype_code(x.dtype), x.ptr, beta.ptr, dy.ptr, dx.ptr, db.ptr,
                                           x.size, int(accumulate)))
        return dx, db

    def row_sum_forward(self, x, average=False, out=None):
        """MatrixSumOperation / MatrixAverageOperation: [rows x 1]."""
        out = out or self.empty((x.shape[0], 1), x.dtype)
        check(self.lib.prad_row_sum_forward(self.ctx, dtype_code(x.dtype), x.ptr, out.ptr, x.shape[0], x.shape[1],
                                            int(average)))
        return out

    def row_sum_backward(self, dy, cols, average=False, out=None):
        out = out or self.empty((dy.shape[0], cols), dy.dtype)
        check(self.lib.prad_row_sum_backward(self.ctx, dtype_code(dy.dtype), dy.ptr, out.ptr, dy.shape[0], cols,
                                             int(average)))
        return out

    def broadcast_forward(self, x, rows, cols, out=None):
        out = out or self.empty((rows, cols), x.dtype)
        check(self.lib.prad_broadcast_forward(self.ctx, dtype_code(x.dtype), x.ptr, x.shape[0], x.shape[1], out.ptr,
                                              rows, cols))
        return out

    def broadcast_backward(self, dy, in_rows, in_cols, out=None):
        out = out or self.empty((in_rows, in_cols), dy.dtype)
        check(self.lib.prad_broadcast_backward(self.ctx, dtype_code(dy.dtype), dy.ptr, dy.shape[0], dy.shape[1],
                                               out.ptr, in_rows, in_cols))
        return out

    def concatenate_forward(self, mats, out=None):
        """MatrixConcatenateOperation: the inputs side by side (same row count)."""
        rows, total = mats[0].shape[0], sum(m.shape[1] for m in mats)
        if any(m.shape[0] != rows for m in mats):
            raise _lib.PradError(_lib.ERR_SHAPE, "All input matrices must have the same number of rows.")
        out = out or self.empty((rows, total), mats[0].dtype)
        es, col = out.dtype.itemsize, 0
        for m in mats:
            check(self.lib.prad_copy_2d(self.ctx, out.ptr + col * es, total * es, m.ptr, m.shape[1] * es,
                                        m.shape[1] * es, rows))
            col += m.shape[1]
        return out

    def concatenate_backward(self, dy, widths):
        """The column ranges of dOutput, one matrix per input."""
        rows, total = dy.shape
        es, col, outs = dy.dtype.itemsize, 0, []
        for w in widths:
            g = self.empty((rows, w), dy.dtype)
            check(self.lib.prad_copy_2d(self.ctx, g.ptr, w * es, dy.ptr + col * es, total * es, w * es, rows))
            outs.append(g)
            col += w
        return outs

    # ------------------------------------------------------------ Tensor elementwise family
    TENSOR_OPS = {"exp": 0, "ln": 1, "log": 2, "abs": 3, "square": 4, "sqrt": 5, "sin": 6, "cos": 7,
                  "reciprocal": 8, "negate": 9, "add": 16, "sub": 17, "mul": 18, "div": 19}

    def tensor_unary(self, op: str, x, out=None):
        out = out or self.empty(x.shape, x.dtype)
        check(self.lib.prad_tensor_unary(self.ctx, dtype_code(x.dtype), self.TENSOR_OPS[op], x.ptr, out.ptr, x.size))
        return out

    def tensor_unary_reverse(self, op: str, saved, dy, out=None):
        out = out or self.empty(dy.shape, dy.dtype)
        check(self.lib.prad_tensor_unary_reverse(self.ctx, dtype_code(dy.dtype), self.TENSOR_OPS[op], saved.ptr, dy.ptr,
                                                 out.ptr, dy.size))
        return out

    def tensor_binary(self, op: str, a, b, out=None):
        out = out or self.empty(a.shape, a.dtype)
        check(self.lib.prad_tensor_binary(self.ctx, dtype_code(a.dtype), self.TENSOR_OPS[op], a.ptr, b.ptr, out.ptr,
                                          a.size))
        return out

    def tensor_binary_reverse(self, op: str, a, b, dy):
        da, db = self.empty(dy.shape, dy.dtype), self.empty(dy.shape, dy.dtype)
        check(self.lib.prad_tensor_binary_reverse(self.ctx, dtype_code(dy.dtype), self.TENSOR_OPS[op], self._p(a),
                                                  self._p(b), dy.ptr, da.ptr, db.ptr, dy.size))
        return da, db

    # ------------------------------------------------------------ Tensor matmul / gather / tile
    def tensor_matmul(self, a, b, alpha=1.0, beta=0.0, out=None):
        """Tensor.MatrixMultiply (src/PRAD/Tensor.cs:572-613); raises PradError(ERR_SHAPE) as it throws."""
        out = out or self.empty((a.shape[0], b.shape[1]), a.dtype)
        check(self.lib.prad_tensor_matmul(self.ctx, dtype_code(a.dtype), a.ptr, a.shape[0], a.shape[1], b.ptr,
                                          b.shape[0], b.shape[1], alpha, beta, out.ptr))
        return out

    def tensor_matmul_reverse(self, a, b, dc):
        da, db = self.empty(a.shape, a.dtype), self.empty(b.shape, a.dtype)
        check(self.lib.prad_tensor_matmul_reverse(self.ctx, dtype_code(a.dtype), a.ptr, a.shape[0], a.shape[1], b.ptr,
                                                  b.shape[0], b.shape[1], dc.ptr, da.ptr, db.ptr))
        return da, db

    @staticmethod
    def _axis_view(shape, axis):
        outer = int(np.prod(shape[:axis], dtype=np.int64))
        inner = int(np.prod(shape[axis + 1:], dtype=np.int64))
        return outer, int(shape[axis]), inner

    def tensor_gather(self, x, indices, axis=0):
        """Tensor.Gather: result shape = x.shape[:axis] + indices.shape + x.shape[axis+1:]."""
        outer, n, inner = self._axis_view(x.shape, axis)
        shape = tuple(x.shape[:axis]) + tuple(indices.shape) + tuple(x.shape[axis + 1:])
        out = self.empty(shape, x.dtype)
        check(self.lib.prad_tensor_gather(self.ctx, dtype_code(x.dtype), x.ptr, outer, n, inner, indices.ptr,
                                          indices.size, out.ptr))
        return out

    def tensor_gather_reverse(self, upstream, indices, input_shape, axis=0):
        outer, n, inner = self._axis_view(input_shape, axis)
        dx = self.empty(input_shape, upstream.dtype)
        check(self.lib.prad_tensor_gather_reverse(self.ctx, dtype_code(upstream.dtype), upstream.ptr, outer, n, inner,
                                                  indices.ptr, indices.size, dx.ptr))
        return dx

    def tensor_tile(self, x, multiples):
        mr, mc = multiples
        out = self.empty((x.shape[0] * mr, x.shape[1] * mc), x.dtype)
        check(self.lib.prad_tensor_tile(self.ctx, dtype_code(x.dtype), x.ptr, x.shape[0], x.shape[1], mr, mc, out.ptr))
        return out

    def tensor_tile_reverse(self, upstream, input_shape, multiples):
        mr, mc = multiples
        dx = self.empty(input_shape, upstream.dtype)
        check(self.lib.prad_tensor_tile_reverse(self.ctx, dtype_code(upstream.dtype), upstream.ptr, input_shape[0],
                                                input_shape[1], mr, mc, dx.ptr))
        return dx

    def batchnorm_forward(self, x, out=None):
        """BatchNormalizationOperation as written.  Returns (y, stats) with stats a device [1 x 4] float64."""
        y = out or self.empty(x.shape, x.dtype)
        stats = self.zeros((1, 4), np.float64)
        check(self.lib.prad_batchnorm_forward(self.ctx, dtype_code(x.dtype), x.ptr, y.ptr, stats.ptr, x.shape[0],
                                              x.shape[1]))
        return y, stats

    def batchnorm_backward(self, x, stats, dy, out=None):
        out = out or self.empty(x.shape, x.dtype)
        check(self.lib.prad_batchnorm_backward(self.ctx, dtype_code(x.dtype), x.ptr, stats.ptr, dy.ptr, out.ptr,
                                               x.shape[0], x.shape[1]))
        return out

    def swiglu_forward(self, x, w, v, b, c, beta, out=None):
        """SwigLUOperation: w, v, b, c hold one value per column of x."""
        out = out or self.empty(x.shape, x.dtype)
        check(self.lib.prad_swiglu_forward(self.ctx, dtype_code(x.dtype), x.ptr, w.ptr, v.ptr, b.ptr, c.ptr, beta,
                                           out.ptr, x.shape[0], x.shape[1]))
        return out

    def swiglu_backward(self, x, w, v, b, c, beta, dy):
        """Returns (dx, dw, dv, db, dc)."""
        dx = self.empty(x.shape, x.dtype)
        g = [self.empty((x.shape[1], 1), x.dtype) for _ in range(4)]
        check(self.lib.prad_swiglu_backward(self.ctx, dtype_code(x.dtype), x.ptr, w.ptr, v.ptr, b.ptr, c.ptr, beta,
                                            dy.ptr, dx.ptr, g[0].ptr, g[1].ptr, g[2].ptr, g[3].ptr, x.shape[0],
                                            x.shape[1]))
        return (dx, *g)

    def scale_shift_forward(self, x, beta, gamma, out=None):
        """ScaleAndShiftOperation: beta, gamma hold one value per row of x."""
        out = out or self.empty(x.shape, x.dtype)
        check(self.lib.prad_scale_shift_forward(self.ctx, dtype_code(x.dtype), x.ptr, beta.ptr, gamma.ptr, out.ptr,
                                                x.shape[0], x.shape[1]))
        return out

    def scale_shift_backward(self, x, beta, dy, out=None):
        """Returns (dx, dbeta[rows], dgamma[rows])."""
        dx, db, dg = out or (self.empty(x.shape, x.dtype), self.empty((x.shape[0], 1), x.dtype),
                             self.empty((x.shape[0], 1), x.dtype))
        check(self.lib.prad_scale_shift_backward(self.ctx, dtype_code(x.dtype), x.ptr, beta.ptr, dy.ptr, dx.ptr,
                                                 db.ptr, dg.ptr, x.shape[0], x.shape[1]))
        return dx, db, dg

    def rmsnorm_forward(self, x, g, out=None):
        out = out or self.empty(x.shape, x.dtype)
        check(self.lib.prad_rmsnorm_forward(self.ctx, dtype_code(x.dtype), x.ptr, g.ptr, out.ptr, x.shape[0],
                                            x.shape[1]))
        return out

    def rmsnorm_backward(self, x, g, dy, out=None):
        """Returns (dx, dg)."""
        dx, dg = out or (self.empty(x.shape, x.dtype), self.empty(x.shape, x.dtype))
        check(self.lib.prad_rmsnorm_backward(self.ctx, dtype_code(x.dtype), x.ptr, g.ptr, dy.ptr, dx.ptr, dg.ptr,
                                             x.shape[0], x.shape[1]))
        return dx, dg

    # ------------------------------------------------------------ losses
    def _loss_fwd(self, fn, out, target):
        loss = self.empty((1, 1), out.dtype)
        check(fn(self.ctx, dtype_code(out.dtype), out.ptr, target.ptr, loss.ptr, out.shape[0],
                 out.shape[1]))
        return loss

    def mse_forward(self, out, target):
        return self._loss_fwd(self.lib.prad_mse_forward, out, target)

    def cce_forward(self, out, target):
        return self._loss_fwd(self.lib.prad_cce_forward, out, target)

    def mse_backward(self, out, target, rows_total=None, grad=None):
        grad = grad or self.empty(out.shape, out.dtype)
        check(self.lib.prad_mse_backward(self.ctx, dtype_code(out.dtype), out.ptr, target.ptr,
                                         grad.ptr, out.shape[0], out.shape[1],
                                         rows_total or out.shape[0]))
        return grad

    def cce_backward(self, out, target, rows_total=None, grad=None):
        grad = grad or self.empty(out.shape, out.dtype)
        check(self.lib.prad_cce_backward(self.ctx, dtype_code(out.dtype), out.ptr, target.ptr,
                                         grad.ptr, out.shape[0], out.shape[1],
                                         rows_total or out.shape[0]))
        return grad

    # ------------------------------------------------------------ embedding
    def embedding_forward(self, index_col, W):
        n = index_col.size
        out = self.empty((n, W.shape[1]), W.dtype)
        check(self.lib.prad_embedding_forward(self.ctx, dtype_code(W.dtype), index_col.ptr, W.ptr,
                                              out.ptr, n, W.shape[0], W.shape[1]))
        return out

    def embedding_backward(self, index_col, dOut, vocab, out=None):
        dW = out or self.empty((vocab, dOut.shape[1]), dOut.dtype)
        check(self.lib.prad_embedding_backward(self.ctx, dtype_code(dOut.dtype), index_col.ptr,
                                               dOut.ptr, dW.ptr, index_col.size, vocab,
                                               dOut.shape[1]))
        return dW

    # ------------------------------------------------------------ accumulation
    def segmented_sum(self, srcs, out=None):
        srcs = list(srcs)
        out = out or self.empty(srcs[0].shape, srcs[0].dtype)
        check(self.lib.prad_segmented_sum(self.ctx, dtype_code(out.dtype), self._ptr_list(srcs),
                                          len(srcs), out.ptr, out.size))
        return out

    def batch_mean(self, srcs, out=None):
        srcs = list(srcs)
        out = out or self.empty(srcs[0].shape, srcs[0].dtype)
        check(self.lib.prad_batch_mean(self.ctx, dtype_code(out.dtype), self._ptr_list(srcs),
                                       len(srcs), out.ptr, out.size))
        return out

    def accumulate(self, dest, src):
        check(self.lib.prad_accumulate(self.ctx, dtype_code(dest.dtype), dest.ptr, src.ptr,
                                       dest.size))

    # ------------------------------------------------------------ clip + Adam
    def clip_reference(self, grads, clip_value, min_value):
        grads = list(grads)
        check(self.lib.prad_clip_reference(self.ctx, dtype_code(grads[0].dtype),
                                           self._ptr_list(grads), self._size_list(grads),
                                           len(grads), clip_value, min_value))

    def clip_global_norm(self, grads, max_norm) -> float:
        grads = list(grads)
        norm = C.c_double()
        check(self.lib.prad_clip_global_norm(self.ctx, dtype_code(grads[0].dtype),
                                             self._ptr_list(grads), self._size_list(grads),
                                             len(grads), max_norm, C.byref(norm)))
        return norm.value

    def clip_adam(self, w, g, m, v, clip_mode, clip_value, min_value, lr, beta1, beta2, eps,
                  iteration, form=ADAM_RMAD, zero_grad=False):
        w, g, m, v = list(w), list(g), list(m), list(v)
        check(self.lib.prad_clip_adam(self.ctx, dtype_code(w[0].dtype), self._ptr_list(w),
                                      self._ptr_list(g), self._ptr_list(m), self._ptr_list(v),
                                      self._size_list(w), len(w), clip_mode, clip_value, min_value,
                                      lr, beta1, beta2, eps, iteration, form, int(zero_grad)))

    def adam(self, w, g, m, v, lr, beta1, beta2, eps, iteration, form=ADAM_RMAD, zero_grad=False):
        self.clip_adam(w, g, m, v, CLIP_NONE, 0.0, 0.0, lr, beta1, beta2, eps, iteration, form,
                       zero_grad)

    # ------------------------------------------------------------ slots, packed transfers, introspection
    @staticmethod
    def _guid_bytes(guid) -> bytes:
        b = guid.bytes if hasattr(guid, "bytes") else bytes(guid)
        if len(b) != 16:
            raise ValueError("a slot id is 16 bytes (System.Guid)")
        return b

    def slot_store(self, guid, mats, copy=False) -> None:
        """IOperationBase.Store(Guid): keep `mats` (references, or device copies) under the id."""
        ptrs = (C.c_void_p * len(mats))(*[m.ptr for m in mats])
        sizes = (C.c_size_t * len(mats))(*[m.nbytes for m in mats])
        check(self.lib.prad_slot_store(self.ctx, self._guid_bytes(guid), ptrs, sizes, len(mats), int(copy)))

    def slot_restore(self, guid, like):
        """IOperationBase.Restore(Guid): the stored buffers as (non-owning) matrices shaped like `like`."""
        out = (C.c_void_p * len(like))()
        check(self.lib.prad_slot_restore(self.ctx, self._guid_bytes(guid), out, len(like)))
        return [DeviceMatrix(self, out[i], m.shape, m.dtype, owned=False) for i, m in enumerate(like)]

    def slot_drop(self, guid) -> None:
        check(self.lib.prad_slot_drop(self.ctx, self._guid_bytes(guid)))

    def slot_count(self) -> int:
        n = C.c_int()
        check(self.lib.prad_slot_count(self.ctx, C.byref(n)))
        return n.value

    def download_many(self, mats) -> List[np.ndarray]:
        """One packed device-to-host transfer of all `mats` (one wait), split back into arrays."""
        total = sum(m.nbytes for m in mats)
        block = np.empty(max(total, 1), np.uint8)
        ptrs = (C.c_void_p * len(mats))(*[m.ptr for m in mats])
        sizes = (C.c_size_t * len(mats))(*[m.nbytes for m in mats])
        check(self.lib.prad_download_many(self.ctx, block.ctypes.data, ptrs, sizes, len(mats)))
        out, off = [], 0
        for m in mats:
            out.append(block[off:off + m.nbytes].view(m.dtype).reshape(m.shape).copy())
            off += m.nbytes
        return out

    def upload_many(self, mats, arrays) -> None:
        block = np.concatenate([np.ascontiguousarray(a, m.dtype).reshape(-1).view(np.uint8) for m, a in zip(mats, arrays)]) \
            if mats else np.empty(1, np.uint8)
        ptrs = (C.c_void_p * len(mats))(*[m.ptr for m in mats])
        sizes = (C.c_size_t * len(mats))(*[m.nbytes for m in mats])
        check(self.lib.prad_upload_many(self.ctx, ptrs, block.ctypes.data, sizes, len(mats)))

    def device_info(self) -> dict:
        info = _lib.DeviceInfo()
        check(self.lib.prad_device_info(self.ctx, C.byref(info)))
        return {k: (getattr(info, k).decode() if k == "name" else getattr(info, k)) for k, _ in info._fields_}

    def pipe_rate(self, pipe: int) -> float:
        """TFLOP/s of a pipe measured now: 0 FP64 FMA, 1 FP64 MMA, 2 FP32 FMA (prad_measure_pipe_rate)."""
        out = C.c_double()
        check(self.lib.prad_measure_pipe_rate(self.ctx, pipe, C.byref(out)))
        return out.value

    def timing_begin(self, label: str) -> None:
        check(self.lib.prad_timing_begin(self.ctx, label.encode()))

    def timing_end(self) -> None:
        check(self.lib.prad_timing_end(self.ctx))

    def get_timings(self):
        """[(label, milliseconds, launches)] of the finished brackets; waits for the stream."""
        n = C.c_int()
        check(self.lib.prad_get_timings(self.ctx, None, 0, C.byref(n)))
        if n.value == 0:
            return []
        buf = (_lib.Timing * n.value)()
        check(self.lib.prad_get_timings(self.ctx, buf, n.value, C.byref(n)))
        return [(t.label.decode(), t.milliseconds, t.launches) for t in buf]

    # ------------------------------------------------------------ data parallel
    @staticmethod
    def dp_unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        check(_lib.load().prad_dp_unique_id(buf))
        return buf.raw

    def dp_init(self, unique_id: bytes, rank: int, world: int) -> None:
        check(self.lib.prad_dp_init(self.ctx, C.create_string_buffer(unique_id, 128), rank, world))

    def dp_allreduce(self, m: DeviceMatrix) -> None:
        check(self.lib.prad_dp_allreduce(self.ctx, dtype_code(m.dtype), m.ptr, m.size))

    def dp_wait(self) -> None:
        check(self.lib.prad_dp_wait(self.ctx))

    def dp_reduce(self, m: DeviceMatrix, root: int) -> None:
        check(self.lib.prad_dp_reduce(self.ctx, dtype_code(m.dtype), m.ptr, m.size, root))

    def dp_broadcast(self, m: DeviceMatrix, root: int) -> None:
        check(self.lib.prad_dp_broadcast(self.ctx, dtype_code(m.dtype), m.ptr, m.size, root))

    def dp_mark(self, slot: int) -> None:
        """Remember, under `slot`, what the communication stream has been given so far."""
        check(self.lib.prad_dp_mark(self.ctx, slot))

    def dp_wait_mark(self, slot: int) -> None:
        """The compute stream waits for the collectives enqueued before dp_mark(slot), not for later ones."""
        check(self.lib.prad_dp_wait_mark(self.ctx, slot))

    def dp_wait_host(self, timeout_ms: float) -> None:
        """Host-side join with a deadline; raises PradError(ERR_TIMEOUT / ERR_COMM) and leaves the
        communicator aborted when a peer never arrives."""
        check(self.lib.prad_dp_wait_host(self.ctx, float(timeout_ms)))

    def dp_shutdown(self) -> None:
        check(self.lib.prad_dp_shutdown(self.ctx))
