"""ctypes binding of ``libprad_cuda.so`` -- the same C ABI a C# caller binds with P/Invoke.

Loading fails loudly when the shared library has not been built; there is no fallback of
any kind.  Every function declared in ``include/prad_cuda.h`` is given its argument types
here, so a signature drift shows up as a ctypes error instead of a corrupted call.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libprad_cuda.so")

vp, i32, i64, f64, sz = C.c_void_p, C.c_int, C.c_int64, C.c_double, C.c_size_t
pvp = C.POINTER(C.c_void_p)
pi64 = C.POINTER(C.c_int64)

# name -> argument types (return type is int32 status unless stated otherwise)
SIGNATURES = {
    "prad_init": [i32, pvp],
    "prad_shutdown": [vp],
    "prad_set_option": [vp, C.c_char_p, C.c_char_p],
    "prad_sync": [vp],
    "prad_launch_count": [vp, pi64],
    "prad_capture_begin": [vp],
    "prad_capture_end": [vp, pvp],
    "prad_sequence_launch": [vp, vp],
    "prad_sequence_launch_count": [vp, pi64],
    "prad_sequence_destroy": [vp, vp],
    "prad_stream": [vp, pvp],
    "prad_use_stream": [vp, vp],
    "prad_alloc": [vp, sz, pvp],
    "prad_free": [vp, vp],
    "prad_zero": [vp, vp, sz],
    "prad_copy": [vp, vp, vp, sz],
    "prad_upload": [vp, vp, vp, sz],
    "prad_download": [vp, vp, vp, sz],
    "prad_upload_prefetch": [vp, vp, vp, sz],
    "prad_upload_join": [vp],
    "prad_upload_rows": [vp, vp, pvp, i32, sz],
    "prad_download_rows": [vp, pvp, vp, i32, sz],
    "prad_alloc_host": [vp, sz, pvp],
    "prad_free_host": [vp, vp],
    "prad_gemm": [vp, i32, i32, i32, i32, i32, i32, f64, vp, i32, vp, i32, f64, vp, i32, i32, i64,
                  i64, i64],
    "prad_packed_create": [vp, i32, i32, i32, i32, i32, pvp],
    "prad_packed_destroy": [vp],
    "prad_packed_shape": [vp, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int),
                          C.POINTER(C.c_int)],
    "prad_pack": [vp, vp, i64],
    "prad_act_forward_pack": [vp, i32, vp, vp, f64],
    "prad_act_backward_pack": [vp, i32, vp, vp, vp, f64],
    "prad_mse_act_backward_pack": [vp, i32, vp, vp, vp, i64, vp, f64],
    "prad_gemm_packed": [vp, vp, i32, vp, i32, f64, f64, vp, i64, vp],
    "prad_matmul_forward": [vp, i32, vp, vp, vp, i32, i32, i32, vp, vp, i32, f64],
    "prad_matmul_backward": [vp, i32, vp, vp, vp, vp, vp, i32, i32, i32, i32, f64, i32, vp, f64],
    "prad_matmul_act_backward": [vp, i32, vp, vp, vp, i32, vp, f64, vp, vp, vp, i32, i32, i32],
    "prad_matmul_act_backward_host": [vp, i32, vp, vp, vp, i32, vp, f64, vp, vp, vp, i32, i32,
                                      i32],
    "prad_batch_matmul_forward": [vp, i32, vp, vp, vp, i32, i32, i32, i32, i32],
    "prad_batch_matmul_backward": [vp, i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32],
    "prad_matmul_and_sum_forward": [vp, i32, vp, vp, vp, i32, i32, i32, i32],
    "prad_matmul_and_sum_backward": [vp, i32, vp, vp, vp, vp, vp, i32, i32, i32, i32],
    "prad_act_forward": [vp, i32, i32, vp, vp, i64, f64],
    "prad_act_backward": [vp, i32, i32, vp, vp, vp, i64, f64],
    "prad_hadamard_forward": [vp, i32, vp, vp, vp, i64],
    "prad_hadamard_backward": [vp, i32, vp, vp, vp, vp, vp, i64],
    "prad_lstm_cell_backward": [vp, i32, i64, vp, vp, f64, pvp, i32, vp, pvp, vp, vp, pvp, vp],
    "prad_add_forward": [vp, i32, vp, vp, vp, vp, i64],
    "prad_add_broadcast_forward": [vp, i32, vp, vp, vp, i32, i32],
    "prad_add_broadcast_backward": [vp, i32, vp, vp, i32, i32, i32],
    "prad_add_broadcast_backward_static": [vp, i32, vp, vp, i32, i32, i32],
    "prad_scale": [vp, i32, vp, vp, i64, f64],
    "prad_transpose": [vp, i32, vp, vp, i32, i32, i32],
    "prad_sine_softmax_forward": [vp, i32, vp, vp, i64, i32],
    "prad_sine_softmax_backward": [vp, i32, vp, vp, vp, i64, i32],
    "prad_softmax_forward": [vp, i32, vp, vp, i64, i32],
    "prad_softmax_backward": [vp, i32, vp, vp, vp, i64, i32],
    "prad_layernorm_forward": [vp, i32, vp, vp, vp, vp, i64, i32],
    "prad_layernorm_backward": [vp, i32, vp, vp, vp, vp, vp, i64, i32],
    "prad_copy_2d": [vp, vp, sz, vp, sz, sz, sz],
    "prad_row_sum_forward": [vp, i32, vp, vp, i64, i32, i32],
    "prad_row_sum_backward": [vp, i32, vp, vp, i64, i32, i32],
    "prad_broadcast_forward": [vp, i32, vp, i32, i32, vp, i32, i32],
    "prad_broadcast_backward": [vp, i32, vp, i32, i32, vp, i32, i32],
    "prad_tensor_unary": [vp, i32, i32, vp, vp, i64],
    "prad_tensor_unary_reverse": [vp, i32, i32, vp, vp, vp, i64],
    "prad_tensor_binary": [vp, i32, i32, vp, vp, vp, i64],
    "prad_tensor_binary_reverse": [vp, i32, i32, vp, vp, vp, vp, vp, i64],
    "prad_tensor_matmul": [vp, i32, vp, i32, i32, vp, i32, i32, f64, f64, vp],
    "prad_tensor_matmul_reverse": [vp, i32, vp, i32, i32, vp, i32, i32, vp, vp, vp],
    "prad_tensor_gather": [vp, i32, vp, i64, i32, i64, vp, i32, vp],
    "prad_tensor_gather_reverse": [vp, i32, vp, i64, i32, i64, vp, i32, vp],
    "prad_tensor_tile": [vp, i32, vp, i32, i32, i32, i32, vp],
    "prad_tensor_tile_reverse": [vp, i32, vp, i32, i32, i32, i32, vp],
    "prad_batchnorm_forward": [vp, i32, vp, vp, vp, i64, i32],
    "prad_batchnorm_backward": [vp, i32, vp, vp, vp, vp, i64, i32],
    "prad_swiglu_forward": [vp, i32, vp, vp, vp, vp, vp, f64, vp, i64, i32],
    "prad_swiglu_backward": [vp, i32, vp, vp, vp, vp, vp, f64, vp, vp, vp, vp, vp, vp, i64, i32],
    "prad_swish_forward": [vp, i32, vp, vp, vp, i64],
    "prad_swish_backward": [vp, i32, vp, vp, vp, vp, vp, i64, i32],
    "prad_scale_shift_forward": [vp, i32, vp, vp, vp, vp, i64, i32],
    "prad_scale_shift_backward": [vp, i32, vp, vp, vp, vp, vp, vp, i64, i32],
    "prad_rmsnorm_forward": [vp, i32, vp, vp, vp, i64, i32],
    "prad_rmsnorm_backward": [vp, i32, vp, vp, vp, vp, vp, i64, i32],
    "prad_mse_forward": [vp, i32, vp, vp, vp, i64, i32],
    "prad_mse_backward": [vp, i32, vp, vp, vp, i64, i32, i64],
    "prad_cce_forward": [vp, i32, vp, vp, vp, i64, i32],
    "prad_cce_backward": [vp, i32, vp, vp, vp, i64, i32, i64],
    "prad_embedding_forward": [vp, i32, vp, vp, vp, i32, i32, i32],
    "prad_embedding_backward": [vp, i32, vp, vp, vp, i32, i32, i32],
    "prad_segmented_sum": [vp, i32, pvp, i32, vp, i64],
    "prad_accumulate": [vp, i32, vp, vp, i64],
    "prad_batch_mean": [vp, i32, pvp, i32, vp, i64],
    "prad_clip_reference": [vp, i32, pvp, pi64, i32, f64, f64],
    "prad_clip_global_norm": [vp, i32, pvp, pi64, i32, f64, C.POINTER(f64)],
    "prad_adam": [vp, i32, pvp, pvp, pvp, pvp, pi64, i32, f64, f64, f64, f64, f64, i32, i32],
    "prad_clip_adam": [vp, i32, pvp, pvp, pvp, pvp, pi64, i32, i32, f64, f64, f64, f64, f64, f64,
                       f64, i32, i32],
    "prad_graph_create": [vp, i32, pvp],
    "prad_graph_destroy": [vp],
    "prad_graph_add_value": [vp, i32, i32, vp, C.POINTER(C.c_int)],
    "prad_graph_add_deep_value": [vp, i32, i32, i32, vp, C.POINTER(C.c_int)],
    "prad_graph_set_gradient_destination": [vp, i32, vp],
    "prad_graph_add_node": [vp, i32, C.POINTER(C.c_int), i32, i32, f64, C.POINTER(C.c_int)],
    "prad_graph_forward": [vp],
    "prad_graph_backward": [vp, i32, vp],
    "prad_graph_backward_multi": [vp, C.POINTER(C.c_int), pvp, i32],
    "prad_graph_value_data": [vp, i32, pvp],
    "prad_graph_value_gradient": [vp, i32, pvp],
    "prad_graph_consumer_count": [vp, i32, C.POINTER(C.c_int)],
    "prad_dp_unique_id": [vp],
    "prad_dp_init": [vp, vp, i32, i32],
    "prad_dp_allreduce": [vp, i32, vp, i64],
    "prad_dp_wait": [vp],
    "prad_dp_reduce": [vp, i32, vp, i64, i32],
    "prad_dp_broadcast": [vp, i32, vp, i64, i32],
    "prad_dp_mark": [vp, i32],
    "prad_dp_wait_mark": [vp, i32],
    "prad_dp_wait_host": [vp, f64],
    "prad_dp_shutdown": [vp],
    "prad_download_many": [vp, vp, pvp, C.POINTER(sz), i32],
    "prad_upload_many": [vp, pvp, vp, C.POINTER(sz), i32],
    "prad_slot_store": [vp, vp, pvp, C.POINTER(sz), i32, i32],
    "prad_slot_restore": [vp, vp, pvp, i32],
    "prad_slot_drop": [vp, vp],
    "prad_slot_count": [vp, C.POINTER(C.c_int)],
    "prad_device_info": [vp, vp],
    "prad_selftest_bounded_wait": [vp, i32],
    "prad_measure_pipe_rate": [vp, i32, C.POINTER(f64)],
    "prad_timing_begin": [vp, C.c_char_p],
    "prad_timing_end": [vp],
    "prad_get_timings": [vp, vp, i32, C.POINTER(C.c_int)],
}
STRING_FUNCS = ("prad_last_error", "prad_version")

class DeviceInfo(C.Structure):
    """prad_device_info_t"""
    _fields_ = [("device", C.c_int32), ("sm_count", C.c_int32), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
                ("l2_bytes", C.c_int32), ("smem_per_block_optin", C.c_int32), ("sm_clock_khz", C.c_int32),
                ("mem_clock_khz", C.c_int32), ("total_bytes", C.c_uint64), ("free_bytes", C.c_uint64),
                ("scratch_bytes", C.c_uint64), ("name", C.c_char * 64)]


class Timing(C.Structure):
    """prad_timing_t"""
    _fields_ = [("label", C.c_char * 48), ("milliseconds", C.c_double), ("launches", C.c_int64)]


_lib = None


class PradError(RuntimeError):
    """A non-zero status from libprad_cuda; ``status`` holds the code."""

    def __init__(self, status: int, message: str):
        super().__init__(f"[prad status {status}] {message}")
        self.status = status


# status codes of include/prad_cuda.h
OK, ERR_INVALID, ERR_SHAPE, ERR_NOT_INITIALIZED, ERR_CUDA, ERR_OOM, ERR_UNSUPPORTED, ERR_COMM, \
    ERR_TIMEOUT = range(9)


def load() -> C.CDLL:
    """Loads the library (once).  Raises if it is missing: there is no other code path."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m parallelreverseautodiff_b200.build` "
            "(nvcc, sm_100a).  This package has no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here == header and library disagree
        fn.argtypes = args
        fn.restype = C.c_int32
    for name in STRING_FUNCS:
        fn = getattr(lib, name)
        fn.argtypes = []
        fn.restype = C.c_char_p
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != 0:
        raise PradError(status, load().prad_last_error().decode("utf-8", "replace"))
