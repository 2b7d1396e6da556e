"""The allocation-free bias-gradient entry point against the ordinary one.

Some users of this library run where device memory may not be requested once the program is
under way (all of it was handed out at start-up, or an allocator call would stall a
latency-bound loop).  For them `prad_add_broadcast_backward_static` keeps its partial sums in
a fixed array inside the library instead of a workspace that grows on demand.  This test
calls it through the C ABI twice in a row, on different data, and requires the same column
sums as `prad_add_broadcast_backward` and as the CPU oracle's restatement of
MatrixAddBroadcastingOperation.Backward, to the tolerance of the other column-sum tests.

It lives in a file that sorts last so that a run stopping at the first failure has already
exercised everything else.
"""
import ctypes as C

import numpy as np
import pytest

import oracle as O
from parallelreverseautodiff_b200 import _lib
from parallelreverseautodiff_b200.engine import dtype_code
from util import assert_close, normal, rng

pytestmark = pytest.mark.gpu


def _static_colsum(engine, dy_dev, accumulate=False, into=None):
    out = into if into is not None else engine.empty((1, dy_dev.shape[1]), dy_dev.dtype)
    _lib.check(engine.lib.prad_add_broadcast_backward_static(
        C.c_void_p(engine.stream()), dtype_code(dy_dev.dtype), dy_dev.ptr, out.ptr,
        dy_dev.shape[0], dy_dev.shape[1], int(accumulate)))
    return out


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_static_matches_allocating_entry_point_twice(engine, dtype):
    r = rng(123)
    # second call is smaller than the first: stale partial sums of call 1 stay in the array
    for shape in [(5000, 513), (333, 96)]:
        dy = normal(r, shape, 1.0, dtype)
        d = engine.upload(dy)
        want = engine.add_broadcast_backward(d).numpy()
        got = _static_colsum(engine, d).numpy()
        scale = np.abs(dy).astype(np.float64).sum(0, keepdims=True)
        assert_close(got, want, scale, f"static column sums {shape}")
        assert_close(got, O.add_broadcast_backward(dy)[1], scale, f"static column sums {shape} vs oracle")
    # accumulate form
    base = normal(r, (1, 96), 1.0, dtype)
    a, b = engine.upload(base), engine.upload(base)
    engine.add_broadcast_backward(d, dbias=a, accumulate=True)
    _static_colsum(engine, d, accumulate=True, into=b)
    assert_close(b.numpy(), a.numpy(), scale + 1.0, "static column sums, accumulate")


@pytest.mark.parametrize("shape", [(3000, 32768), (1, 777), (70000, 7)])
def test_static_edge_shapes_against_the_oracle(engine, shape):
    """The widest matrix the fixed array admits, a single row, and a tall narrow matrix."""
    r = rng(7)
    dy = normal(r, shape, 1.0, np.float32)
    d = engine.upload(dy)
    got = _static_colsum(engine, d).numpy()
    scale = np.abs(dy).astype(np.float64).sum(0, keepdims=True)
    assert_close(got, O.add_broadcast_backward(dy)[1], scale, f"static column sums {shape} vs oracle")
    assert_close(got, engine.add_broadcast_backward(d).numpy(), scale, f"static column sums {shape}")


def test_static_rejects_sizes_beyond_its_array(engine):
    d = engine.empty((2, 40000), np.float32)
    out = engine.empty((1, 40000), np.float32)
    st = engine.lib.prad_add_broadcast_backward_static(C.c_void_p(engine.stream()), 0, d.ptr, out.ptr,
                                                       2, 40000, 0)
    assert st == _lib.ERR_UNSUPPORTED
    assert b"exceed" in engine.lib.prad_last_error()
