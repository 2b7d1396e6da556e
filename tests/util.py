"""Shared helpers of the test-suite: seeded inputs and the stated tolerances."""
import numpy as np

# Tolerances of the parity contract.
#   double (PRAD):     |got - ref| <= 1e-12*|ref| + 1e-14*scale
#   float (PRADLite):  |got - ref| <= 1e-5*|ref|  + 1e-5*scale
# `scale` is 1 unless the caller passes the magnitude the rounding error is proportional to
# (for a dot product: sum_k |a_k||b_k|; for an elementwise tensor: its rms).  A plain
# element-wise relative test is meaningless where a sum cancels to ~0, so the absolute term
# carries that magnitude; it is never looser than the stated relative figure times it.
RTOL = {np.dtype(np.float64): 1e-12, np.dtype(np.float32): 1e-5}
ATOL = {np.dtype(np.float64): 1e-14, np.dtype(np.float32): 1e-5}


# Largest err / limit seen per `what` label in this session (1.0 = the tolerance is used up);
# conftest.py prints the table at the end of the run so that bounds can be tightened knowingly.
HEADROOM = {}


def assert_close(got, ref, scale=1.0, what=""):
    got = np.asarray(got)
    ref = np.asarray(ref)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert got.dtype == ref.dtype, f"{what}: dtype {got.dtype} vs {ref.dtype}"
    dt = ref.dtype
    g = got.astype(np.float64)
    r = ref.astype(np.float64)
    nan_mismatch = np.isnan(g) != np.isnan(r)
    assert not nan_mismatch.any(), f"{what}: NaN pattern differs"
    ok = np.isnan(r)
    err = np.abs(g - r)
    lim = RTOL[dt] * np.abs(r) + ATOL[dt] * np.maximum(np.asarray(scale, dtype=np.float64), 0)
    bad = ~ok & ~(err <= lim)
    if what and err.size:
        with np.errstate(divide="ignore", invalid="ignore"):
            ratio = np.where(ok | (err == 0), 0.0, err / np.broadcast_to(lim, err.shape))
        used = float(np.nanmax(ratio)) if ratio.size else 0.0
        HEADROOM[what] = max(HEADROOM.get(what, 0.0), used)
    if bad.any():
        i = np.unravel_index(np.argmax(np.where(bad, err - lim, -np.inf)), err.shape)
        raise AssertionError(
            f"{what}: {bad.sum()} of {bad.size} elements outside tolerance; worst at {i}: "
            f"got {g[i]!r} ref {r[i]!r} err {err[i]:.3e} lim {np.broadcast_to(lim, err.shape)[i]:.3e}")


def rms(x):
    x = np.asarray(x, dtype=np.float64)
    return float(np.sqrt(np.mean(x * x))) if x.size else 0.0


def rng(seed):
    return np.random.default_rng(seed)


def uniform(r, shape, lo, hi, dtype):
    return (r.random(shape) * (hi - lo) + lo).astype(dtype)


def normal(r, shape, std, dtype):
    return (r.standard_normal(shape) * std).astype(dtype)
