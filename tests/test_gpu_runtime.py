"""Runtime services of the C ABI on a GPU: intermediate slots (Store / Restore by Guid), packed
download / upload of weights and Adam moments, device facts and CUDA-event timing brackets."""
import uuid

import numpy as np
import pytest

import oracle as O
from parallelreverseautodiff_b200 import _lib
from parallelreverseautodiff_b200 import engine as E
from parallelreverseautodiff_b200.networks import FeedForwardNetwork
from util import rng

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("copy", [False, True], ids=["references", "device copies"])
def test_two_forwards_stored_then_two_backwards_in_reverse_order(engine, copy):
    """ComputationGraph.StoreOperationIntermediates(id) after each of two forward passes, then
    RestoreOperationIntermediates(id) + Backward for the second pass first and the first pass last
    (src/RMAD/ComputationGraph.cs:161-181, MatrixMultiplyOperation.cs:31-42): a MatMul -> Tanh node."""
    r = rng(1)
    W = r.standard_normal((24, 16))
    xs = [r.standard_normal((10, 24)), r.standard_normal((10, 24))]
    ds = [r.standard_normal((10, 16)), r.standard_normal((10, 16))]
    Wd = engine.upload(W)
    ids = [uuid.uuid4(), uuid.uuid4()]
    x_buf = engine.empty((10, 24), np.float64)       # with copies the SAME buffers serve both passes
    y_buf = engine.empty((10, 16), np.float64)
    keep = []
    n_before = engine.slot_count()
    for k in range(2):
        if copy:
            x, y = x_buf, y_buf
            engine.upload(xs[k], out=x)
        else:                                        # references: fresh buffers per pass, as `new Matrix`
            x = engine.upload(xs[k])
            y = engine.empty((10, 16), np.float64)
            keep += [x, y]
        z = engine.matmul_forward(x, Wd)
        engine.act_forward(E.ACT_TANH, z, out=y)
        engine.slot_store(ids[k], [x, y], copy=copy)
    assert engine.slot_count() == n_before + 2
    for k in (1, 0):
        x, y = engine.slot_restore(ids[k], [x_buf, y_buf])
        dz = engine.act_backward(E.ACT_TANH, y, engine.upload(ds[k]))
        dA, dW = engine.matmul_backward(x, Wd, dz)
        y_ref = O.tanh_forward(O.matmul_forward(xs[k], W))
        dz_ref = O.tanh_backward(y_ref, ds[k])
        dA_ref, dW_ref = O.matmul_backward(xs[k], W, dz_ref)
        np.testing.assert_allclose(y.numpy(), y_ref, rtol=1e-12, atol=1e-14)
        np.testing.assert_allclose(dA.numpy(), dA_ref, rtol=1e-12, atol=1e-13)
        np.testing.assert_allclose(dW.numpy(), dW_ref, rtol=1e-12, atol=1e-13)
    # AddOrUpdate: storing again under the first id replaces it
    engine.slot_store(ids[0], [Wd], copy=copy)
    (w_back,) = engine.slot_restore(ids[0], [Wd])
    np.testing.assert_array_equal(w_back.numpy(), W)
    with pytest.raises(_lib.PradError) as e:         # two buffers asked of a one-buffer slot
        engine.slot_restore(ids[0], [x_buf, y_buf])
    assert e.value.status == _lib.ERR_SHAPE
    for i in ids:
        engine.slot_drop(i)
    assert engine.slot_count() == n_before
    with pytest.raises(_lib.PradError) as e:
        engine.slot_restore(ids[1], [x_buf, y_buf])
    assert e.value.status == _lib.ERR_INVALID and "KeyNotFound" in str(e.value)


def test_weights_and_moments_round_trip_in_the_save_order(engine):
    """ModelLayer.SaveWeightsAndMoments writes (weights, first moments, second moments), each in element
    order (src/RMAD/ModelLayer.cs:282-299); LoadWeightsAndMoments reads them back."""
    r = rng(2)
    f = np.float32
    sizes = [12, 20, 7]
    net = FeedForwardNetwork(engine, f, sizes, hidden_act=E.ACT_LEAKY_RELU, loss="mse")
    net.set_weights([r.standard_normal((sizes[i], sizes[i + 1])).astype(f) for i in range(2)])
    x, t = r.standard_normal((9, 12)).astype(f), r.standard_normal((9, 7)).astype(f)
    net.train_step_host(x, t)                      # one step so that the moments are not zero
    order = net.params + net.m + net.v
    saved = engine.download_many(order)
    for got, m in zip(saved, order):
        np.testing.assert_array_equal(got, m.numpy())
    assert any(np.abs(a).max() > 0 for a in saved[len(net.params):])
    other = FeedForwardNetwork(engine, f, sizes, hidden_act=E.ACT_LEAKY_RELU, loss="mse")
    engine.upload_many(other.params + other.m + other.v, saved)
    a = net.train_step_host(x, t)
    b = other.train_step_host(x, t)                # resumes bit for bit
    assert a == b
    for p, q in zip(net.params + net.m + net.v, other.params + other.m + other.v):
        np.testing.assert_array_equal(p.numpy(), q.numpy())


def test_device_info(engine):
    info = engine.device_info()
    assert info["cc_major"] == 10 and info["sm_count"] >= 100
    assert info["total_bytes"] > info["free_bytes"] > 0
    assert info["l2_bytes"] > 0 and info["smem_per_block_optin"] >= 200 * 1024
    assert info["name"]


def test_timing_brackets(engine):
    a = engine.upload(rng(3).standard_normal((512, 512)).astype(np.float32))
    engine.get_timings()                            # forget whatever earlier tests left
    engine.timing_begin("product")
    engine.matmul_forward(a, a)
    engine.timing_end()
    engine.timing_begin("nothing")
    engine.timing_end()
    with pytest.raises(_lib.PradError):
        engine.timing_end()                         # no bracket is open
    rows = engine.get_timings()
    assert [r[0] for r in rows] == ["product", "nothing"]
    assert rows[0][1] > 0 and rows[0][2] >= 1 and rows[1][2] == 0
    assert rows[0][1] > rows[1][1]
    assert engine.get_timings() == []


def test_pipe_rates_are_plausible(engine):
    fma64, mma64, fma32 = engine.pipe_rate(0), engine.pipe_rate(1), engine.pipe_rate(2)
    assert 5 < fma64 < 200 and 5 < mma64 < 400 and 20 < fma32 < 400


def test_a_wait_that_runs_out_is_reported_and_leaves_the_context_usable(engine):
    """The give-up path without a fault or a hang: a one-CTA kernel waits a few polls on a barrier nobody
    arrives on.  Until the host has seen the error, the optimiser must not touch weights or moments
    (the gradients on the stream may be garbage); afterwards everything works again."""
    r = rng(6)
    f = np.float32
    w0 = r.standard_normal((64, 48)).astype(f)
    g0 = r.standard_normal((64, 48)).astype(f)
    w, g = engine.upload(w0), engine.upload(g0)
    m, v = engine.zeros((64, 48), f), engine.zeros((64, 48), f)
    engine.sync()
    _lib.check(engine.lib.prad_selftest_bounded_wait(engine.ctx, 16))
    engine.clip_adam([w], [g], [m], [v], E.CLIP_REFERENCE, 4.0, 1e-8, 1e-3, 0.9, 0.999, 1e-8, 1.0, zero_grad=True)
    with pytest.raises(_lib.PradError) as e:
        engine.sync()
    assert e.value.status == _lib.ERR_TIMEOUT and "self-test" in str(e.value)
    np.testing.assert_array_equal(w.numpy(), w0)          # the step was skipped ...
    np.testing.assert_array_equal(g.numpy(), g0)          # ... gradients not cleared, moments still zero
    assert not m.numpy().any() and not v.numpy().any()
    engine.sync()                                         # the flag was cleared by the failed sync
    engine.clip_adam([w], [g], [m], [v], E.CLIP_REFERENCE, 4.0, 1e-8, 1e-3, 0.9, 0.999, 1e-8, 1.0, zero_grad=True)
    assert np.abs(w.numpy() - w0).max() > 0 and not g.numpy().any()
    # and a tensor-core product afterwards is correct
    a = r.standard_normal((256, 512)).astype(f)
    b = r.standard_normal((512, 256)).astype(f)
    engine.set_option("gemm_f32", "fp16x3")
    try:
        got = engine.matmul_forward(engine.upload(a), engine.upload(b)).numpy()
    finally:
        engine.set_option("gemm_f32", "auto")
    ref = a.astype(np.float64) @ b.astype(np.float64)
    assert np.abs(got - ref).max() <= 1e-5 * (np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)).max()
