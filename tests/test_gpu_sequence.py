"""Recorded launch sequences (prad_capture_begin / prad_capture_end / prad_sequence_launch):
a replay produces bit-identical results to the direct calls, counts its launches, and the
entry points that cannot be recorded say so without spoiling the recording."""
import numpy as np
import pytest

from parallelreverseautodiff_b200 import engine as E
from parallelreverseautodiff_b200._lib import ERR_INVALID, PradError
from parallelreverseautodiff_b200.workloads import C2Runner, C3Runner, make_c2, make_c3

pytestmark = pytest.mark.gpu


def test_replay_equals_direct_calls(engine):
    r = np.random.default_rng(5)
    A = engine.upload(r.standard_normal((96, 80)))
    B = engine.upload(r.standard_normal((80, 64)))
    dC = engine.upload(r.standard_normal((96, 64)))
    Z = engine.empty((96, 64), np.float64)
    dA, dB = engine.empty((96, 80), np.float64), engine.empty((80, 64), np.float64)
    dZ = engine.empty((96, 64), np.float64)

    def step():
        engine.matmul_forward(A, B, Y=Z)
        engine.act_backward(E.ACT_TANH, Z, dC, out=dZ)
        engine.matmul_backward(A, B, dZ, dA=dA, dB=dB)

    step()
    want = [dZ.numpy(), dA.numpy(), dB.numpy()]
    seq = engine.record(step)
    assert seq.launches >= 4
    for m in (dZ, dA, dB):
        engine.zero_(m)
    n0 = engine.launch_count()
    seq.launch()
    assert engine.launch_count() - n0 == seq.launches
    for got, ref in zip([dZ.numpy(), dA.numpy(), dB.numpy()], want):
        np.testing.assert_array_equal(got, ref)
    # the replay reads the buffers as they are when it runs
    engine.upload(2.0 * dC.numpy(), out=dC)
    seq.launch()
    np.testing.assert_array_equal(dZ.numpy(), 2.0 * want[0])
    seq.close()


def test_unrecordable_calls_are_refused_and_the_recording_survives(engine):
    x = engine.upload(np.ones((8, 8), np.float32))
    y = engine.empty((8, 8), np.float32)

    def bad():
        engine.scale(x, 2.0, out=y)
        engine.sync()

    with pytest.raises(PradError) as ei:
        engine.record(bad)
    assert ei.value.status == ERR_INVALID and "cannot be recorded" in str(ei.value)
    seq = engine.record(lambda: engine.scale(x, 3.0, out=y))      # a new recording works
    seq.launch()
    np.testing.assert_array_equal(y.numpy(), np.full((8, 8), 3.0, np.float32))
    seq.close()


def test_c2_step_replayed_matches_direct_steps(engine):
    """Two training steps of C2 (backward + clip + Adam), once by direct calls and once as
    replays of one recording, from the same start: identical weights afterwards."""
    inp = make_c2()
    a, b = C2Runner(engine, inp), C2Runner(engine, inp)
    for _ in range(2):
        a.backward()
    b.backward()                       # unrecorded once: scratch reaches its size, moments advance
    seq = engine.record(b.backward)
    seq.launch()
    for wa, wb in zip(a.net.params, b.net.params):
        np.testing.assert_array_equal(wa.numpy(), wb.numpy())
    seq.close()


def test_c3_bptt_replayed(engine):
    inp = make_c3(T=8, B=4, n_in=16, nh=24)
    a, b = C3Runner(engine, inp), C3Runner(engine, inp)
    a.backward()
    b.backward()
    seq = engine.record(b.backward)
    grads = lambda n: [n.dW[g] for g in n.GATES] + [n.dU[g] for g in n.GATES] + [n.db[g] for g in n.GATES]  # noqa: E731
    for g in grads(b.net):
        engine.zero_(g)
    seq.launch()
    for ga, gb in zip(grads(a.net), grads(b.net)):
        np.testing.assert_array_equal(ga.numpy(), gb.numpy())
    seq.close()


def test_tensor_core_product_replayed(engine):
    """The persistent tensor-core GEMM (operand passes, dynamic tile hand-out, split-K combine)
    inside a recorded sequence: replays give the bits of the direct call, every time."""
    engine.set_option("gemm_f32", "fp16x3")
    try:
        r = np.random.default_rng(9)
        A = engine.upload(r.standard_normal((640, 1100)).astype(np.float32))
        B = engine.upload(r.standard_normal((1100, 520)).astype(np.float32))
        dC = engine.upload(r.standard_normal((640, 520)).astype(np.float32))
        dA, dB = engine.empty((640, 1100), np.float32), engine.empty((1100, 520), np.float32)

        def step():
            engine.matmul_backward(A, B, dC, dA=dA, dB=dB)

        step()
        want = dA.numpy(), dB.numpy()
        seq = engine.record(step)
        for _ in range(3):
            engine.zero_(dA)
            engine.zero_(dB)
            seq.launch()
            np.testing.assert_array_equal(dA.numpy(), want[0])
            np.testing.assert_array_equal(dB.numpy(), want[1])
        seq.close()
    finally:
        engine.set_option("gemm_f32", "auto")
