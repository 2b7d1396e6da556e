"""CUDA kernels against the committed golden vectors (tests/golden/ops_*.npz)."""
import numpy as np
import pytest

from parallelreverseautodiff_b200 import engine as E
from tests_golden import load_golden
from util import assert_close, rms

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["f32", "f64"])
def test_kernels_reproduce_golden_vectors(engine, name):
    g = load_golden(name)
    up = engine.upload
    A, B, dC = up(g["mm_A"]), up(g["mm_B"]), up(g["mm_dC"])
    bound = 40.0
    assert_close(engine.matmul_forward(A, B).numpy(), g["mm_C"], bound, "C")
    dA, dB = engine.matmul_backward(A, B, dC)
    assert_close(dA.numpy(), g["mm_dA"], bound, "dA")
    assert_close(dB.numpy(), g["mm_dB"], bound, "dB")
    dPre, dA, dB = engine.matmul_act_backward(A, B, dC, E.ACT_LEAKY_RELU, up(g["mm_C"]), 0.01)
    np.testing.assert_array_equal(dPre.numpy(), g["node_dPre"])
    assert_close(dA.numpy(), g["node_dA"], bound, "node dA")
    assert_close(dB.numpy(), g["node_dB"], bound, "node dB")
    bA, bB, bdC = up(g["bmm_A"]), up(g["bmm_B"]), up(g["bmm_dC"])
    assert_close(engine.batch_matmul_forward(bA, bB).numpy(), g["bmm_C"], bound, "bmm C")
    dA, dB, _ = engine.batch_matmul_backward(bA, bB, bdC)
    assert_close(dA.numpy(), g["bmm_dA"], bound, "bmm dA")
    assert_close(dB.numpy(), g["bmm_dB"], bound, "bmm dB")
    x, dy = up(g["x"]), up(g["dy"])
    for act, key, saved in ((E.ACT_LEAKY_RELU, "leaky", x), (E.ACT_SIGMOID, "sigmoid", up(g["sigmoid_y"])),
                            (E.ACT_TANH, "tanh", up(g["tanh_y"])), (E.ACT_GELU, "gelu", x)):
        assert_close(engine.act_forward(act, x, 0.01).numpy(), g[f"{key}_y"], 1.0, key)
        assert_close(engine.act_backward(act, saved, dy, 0.01).numpy(), g[f"{key}_dx"], 1.0, key + " bwd")
    for act, key in ((E.ACT_RELU, "relu"), (E.ACT_AMPLIFIED_SIGMOID, "ampsig")):
        assert_close(engine.act_forward(act, x).numpy(), g[f"{key}_y"], 1.0, key)
        assert_close(engine.act_backward(act, x, dy).numpy(), g[f"{key}_dx"], 1.0, key + " bwd")
    beta, gamma, gain = up(g["ss_beta"]), up(g["ss_gamma"]), up(g["rms_g"])
    np.testing.assert_array_equal(engine.scale_shift_forward(x, beta, gamma).numpy(), g["ss_y"])
    sdx, sdb, sdg = engine.scale_shift_backward(x, beta, dy)
    np.testing.assert_array_equal(sdx.numpy(), g["ss_dx"])
    assert_close(sdb.numpy().reshape(-1), g["ss_dbeta"], 10.0, "scale-and-shift dbeta")
    assert_close(sdg.numpy().reshape(-1), g["ss_dgamma"], 10.0, "scale-and-shift dgamma")
    assert_close(engine.rmsnorm_forward(x, gain).numpy(), g["rms_y"], 3.0, "rmsnorm")
    rdx, rdg = engine.rmsnorm_backward(x, gain, dy)
    assert_close(rdx.numpy(), g["rms_dx"], 3.0, "rmsnorm dx")
    assert_close(rdg.numpy(), g["rms_dg"], 3.0, "rmsnorm dg")
    da, db = engine.hadamard_backward(x, dy, dy)
    np.testing.assert_array_equal(da.numpy(), g["had_da"])
    np.testing.assert_array_equal(db.numpy(), g["had_db"])
    assert_close(engine.add_broadcast_backward(dy).numpy(), g["bias_db"], 20.0, "bias")
    assert_close(engine.softmax_forward(x).numpy(), g["softmax_y"], 1.0, "softmax")
    assert_close(engine.softmax_backward(up(g["softmax_y"]), dy).numpy(), g["softmax_dx"], 1.0, "softmax bwd")
    y, mean, std = engine.layernorm_forward(x)
    assert_close(y.numpy(), g["ln_y"], 1.0, "ln")
    assert_close(engine.layernorm_backward(x, up(g["ln_mean"]), up(g["ln_std"]), dy).numpy(), g["ln_dx"],
                 rms(g["ln_dx"]), "ln bwd")
    np.testing.assert_array_equal(engine.mse_backward(x, dy).numpy(), g["mse_grad"])
    assert_close(engine.mse_forward(x, dy).numpy().reshape(()), g["mse_loss"], 1.0, "mse")
    p, h = up(g["softmax_y"]), up(g["onehot"])
    np.testing.assert_array_equal(engine.cce_backward(p, h).numpy(), g["cce_grad"])
    assert_close(engine.cce_forward(p, h).numpy().reshape(()), g["cce_loss"], 1.0, "cce")
    idx = up(g["emb_idx"])
    np.testing.assert_array_equal(engine.embedding_forward(idx, up(g["emb_W"])).numpy(), g["emb_out"])
    np.testing.assert_array_equal(engine.embedding_backward(idx, up(g["emb_dOut"]), 7).numpy(), g["emb_dW"])
    srcs = [up(s) for s in g["acc_srcs"]]
    np.testing.assert_array_equal(engine.segmented_sum(srcs).numpy(), g["acc_sum"])
    np.testing.assert_array_equal(engine.batch_mean(srcs).numpy(), g["acc_mean"])
    grad = up(g["clip_in"])
    minv = 1e-8 if name == "f32" else 1e-16
    engine.clip_reference([grad], 4.0, minv)
    assert_close(grad.numpy(), g["clip_out"], 1.0, "clip")
    w, m, v = up(g["adam_w0"]), up(g["adam_m0"]), up(g["adam_v0"])
    engine.adam([w], [up(g["clip_out"])], [m], [v], 1e-3, 0.9, 0.999, 1e-8, 3.0)
    np.testing.assert_array_equal(w.numpy(), g["adam_w1"])
    np.testing.assert_array_equal(m.numpy(), g["adam_m1"])
    np.testing.assert_array_equal(v.numpy(), g["adam_v1"])
