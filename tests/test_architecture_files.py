"""The architectures spelled out in tests/architectures.py ARE the reference's JSON files (checked
wherever the reference tree is present), and the CPU interpreter of the schema agrees with a
hand-written composition of oracle operations.  No GPU."""
import json
import os

import numpy as np
import pytest

import architectures as A
import oracle as O
from util import rng

# the reference tree: named by PRAD_REFERENCE_TREE, else a directory "reference" beside the repository
REF = os.environ.get("PRAD_REFERENCE_TREE") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
FILES = {
    "test/ParallelReverseAutoDiff.Test/FeedForward/Architecture/FeedForwardArchitecture.json":
        lambda: A.feedforward_architecture("GpuMatrixMultiplyOperation"),
    "lite/test/ParallelReverseAutoDiffLite.Test/FeedForward/Architecture/FeedForwardArchitecture.json":
        lambda: A.feedforward_architecture("GpuMatrixMultiplyOperation"),
    "examples/lstm/ParallelReverseAutoDiff.LstmExample/architecture/SelfAttentionMultiLayerLSTMArchitectureAmplified.json":
        A.lstm_architecture,
    "test/ParallelReverseAutoDiff.Test/GraphAttentionPaths/LSTM/Architecture/NodeProcessing.json":
        lambda: A.lstm_architecture(batch=True),
}


@pytest.mark.parametrize("path", sorted(FILES))
def test_built_architectures_equal_the_reference_files(path):
    full = os.path.join(REF, path)
    if not os.path.exists(full):
        pytest.skip("the reference tree is not on this machine")
    with open(full, encoding="utf-8-sig") as f:
        ref = json.load(f)
    assert A.strip_descriptions(ref) == FILES[path]()


def test_the_example_file_with_a_destination_beyond_the_results():
    """examples/feedforward/.../FeedForwardArchitecture.json lists three gradient destinations for the
    two-input MatrixAddOperation `h_add`; the managed AccumulateGradient throws for it
    (src/RMAD/OperationBase.cs:283-286).  Everything else equals the test network's file."""
    full = os.path.join(REF, "examples/feedforward/ParallelReverseAutoDiff.FeedForwardExample/architecture/FeedForwardArchitecture.json")
    if not os.path.exists(full):
        pytest.skip("the reference tree is not on this machine")
    with open(full, encoding="utf-8-sig") as f:
        ref = A.strip_descriptions(json.load(f))
    mine = A.feedforward_architecture("CudaMatrixMultiplyOperation")
    assert ref["timeSteps"][0]["layers"][0]["operations"][1]["gradientResultTo"] == [None, None, "DB[layerIndex]"]
    ref["timeSteps"][0]["layers"][0]["operations"][1]["gradientResultTo"] = [None, "DB[layerIndex]"]
    assert ref == mine


def test_interpreter_against_a_hand_written_composition():
    r = rng(3)
    n_in, nh, n_out, L = 5, 7, 3, 2
    We, Be = r.standard_normal((nh, n_in)), r.standard_normal((nh, 1))
    W = [r.standard_normal((nh, nh)) for _ in range(L)]
    B = [r.standard_normal((nh, 1)) for _ in range(L)]
    V, Bo = r.standard_normal((n_out, nh)), r.standard_normal((n_out, 1))
    x, d_out = r.standard_normal((n_in, 1)), r.standard_normal((n_out, 1))
    g = {k: np.zeros_like(v) for k, v in dict(DWe=We, DBe=Be, DV=V, DBo=Bo).items()}
    gW, gB = [np.zeros_like(w) for w in W], [np.zeros_like(b) for b in B]
    H = [np.zeros((nh, 1)) for _ in range(L)]
    leaves = {"We": lambda t, l: We, "Be": lambda t, l: Be, "W": lambda t, l: W[l], "B": lambda t, l: B[l], "V": lambda t, l: V,
              "Bo": lambda t, l: Bo, "Input": lambda t, l: x,
              "currentInput": lambda t, l: ("op", "embeddedInput_0_0" if l == 0 else f"h_act_0_{l - 1}"),
              "HFromLastLayer": lambda t, l: ("op", f"h_act_0_{L - 1}")}
    grads = {"DWe": lambda t, l: g["DWe"], "DBe": lambda t, l: g["DBe"], "DW": lambda t, l: gW[l], "DB": lambda t, l: gB[l],
             "DV": lambda t, l: g["DV"], "DBo": lambda t, l: g["DBo"]}
    it = A.OracleInterpreter(A.feedforward_architecture(), leaves, grads, L)
    it.forward()
    it.backward({"output_t_0_0": d_out})
    # by hand
    cur = O.add_forward(O.matmul_forward(We, x), Be)
    emb = cur
    pre, hs = [], []
    for l in range(L):
        z = O.add_forward(O.matmul_forward(W[l], cur), B[l])
        zt = O.transpose(z)
        ln, mu, sd = O.layernorm_forward(zt)
        cur = O.sigmoid_forward(O.transpose(ln))
        pre.append((zt, mu, sd))
        hs.append(cur)
    out = O.sigmoid_forward(O.add_forward(O.matmul_forward(V, cur), Bo))
    np.testing.assert_array_equal(it.by_id["output_t_0_0"]["out"], out)
    d = O.sigmoid_backward(out, d_out)
    np.testing.assert_array_equal(g["DBo"], d)
    dV_ref = O.matmul_backward(V, hs[-1], d)
    np.testing.assert_array_equal(g["DV"], dV_ref[0])
    d = dV_ref[1]
    for l in range(L - 1, -1, -1):
        d = O.sigmoid_backward(hs[l], d)
        d = O.transpose(O.layernorm_backward(pre[l][0], pre[l][1], pre[l][2], O.transpose(d)))
        np.testing.assert_array_equal(gB[l], d)
        dWl, d = O.matmul_backward(W[l], hs[l - 1] if l > 0 else emb, d)
        np.testing.assert_array_equal(gW[l], dWl)
    np.testing.assert_array_equal(g["DBe"], d)
