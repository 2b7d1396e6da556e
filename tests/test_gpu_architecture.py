"""The reference's architecture files loaded into graph mode (ArchitectureGraph -> prad_graph_*) and run
on the GPU, against the CPU interpreter of the same schema over the oracle's operations: the feed-forward
test network's file and the self-attention LSTM example's file (tests/architectures.py builds them and a
CPU test shows they equal the files)."""
import numpy as np
import pytest

import architectures as A
from parallelreverseautodiff_b200.architecture import ArchitectureError, ArchitectureGraph
from util import assert_close, rms, rng

pytestmark = pytest.mark.gpu


def _both(engine, arrays):
    """name -> (numpy copy for the interpreter, device matrix for the loader)"""
    return {k: (v.copy(), engine.upload(v)) for k, v in arrays.items()}


@pytest.mark.parametrize("dtype,cols", [(np.float64, 1), (np.float32, 1), (np.float64, 3)])
def test_feedforward_architecture_file(engine, dtype, cols):
    r = rng(5)
    n_in, nh, n_out, L = 10, 16, 4, 3
    mk = lambda *s: r.standard_normal(s).astype(dtype)
    P = _both(engine, dict(We=mk(nh, n_in) * 0.3, Be=mk(nh, cols) * 0.1, V=mk(n_out, nh) * 0.3, Bo=mk(n_out, cols) * 0.1,
                           Input=mk(n_in, cols)))
    Wl = [_both(engine, dict(W=mk(nh, nh) * 0.3, B=mk(nh, cols) * 0.1)) for _ in range(L)]
    G = _both(engine, dict(DWe=np.zeros((nh, n_in), dtype), DBe=np.zeros((nh, cols), dtype), DV=np.zeros((n_out, nh), dtype),
                           DBo=np.zeros((n_out, cols), dtype)))
    Gl = [_both(engine, dict(DW=np.zeros((nh, nh), dtype), DB=np.zeros((nh, cols), dtype))) for _ in range(L)]
    H = [engine.zeros((nh, cols), dtype) for _ in range(L)]
    out_dev = engine.zeros((n_out, cols), dtype)
    d_out = mk(n_out, cols)

    g = ArchitectureGraph(engine, dtype)
    for k in ("We", "Be", "V", "Bo"):
        g.AddWeight(k, lambda li, k=k: P[k][1])
    g.AddWeight("W", lambda li: Wl[li.Layer]["W"][1]).AddWeight("B", lambda li: Wl[li.Layer]["B"][1])
    for k in ("DWe", "DBe", "DV", "DBo"):
        g.AddGradient(k, lambda li, k=k: G[k][1])
    g.AddGradient("DW", lambda li: Gl[li.Layer]["DW"][1]).AddGradient("DB", lambda li: Gl[li.Layer]["DB"][1])
    g.AddIntermediate("Input", lambda li: P["Input"][1]).AddIntermediate("Output", lambda li: out_dev)
    g.AddIntermediate("H", lambda li: H[li.Layer])
    g.AddOperationFinder("HFromLastLayer", lambda li: g[f"h_act_0_{L - 1}"])
    g.AddOperationFinder("currentInput", lambda li: g["embeddedInput_0_0"] if li.Layer == 0 else g[f"h_act_0_{li.Layer - 1}"])
    g.ConstructFromArchitecture(A.feedforward_architecture(), L)
    assert [o.SpecificId for o in g.order][:3] == ["projectedInput_0_0", "embeddedInput_0_0", "w1_currentInput_0_0"]
    assert len(g.order) == 2 + 6 * L + 3

    leaves = {k: (lambda t, l, k=k: P[k][0]) for k in P}
    leaves.update(W=lambda t, l: Wl[l]["W"][0], B=lambda t, l: Wl[l]["B"][0],
                  currentInput=lambda t, l: ("op", "embeddedInput_0_0" if l == 0 else f"h_act_0_{l - 1}"),
                  HFromLastLayer=lambda t, l: ("op", f"h_act_0_{L - 1}"))
    grads = {k: (lambda t, l, k=k: G[k][0]) for k in G}
    grads.update(DW=lambda t, l: Gl[l]["DW"][0], DB=lambda t, l: Gl[l]["DB"][0])
    it = A.OracleInterpreter(A.feedforward_architecture(), leaves, grads, L)

    g.forward()
    it.forward()
    assert_close(g.output("output_t_0_0").numpy(), it.by_id["output_t_0_0"]["out"], 1.0, "ff architecture output")
    assert_close(out_dev.numpy(), it.by_id["output_t_0_0"]["out"], 1.0, "ff architecture setResultTo Output")
    for l in range(L):
        assert_close(H[l].numpy(), it.by_id[f"h_act_0_{l}"]["out"], 1.0, "ff architecture setResultTo H")
    g.backward("output_t_0_0", engine.upload(d_out))
    it.backward({"output_t_0_0": d_out})
    for k in G:
        assert_close(G[k][1].numpy(), G[k][0], 10 * rms(G[k][0]) + 1e-3, f"ff architecture {k}")
    for l in range(L):
        for k in ("DW", "DB"):
            assert_close(Gl[l][k][1].numpy(), Gl[l][k][0], 10 * rms(Gl[l][k][0]) + 1e-3, f"ff architecture {k}[{l}]")
    # BackwardDependencyCounts: a chain, every operation on the path has one consumer
    assert g.dependency_count("h_act_0_0") == 1 and g.dependency_count("embeddedInput_0_0") == 1
    g.close()


def test_destination_beyond_the_results_is_refused(engine):
    arch = A.feedforward_architecture("CudaMatrixMultiplyOperation")
    arch["timeSteps"][0]["layers"][0]["operations"][1]["gradientResultTo"] = [None, None, "DB[layerIndex]"]   # as the example's file
    z = engine.zeros((4, 4), np.float64)
    col = engine.zeros((4, 1), np.float64)
    g = ArchitectureGraph(engine, np.float64)
    for k in ("We", "W", "V"):
        g.AddWeight(k, lambda li: z)
    for k in ("Be", "B", "Bo"):
        g.AddWeight(k, lambda li: col)
    for k in ("DWe", "DW", "DV"):
        g.AddGradient(k, lambda li: z)
    for k in ("DBe", "DB", "DBo"):
        g.AddGradient(k, lambda li: col)
    g.AddIntermediate("Input", lambda li: col).AddIntermediate("Output", lambda li: col).AddIntermediate("H", lambda li: col)
    g.AddOperationFinder("currentInput", lambda li: g["embeddedInput_0_0"])
    g.AddOperationFinder("HFromLastLayer", lambda li: g["h_act_0_0"])
    with pytest.raises(ArchitectureError, match="output gradient must be non-null"):
        g.ConstructFromArchitecture(arch, 1)
    g.close()


@pytest.mark.parametrize("one_walk", [True, False], ids=["all time steps in one walk", "one walk per time step"])
def test_lstm_example_architecture_file(engine, one_walk):
    """SelfAttentionMultiLayerLSTM: T time steps x L layers unrolled by ConstructFromArchitecture(arch, T, L), with
    the registrations of examples/lstm/.../SelfAttentionMultiLayerLSTM.cs:295-328; shared weights accumulate
    over time steps; fan-out at h, c, the embedded input, the attention sources."""
    _lstm_architecture_case(engine, one_walk, depth=0)


def test_node_processing_architecture_file(engine):
    """test/.../GraphAttentionPaths/LSTM/Architecture/NodeProcessing.json: the same network on DeepMatrix values
    (one slice per sample) with Batch* operations, BatchGpuMatrixMultiplyOperation(Matrix, DeepMatrix) products
    whose weights are shared by the slices (their gradient is the mean over the slices), and
    BatchSineSoftmaxOperation attention weights."""
    _lstm_architecture_case(engine, True, depth=3)


def _lstm_architecture_case(engine, one_walk, depth):
    dtype = np.float64
    r = rng(8)
    T, L, n_in, nh, n_out, B = 3, 2, 6, 8, 5, 2
    batch = depth > 0
    mk = lambda *s: r.standard_normal(s) * 0.4
    deep = (lambda *s: mk(depth, *s)) if batch else mk          # per-sample values
    names_l = []
    for w in "fico":
        names_l += [f"W{w}", f"U{w}", f"b{w}"]
    names_l += ["Wq", "Wk", "Wv"]

    def shape_of(name, l):
        return (nh, B) if name.startswith("b") else (nh, nh)

    layer_p = [_both(engine, {n: mk(*shape_of(n, l)) for n in names_l}) for l in range(L)]
    layer_g = [_both(engine, {"d" + n: np.zeros(shape_of(n, l)) for n in names_l}) for l in range(L)]
    glob_p = _both(engine, dict(We=mk(nh, n_in), be=mk(nh, B), V=mk(n_out, nh), b=mk(n_out, B)))
    glob_g = _both(engine, dict(dWe=np.zeros((nh, n_in)), dbe=np.zeros((nh, B)), dV=np.zeros((n_out, nh)), db=np.zeros((n_out, B))))
    xs = [deep(n_in, B) for _ in range(T)]
    xs_dev = [engine.upload(x) for x in xs]
    lead = (depth,) if batch else ()
    zero_h = engine.zeros(lead + (nh, B), dtype)
    zero_np = np.zeros(lead + (nh, B))
    out_dev = [engine.zeros(lead + (n_out, B), dtype) for _ in range(T)]
    c_dev = [[engine.zeros((nh, B), dtype) for _ in range(L)] for _ in range(T)]
    h_dev = [[engine.zeros((nh, B), dtype) for _ in range(L)] for _ in range(T)]
    scalar = 1.0 / np.sqrt(nh)
    in_name, out_name = ("InputNodeFeatures", "OutputPathFeatures") if batch else ("inputSequence", "output")
    arch = A.lstm_architecture(batch=batch)

    g = ArchitectureGraph(engine, dtype, leaky_relu_alpha=0.01)
    g.AddIntermediate(in_name, lambda x: xs_dev[x.TimeStep]).AddIntermediate(out_name, lambda x: out_dev[x.TimeStep])
    g.AddIntermediate("c", lambda x: c_dev[x.TimeStep][x.Layer]).AddIntermediate("h", lambda x: h_dev[x.TimeStep][x.Layer])
    g.AddScalar("scaledDotProductScalar", lambda x: scalar)
    for n in names_l:
        g.AddWeight(n, lambda x, n=n: layer_p[x.Layer][n][1]).AddGradient("d" + n, lambda x, n=n: layer_g[x.Layer]["d" + n][1])
    for n in glob_p:
        g.AddWeight(n, lambda x, n=n: glob_p[n][1]).AddGradient("d" + n, lambda x, n=n: glob_g["d" + n][1])
    for n in ("i", "f", "cHat", "o"):
        g.AddOperationFinder(n, lambda x, n=n: g[f"{n}_{x.TimeStep}_{x.Layer}"])
    g.AddOperationFinder("embeddedInput", lambda x: g[f"embeddedInput_{x.TimeStep}_0"])
    g.AddOperationFinder("hFromCurrentTimeStepAndLastLayer", lambda x: g[f"h_{x.TimeStep}_{L - 1}"])
    g.AddOperationFinder("currentInput", lambda x: g[f"embeddedInput_{x.TimeStep}_0"] if x.Layer == 0 else g[f"h_{x.TimeStep}_{x.Layer - 1}"])
    g.AddOperationFinder("previousHiddenState", lambda x: zero_h if x.TimeStep == 0 else g[f"h_{x.TimeStep - 1}_{x.Layer}"])
    g.AddOperationFinder("previousMemoryCellState", lambda x: zero_h if x.TimeStep == 0 else g[f"c_{x.TimeStep - 1}_{x.Layer}"])
    g.ConstructFromArchitecture(arch, L, T)
    assert len(g.order) == T * (2 + 46 * L + 3)

    leaves = {n: (lambda t, l, n=n: layer_p[l][n][0]) for n in names_l}
    leaves.update({n: (lambda t, l, n=n: glob_p[n][0]) for n in glob_p})
    leaves.update({in_name: lambda t, l: xs[t]}, scaledDotProductScalar=lambda t, l: scalar,
                  embeddedInput=lambda t, l: ("op", f"embeddedInput_{t}_0"),
                  hFromCurrentTimeStepAndLastLayer=lambda t, l: ("op", f"h_{t}_{L - 1}"),
                  currentInput=lambda t, l: ("op", f"embeddedInput_{t}_0" if l == 0 else f"h_{t}_{l - 1}"),
                  previousHiddenState=lambda t, l: zero_np if t == 0 else ("op", f"h_{t - 1}_{l}"),
                  previousMemoryCellState=lambda t, l: zero_np if t == 0 else ("op", f"c_{t - 1}_{l}"))
    for n in ("i", "f", "cHat", "o"):
        leaves[n] = lambda t, l, n=n: ("op", f"{n}_{t}_{l}")
    grads = {"d" + n: (lambda t, l, n=n: layer_g[l]["d" + n][0]) for n in names_l}
    grads.update({"d" + n: (lambda t, l, n=n: glob_g["d" + n][0]) for n in glob_p})
    it = A.OracleInterpreter(arch, leaves, grads, L, T)

    g.forward()
    it.forward()
    what = "node processing" if batch else "lstm architecture"
    for t in range(T):
        ref = it.by_id[f"output_t_{t}_0"]["out"]
        assert_close(out_dev[t].numpy(), ref, 1.0, f"{what} output[t]")
        for l in range(L):
            got = g.output(f"h_{t}_{l}") if batch else h_dev[t][l]       # the batch file copies neither c nor h out
            assert_close(got.numpy(), it.by_id[f"h_{t}_{l}"]["out"], 10.0, f"{what} h[t][l]")
    ups = [deep(n_out, B) for _ in range(T)]
    starts = [f"output_t_{t}_0" for t in range(T)]
    if one_walk:
        g.backward(starts, [engine.upload(u) for u in ups])
    else:
        for t in range(T - 1, -1, -1):            # the managed code: one visitor per time step, last step first
            g.backward(starts[t], engine.upload(ups[t]))
    it.backward(dict(zip(starts, ups)))
    for l in range(L):
        for n in names_l:
            ref = layer_g[l]["d" + n][0]
            assert_close(layer_g[l]["d" + n][1].numpy(), ref, 20 * rms(ref) + 1e-6, f"{what} d{n}[{l}]")
    for n in glob_p:
        ref = glob_g["d" + n][0]
        assert_close(glob_g["d" + n][1].numpy(), ref, 20 * rms(ref) + 1e-6, f"{what} d{n}")
    if one_walk:
        # h of a time step feeds the four gates and the attention queries of the next, the layer above and the output
        assert g.dependency_count("h_0_0") >= 5 and g.dependency_count("embeddedInput_0_0") >= 3
    g.close()


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_batch_operations_on_deep_matrices(engine, dtype):
    """Batch* operations (one slice per sample) with weights and biases shared by the samples: the shared
    matrices receive the mean over the samples; deep values fan out (z, embeddedInput, hLast)."""
    r = rng(21)
    B, n_in, nh, n_out, L = 6, 9, 12, 4, 2
    mk = lambda *s: (r.standard_normal(s) * 0.5).astype(dtype)
    glob = _both(engine, dict(We=mk(nh, n_in), be=mk(nh, 1), V=mk(n_out, nh), bo=mk(n_out, 1)))
    lay = [_both(engine, dict(W=mk(nh, nh), U=mk(nh, nh), b=mk(nh, 1))) for _ in range(L)]
    gg = _both(engine, {"d" + k: np.zeros_like(v[0]) for k, v in glob.items()})
    gl = [_both(engine, {"d" + k: np.zeros_like(v[0]) for k, v in lay[l].items()}) for l in range(L)]
    x = mk(B, n_in, 1)
    x_dev = engine.upload(x)
    H = [engine.zeros((B, nh, 1), dtype) for _ in range(L)]
    out_dev = engine.zeros((B, n_out, 1), dtype)
    scale = 1.0 / np.sqrt(nh)

    g = ArchitectureGraph(engine, dtype)
    for k in glob:
        g.AddWeight(k, lambda li, k=k: glob[k][1]).AddGradient("d" + k, lambda li, k=k: gg["d" + k][1])
    for k in ("W", "U", "b"):
        g.AddWeight(k, lambda li, k=k: lay[li.Layer][k][1]).AddGradient("d" + k, lambda li, k=k: gl[li.Layer]["d" + k][1])
    g.AddIntermediate("Input", lambda li: x_dev).AddIntermediate("Output", lambda li: out_dev)
    g.AddIntermediate("H", lambda li: H[li.Layer]).AddScalar("scale", lambda li: scale)
    g.AddOperationFinder("currentInput", lambda li: g["embeddedInput_0_0"] if li.Layer == 0 else g[f"h_0_{li.Layer - 1}"])
    g.AddOperationFinder("embeddedInput", lambda li: g["embeddedInput_0_0"])
    g.AddOperationFinder("hLast", lambda li: g[f"h_0_{L - 1}"])
    g.ConstructFromArchitecture(A.batch_network_architecture(), L)

    leaves = {k: (lambda t, l, k=k: glob[k][0]) for k in glob}
    leaves.update({k: (lambda t, l, k=k: lay[l][k][0]) for k in ("W", "U", "b")})
    leaves.update(Input=lambda t, l: x, scale=lambda t, l: scale,
                  currentInput=lambda t, l: ("op", "embeddedInput_0_0" if l == 0 else f"h_0_{l - 1}"),
                  embeddedInput=lambda t, l: ("op", "embeddedInput_0_0"), hLast=lambda t, l: ("op", f"h_0_{L - 1}"))
    grads = {"d" + k: (lambda t, l, k=k: gg["d" + k][0]) for k in glob}
    grads.update({"d" + k: (lambda t, l, k=k: gl[l]["d" + k][0]) for k in ("W", "U", "b")})
    it = A.OracleInterpreter(A.batch_network_architecture(), leaves, grads, L)

    g.forward()
    it.forward()
    assert_close(out_dev.numpy(), it.by_id["output_0_0"]["out"], 10.0, "batch architecture Output")
    for l in range(L):
        assert_close(H[l].numpy(), it.by_id[f"h_0_{l}"]["out"], 10.0, "batch architecture H")
    up = mk(B, n_out, 1)
    g.backward("output_0_0", engine.upload(up))
    it.backward({"output_0_0": up})
    for k in gg:
        assert_close(gg[k][1].numpy(), gg[k][0], 10 * rms(gg[k][0]) + 1e-3, f"batch architecture {k}")
    for l in range(L):
        for k in gl[l]:
            assert_close(gl[l][k][1].numpy(), gl[l][k][0], 10 * rms(gl[l][k][0]) + 1e-3, f"batch architecture {k}[{l}]")
    assert g.dependency_count("embeddedInput_0_0") == 1 + L      # the first layer's input and every layer's u_x
    g.close()
