"""Architectures in the reference's JSON schema, built by code, plus a CPU interpreter of the schema
over the oracle's operations.

`feedforward_architecture()` and `lstm_architecture()` spell out, operation by operation, the graphs of
the reference's feed-forward test network and of its self-attention LSTM example.  A CPU test compares
them with the reference's own JSON files wherever the reference tree is present (descriptions aside,
they are identical), so loading these dictionaries is loading those files; GPU tests cannot read the
reference tree.

`OracleInterpreter` runs such an architecture on numpy arrays with the oracle's operations: forward in
list order, backward with the visitor's semantics (each operation's Backward once, the gradients of an
operation with several consumers summed in consumer registration order, `destination += gradient`).
It shares no code with the device-side loader.
"""
import numpy as np

import oracle as O


def _op(id_, type_, inputs, grads=None, result=None):
    d = {"id": id_, "type": type_, "inputs": list(inputs)}
    if grads is not None:
        d["gradientResultTo"] = list(grads)
    if result is not None:
        d["setResultTo"] = result
    return d


def feedforward_architecture(matmul="GpuMatrixMultiplyOperation"):
    """test/ParallelReverseAutoDiff.Test/FeedForward/Architecture/FeedForwardArchitecture.json"""
    start = [_op("projectedInput", matmul, ["We", "Input"], ["DWe", None]),
             _op("embeddedInput", "MatrixAddOperation", ["projectedInput", "Be"], [None, "DBe"])]
    layer = [_op("w1_currentInput", matmul, ["W[layerIndex]", "currentInput"], ["DW[layerIndex]", None]),
             _op("h_add", "MatrixAddOperation", ["w1_currentInput", "B[layerIndex]"], [None, "DB[layerIndex]"]),
             _op("intermediate_h_1", "MatrixTransposeOperation", ["h_add"]),
             _op("intermediate_h_2", "LayerNormalizationOperation", ["intermediate_h_1"]),
             _op("intermediate_h_3", "MatrixTransposeOperation", ["intermediate_h_2"]),
             _op("h_act", "SigmoidOperation", ["intermediate_h_3"], result="H[layerIndex]")]
    end = [_op("v_h", matmul, ["V", "HFromLastLayer"], ["DV", None]),
           _op("v_h_b", "MatrixAddOperation", ["v_h", "Bo"], [None, "DBo"]),
           _op("output_t", "SigmoidOperation", ["v_h_b"], result="Output")]
    return {"timeSteps": [{"startOperations": start, "layers": [{"operations": layer}], "endOperations": end}]}


def lstm_architecture(batch=False):
    """examples/lstm/ParallelReverseAutoDiff.LstmExample/architecture/SelfAttentionMultiLayerLSTMArchitectureAmplified.json,
    or with batch=True its DeepMatrix twin
    test/ParallelReverseAutoDiff.Test/GraphAttentionPaths/LSTM/Architecture/NodeProcessing.json: every operation
    is the Batch* one, the products are BatchGpuMatrixMultiplyOperation, the attention weights come from
    BatchSineSoftmaxOperation, c and h are not copied out, and the output is a LeakyReLU."""
    pre = "Batch" if batch else ""
    mm = "BatchGpuMatrixMultiplyOperation" if batch else "MatrixMultiplyOperation"
    tr, ln = pre + "MatrixTransposeOperation", pre + "LayerNormalizationOperation"
    add, add3, had = pre + "MatrixAddOperation", pre + "MatrixAddThreeOperation", pre + "HadamardProductOperation"
    start = [_op("projectedInput", mm, ["We", "InputNodeFeatures[t]" if batch else "inputSequence[t]"], ["dWe", None]),
             _op("embeddedInput", add, ["projectedInput", "be"], [None, "dbe"])]
    ops = []

    def gate(name, w, act, normalized=True):
        ops.append(_op(f"w{w}_currentInput", mm, [f"W{w}[layerIndex]", "currentInput"], [f"dW{w}[layerIndex]", None]))
        ops.append(_op(f"u{w}_previousHiddenState", mm, [f"U{w}[layerIndex]", "previousHiddenState"], [f"dU{w}[layerIndex]", None]))
        ops.append(_op(f"{name}_add", add3,
                       [f"w{w}_currentInput", f"u{w}_previousHiddenState", f"b{w}[layerIndex]"], [None, None, f"db{w}[layerIndex]"]))
        last = f"{name}_add"
        if normalized:
            ops.append(_op(f"intermediate_{name}_1", tr, [f"{name}_add"]))
            ops.append(_op(f"intermediate_{name}_2", ln, [f"intermediate_{name}_1"]))
            ops.append(_op(f"intermediate_{name}_3", tr, [f"intermediate_{name}_2"]))
            last = f"intermediate_{name}_3"
        ops.append(_op(name, pre + act, [last]))

    gate("f", "f", "AmplifiedSigmoidOperation")
    gate("i", "i", "AmplifiedSigmoidOperation")
    gate("cHat", "c", "TanhOperation")
    ops += [_op("f_previousMemoryCellState", had, ["f[t][layerIndex]", "previousMemoryCellState"]),
            _op("i_cHat", had, ["i[t][layerIndex]", "cHat[t][layerIndex]"]),
            _op("newC", add, ["f_previousMemoryCellState", "i_cHat"]),
            _op("newCTransposed", tr, ["newC"]),
            _op("newCNormalized", ln, ["newCTransposed"]),
            _op("c", tr, ["newCNormalized"], result=None if batch else "c[t][layerIndex]")]
    gate("o", "o", "LeakyReLUOperation", normalized=False)
    ops += [_op("c_tanh", pre + "TanhOperation", ["c"]),
            _op("newH", had, ["o[t][layerIndex]", "c_tanh"]),
            _op("keys", mm, ["Wk[layerIndex]", "embeddedInput"], ["dWk[layerIndex]", None]),
            _op("queries", mm, ["Wq[layerIndex]", "previousHiddenState"], ["dWq[layerIndex]", None]),
            _op("values", mm, ["Wv[layerIndex]", "embeddedInput"], ["dWv[layerIndex]", None]),
            _op("queriesTranspose", tr, ["queries"]),
            _op("dotProduct", mm, ["keys", "queriesTranspose"]),
            _op("scaledDotProduct", pre + "MatrixMultiplyScalarOperation", ["dotProduct", "scaledDotProductScalar"]),
            _op("scaledDotProductTranspose", tr, ["scaledDotProduct"]),
            _op("attentionWeights", "BatchSineSoftmaxOperation" if batch else "SoftmaxOperation", ["scaledDotProductTranspose"]),
            _op("attentionOutput", mm, ["attentionWeights", "values"]),
            _op("newHWithAttentionOutput", add, ["newH", "attentionOutput"]),
            _op("newHWithAttentionOutputTranspose", tr, ["newHWithAttentionOutput"]),
            _op("normalizedNewH", ln, ["newHWithAttentionOutputTranspose"]),
            _op("h", tr, ["normalizedNewH"], result=None if batch else "h[t][layerIndex]")]
    end = [_op("v_h", mm, ["V", "hFromCurrentTimeStepAndLastLayer"], ["dV", None]),
           _op("v_h_b", add, ["v_h", "b"], [None, "db"]),
           _op("output_t", "BatchLeakyReLUOperation" if batch else "AmplifiedSigmoidOperation", ["v_h_b"],
               result="OutputPathFeatures[t]" if batch else "output[t]")]
    return {"timeSteps": [{"startOperations": start, "layers": [{"operations": ops}], "endOperations": end}]}


def strip_descriptions(arch):
    """The same architecture without the free-text "description" entries."""
    if isinstance(arch, dict):
        return {k: strip_descriptions(v) for k, v in arch.items() if k != "description"}
    if isinstance(arch, list):
        return [strip_descriptions(v) for v in arch]
    return arch


# ------------------------------------------------------------------------------------------------
class OracleInterpreter:
    """numpy / oracle execution of an architecture.  `leaves` maps a name (the part before "[") to a function
    (time step, layer) -> numpy array, float, or ("op", specific id) for an operation finder."""

    def __init__(self, arch, leaves, grads, num_layers, num_time_steps=None, alpha=0.01):
        self.leaves, self.grads, self.alpha = leaves, grads, alpha
        self.nodes, self.by_id = [], {}
        for t in range(1 if num_time_steps is None else num_time_steps):
            for ts in arch["timeSteps"]:
                for info in ts.get("startOperations") or []:
                    self._add(info, t, 0)
                for l in range(num_layers):
                    for layer in ts["layers"]:
                        for info in layer["operations"]:
                            self._add(info, t, l)
                for info in ts.get("endOperations") or []:
                    self._add(info, t, 0)

    def _add(self, info, t, l):
        sid = f"{info['id']}_{t}_{l}"
        ins = []
        for name in info["inputs"]:
            key = name.split("[")[0]
            same = f"{key}_{t}_{l}"
            if same in self.by_id:
                ins.append(("op", same))
                continue
            found = self.leaves[key](t, l)
            ins.append(found if isinstance(found, tuple) else ("leaf", found))
        dests = [None if g is None else self.grads[g.split("[")[0]](t, l) for g in info.get("gradientResultTo") or []]
        node = dict(id=sid, type=info["type"].replace("Gpu", "").replace("Cuda", ""), ins=ins, dests=dests, out=None)
        self.by_id[sid] = node
        self.nodes.append(node)

    def _val(self, ref):
        return self.by_id[ref[1]]["out"] if ref[0] == "op" else ref[1]

    def _fwd_one(self, t, x, n, slot):
        """One Forward on matrices; `slot` keeps what the Backward of that slice needs."""
        if t == "MatrixMultiplyOperation": return O.matmul_forward(x[0], x[1])
        if t == "MatrixAddOperation": return O.add_forward(x[0], x[1])
        if t == "MatrixAddThreeOperation": return O.add3_forward(x[0], x[1], x[2])
        if t == "MatrixTransposeOperation": return O.transpose(x[0])
        if t == "LayerNormalizationOperation":
            y, slot["mean"], slot["std"] = O.layernorm_forward(x[0])
            return y
        if t == "SigmoidOperation": return O.sigmoid_forward(x[0])
        if t == "TanhOperation": return O.tanh_forward(x[0])
        if t == "AmplifiedSigmoidOperation": return O.amplified_sigmoid_forward(x[0])
        if t == "LeakyReLUOperation": return O.leaky_relu_forward(x[0], self.alpha)
        if t == "HadamardProductOperation": return O.hadamard_forward(x[0], x[1])
        if t == "MatrixMultiplyScalarOperation": return O.scale(x[0], x[1])
        if t == "SoftmaxOperation": return O.softmax_forward(x[0])
        if t == "SineSoftmaxOperation": return O.sine_softmax_forward(x[0])
        raise KeyError(t)

    def _bwd_one(self, t, x, y, d, slot):
        if t == "MatrixMultiplyOperation": return list(O.matmul_backward(x[0], x[1], d))
        if t == "MatrixAddOperation": return [d, d]
        if t == "MatrixAddThreeOperation": return [d, d, d]
        if t == "MatrixTransposeOperation": return [O.transpose(d)]
        if t == "LayerNormalizationOperation": return [O.layernorm_backward(x[0], slot["mean"], slot["std"], d)]
        if t == "SigmoidOperation": return [O.sigmoid_backward(y, d)]
        if t == "TanhOperation": return [O.tanh_backward(y, d)]
        if t == "AmplifiedSigmoidOperation": return [O.amplified_sigmoid_backward(x[0], d)]
        if t == "LeakyReLUOperation": return [O.leaky_relu_backward(x[0], d, self.alpha)]
        if t == "HadamardProductOperation": return list(O.hadamard_backward(x[0], x[1], d))
        if t == "MatrixMultiplyScalarOperation": return [O.scale(d, x[1])]
        if t == "SoftmaxOperation": return [O.softmax_backward(y, d)]
        if t == "SineSoftmaxOperation": return [O.sine_softmax_backward(x[0], d)]
        raise KeyError(t)

    @staticmethod
    def _slice(v, k):
        return v[k] if isinstance(v, np.ndarray) and v.ndim == 3 else v

    def forward(self):
        for n in self.nodes:
            x = [self._val(r) for r in n["ins"]]
            t = n["type"]
            if t.startswith("Batch"):      # BatchOperation: one operation object per slice
                depth = max(v.shape[0] for v in x if isinstance(v, np.ndarray) and v.ndim == 3)
                n["slots"] = [dict() for _ in range(depth)]
                n["out"] = np.stack([self._fwd_one(t[5:], [self._slice(v, k) for v in x], n, n["slots"][k])
                                     for k in range(depth)])
            else:
                n["slots"] = [dict()]
                n["out"] = self._fwd_one(t, x, n, n["slots"][0])

    def backward(self, starts):
        """starts: {specific id: upstream gradient}.  One reverse walk; contributions of the consumers of an
        operation are summed in the order the consumers were added.  A Batch* operation runs its slices'
        Backward one by one; a Matrix shared by the slices receives the visitor's combined gradient, the
        left-fold sum of the slices' gradients times 1 / depth."""
        order = {n["id"]: k for k, n in enumerate(self.nodes)}
        contrib = {n["id"]: [] for n in self.nodes}           # (consumer index, gradient)
        for sid, g in starts.items():
            contrib[sid].append((-1, g))
        for n in reversed(self.nodes):
            cs = sorted(contrib[n["id"]], key=lambda kv: kv[0])
            if not cs:
                continue
            d = cs[0][1] if len(cs) == 1 else O.accumulate_gradients([g for _, g in cs])
            n["grad"] = d
            x = [self._val(r) for r in n["ins"]]
            t = n["type"]
            if t.startswith("Batch"):
                depth = n["out"].shape[0]
                per = [self._bwd_one(t[5:], [self._slice(v, k) for v in x], n["out"][k], d[k], n["slots"][k]) for k in range(depth)]
                gs = []
                for j, v in enumerate(x):
                    if j >= len(per[0]):
                        break
                    if isinstance(v, np.ndarray) and v.ndim == 3:
                        gs.append(np.stack([per[k][j] for k in range(depth)]))
                    else:
                        gs.append(O.batch_mean([np.ascontiguousarray(per[k][j]) for k in range(depth)]))
            else:
                gs = self._bwd_one(t, x, n["out"], d, n["slots"][0])
            for j, g in enumerate(gs):
                if j < len(n["dests"]) and n["dests"][j] is not None:
                    O.accumulate_into(n["dests"][j], g)
                if n["ins"][j][0] == "op":
                    contrib[n["ins"][j][1]].append((order[n["id"]], g))


def batch_network_architecture():
    """A small network in the spelling of test/.../GraphAttentionPaths/*/Architecture/*.json: Batch* operations
    over per-sample column vectors held in DeepMatrix values, weights and biases shared by the samples."""
    bmm = "BatchGpuMatrixMultiplyOperation"
    start = [_op("projectedInput", bmm, ["We", "Input"], ["dWe", None]),
             _op("embeddedInput", "BatchMatrixAddOperation", ["projectedInput", "be"], [None, "dbe"])]
    layer = [_op("w_x", bmm, ["W[layerIndex]", "currentInput"], ["dW[layerIndex]", None]),
             _op("u_x", bmm, ["U[layerIndex]", "embeddedInput"], ["dU[layerIndex]", None]),
             _op("z", "BatchMatrixAddThreeOperation", ["w_x", "u_x", "b[layerIndex]"], [None, None, "db[layerIndex]"]),
             _op("zT", "BatchMatrixTransposeOperation", ["z"]),
             _op("zN", "BatchLayerNormalizationOperation", ["zT"]),
             _op("zNT", "BatchMatrixTransposeOperation", ["zN"]),
             _op("gate", "BatchAmplifiedSigmoidOperation", ["zNT"]),
             _op("cand", "BatchTanhOperation", ["z"]),
             _op("mix", "BatchHadamardProductOperation", ["gate", "cand"]),
             _op("h", "BatchLeakyReLUOperation", ["mix"], result="H[layerIndex]")]
    end = [_op("hT", "BatchMatrixTransposeOperation", ["hLast"]),
           _op("outer", "BatchMatrixMultiplyOperation", ["hLast", "hT"]),
           _op("scaled", "BatchMatrixMultiplyScalarOperation", ["outer", "scale"]),
           _op("attn", "BatchSoftmaxOperation", ["scaled"]),
           _op("mixed", "BatchMatrixMultiplyOperation", ["attn", "hLast"]),
           _op("v_h", bmm, ["V", "mixed"], ["dV", None]),
           _op("output", "BatchMatrixAddOperation", ["v_h", "bo"], [None, "dbo"], result="Output")]
    return {"timeSteps": [{"startOperations": start, "layers": [{"operations": layer}], "endOperations": end}]}
