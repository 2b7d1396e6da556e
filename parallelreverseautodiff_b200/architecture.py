"""JSON architecture -> operation DAG on the device (host logic only; every operation is a node of
``prad_graph_*``).

This is the counterpart of the reference's ``ComputationGraph`` for callers that have no managed
runtime: the same registration calls and the same JSON schema, so an architecture file of the
reference loads unmodified.

    schema     JsonArchitecture { timeSteps: [ { startOperations, layers: [ { operations } ], endOperations } ] }
               OperationInfo { id, description, type, inputs, setResultTo, gradientResultTo }
               (src/RMAD/JsonArchitecture.cs, src/RMAD/OperationInfo.cs:11-46)
    unrolling  ConstructFromArchitecture(architecture, numLayers)                 src/RMAD/ComputationGraph.cs:219-256
               ConstructFromArchitecture(architecture, numTimeSteps, numLayers)   src/RMAD/ComputationGraph.cs:808-849
    ids        SpecificId = id + "_" + timeStep + "_" + layer                     src/RMAD/LayerInfo.cs:81-84
    inputs     resolved by name, the part before "[" only, in this order: an operation of the same
               (time step, layer), an operation finder, a weight, an intermediate, a scalar
               (DependenciesSetup, src/RMAD/ComputationGraph.cs:1330-1422)
    gradients  gradientResultTo[i] names the matrix that receives `+=` the gradient of input i
               (OperationBase.InitializeFrom :208-236, AccumulateGradient :273-304)
    results    setResultTo names the intermediate the operation's output is copied to after its
               Forward (NeuralNetwork.AutomaticForwardPropagate -> CopyResult)
    types      the JSON "type" is a class name of namespace ParallelReverseAutoDiff.RMAD
               (TypeRetrieved :1114-1117); Gpu* / Cuda* matrix products are the same node here
    batches    Batch* operations (src/RMAD/BatchOperation.cs:11-58) work on DeepMatrix values, one slice per
               sample: register such a matrix with a 3-D shape (depth, rows, cols).  A Matrix given where a
               Batch* operation has a (DeepMatrix, Matrix) overload is shared by the slices, and its
               gradient destination receives the mean over the slices (OperationNeuralNetworkVisitor
               .CombineResults :449-478)
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Union

import numpy as np

from . import engine as E
from ._lib import check
from .graph import OPS as _NODE_CODES


@dataclass(frozen=True)
class LayerInfo:
    """src/RMAD/LayerInfo.cs: the (time step, layer) an operation instance belongs to."""
    TimeStep: int = 0
    Layer: int = 0

    def __str__(self) -> str:
        return f"_{self.TimeStep}_{self.Layer}"


@dataclass
class OperationRef:
    """An operation instance of the graph: what ``graph["id_t_l"]`` returns to an operation finder."""
    SpecificId: str
    Id: str
    Type: str
    LayerInfo: LayerInfo
    value: int                    # graph value id of its output
    shape: tuple
    inputs: List[str]
    gradient_destinations: List[Optional[E.DeviceMatrix]]
    result_to: Optional[str] = None


# JSON type name -> node code.  The three spellings of the matrix product are one node, and every
# operation has its Batch* twin (the same node on DeepMatrix values).
def _canonical(type_name: str) -> str:
    name = type_name[5:] if type_name.startswith("Batch") else type_name
    return {"GpuMatrixMultiplyOperation": "MatrixMultiplyOperation",
            "CudaMatrixMultiplyOperation": "MatrixMultiplyOperation"}.get(name, name)


TYPE_CODES = dict(_NODE_CODES)
for _name in ("GpuMatrixMultiplyOperation", "CudaMatrixMultiplyOperation"):
    TYPE_CODES[_name] = TYPE_CODES["MatrixMultiplyOperation"]
for _name in list(TYPE_CODES):
    TYPE_CODES["Batch" + _name] = TYPE_CODES[_name]

_ARITY = {"MatrixMultiplyOperation": 2, "MatrixAddOperation": 2, "MatrixAddThreeOperation": 3,
          "MatrixAddBroadcastingOperation": 2, "HadamardProductOperation": 2, "MatrixMultiplyScalarOperation": 2}


class ArchitectureError(ValueError):
    """InvalidOperationException of the managed graph builder."""


class ArchitectureGraph:
    def __init__(self, eng: E.Engine, dtype, leaky_relu_alpha: float = 0.01):
        self.eng, self.dtype = eng, np.dtype(dtype)
        self.leaky_relu_alpha = leaky_relu_alpha          # NeuralNetworkParameters.LeakyReLUAlpha
        h = C.c_void_p()
        check(eng.lib.prad_graph_create(eng.ctx, E.dtype_code(dtype), C.byref(h)))
        self.h = h
        self._weights: Dict[str, Callable] = {}
        self._gradients: Dict[str, Callable] = {}
        self._intermediates: Dict[str, Callable] = {}
        self._scalars: Dict[str, Callable] = {}
        self._finders: Dict[str, Callable] = {}
        self.operations: Dict[str, OperationRef] = {}
        self.order: List[OperationRef] = []               # StartOperation, .Next, ...
        self._keep = []
        self._copies = []                                 # (operation, destination matrix) of setResultTo

    def close(self) -> None:
        if self.h:
            check(self.eng.lib.prad_graph_destroy(self.h))
            self.h = None

    # ------------------------------------------------------------ registration (fluent, as the reference)
    def AddWeight(self, name: str, fn: Callable[[LayerInfo], E.DeviceMatrix]) -> "ArchitectureGraph":
        self._weights[name] = fn
        return self

    def AddGradient(self, name: str, fn: Callable[[LayerInfo], E.DeviceMatrix]) -> "ArchitectureGraph":
        self._gradients[name] = fn
        return self

    def AddIntermediate(self, name: str, fn: Callable[[LayerInfo], E.DeviceMatrix]) -> "ArchitectureGraph":
        self._intermediates[name] = fn
        return self

    def AddScalar(self, name: str, fn: Callable[[LayerInfo], float]) -> "ArchitectureGraph":
        self._scalars[name] = fn
        return self

    def AddOperationFinder(self, name: str, fn: Callable[[LayerInfo], Union[OperationRef, E.DeviceMatrix]]):
        self._finders[name] = fn
        return self

    def __getitem__(self, specific_id: str) -> OperationRef:
        try:
            return self.operations[specific_id]
        except KeyError:
            raise ArchitectureError(f"The given key '{specific_id}' was not present in the dictionary.") from None

    # ------------------------------------------------------------ construction
    def ConstructFromArchitecture(self, architecture: dict, numLayers: int, numTimeSteps: Optional[int] = None):
        steps = architecture.get("timeSteps") or architecture.get("TimeSteps")
        if not steps:
            raise ArchitectureError("the architecture has no timeSteps")
        for t in range(1 if numTimeSteps is None else numTimeSteps):
            for ts in steps:
                for info in ts.get("startOperations") or []:
                    self._add_operation(info, LayerInfo(t, 0))
                for l in range(numLayers):
                    for layer in ts.get("layers") or []:
                        for info in layer.get("operations") or []:
                            self._add_operation(info, LayerInfo(t, l))
                for info in ts.get("endOperations") or []:
                    self._add_operation(info, LayerInfo(t, 0))
        return self

    def _leaf(self, m: E.DeviceMatrix, grad: Optional[E.DeviceMatrix]):
        """A caller-owned matrix as a graph value.  Every USE gets its own value, because a gradient
        destination belongs to (operation, input position), not to the matrix."""
        if len(m.shape) not in (2, 3):
            raise ArchitectureError("graph values are matrices (rows, cols) or deep matrices (depth, rows, cols)")
        v = C.c_int()
        if len(m.shape) == 3:
            check(self.eng.lib.prad_graph_add_deep_value(self.h, m.shape[0], m.shape[1], m.shape[2], C.c_void_p(m.ptr),
                                                         C.byref(v)))
        else:
            check(self.eng.lib.prad_graph_add_value(self.h, m.shape[0], m.shape[1], C.c_void_p(m.ptr), C.byref(v)))
        self._keep.append(m)
        if grad is not None:
            if tuple(grad.shape) != tuple(m.shape):
                raise ArchitectureError("a gradient destination has the shape of the matrix it belongs to")
            check(self.eng.lib.prad_graph_set_gradient_destination(self.h, v.value, C.c_void_p(grad.ptr)))
            self._keep.append(grad)
        return v.value, tuple(m.shape)

    def _add_operation(self, info: dict, li: LayerInfo) -> None:
        type_name = info["type"]
        if info["id"] + str(li) in self.operations:
            raise ArchitectureError(f"operation id '{info['id'] + str(li)}' occurs twice")
        if type_name not in TYPE_CODES:
            raise ArchitectureError(f"operation type '{type_name}' (operation '{info['id']}') is not available as a device node")
        canonical = _canonical(type_name)
        inputs = list(info["inputs"])
        arity = _ARITY.get(canonical, 1)
        if len(inputs) != arity:
            raise ArchitectureError(f"operation '{info['id']}' of type {type_name} takes {arity} inputs, the architecture lists {len(inputs)}")
        dests: List[Optional[E.DeviceMatrix]] = []
        for name in info.get("gradientResultTo") or []:
            if name is None:
                dests.append(None)
            else:
                key = name.split("[")[0]
                if key not in self._gradients:
                    raise ArchitectureError(f"gradient '{key}' of operation '{info['id']}' is not registered")
                dests.append(self._gradients[key](li))
        # AccumulateGradient throws when a destination sits beyond the operation's results
        n_results = arity if canonical != "MatrixMultiplyScalarOperation" else 1
        for pos, d in enumerate(dests):
            if d is not None and pos >= n_results:
                raise ArchitectureError(f"operation '{info['id']}': The output gradient must be non-null. "
                                        f"(gradientResultTo[{pos}] has no matching input gradient)")
        values, shapes, scalar = [], [], 0.0
        for j, name in enumerate(inputs):
            key = name.split("[")[0]
            dest = dests[j] if j < len(dests) else None
            same_level = key + str(li)
            if same_level in self.operations:
                ref = self.operations[same_level]
                values.append(ref.value)
                shapes.append(ref.shape)
                continue
            if key in self._finders:
                found = self._finders[key](li)
                if isinstance(found, OperationRef):
                    values.append(found.value)
                    shapes.append(found.shape)
                elif isinstance(found, E.DeviceMatrix):
                    v, shp = self._leaf(found, dest)
                    values.append(v)
                    shapes.append(shp)
                else:
                    raise ArchitectureError(f"operation finder '{key}' returned {type(found).__name__}")
                continue
            if key in self._weights or key in self._intermediates:
                m = (self._weights.get(key) or self._intermediates[key])(li)
                v, shp = self._leaf(m, dest)
                values.append(v)
                shapes.append(shp)
                continue
            if key in self._scalars:
                if canonical != "MatrixMultiplyScalarOperation" or j != 1:
                    raise ArchitectureError(f"scalar '{key}' can only be the second input of MatrixMultiplyScalarOperation")
                scalar = float(self._scalars[key](li))
                continue
            raise ArchitectureError(f"Input name {key} not found in value map")
        depth = max((s[0] for s in shapes if len(s) == 3), default=0)     # 0: plain matrices
        a = shapes[0][-2:]
        if canonical == "MatrixMultiplyOperation":
            out_shape = (a[0], shapes[1][-1])
        elif canonical == "MatrixTransposeOperation":
            out_shape = (a[1], a[0])
        else:
            out_shape = a
        if canonical == "LeakyReLUOperation":
            scalar = self.leaky_relu_alpha
        out = C.c_int()
        if depth:
            check(self.eng.lib.prad_graph_add_deep_value(self.h, depth, out_shape[0], out_shape[1], None, C.byref(out)))
            out_shape = (depth,) + tuple(out_shape)
        else:
            check(self.eng.lib.prad_graph_add_value(self.h, out_shape[0], out_shape[1], None, C.byref(out)))
        arr = (C.c_int * len(values))(*values)
        check(self.eng.lib.prad_graph_add_node(self.h, TYPE_CODES[type_name], arr, len(values), out.value, scalar, None))
        ref = OperationRef(info["id"] + str(li), info["id"], type_name, li, out.value, out_shape, inputs, dests,
                           info.get("setResultTo"))
        self.operations[ref.SpecificId] = ref
        self.order.append(ref)
        if ref.result_to:
            key = ref.result_to.split("[")[0]
            if key not in self._intermediates:
                raise ArchitectureError(f"intermediate '{key}' named by setResultTo of '{ref.Id}' is not registered")
            dst = self._intermediates[key](li)
            if tuple(dst.shape) != tuple(out_shape):
                raise ArchitectureError(f"setResultTo '{key}' of '{ref.Id}': shape {dst.shape} does not match {out_shape}")
            self._copies.append((ref, dst))

    # ------------------------------------------------------------ execution
    def forward(self) -> None:
        """Every operation's Forward in list order, then the setResultTo copies."""
        check(self.eng.lib.prad_graph_forward(self.h))
        for ref, dst in self._copies:
            self.eng.copy(dst, self.output(ref.SpecificId))

    def backward(self, starts: Union[str, Sequence[str]], gradients: Union[E.DeviceMatrix, Sequence[E.DeviceMatrix]]) -> None:
        """Backward from one operation (``BackwardInput = dLoss`` + visitor traversal) or from several at
        once (the per-time-step losses of an unrolled network, one walk instead of one per time step)."""
        if isinstance(starts, str):
            starts, gradients = [starts], [gradients]
        ids = (C.c_int * len(starts))(*[self[s].value for s in starts])
        ptrs = (C.c_void_p * len(starts))(*[g.ptr for g in gradients])
        check(self.eng.lib.prad_graph_backward_multi(self.h, ids, ptrs, len(starts)))

    def _matrix(self, fn, ref: OperationRef) -> Optional[E.DeviceMatrix]:
        p = C.c_void_p()
        check(fn(self.h, ref.value, C.byref(p)))
        return E.DeviceMatrix(self.eng, p.value, ref.shape, self.dtype, owned=False) if p.value else None

    def output(self, specific_id: str) -> E.DeviceMatrix:
        """GetOutput() of an operation."""
        return self._matrix(self.eng.lib.prad_graph_value_data, self[specific_id])

    def gradient(self, specific_id: str) -> Optional[E.DeviceMatrix]:
        """The upstream gradient the operation received in the last backward (None if not reached)."""
        return self._matrix(self.eng.lib.prad_graph_value_gradient, self[specific_id])

    def dependency_count(self, specific_id: str) -> int:
        """BackwardDependencyCounts of the last backward (OperationGraphVisitor.cs:124-162)."""
        n = C.c_int()
        check(self.eng.lib.prad_graph_consumer_count(self.h, self[specific_id].value, C.byref(n)))
        return n.value
