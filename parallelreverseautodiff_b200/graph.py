"""Graph mode over the C ABI: hand an operation DAG to ``prad_graph_*`` and run the
static-schedule forward / backward (the replacement of OperationNeuralNetworkVisitor).

The managed library keeps building the DAG from its JSON architecture
(ComputationGraph.ConstructFromArchitecture); this class is the thin host mirror used by the
tests: values are matrices, nodes are operations named like the reference's classes.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import engine as E
from ._lib import check

OPS = {
    "MatrixMultiplyOperation": 0, "MatrixAddOperation": 1, "MatrixAddThreeOperation": 2,
    "MatrixAddBroadcastingOperation": 3, "HadamardProductOperation": 4, "LeakyReLUOperation": 5,
    "SigmoidOperation": 6, "TanhOperation": 7, "GELUOperation": 8, "SoftmaxOperation": 9,
    "LayerNormalizationOperation": 10, "MatrixMultiplyScalarOperation": 11, "MatrixTransposeOperation": 12,
    "ReLUOperation": 13, "AmplifiedSigmoidOperation": 14, "SineSoftmaxOperation": 15,
}


class Graph:
    def __init__(self, eng: E.Engine, dtype):
        self.eng, self.dtype = eng, np.dtype(dtype)
        h = C.c_void_p()
        check(eng.lib.prad_graph_create(eng.ctx, E.dtype_code(dtype), C.byref(h)))
        self.h = h
        self.shapes = {}
        self._keep = []          # caller-owned matrices must outlive the graph

    def close(self):
        if self.h:
            check(self.eng.lib.prad_graph_destroy(self.h))
            self.h = None

    def value(self, rows: int, cols: int, data: Optional[E.DeviceMatrix] = None) -> int:
        out = C.c_int()
        check(self.eng.lib.prad_graph_add_value(self.h, rows, cols, C.c_void_p(data.ptr) if data else None, C.byref(out)))
        if data is not None:
            self._keep.append(data)
        self.shapes[out.value] = (rows, cols)
        return out.value

    def input(self, m: E.DeviceMatrix) -> int:
        return self.value(m.shape[0], m.shape[1], m)

    def weight(self, m: E.DeviceMatrix, grad: E.DeviceMatrix) -> int:
        v = self.input(m)
        check(self.eng.lib.prad_graph_set_gradient_destination(self.h, v, C.c_void_p(grad.ptr)))
        self._keep.append(grad)
        return v

    def node(self, op: str, inputs: Sequence[int], out_shape=None, scalar: float = 0.0) -> int:
        a = self.shapes[inputs[0]]
        if out_shape is None:
            if op == "MatrixMultiplyOperation":
                out_shape = (a[0], self.shapes[inputs[1]][1])
            elif op == "MatrixTransposeOperation":
                out_shape = (a[1], a[0])
            else:
                out_shape = a
        out = self.value(*out_shape)
        arr = (C.c_int * len(inputs))(*inputs)
        check(self.eng.lib.prad_graph_add_node(self.h, OPS[op], arr, len(inputs), out, scalar, None))
        return out

    def forward(self):
        check(self.eng.lib.prad_graph_forward(self.h))

    def backward(self, start: int, d_start: E.DeviceMatrix):
        check(self.eng.lib.prad_graph_backward(self.h, start, C.c_void_p(d_start.ptr)))

    def _matrix(self, fn, v) -> Optional[E.DeviceMatrix]:
        p = C.c_void_p()
        check(fn(self.h, v, C.byref(p)))
        if not p.value:
            return None
        return E.DeviceMatrix(self.eng, p.value, self.shapes[v], self.dtype, owned=False)

    def data(self, v: int):
        return self._matrix(self.eng.lib.prad_graph_value_data, v)

    def gradient(self, v: int):
        return self._matrix(self.eng.lib.prad_graph_value_gradient, v)

    def consumers(self, v: int) -> int:
        n = C.c_int()
        check(self.eng.lib.prad_graph_consumer_count(self.h, v, C.byref(n)))
        return n.value
