"""Feed-forward network driver over the C ABI (host logic only; all arithmetic is in
libprad_cuda).

It plays the part of the reference's hand-written network classes
(examples/feedforward/.../FeedForwardNeuralNetwork.cs; AutomaticForwardPropagate :208-247,
AutomaticBackwardPropagate :249-299, then ``clipper.Clip(layers)`` and
``optimizer.Optimize(layers)``) for the graph spelling that keeps the whole batch in one
matrix: ``Z_l = A_{l-1} W_l (+ bias_l)``, ``A_l = act(Z_l)``; weight and bias gradients are
sums over the batch rows (MatrixMultiplyOperation.Backward, MatrixAddBroadcastingOperation
.Backward), which is also what makes batch sharding over GPUs exact up to summation order:
every rank holds a contiguous block of rows and the weight gradients are all-reduced (SUM).

Backward schedule per layer, last to first:
    dW_l = A_{l-1}^T dZ_l          -> all-reduce of dW_l starts on the communication stream
    db_l = column sums of dZ_l     -> all-reduce likewise
    dZ_{l-1} = (dZ_l W_l^T) (.) act'(saved_{l-1})   (derivative fused into the GEMM epilogue)
so a layer's collective overlaps with the GEMMs of the layers below it.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import numpy as np

from . import engine as E


class NeuralNetworkParameters:
    """Property bag of src/RMAD/NeuralNetworkParameters.cs:13-119 (lite defaults in float)."""

    def __init__(self, dtype=np.float32):
        lite = np.dtype(dtype) == np.float32
        self.LeakyReLUAlpha = 0.01
        self.LearningRate = 0.001
        self.AdamIteration = 1.0
        self.AdamBeta1 = 0.9
        self.AdamBeta2 = 0.999
        self.AdamEpsilon = 1e-8
        self.ClipValue = 4.0
        self.MinimumClipValue = 1e-8 if lite else 1e-16


_SAVES_OUTPUT = {E.ACT_SIGMOID, E.ACT_TANH}


def row_shard(total_rows: int, rank: int, world: int):
    """Contiguous block of batch rows owned by `rank`: the first `total % world` ranks get one
    extra row.  Returns (start, stop)."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(total_rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


class FeedForwardNetwork:
    def __init__(self, eng: E.Engine, dtype, sizes: Sequence[int], hidden_act=E.ACT_LEAKY_RELU,
                 output_act=E.ACT_NONE, softmax_output=False, loss="mse", use_bias=True,
                 clip_mode=E.CLIP_REFERENCE, rank=0, world=1):
        self.eng = eng
        self.dtype = np.dtype(dtype)
        self.sizes = list(sizes)
        self.L = len(sizes) - 1
        self.acts = [hidden_act] * (self.L - 1) + [output_act]
        self.softmax_output = softmax_output
        self.loss = loss
        self.use_bias = use_bias
        self.clip_mode = clip_mode
        self.rank, self.world = rank, world
        self.Parameters = NeuralNetworkParameters(dtype)
        self.W: List[E.DeviceMatrix] = []
        self.b: List[E.DeviceMatrix] = []
        for l in range(self.L):
            self.W.append(eng.zeros((sizes[l], sizes[l + 1]), dtype))
            if use_bias:
                self.b.append(eng.zeros((1, sizes[l + 1]), dtype))
        params = self.W + self.b
        self.params = params
        self.grads = [eng.zeros(p.shape, dtype) for p in params]
        self.m = [eng.zeros(p.shape, dtype) for p in params]
        self.v = [eng.zeros(p.shape, dtype) for p in params]
        self.dW = self.grads[: self.L]
        self.db = self.grads[self.L:]
        self.rows = 0
        self.A: List[Optional[E.DeviceMatrix]] = []
        self.Z: List[Optional[E.DeviceMatrix]] = []
        self.probs = None
        self.dZ = [None, None]
        self.dX = None
        self.loss_dev = eng.zeros((1, 1), dtype)

    # ---------------------------------------------------------------- set-up
    def set_weights(self, weights: Sequence[np.ndarray], biases: Optional[Sequence[np.ndarray]] = None):
        for l, w in enumerate(weights):
            self.eng.upload(np.ascontiguousarray(w, self.dtype), out=self.W[l])
        if biases is not None:
            for l, b in enumerate(biases):
                self.eng.upload(np.ascontiguousarray(b, self.dtype).reshape(1, -1), out=self.b[l])

    def _ensure_buffers(self, rows: int) -> None:
        if rows == self.rows:
            return
        e, dt = self.eng, self.dtype
        self.rows = rows
        self.A = [e.empty((rows, self.sizes[0]), dt)] + [e.empty((rows, n), dt) for n in self.sizes[1:]]
        self.Z = [None] + [e.empty((rows, n), dt) if self.acts[l] != E.ACT_NONE else None
                           for l, n in enumerate(self.sizes[1:])]
        widest = max(self.sizes)
        self.dZ = [e.empty((rows * widest,), dt), e.empty((rows * widest,), dt)]
        self.target = e.empty((rows, self.sizes[-1]), dt)
        if self.softmax_output:
            self.probs = e.empty((rows, self.sizes[-1]), dt)

    # ---------------------------------------------------------------- forward
    def forward(self, x: Optional[E.DeviceMatrix] = None) -> E.DeviceMatrix:
        """Forward through every layer; keeps Z_l (pre-activation) and A_l for the backward."""
        e = self.eng
        if x is not None:
            self._ensure_buffers(x.shape[0])
            e.copy(self.A[0], x)
        for l in range(self.L):
            e.matmul_forward(self.A[l], self.W[l], Y=self.A[l + 1],
                             bias=self.b[l] if self.use_bias else None, Z_out=self.Z[l + 1],
                             act=self.acts[l], act_alpha=self.Parameters.LeakyReLUAlpha)
        out = self.A[self.L]
        if self.softmax_output:
            e.softmax_forward(out, out=self.probs)
            out = self.probs
        return out

    def loss_value(self, target: Optional[E.DeviceMatrix] = None) -> E.DeviceMatrix:
        t = target or self.target
        out = self.probs if self.softmax_output else self.A[self.L]
        fn = self.eng.lib.prad_mse_forward if self.loss == "mse" else self.eng.lib.prad_cce_forward
        E.check(fn(self.eng.ctx, E.dtype_code(self.dtype), out.ptr, t.ptr, self.loss_dev.ptr,
                   out.shape[0], out.shape[1]))
        return self.loss_dev

    # ---------------------------------------------------------------- backward
    def _saved(self, l: int):
        """Tensor the activation of layer l keeps for Backward (1-based l)."""
        return self.A[l] if self.acts[l - 1] in _SAVES_OUTPUT else self.Z[l]

    def backward(self, target: Optional[E.DeviceMatrix] = None, rows_total: Optional[int] = None,
                 probe: Optional[Callable[[str, bool], None]] = None, need_dx: bool = True):
        """Loss gradient, then every layer's Backward; starts the all-reduces when world > 1."""
        e, L = self.eng, self.L
        rows = self.rows
        rows_total = rows_total or rows * self.world
        t = target or self.target
        alpha = self.Parameters.LeakyReLUAlpha
        cur = self.dZ[0].view((rows, self.sizes[L]))
        out = self.probs if self.softmax_output else self.A[L]
        if self.loss == "mse":
            e.mse_backward(out, t, rows_total=rows_total, grad=cur)
        else:
            e.cce_backward(out, t, rows_total=rows_total, grad=cur)
        if self.softmax_output:
            nxt = self.dZ[1].view((rows, self.sizes[L]))
            e.softmax_backward(self.probs, cur, out=nxt)
            self.dZ.reverse()
            cur = nxt
        if self.acts[L - 1] != E.ACT_NONE:
            e.act_backward(self.acts[L - 1], self._saved(L), cur, alpha, out=cur)
        for l in range(L, 0, -1):
            if probe:
                probe("gemm", True)
            e.matmul_backward(self.A[l - 1], None, cur, dB=self.dW[l - 1], need_dA=False)
            if probe:
                probe("gemm", False)
            if self.world > 1:
                e.dp_allreduce(self.dW[l - 1])
            if self.use_bias:
                e.add_broadcast_backward(cur, dbias=self.db[l - 1])
                if self.world > 1:
                    e.dp_allreduce(self.db[l - 1])
            if l > 1 or need_dx:
                below = self.acts[l - 2] if l > 1 else E.ACT_NONE
                nxt = self.dZ[1].view((rows, self.sizes[l - 1]))
                if probe:
                    probe("gemm", True)
                e.matmul_backward(None, self.W[l - 1], cur, dA=nxt, need_dB=False,
                                  act_below=below,
                                  saved_below=self._saved(l - 1) if below != E.ACT_NONE else None,
                                  act_alpha=alpha)
                if probe:
                    probe("gemm", False)
                self.dZ.reverse()
                cur = nxt
        self.dX = cur
        if self.world > 1:
            e.dp_wait()

    # ---------------------------------------------------------------- clip + Adam
    def clip_and_optimize(self, zero_grad: bool = True):
        p = self.Parameters
        self.eng.clip_adam(self.params, self.grads, self.m, self.v, self.clip_mode, p.ClipValue,
                           p.MinimumClipValue, p.LearningRate, p.AdamBeta1, p.AdamBeta2,
                           p.AdamEpsilon, p.AdamIteration, E.ADAM_RMAD, zero_grad)

    # ---------------------------------------------------------------- end to end
    def train_step_host(self, x_host: np.ndarray, t_host: np.ndarray, rows_total=None) -> float:
        """Host batch in, loss out: upload, forward, loss, backward, clip + Adam, download."""
        e = self.eng
        self._ensure_buffers(x_host.shape[0])
        e.upload(x_host, out=self.A[0])
        e.upload(t_host, out=self.target)
        self.forward()
        loss = self.loss_value()
        self.backward(rows_total=rows_total)
        self.clip_and_optimize()
        return float(loss.numpy()[0, 0])
