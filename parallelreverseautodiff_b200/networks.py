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
    dZ_{l-1} = (dZ_l W_l^T) (.) act'(saved_{l-1})
so a layer's collective overlaps with the GEMMs of the layers below it.

Large float networks run "packed": every tensor that feeds a product is written once, by the kernel
that computes it, in the operand form of the tensor-core GEMM (prad_packed), in both orientations --
the activation A_l by the forward activation pass (for Z_{l+1} = A_l W and, later, dW = A_l^T dZ), the
gradient dZ_l by the activation's Backward (for dW and for dA = dZ_l W^T) -- so no product has to
read an FP32 tensor back, find its maxima and convert it first.
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
                 clip_mode=E.CLIP_REFERENCE, rank=0, world=1, dp_overlap=True, dp_sharded=False, packed="auto",
                 pack_block_cols=0):
        """dp_overlap: all-reduce each weight gradient right after its product (on the communication
        stream, beside the rest of the backward), or all gradients in one collective at the end.
        dp_sharded: sharded optimiser -- parameter tensor p belongs to rank p % world: its gradient is
        reduced to that rank only, which alone clips and updates it (and alone keeps its Adam moments)
        and broadcasts the new weights while the next step has already begun.  Needs a clip whose
        statistics are per tensor (the reference's z-score clip, or none)."""
        self.eng = eng
        self.packed_mode = packed          # "auto" | True | False: operands packed where they are produced
        self.pack_block_cols = pack_block_cols   # block length of the by-columns forms (0 = the library's default)
        self.packed = False                # decided per batch size in _ensure_buffers
        self.dp_overlap = dp_overlap
        self.dp_sharded = bool(dp_sharded) and world > 1
        if self.dp_sharded and clip_mode == E.CLIP_GLOBAL_NORM:
            raise ValueError("the sharded optimiser needs per-tensor clip statistics; the global-norm clip "
                             "sums over all tensors")
        self._bcast_pending = False
        self._bcast_marks = set()          # parameters whose broadcast has been enqueued and not joined yet
        self.forward_follows = False       # which pass follows an optimiser step: owners broadcast in that pass's order
        self.dtype = np.dtype(dtype)
        self.sizes = list(sizes)
        self.L = len(sizes) - 1
        self._w_dirty = [True] * self.L    # packed weight forms (by rows / by columns) older than the weights
        self._wc_dirty = [True] * self.L
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
        # one allocation for all gradients, so that they can also travel as one collective
        sizes_ = [int(np.prod(p.shape)) for p in params]
        self._grad_all = eng.zeros((sum(sizes_),), dtype)
        self.grads, off = [], 0
        for p, n in zip(params, sizes_):
            self.grads.append(self._grad_all.view(p.shape, off))
            off += n
        # Adam moments: every rank keeps all of them, or only those of the tensors it owns
        self.owned = [i for i in range(len(params)) if not self.dp_sharded or i % world == rank]
        self.m = [eng.zeros(p.shape, dtype) if i in self.owned else None for i, p in enumerate(params)]
        self.v = [eng.zeros(p.shape, dtype) if i in self.owned else None for i, p in enumerate(params)]
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
        self._w_dirty = [True] * self.L
        self._wc_dirty = [True] * self.L
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
        self.packed = self._wants_packed(rows)
        if self.packed:
            self._make_packed(rows)
            return
        self.A = [e.empty((rows, self.sizes[0]), dt)] + [e.empty((rows, n), dt) for n in self.sizes[1:]]
        self.Z = [None] + [e.empty((rows, n), dt) if self.acts[l] != E.ACT_NONE else None
                           for l, n in enumerate(self.sizes[1:])]
        widest = max(self.sizes)
        self.dZ = [e.empty((rows * widest,), dt), e.empty((rows * widest,), dt)]
        self.target = e.empty((rows, self.sizes[-1]), dt)
        if self.softmax_output:
            self.probs = e.empty((rows, self.sizes[-1]), dt)

    # ---------------------------------------------------------------- packed operands
    def _wants_packed(self, rows: int) -> bool:
        if self.packed_mode is False or self.dtype != np.float32 or self.softmax_output:
            return False
        if self.packed_mode is True:
            return True
        big = all(rows * a * b >= (1 << 27) for a, b in zip(self.sizes[:-1], self.sizes[1:]))
        return big and rows >= 256 and min(self.sizes) >= 256 and self.eng.packs_large_float_products()

    def _make_packed(self, rows: int) -> None:
        e, dt, L = self.eng, self.dtype, self.L
        both = E.PACK_ROWS | E.PACK_COLS
        bc = self.pack_block_cols
        # FP32 tensors that are still needed: the input, the saved tensor of every activation, the output
        self.A = [e.empty((rows, self.sizes[0]), dt)] + [None] * L
        self.Z = [None] * (L + 1)
        for l in range(1, L + 1):
            act = self.acts[l - 1]
            if act != E.ACT_NONE and act not in _SAVES_OUTPUT:
                self.Z[l] = e.empty((rows, self.sizes[l]), dt)
            if l == L or act in _SAVES_OUTPUT or act == E.ACT_NONE:
                self.A[l] = e.empty((rows, self.sizes[l]), dt)
        widest = max(self.sizes)
        self.dZ = [e.empty((rows * widest,), dt), e.empty((rows * widest,), dt)]
        self.target = e.empty((rows, self.sizes[-1]), dt)
        # A_0 .. A_{L-1}: by rows for the forward product, by columns for the weight gradient
        self.PA = [e.packed(rows, self.sizes[l], both, 0, bc) for l in range(L)]
        # dZ_l: by columns for the weight gradient, by rows for the gradient of the layer below; one object
        # per width (layer l's is dead when layer l-1's is written)
        self.PD = {}
        for l in range(1, L + 1):
            if self.sizes[l] not in self.PD:
                self.PD[self.sizes[l]] = e.packed(rows, self.sizes[l], both, 0, bc)
        # W_l: by columns it multiplies A_l (forward), by rows it multiplies dZ_{l+1} (backward); its block
        # lengths are those of the by-rows forms it meets
        blk_a = self.PA[0].blocks()[0]
        blk_d = next(iter(self.PD.values())).blocks()[0]
        # (two objects: the backward needs only the by-rows form, and packs it again after every optimiser step)
        self.PWr = [e.packed(self.sizes[l], self.sizes[l + 1], E.PACK_ROWS, blk_d, 0) for l in range(L)]
        self.PWc = [e.packed(self.sizes[l], self.sizes[l + 1], E.PACK_COLS, 0, blk_a) for l in range(L)]
        self._w_dirty = [True] * L
        self._wc_dirty = [True] * L

    def _pack_weight(self, l: int, forward: bool) -> None:
        """Packed form of W_l for the forward (by columns) or the backward (by rows) product, refreshed after
        an optimiser step; waits for that tensor's broadcast only."""
        dirty = self._wc_dirty if forward else self._w_dirty
        if dirty[l]:
            self._join_tensor(l)
            (self.PWc if forward else self.PWr)[l].pack(self.W[l])
            dirty[l] = False

    def _forward_packed(self) -> E.DeviceMatrix:
        e, L = self.eng, self.L
        alpha = self.Parameters.LeakyReLUAlpha
        self.PA[0].pack(self.A[0])
        for l in range(L):
            act = self.acts[l]
            pre = self.Z[l + 1] if self.Z[l + 1] is not None else self.A[l + 1]
            self._pack_weight(l, forward=True)
            if self.use_bias:
                self._join_tensor(L + l)
            e.gemm_packed(self.PA[l], E.PACK_ROWS, self.PWc[l], E.PACK_COLS, pre,
                          bias=self.b[l] if self.use_bias else None)
            if l + 1 < L:      # the activation writes the next layer's operand (and A_{l+1} in FP32 if kept)
                self.PA[l + 1].act_forward(act, pre, self.A[l + 1], alpha)
            elif act != E.ACT_NONE:
                e.act_forward(act, pre, alpha, out=self.A[L])
        return self.A[L]

    def _backward_packed(self, g: Optional[E.DeviceMatrix], probe, need_dx: bool, mse=None) -> None:
        """g = gradient of the loss with respect to A_L (FP32), or mse = (output, target, rows_total) to have
        the mean-squared-error gradient formed on the fly."""
        e, L, rows = self.eng, self.L, self.rows
        alpha = self.Parameters.LeakyReLUAlpha
        for l in range(L, 0, -1):
            act = self.acts[l - 1]
            pd = self.PD[self.sizes[l]]
            dz32 = None
            if self.use_bias:                        # the bias gradient sums the FP32 gradient's columns
                dz32 = self.dZ[1].view((rows, self.sizes[l]))
            saved = self._saved(l) if act != E.ACT_NONE else None
            if probe:
                probe("pack", True)
            if l == L and mse is not None:
                pd.mse_act_backward(act, saved, mse[0], mse[1], mse[2], dz32, alpha)
            else:
                pd.act_backward(act, saved, g, dz32, alpha)
            if probe:
                probe("pack", False)
            if probe:
                probe("gemm", True)
            e.gemm_packed(self.PA[l - 1], E.PACK_COLS, pd, E.PACK_COLS, self.dW[l - 1])
            if probe:
                probe("gemm", False)
            if self.world > 1 and self.dp_overlap:
                self._reduce_grad(l - 1)
            if self.use_bias:
                e.add_broadcast_backward(dz32, dbias=self.db[l - 1])
                if self.world > 1 and self.dp_overlap:
                    self._reduce_grad(L + l - 1)
            if l > 1 or need_dx:
                g = self.dZ[0].view((rows, self.sizes[l - 1]))
                # the weight-gradient product above read no weights: the previous step's weight broadcasts ran
                # beside it, owner by owner in the order this loop needs them; only W_{l-1}'s is joined here
                if probe:
                    probe("pack", True)
                self._pack_weight(l - 1, forward=False)
                if probe:
                    probe("pack", False)
                if probe:
                    probe("gemm", True)
                e.gemm_packed(pd, E.PACK_ROWS, self.PWr[l - 1], E.PACK_ROWS, g)
                if probe:
                    probe("gemm", False)
        self.dX = g

    # ---------------------------------------------------------------- forward
    def forward(self, x: Optional[E.DeviceMatrix] = None) -> E.DeviceMatrix:
        """Forward through every layer; keeps Z_l (pre-activation) and A_l for the backward."""
        e = self.eng
        packed = self.packed or (x is not None and self._wants_packed(x.shape[0]))
        if not packed:               # (the packed path joins tensor by tensor, as it reaches them)
            self._join_broadcasts()
        if packed:
            if x is not None:
                self._ensure_buffers(x.shape[0])
                e.copy(self.A[0], x)
            return self._forward_packed()
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
    def _owner(self, p: int) -> int:
        """Rank that owns parameter tensor p (index into self.params) under the sharded optimiser."""
        return p % self.world

    def _reduce_grad(self, p: int) -> None:
        if self.dp_sharded:
            self.eng.dp_reduce(self.grads[p], self._owner(p))
        else:
            self.eng.dp_allreduce(self.grads[p])

    def _join_broadcasts(self) -> None:
        """The weights broadcast by their owners after the last optimiser step must have arrived
        before a kernel reads them."""
        if self._bcast_pending:
            self.eng.dp_wait()
            self._bcast_pending = False
            self._bcast_marks.clear()

    def _join_tensor(self, p: int) -> None:
        """Wait for the broadcast of parameter p alone (the others may still be on their way)."""
        if p in self._bcast_marks:
            self.eng.dp_wait_mark(p)
            self._bcast_marks.discard(p)
        elif self._bcast_pending and p >= E.DP_MARKS:
            self._join_broadcasts()

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
        if self.packed and self.loss == "mse":
            # the loss gradient is formed inside the pass that packs dZ_L (never stored)
            self._backward_packed(None, probe, need_dx, mse=(out, t, rows_total))
            self._finish_backward(probe)
            return
        if self.loss == "mse":
            e.mse_backward(out, t, rows_total=rows_total, grad=cur)
        else:
            e.cce_backward(out, t, rows_total=rows_total, grad=cur)
        if self.softmax_output:
            nxt = self.dZ[1].view((rows, self.sizes[L]))
            e.softmax_backward(self.probs, cur, out=nxt)
            self.dZ.reverse()
            cur = nxt
        if self.packed:
            self._backward_packed(cur, probe, need_dx)
            self._finish_backward(probe)
            return
        if self.acts[L - 1] != E.ACT_NONE:
            e.act_backward(self.acts[L - 1], self._saved(L), cur, alpha, out=cur)
        for l in range(L, 0, -1):
            if probe:
                probe("gemm", True)
            e.matmul_backward(self.A[l - 1], None, cur, dB=self.dW[l - 1], need_dA=False)
            if probe:
                probe("gemm", False)
            # the first weight-gradient product reads no weights: the broadcasts of the previous step's
            # new weights run beside it and are joined here, before the first collective of this step
            self._join_broadcasts()
            if self.world > 1 and self.dp_overlap:
                self._reduce_grad(l - 1)
            if self.use_bias:
                e.add_broadcast_backward(cur, dbias=self.db[l - 1])
                if self.world > 1 and self.dp_overlap:
                    self._reduce_grad(L + l - 1)
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
        self._finish_backward(probe)

    def _finish_backward(self, probe=None) -> None:
        e = self.eng
        if self.world > 1:
            if not self.dp_overlap:
                if self.dp_sharded:
                    for p in range(len(self.params)):
                        self._reduce_grad(p)
                else:
                    e.dp_allreduce(self._grad_all)
            if probe:
                probe("join", True)
            e.dp_wait()                  # every collective so far, the previous step's broadcasts included
            self._bcast_marks.clear()
            self._bcast_pending = False
            if probe:
                probe("join", False)

    # ---------------------------------------------------------------- clip + Adam
    def clip_and_optimize(self, zero_grad: bool = True):
        p = self.Parameters
        self._w_dirty = [True] * self.L
        self._wc_dirty = [True] * self.L
        own = self.owned
        pick = lambda xs: [xs[i] for i in own]
        if own:
            self.eng.clip_adam(pick(self.params), pick(self.grads), pick(self.m), pick(self.v), self.clip_mode,
                               p.ClipValue, p.MinimumClipValue, p.LearningRate, p.AdamBeta1, p.AdamBeta2,
                               p.AdamEpsilon, p.AdamIteration, E.ADAM_RMAD, zero_grad)
        if self.dp_sharded:
            # owners publish their new weights; the tensors the next backward needs first go first.
            # (Gradients of tensors owned elsewhere keep this rank's partial sums: the next backward
            # overwrites them.)
            if self.forward_follows:     # W_0 (and its bias) first
                order = [i for l in range(self.L) for i in ([l, self.L + l] if self.use_bias else [l])]
            else:
                order = list(range(self.L - 1, -1, -1)) + list(range(self.L, len(self.params)))
            for i in order:
                self.eng.dp_broadcast(self.params[i], self._owner(i))
                if i < E.DP_MARKS:               # (a network with more tensors than marks joins the rest as a whole)
                    self.eng.dp_mark(i)
                    self._bcast_marks.add(i)
            self._bcast_pending = True

    # ---------------------------------------------------------------- end to end
    def train_step_host(self, x_host: np.ndarray, t_host: np.ndarray, rows_total=None) -> float:
        """Host batch in, loss out: upload, forward, loss, backward, clip + Adam, download."""
        e = self.eng
        self.forward_follows = True
        self._ensure_buffers(x_host.shape[0])
        e.upload(x_host, out=self.A[0])
        e.upload(t_host, out=self.target)
        self.forward()
        loss = self.loss_value()
        self.backward(rows_total=rows_total)
        self.clip_and_optimize()
        return float(loss.numpy()[0, 0])

    def train_steps_host(self, batches, rows_total=None):
        """Same as train_step_host over a sequence of (x_host, t_host) page-locked batches, with
        the upload of batch i+1 running on the copy stream while batch i is computed (two input
        buffers alternate).  Every batch is still copied host->device and every loss read back;
        yields the losses."""
        e = self.eng
        self.forward_follows = True
        batches = list(batches)
        if not batches:
            return
        rows = batches[0][0].shape[0]
        self._ensure_buffers(rows)
        if getattr(self, "_stage_rows", None) != rows:
            self._in = [self.A[0], e.empty(self.A[0].shape, self.dtype)]
            self._tg = [self.target, e.empty(self.target.shape, self.dtype)]
            self._stage_rows = rows
        e.upload_prefetch(batches[0][0], self._in[0])
        e.upload_prefetch(batches[0][1], self._tg[0])
        for i in range(len(batches)):
            self.A[0], self.target = self._in[i % 2], self._tg[i % 2]
            e.upload_join()                       # batch i is on the device before its first use
            if i + 1 < len(batches):              # step i-1 has completed (its loss was read back)
                e.upload_prefetch(batches[i + 1][0], self._in[(i + 1) % 2])
                e.upload_prefetch(batches[i + 1][1], self._tg[(i + 1) % 2])
            self.forward()
            loss = self.loss_value()
            self.backward(rows_total=rows_total)
            self.clip_and_optimize()
            yield float(loss.numpy()[0, 0])


class LstmNetwork:
    """Single-layer LSTM with full BPTT over the C ABI (benchmark config 3, PRAD double).

    Reference graph (test/.../GraphAttentionPaths/LSTM/Architecture/NodeProcessing.json style,
    README.md:396-430): per sample a column vector, gates through
    BatchGpuMatrixMultiplyOperation(W, x) + (U, h) + bias, Sigmoid / Tanh, HadamardProduct,
    MatrixAdd; weight gradients are averaged over the batch by the visitor
    (OperationNeuralNetworkVisitor.cs:449-478) and added up over the time steps
    (OperationBase.cs:295-303).

    Device layout: one row per sample (batch-major), time steps stacked along the rows, so the
    input contribution of every gate for ALL steps is one GEMM, and every shared weight's
    gradient is ONE long-K product over the T*B stacked rows with alpha = 1/B -- the
    deterministic replacement of the visitor's per-step `+=`.  The fan-in at h_t (loss + four
    gate products of step t+1) and at c_t is a fixed-order prad_segmented_sum.
    """

    GATES = ("i", "f", "g", "o")

    def __init__(self, eng: E.Engine, dtype, n_in: int, n_hidden: int, steps: int, batch: int, fused_cell: bool = True):
        self.eng, self.dtype = eng, np.dtype(dtype)
        self.fused_cell = fused_cell      # one kernel per time step for the elementwise part of the backward
        self.n_in, self.n_h, self.T, self.B = n_in, n_hidden, steps, batch
        e, dt = eng, self.dtype
        z = lambda *s: e.zeros(s, dt)  # noqa: E731
        TB = steps * batch
        G = len(self.GATES)

        def stacked(rows, cols):
            """The four gates' matrices in one allocation, so that one strided-batched product serves all."""
            whole = z(G * rows, cols)
            return whole, {g: whole.view((rows, cols), k * rows * cols) for k, g in enumerate(self.GATES)}

        self._W_all, self.W = stacked(n_hidden, n_in)             # [hidden x in], as in the reference
        self._U_all, self.U = stacked(n_hidden, n_hidden)
        self.b = {g: z(1, n_hidden) for g in self.GATES}
        self._dW_all, self.dW = stacked(n_hidden, n_in)
        self._dU_all, self.dU = stacked(n_hidden, n_hidden)
        self.db = {g: z(1, n_hidden) for g in self.GATES}
        self.X = z(TB, n_in)
        self.Y = z(TB, n_hidden)                                  # targets
        self._pre_all, self.pre = stacked(TB, n_hidden)           # gate pre-activations
        self.gate = {g: z(TB, n_hidden) for g in self.GATES}     # gate outputs
        self.C = z(TB, n_hidden)
        self.tanhC = z(TB, n_hidden)
        self.H = z(TB, n_hidden)
        self.Hprev = z(TB, n_hidden)                              # H shifted by one step (h_{-1} = 0)
        self.FC = z(TB, n_hidden)                                 # f (.) c_{t-1}
        self.IG = z(TB, n_hidden)                                 # i (.) g
        self._dpre_all, self.dpre = stacked(TB, n_hidden)
        self.dX = z(TB, n_in)
        self._tmp = [z(batch, n_hidden) for _ in range(18)]
        self._rec_all, rec = stacked(batch, n_hidden)             # dZ_g(t) U_g for the four gates
        for k, g in enumerate(self.GATES):
            self._tmp[8 + k] = rec[g]

    def set_parameters(self, W, U, b):
        for g in self.GATES:
            self.eng.upload(np.ascontiguousarray(W[g], self.dtype), out=self.W[g])
            self.eng.upload(np.ascontiguousarray(U[g], self.dtype), out=self.U[g])
            self.eng.upload(np.ascontiguousarray(b[g], self.dtype).reshape(1, -1), out=self.b[g])

    def _step(self, m: E.DeviceMatrix, t: int) -> E.DeviceMatrix:
        return m.view((self.B, m.shape[1]), t * self.B * m.shape[1])

    def forward(self, x_host: np.ndarray, y_host: np.ndarray):
        """x_host [T, B, in], y_host [T, B, hidden]."""
        e, T, B = self.eng, self.T, self.B
        e.upload(np.ascontiguousarray(x_host, self.dtype).reshape(T * B, -1), out=self.X)
        e.upload(np.ascontiguousarray(y_host, self.dtype).reshape(T * B, -1), out=self.Y)
        e.zero_(self.Hprev)
        nh, n_in, TB, G = self.n_h, self.n_in, T * B, len(self.GATES)
        first = self.GATES[0]
        # input contribution of all steps and gates: X_all * W_g^T, one strided-batched product
        e.gemm(self.X, self.W[first], self.pre[first], transB=True, batch=G, strideA=0, strideB=nh * n_in,
               strideC=TB * nh)
        acts = {"i": E.ACT_SIGMOID, "f": E.ACT_SIGMOID, "g": E.ACT_TANH, "o": E.ACT_SIGMOID}
        for t in range(T):
            hp = self._step(self.Hprev, t)
            if t > 0:           # + h_{t-1} * U_g^T for the four gates (MatrixAddThree: (Wx + Uh) + b)
                e.gemm(hp, self.U[first], self._step(self.pre[first], t), transB=True, beta=1.0, batch=G,
                       strideA=0, strideB=nh * nh, strideC=TB * nh)
            for g in self.GATES:
                p = self._step(self.pre[g], t)
                e.add_broadcast_forward(p, self.b[g], out=p)
                e.act_forward(acts[g], p, out=self._step(self.gate[g], t))
            c, fc, ig = self._step(self.C, t), self._step(self.FC, t), self._step(self.IG, t)
            e.hadamard_forward(self._step(self.gate["i"], t), self._step(self.gate["g"], t), out=ig)
            if t > 0:
                e.hadamard_forward(self._step(self.gate["f"], t), self._step(self.C, t - 1), out=fc)
            else:
                e.zero_(fc)
            e.add_forward(fc, ig, out=c)
            tc = self._step(self.tanhC, t)
            e.act_forward(E.ACT_TANH, c, out=tc)
            h = self._step(self.H, t)
            e.hadamard_forward(self._step(self.gate["o"], t), tc, out=h)
            if t + 1 < T:
                e.copy(self._step(self.Hprev, t + 1), h)
        return self.H

    def backward(self):
        """MSE per sample and step (MeanSquaredErrorLossOperation on each [hidden x 1] column),
        BPTT, then the time- and batch-reduced weight gradients."""
        e, T, B, nh = self.eng, self.T, self.B, self.n_h
        tmp = self._tmp
        if not self.fused_cell:
            self._backward_steps_by_operation()
        else:
            # one launch per time step for everything elementwise (prad_lstm_cell_backward), one strided-batched
            # product for the four recurrent gradients; bit-identical to the operation-by-operation path
            dh_rec, dc_next = [], None
            g0 = self.GATES[0]
            for t in range(T - 1, -1, -1):
                st = lambda m: self._step(m, t)        # noqa: E731
                dc_prev = tmp[15 + (t & 1)] if t > 0 else None
                e.lstm_cell_backward(st(self.H), st(self.Y), 2.0 / nh, dh_rec, dc_next,
                                     [st(self.gate[k]) for k in ("i", "f", "g", "o")], st(self.tanhC),
                                     self._step(self.C, t - 1) if t > 0 else None,
                                     [st(self.dpre[k]) for k in ("i", "f", "g", "o")], dc_prev)
                dc_next = dc_prev
                if t > 0:           # gradient w.r.t. h_{t-1}: one product per gate, summed by the next call
                    e.gemm(st(self.dpre[g0]), self.U[g0], tmp[8], batch=len(self.GATES),
                           strideA=T * B * nh, strideB=nh * nh, strideC=B * nh)
                    dh_rec = [tmp[8 + k] for k in range(len(self.GATES))]
        inv_b = 1.0 / B
        first = True
        g0, G, TB = self.GATES[0], len(self.GATES), T * B
        # dW_g = (1/B) * dZ_all^T X_all ; dU_g = (1/B) * dZ_all^T Hprev_all : the four gates per launch
        e.gemm(self.dpre[g0], self.X, self.dW[g0], transA=True, alpha=inv_b, batch=G, strideA=TB * nh, strideB=0,
               strideC=nh * self.n_in)
        e.gemm(self.dpre[g0], self.Hprev, self.dU[g0], transA=True, alpha=inv_b, batch=G, strideA=TB * nh,
               strideB=0, strideC=nh * nh)
        for g in self.GATES:
            # db_g = (1/B) colsum
            e.add_broadcast_backward(self.dpre[g], dbias=self.db[g])
            e.scale(self.db[g], inv_b, out=self.db[g])
            # dX_all = sum over gates of dZ_g W_g (left fold in gate order)
            e.gemm(self.dpre[g], self.W[g], self.dX, beta=0.0 if first else 1.0)
            first = False



    def _backward_steps_by_operation(self):
        """The time loop of the backward with one library call per managed operation."""
        e, T, B, nh = self.eng, self.T, self.B, self.n_h
        tmp = self._tmp
        dh_rec = None           # four buffers: dZ_g(t+1) * U_g
        dc_next = None          # dc_{t+1} (.) f_{t+1}
        for t in range(T - 1, -1, -1):
            # per-sample MSE over a [hidden x 1] column: 2/(hidden*1) * (h - y)
            dloss = tmp[0]
            e.mse_backward(self._step(self.H, t), self._step(self.Y, t), rows_total=1, grad=dloss)
            dh = tmp[1]
            if dh_rec is None:
                e.copy(dh, dloss)
            else:
                e.segmented_sum([dloss] + dh_rec, out=dh)
            o, tc = self._step(self.gate["o"], t), self._step(self.tanhC, t)
            d_o, d_tc = tmp[2], tmp[3]
            e.hadamard_backward(o, tc, dh, out=(d_o, d_tc))
            dc_a = tmp[4]
            e.act_backward(E.ACT_TANH, tc, d_tc, out=dc_a)
            dc = tmp[5]
            if dc_next is None:
                e.copy(dc, dc_a)
            else:
                e.segmented_sum([dc_a, dc_next], out=dc)
            # c = f*c_prev + i*g : MatrixAdd copies dc to both products
            i_, g_, f_ = (self._step(self.gate[k], t) for k in ("i", "g", "f"))
            d_i, d_g = e.hadamard_backward(i_, g_, dc, out=(tmp[12], tmp[13]))
            if t > 0:
                # dc_next alternates between two buffers: the one read as dc_next above stays intact
                d_f, dc_next = e.hadamard_backward(f_, self._step(self.C, t - 1), dc,
                                                   out=(tmp[14], tmp[15 + (t & 1)]))
            else:
                d_f = tmp[7]
                e.zero_(d_f)    # c_{-1} = 0 -> dc (.) 0
            e.act_backward(E.ACT_SIGMOID, i_, d_i, out=self._step(self.dpre["i"], t))
            e.act_backward(E.ACT_SIGMOID, f_, d_f, out=self._step(self.dpre["f"], t))
            e.act_backward(E.ACT_TANH, g_, d_g, out=self._step(self.dpre["g"], t))
            e.act_backward(E.ACT_SIGMOID, o, d_o, out=self._step(self.dpre["o"], t))
            if t > 0:           # gradient w.r.t. h_{t-1}: one product per gate, summed above
                g0 = self.GATES[0]
                e.gemm(self._step(self.dpre[g0], t), self.U[g0], tmp[8], batch=len(self.GATES),
                       strideA=T * B * nh, strideB=nh * nh, strideC=B * nh)
                dh_rec = [tmp[8 + k] for k in range(len(self.GATES))]


class SwinBlock:
    """One Swin-style windowed self-attention block, forward and full backward (benchmark
    config 4, PRADLite float).  Composition of the RMAD operations: LayerNormalization,
    MatrixMultiply + MatrixAddBroadcasting (QKV / output projection / MLP), BatchMatrixMultiply
    (Q K^T and P V per window and head), MatrixMultiplyScalar (1/sqrt(d)), Softmax, GELU,
    MatrixAdd (residuals).  The Swin *example* of the reference cannot run its attention
    (Tensor.MatrixMultiply throws for non-2-D input, src/PRAD/Tensor.cs:572-577), so the RMAD
    composition is the semantics.

    Heads are never materialised: every per-(window, head) product is a strided-batched GEMM
    addressing the [tokens x 3*dim] QKV matrix in place (leading dimension 3*dim, window stride
    ws*3*dim, one call per head), so head split / merge and all transposes cost no copies.
    """

    def __init__(self, eng: E.Engine, dtype, dim=96, heads=3, window=49, mlp_ratio=4):
        self.eng, self.dtype = eng, np.dtype(dtype)
        self.dim, self.heads, self.ws, self.hd = dim, heads, window, dim // heads
        self.hidden = dim * mlp_ratio
        z = lambda *s: eng.zeros(s, dtype)  # noqa: E731
        d, h = dim, self.hidden
        self.p = {"Wqkv": z(d, 3 * d), "bqkv": z(1, 3 * d), "Wproj": z(d, d), "bproj": z(1, d),
                  "W1": z(d, h), "b1": z(1, h), "W2": z(h, d), "b2": z(1, d)}
        self.g = {k: z(*v.shape) for k, v in self.p.items()}
        self.scale = 1.0 / float(np.sqrt(self.hd))
        self._cache = {}

    def _buf(self, name, shape):
        """Device buffer reused across calls (no allocation in the steady state)."""
        b = self._cache.get(name)
        if b is None or b.shape != tuple(shape):
            b = self.eng.empty(shape, self.dtype)
            self._cache[name] = b
        return b

    def set_parameters(self, params):
        for k, v in params.items():
            self.eng.upload(np.ascontiguousarray(v, self.dtype).reshape(self.p[k].shape), out=self.p[k])

    def _attn_gemm(self, A, a_off, lda, sA, Bm, b_off, ldb, sB, Cm, c_off, ldc, sC, M, N, K, transA=False,
                   transB=False, alpha=1.0, beta=0.0, batch=1):
        e = self.eng
        e.gemm(A.view((1, 1), a_off), Bm.view((1, 1), b_off), Cm.view((1, 1), c_off), transA=transA, transB=transB,
               alpha=alpha, beta=beta, M=M, N=N, K=K, lda=lda, ldb=ldb, ldc=ldc, batch=batch, strideA=sA,
               strideB=sB, strideC=sC)

    def forward(self, x: E.DeviceMatrix):
        e, d, ws, H, hd = self.eng, self.dim, self.ws, self.heads, self.hd
        T = x.shape[0]
        nw = T // ws
        self.x, self.nw = x, nw
        self.ln1, self.mu1, self.sd1 = e.layernorm_forward(x)
        self.qkv = e.matmul_forward(self.ln1, self.p["Wqkv"], bias=self.p["bqkv"])
        self.S = e.empty((nw * H * ws, ws), self.dtype)           # [window][head][ws x ws]
        for h in range(H):                                        # S = (Q K^T) * scale
            self._attn_gemm(self.qkv, h * hd, 3 * d, ws * 3 * d, self.qkv, d + h * hd, 3 * d, ws * 3 * d,
                            self.S, h * ws * ws, ws, H * ws * ws, ws, ws, hd, transB=True, alpha=self.scale, batch=nw)
        self.P = e.softmax_forward(self.S)
        self.attn = e.empty((T, d), self.dtype)
        for h in range(H):                                        # O_h = P V, written at column h*hd
            self._attn_gemm(self.P, h * ws * ws, ws, H * ws * ws, self.qkv, 2 * d + h * hd, 3 * d, ws * 3 * d,
                            self.attn, h * hd, d, ws * d, ws, hd, ws, batch=nw)
        self.proj = e.matmul_forward(self.attn, self.p["Wproj"], bias=self.p["bproj"])
        self.r1 = e.add_forward(x, self.proj)
        self.ln2, self.mu2, self.sd2 = e.layernorm_forward(self.r1)
        self.z1 = e.empty((T, self.hidden), self.dtype)
        self.a1 = e.matmul_forward(self.ln2, self.p["W1"], bias=self.p["b1"], Z_out=self.z1, act=E.ACT_GELU)
        self.m2 = e.matmul_forward(self.a1, self.p["W2"], bias=self.p["b2"])
        self.out = e.add_forward(self.r1, self.m2)
        return self.out

    def backward(self, d_out: E.DeviceMatrix):
        e, d, ws, H, hd, nw = self.eng, self.dim, self.ws, self.heads, self.hd, self.nw
        g, p = self.g, self.p
        T = d_out.shape[0]
        # out = r1 + m2 : both receive d_out (MatrixAddOperation.Backward)
        e.add_broadcast_backward(d_out, dbias=g["b2"])
        B_ = self._buf
        d_z1, _ = e.matmul_backward(self.a1, p["W2"], d_out, dA=B_("d_z1", (T, self.hidden)), dB=g["W2"],
                                    act_below=E.ACT_GELU, saved_below=self.z1)
        e.add_broadcast_backward(d_z1, dbias=g["b1"])
        d_ln2, _ = e.matmul_backward(self.ln2, p["W1"], d_z1, dA=B_("d_ln2", (T, d)), dB=g["W1"])
        d_r1_b = e.layernorm_backward(self.r1, self.mu2, self.sd2, d_ln2, out=B_("d_r1_b", (T, d)))
        d_r1 = e.segmented_sum([d_out, d_r1_b], out=B_("d_r1", (T, d)))   # fan-in at r1: residual + LN2 branch
        # r1 = x + proj
        e.add_broadcast_backward(d_r1, dbias=g["bproj"])
        d_attn, _ = e.matmul_backward(self.attn, p["Wproj"], d_r1, dA=B_("d_attn", (T, d)), dB=g["Wproj"])
        d_qkv = B_("d_qkv", (T, 3 * d))     # every element is written by the three per-head products below
        dP = B_("dP", self.P.shape)
        for h in range(H):
            # O_h = P_h V_h :  dP_h = dO_h V_h^T ,  dV_h = P_h^T dO_h
            self._attn_gemm(d_attn, h * hd, d, ws * d, self.qkv, 2 * d + h * hd, 3 * d, ws * 3 * d,
                            dP, h * ws * ws, ws, H * ws * ws, ws, ws, hd, transB=True, batch=nw)
            self._attn_gemm(self.P, h * ws * ws, ws, H * ws * ws, d_attn, h * hd, d, ws * d,
                            d_qkv, 2 * d + h * hd, 3 * d, ws * 3 * d, ws, hd, ws, transA=True, batch=nw)
        dS = e.softmax_backward(self.P, dP, out=B_("dS", self.P.shape))
        for h in range(H):
            # S_h = scale * Q_h K_h^T :  dQ_h = scale * dS_h K_h ,  dK_h = scale * dS_h^T Q_h
            self._attn_gemm(dS, h * ws * ws, ws, H * ws * ws, self.qkv, d + h * hd, 3 * d, ws * 3 * d,
                            d_qkv, h * hd, 3 * d, ws * 3 * d, ws, hd, ws, alpha=self.scale, batch=nw)
            self._attn_gemm(dS, h * ws * ws, ws, H * ws * ws, self.qkv, h * hd, 3 * d, ws * 3 * d,
                            d_qkv, d + h * hd, 3 * d, ws * 3 * d, ws, hd, ws, transA=True, alpha=self.scale, batch=nw)
        e.add_broadcast_backward(d_qkv, dbias=g["bqkv"])
        d_ln1, _ = e.matmul_backward(self.ln1, p["Wqkv"], d_qkv, dA=B_("d_ln1", (T, d)), dB=g["Wqkv"])
        d_x_b = e.layernorm_backward(self.x, self.mu1, self.sd1, d_ln1, out=B_("d_x_b", (T, d)))
        self.d_x = e.segmented_sum([d_r1, d_x_b], out=B_("d_x", (T, d)))  # fan-in at x: residual + LN1 branch
        self.d_qkv, self.dS, self.dP, self.d_attn = d_qkv, dS, dP, d_attn
        return self.d_x
