"""Data-parallel semantics on CPU with two gloo ranks: row shards + SUM all-reduce of the
weight gradients reproduce the single-process gradients, and clip + Adam then give the same
weights on every rank.  The arithmetic on each rank is the CPU oracle (the checker); what is
under test is the sharding rule, the global-row-count loss normaliser and the reduction."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from parallelreverseautodiff_b200.networks import row_shard


def test_row_shard_partitions_exactly():
    for total in (0, 1, 7, 64, 65536, 65537):
        for world in (1, 2, 3, 8):
            spans = [row_shard(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for a, b in zip(spans, spans[1:]):
                assert a[1] == b[0]
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        row_shard(10, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _mlp_grads(O, x, t, Ws, rows_total):
    """Forward + backward of a 2-layer GELU MLP with the oracle; returns weight gradients."""
    acts, pres = [x], []
    for W in Ws:
        z = O.matmul_forward(acts[-1], W)
        pres.append(z)
        acts.append(O.gelu_forward(z))
    d = O.mse_backward(acts[-1], t, rows_total=rows_total)
    grads = [None] * len(Ws)
    for l in range(len(Ws) - 1, -1, -1):
        d = O.gelu_backward(pres[l], d)
        dA, dW = O.matmul_backward(acts[l], Ws[l], d)
        grads[l] = dW
        d = dA
    return grads


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle as O

    r = np.random.default_rng(42)
    batch, width = 37, 24                      # odd batch: shards differ in size
    x = r.standard_normal((batch, width))
    t = r.standard_normal((batch, width))
    Ws = [r.standard_normal((width, width)) * np.sqrt(2.0 / width) for _ in range(2)]
    a, b = row_shard(batch, rank, world)
    grads = _mlp_grads(O, x[a:b], t[a:b], Ws, rows_total=batch)
    for g in grads:
        tg = torch.from_numpy(g)
        dist.all_reduce(tg, op=dist.ReduceOp.SUM)
    ws = [w.copy() for w in Ws]
    for w, g in zip(ws, grads):
        O.clip_reference(g, 4.0, 1e-16)
        O.adam_rmad(w, np.zeros_like(w), np.zeros_like(w), g, 1e-3, 0.9, 0.999, 1e-8, 1.0)
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), *grads, *ws)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gradients_match_single_process(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    import oracle as O

    r = np.random.default_rng(42)
    batch, width = 37, 24
    x = r.standard_normal((batch, width))
    t = r.standard_normal((batch, width))
    Ws = [r.standard_normal((width, width)) * np.sqrt(2.0 / width) for _ in range(2)]
    full = _mlp_grads(O, x, t, Ws, rows_total=batch)
    r0 = np.load(tmp_path / "rank0.npz")
    r1 = np.load(tmp_path / "rank1.npz")
    for k in r0.files:
        np.testing.assert_array_equal(r0[k], r1[k])       # ranks agree bit for bit
    for i, g in enumerate(full):
        got = r0[f"arr_{i}"]
        ref = O.clip_reference(g.copy(), 4.0, 1e-16)
        assert np.abs(got - ref).max() <= 1e-12 * np.abs(ref).max() + 1e-14
