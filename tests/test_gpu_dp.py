"""Data parallel on real GPUs (needs >= 2): two ranks, one process per GPU, NCCL all-reduce of
the weight gradients through prad_dp_*; the reduced gradients and the updated weights must
match the single-process CPU oracle on the whole batch.  Skipped on a one-GPU box."""
import os

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, id_path, out_dir, overlap=True, sharded=False, packed=False):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import time

    from parallelreverseautodiff_b200 import engine as E
    from parallelreverseautodiff_b200.networks import FeedForwardNetwork, row_shard

    eng = E.Engine(rank)
    if rank == 0:
        uid = E.Engine.dp_unique_id()
        with open(id_path + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(id_path + ".tmp", id_path)
    else:
        for _ in range(600):
            if os.path.exists(id_path):
                break
            time.sleep(0.05)
        uid = open(id_path, "rb").read()
    eng.dp_init(uid, rank, world)
    r = np.random.default_rng(42)
    batch, sizes = 96, [40, 64, 24]
    x = r.standard_normal((batch, sizes[0])).astype(np.float32)
    t = r.standard_normal((batch, sizes[-1])).astype(np.float32)
    Ws = [(r.standard_normal((sizes[i], sizes[i + 1])) * np.sqrt(2.0 / sizes[i])).astype(np.float32) for i in range(2)]
    net = FeedForwardNetwork(eng, np.float32, sizes, hidden_act=E.ACT_GELU, output_act=E.ACT_GELU, loss="mse",
                             use_bias=True, clip_mode=E.CLIP_REFERENCE, rank=rank, world=world, dp_overlap=overlap,
                             dp_sharded=sharded, packed=True if packed else "auto")
    net.forward_follows = packed == "forward first"     # order in which the owners publish their tensors
    net.set_weights(Ws)
    a, b = row_shard(batch, rank, world)
    net._ensure_buffers(b - a)
    eng.upload(x[a:b], out=net.A[0])
    eng.upload(t[a:b], out=net.target)
    net.forward()
    net.backward(rows_total=batch)
    grads = [g.numpy() for g in net.grads]
    net.clip_and_optimize(zero_grad=False)
    net._join_broadcasts()
    weights = [w.numpy() for w in net.params]
    # a second step exercises the hand-over of the broadcast weights to the next forward / backward
    net.forward()
    net.backward(rows_total=batch)
    net.clip_and_optimize(zero_grad=False)
    net._join_broadcasts()
    weights2 = [w.numpy() for w in net.params]
    owned = np.array(net.owned)
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), *grads, *weights, *weights2, owned=owned)
    eng.dp_shutdown()
    eng.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("overlap,sharded,packed",
                         [(True, False, False), (False, False, False), (True, True, False), (False, True, False),
                          (True, True, "backward first"), (True, True, "forward first")],
                         ids=["per-layer all-reduce", "one collective after the backward",
                              "sharded optimiser, per-layer reduce", "sharded optimiser, reduces after the backward",
                              "sharded optimiser on packed operands, tensors joined one by one",
                              "the same with the broadcasts in forward order"])
def test_two_gpu_gradients_match_oracle(tmp_path, overlap, sharded, packed):
    import oracle as O

    world = 2
    mp.spawn(_worker, args=(world, str(tmp_path / "nccl_id"), str(tmp_path), overlap, sharded, packed), nprocs=world, join=True)
    r = np.random.default_rng(42)
    batch, sizes = 96, [40, 64, 24]
    x = r.standard_normal((batch, sizes[0])).astype(np.float32)
    t = r.standard_normal((batch, sizes[-1])).astype(np.float32)
    Ws = [(r.standard_normal((sizes[i], sizes[i + 1])) * np.sqrt(2.0 / sizes[i])).astype(np.float32) for i in range(2)]
    acts, pres = [x], []
    for W in Ws:
        z = O.add_broadcast_forward(O.matmul_forward(acts[-1], W), np.zeros((1, W.shape[1]), np.float32))
        pres.append(z)
        acts.append(O.gelu_forward(z))
    d = O.mse_backward(acts[-1], t)
    dW, db = [None, None], [None, None]
    for l in (1, 0):
        d = O.gelu_backward(pres[l], d)
        db[l] = O.add_broadcast_backward(d)[1]
        dA, dW[l] = O.matmul_backward(acts[l], Ws[l], d)
        d = dA
    ref = dW + db
    ranks = [np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")]
    n = len(ref)
    for i, g in enumerate(ref):
        # the summed gradient lives on every rank (all-reduce) or on the tensor's owner (sharded)
        holders = [rk for rk in ranks if not sharded or i in rk["owned"]]
        assert holders
        for rk in holders:
            got = rk[f"arr_{i}"]
            # (packed operands: tensor-core products, 22-bit pieces)
            assert np.abs(got - g).max() <= (1e-4 if packed else 1e-5) * np.abs(g).max() + 1e-7, i
        if not sharded:
            np.testing.assert_array_equal(ranks[0][f"arr_{i}"], ranks[1][f"arr_{i}"])
    # weights after clip + Adam: identical on both ranks (they were broadcast, or computed from identical
    # gradients), and equal to the oracle's clip_reference + adam_rmad on the whole-batch gradients
    params0 = Ws + [np.zeros((1, W.shape[1]), np.float32) for W in Ws]
    for i in range(n):
        w_ref, g_ref = params0[i].copy(), ref[i].copy()
        O.clip_reference(g_ref, np.float32(4.0), np.float32(1e-8))
        O.adam_rmad(w_ref, np.zeros_like(w_ref), np.zeros_like(w_ref), g_ref, 1e-3, 0.9, 0.999, 1e-8, 1.0)
        for step in (0, 1):
            np.testing.assert_array_equal(ranks[0][f"arr_{n * (1 + step) + i}"], ranks[1][f"arr_{n * (1 + step) + i}"])
        got = ranks[0][f"arr_{n + i}"]
        upd, upd_ref = got - params0[i], w_ref - params0[i]
        big = np.abs(g_ref) > 1e-6            # where g ~ 0 the direction of the first Adam step is rounding noise
        # the update itself is ~lr * sign(g); what can differ is the last bit of the updated weight
        lim = 1e-5 * 1e-3 + 1e-5 * np.abs(upd_ref[big]) + np.spacing(np.abs(params0[i][big]) + 1e-3)
        assert (np.abs(upd[big] - upd_ref[big]) <= lim).all(), i
