"""Host-side logic of the multi-GPU path, on CPU: shard arithmetic, and the all-gather + merge
plumbing run as two gloo ranks with the merge kernel replaced by a NumPy stand-in."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from project_tensor_b200.sharded import gather_score_slabs, merge_topk_across_ranks, scatter_merge_topk, shard_range


def test_shard_range_covers_everything_once():
    for n in (0, 1, 7, 8, 134217728, 1000003):
        for world in (1, 2, 4, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(10, 2, 2)


def numpy_merge(gs, gi):
    """Stand-in for tq_topk_merge: descending by score, ties to the earlier list / slot."""
    gs, gi = gs.numpy(), gi.numpy()
    lists, queries, k = gs.shape
    out_s = np.full((queries, k), -np.inf, np.float32)
    out_i = np.full((queries, k), -1, np.int64)
    for q in range(queries):
        s = gs[:, q, :].reshape(-1)
        i = gi[:, q, :].reshape(-1)
        valid = i >= 0
        order = np.lexsort((np.arange(s.size), -s))
        order = [o for o in order if valid[o]][:k]
        out_s[q, :len(order)] = s[order]
        out_i[q, :len(order)] = i[order]
    return torch.from_numpy(out_s), torch.from_numpy(out_i)


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(7)
        n, q, k = 64, 3, 5
        scores = rng.standard_normal((q, n)).astype(np.float32)
        scores[:, 10] = scores[:, 40]                       # a tie across the two shards
        lo, hi = shard_range(n, rank, world)
        local = scores[:, lo:hi]
        order = np.argsort(-local, axis=1, kind="stable")[:, :k]
        top_s = torch.from_numpy(np.take_along_axis(local, order, axis=1))
        top_i = torch.from_numpy(order.astype(np.int64) + lo)
        got_s, got_i = merge_topk_across_ranks(top_s, top_i, merge=numpy_merge)
        want = np.argsort(-scores, axis=1, kind="stable")[:, :k]
        assert np.array_equal(got_i.numpy(), want)
        assert np.array_equal(got_s.numpy(), np.take_along_axis(scores, want, axis=1))
        slab = gather_score_slabs(torch.from_numpy(local.copy()))
        assert np.array_equal(slab.numpy(), scores)
        # the scatter form: every rank merges only its own slice of the queries
        q4 = 4
        scores4 = rng.standard_normal((q4, n)).astype(np.float32)
        local4 = scores4[:, lo:hi]
        order4 = np.argsort(-local4, axis=1, kind="stable")[:, :k]
        s_s, s_i, first = scatter_merge_topk(torch.from_numpy(np.take_along_axis(local4, order4, axis=1)),
                                             torch.from_numpy(order4.astype(np.int64) + lo), merge=numpy_merge)
        want4 = np.argsort(-scores4, axis=1, kind="stable")[:, :k]
        assert first == rank * (q4 // world) and s_i.shape == (q4 // world, k)
        assert np.array_equal(s_i.numpy(), want4[first:first + q4 // world])
        ret[rank] = True
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_and_merge_over_gloo():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
        assert ret.get(0) and ret.get(1)


def _absent_rank_worker(rank, world, port, ret):
    """Rank 1 initialises the group and then never enters the collective (it sleeps and leaves); rank 0 must get
    ShardExchangeTimeout after its limit instead of waiting forever.  Host-side failure only: no device involved."""
    import time
    from project_tensor_b200.sharded import ShardExchangeTimeout, TopkExchange
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    if rank == 1:
        time.sleep(4.0)
        ret[1] = "left without joining"
        os._exit(0)
    ex = TopkExchange(3, 5, torch.device("cpu"))
    ex.top_scores.copy_(torch.arange(15, dtype=torch.float32).view(3, 5))
    ex.top_idx.copy_(torch.arange(15, dtype=torch.int64).view(3, 5))
    t0 = time.monotonic()
    try:
        ex.start().finish(merge=numpy_merge, timeout_s=1.0)
        ret[0] = "returned"
    except ShardExchangeTimeout as exc:
        ret[0] = ("timeout", time.monotonic() - t0, str(exc))
    os._exit(0)      # the group is unusable after the time-out; do not wait for the absent rank on the way out


def test_exchange_times_out_when_a_rank_never_joins():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_absent_rank_worker, args=(2, port, ret), nprocs=2, join=True)
        assert ret.get(1) == "left without joining"
        kind, waited, msg = ret.get(0)
        assert kind == "timeout" and 0.9 <= waited < 3.0, (kind, waited)
        assert "did not complete within" in msg and "2 ranks" in msg


def test_exchange_block_layout():
    """The send block holds scores and indices at the offsets tq_topk_merge_gathered is told about."""
    from project_tensor_b200.sharded import TopkExchange
    ex = TopkExchange(3, 5, torch.device("cpu"))
    assert ex.idx_offset % 16 == 0 and ex.idx_offset >= 4 * 15 and ex.block_bytes == ex.idx_offset + 8 * 15
    ex.top_scores.fill_(1.5)
    ex.top_idx.fill_(7)
    assert ex.send[:60].view(torch.float32).eq(1.5).all()
    assert ex.send[ex.idx_offset:].view(torch.int64).eq(7).all()
    got_s, got_i = ex.start().finish(merge=numpy_merge)      # world of one: nothing to gather
    assert got_s.shape == (3, 5) and bool((got_i == 7).all())
