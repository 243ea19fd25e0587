"""Key shards across the GPUs of one box.

Every key is independent, so quantizing and scoring shard with no exchange at all: rank r of W
owns the contiguous key range ``shard_range(n, r, W)`` and holds the (small) rotation, codebook and
projection itself.  The one collective on the path is the all-gather of per-shard results -- score
slabs, or the k best (score, global index) pairs per query -- followed by a merge kernel that every
rank runs on the gathered lists.  ``torch.distributed`` (NCCL on GPUs) does the gather; nothing here
touches a peer's memory directly.

The reference (Project-Tensor) is single-device and has no counterpart for this module.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

from . import _native


def shard_range(n: int, rank: int, world: int) -> Tuple[int, int]:
    """[start, stop) of the keys owned by ``rank`` when ``n`` keys are split as evenly as possible
    into ``world`` contiguous ranges (the first ``n % world`` ranks hold one key more)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of size {world}")
    base, extra = divmod(int(n), world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


class ShardExchangeTimeout(RuntimeError):
    """The all-gather of a TopkExchange did not complete in time: a rank is missing, hung or gone.  The
    process group is unusable afterwards (its abort has been asked for where the backend has one)."""


def _merge_on_gpu(gathered_scores, gathered_idx):
    """[W, Q, k] candidate lists -> ([Q, k], [Q, k]) through tq_topk_merge."""
    import torch
    lists, queries, k = gathered_scores.shape
    out_s = torch.empty((queries, k), dtype=torch.float32, device=gathered_scores.device)
    out_i = torch.empty((queries, k), dtype=torch.int64, device=gathered_scores.device)
    with torch.cuda.device(gathered_scores.device):
        stream = torch.cuda.current_stream(gathered_scores.device).cuda_stream
        _native.check(_native.load().tq_topk_merge(gathered_scores.data_ptr(), gathered_idx.data_ptr(), lists,
                                                   queries, k, out_s.data_ptr(), out_i.data_ptr(), stream))
    return out_s, out_i


class TopkExchange:
    """The one collective of the path: every rank's per-query top-k -> the global top-k on every rank.

    A rank owns one send block of bytes, float32 [Q][k] scores at offset 0 and int64 [Q][k] global indices at
    a 16-byte aligned offset behind them.  ``top_scores`` / ``top_idx`` are views of that block: hand them to
    ``TurboQuantProd.attention_scores(..., out=(ex.top_scores, ex.top_idx))`` and the scoring call writes the
    candidates where the collective reads them.  ``start()`` enqueues ONE all-gather of the blocks without
    blocking the host or the compute stream; ``finish()`` makes the current stream wait for it and runs the merge
    kernel straight on the gathered blocks (``tq_topk_merge_gathered``).  Between the two the caller may enqueue the
    next step's work, which then overlaps the collective.

    ``timeout_s``: with a value, ``finish()`` waits on the host, at most that long, for the collective; when the
    time runs out it asks the backend to abort the group and raises ``ShardExchangeTimeout`` instead of hanging on
    a rank that never joined.  ``merge`` replaces the GPU merge kernel by a function of the gathered
    ``(scores [W, Q, k], idx [W, Q, k])``; the CPU tests run the plumbing over gloo that way.
    """

    def __init__(self, queries: int, k: int, device, group=None):
        import torch
        import torch.distributed as dist
        self.queries, self.k, self.group = int(queries), int(k), group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        cnt = self.queries * self.k
        self.idx_offset = (4 * cnt + 15) // 16 * 16
        self.block_bytes = self.idx_offset + 8 * cnt
        self.send = torch.empty((self.block_bytes,), dtype=torch.uint8, device=device)
        self.top_scores = self.send[:4 * cnt].view(torch.float32).view(self.queries, self.k)
        self.top_idx = self.send[self.idx_offset:].view(torch.int64).view(self.queries, self.k)
        self.gathered = (self.send[None] if self.world == 1 else
                         torch.empty((self.world, self.block_bytes), dtype=torch.uint8, device=device))
        self._work = None

    def start(self):
        import torch.distributed as dist
        if self.world > 1:
            if self.send.is_cuda:
                self._work = dist.all_gather_into_tensor(self.gathered, self.send, group=self.group, async_op=True)
            else:  # gloo
                self._work = dist.all_gather(list(self.gathered.unbind(0)), self.send, group=self.group, async_op=True)
        return self

    def _abort_group(self):
        import torch.distributed as dist
        try:
            pg = self.group if self.group is not None else dist.group.WORLD
            backend = pg._get_backend(self.send.device)
            if hasattr(backend, "abort"):
                backend.abort()
        except Exception:
            pass    # best effort: the caller gets the time-out either way

    def finish(self, merge: Optional[Callable] = None, timeout_s: Optional[float] = None):
        import time
        import torch
        work, self._work = self._work, None
        if work is not None:
            if timeout_s is not None:
                deadline = time.monotonic() + float(timeout_s)
                while not work.is_completed():
                    if time.monotonic() > deadline:
                        self._abort_group()
                        raise ShardExchangeTimeout(
                            f"all-gather of the top-{self.k} candidates did not complete within {timeout_s} s "
                            f"({self.world} ranks expected)")
                    time.sleep(0.0005)
            work.wait()     # NCCL: the current stream waits for the collective; gloo: the host does
        cnt = self.queries * self.k
        if merge is not None:
            gs = self.gathered[:, :4 * cnt].contiguous().view(torch.float32).view(self.world, self.queries, self.k)
            gi = self.gathered[:, self.idx_offset:].contiguous().view(torch.int64).view(self.world, self.queries, self.k)
            return merge(gs, gi)
        dev = self.send.device
        out_s = torch.empty((self.queries, self.k), dtype=torch.float32, device=dev)
        out_i = torch.empty((self.queries, self.k), dtype=torch.int64, device=dev)
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream(dev).cuda_stream
            _native.check(_native.load().tq_topk_merge_gathered(
                self.gathered.data_ptr(), self.block_bytes, self.idx_offset, self.world, self.queries, self.k,
                out_s.data_ptr(), out_i.data_ptr(), stream))
        return out_s, out_i


def merge_topk_across_ranks(top_scores, top_idx, group=None, merge: Optional[Callable] = None,
                            timeout_s: Optional[float] = None):
    """All-gather every rank's per-query top-k (``top_scores`` float32 [Q, k] descending, ``top_idx``
    int64 [Q, k] global key indices) and merge them into the global top-k, identical on all ranks.
    Ties go to the lower rank, i.e. to the lower global index for contiguous shards.

    Convenience form of ``TopkExchange`` for results that already exist as two tensors (they are copied into
    a send block first); see there for ``merge`` and ``timeout_s``."""
    ex = TopkExchange(top_scores.shape[0], top_scores.shape[1], top_scores.device, group=group)
    ex.top_scores.copy_(top_scores)
    ex.top_idx.copy_(top_idx)
    return ex.start().finish(merge=merge, timeout_s=timeout_s)


def scatter_merge_topk(top_scores, top_idx, group=None, merge: Optional[Callable] = None):
    """Global top-k for many queries without every rank merging every query: rank r of W receives all ranks'
    candidates for queries [r*Q/W, (r+1)*Q/W) only (one all-to-all of the candidate lists, the exchange pattern of a
    reduce-scatter) and merges those; returns ``(scores [Q/W, k], idx [Q/W, k], first_query)``.  Compared with the
    all-gather form, every rank receives and merges 1/W of the candidates, which matters once Q * k * W entries no
    longer fit a small message.  Q must be a multiple of W.  ``merge`` as in TopkExchange."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    nq, k = top_scores.shape
    if nq % world:
        raise ValueError(f"{nq} queries do not split evenly over {world} ranks")
    per = nq // world
    send_s = top_scores.contiguous().view(world, per, k)
    send_i = top_idx.contiguous().view(world, per, k)
    if world == 1:
        recv_s, recv_i = send_s, send_i
    else:
        recv_s, recv_i = torch.empty_like(send_s), torch.empty_like(send_i)
        if send_s.is_cuda:
            dist.all_to_all_single(recv_s, send_s, group=group)      # block j of the result comes from rank j
            dist.all_to_all_single(recv_i, send_i, group=group)
        else:  # gloo has no all-to-all for every build: W broadcast-free point exchanges through all_gather
            all_s = [torch.empty_like(send_s) for _ in range(world)]
            all_i = [torch.empty_like(send_i) for _ in range(world)]
            dist.all_gather(all_s, send_s, group=group)
            dist.all_gather(all_i, send_i, group=group)
            recv_s = torch.stack([a[rank] for a in all_s])
            recv_i = torch.stack([a[rank] for a in all_i])
    out_s, out_i = (merge or _merge_on_gpu)(recv_s.contiguous(), recv_i.contiguous())
    return out_s, out_i, rank * per


def gather_score_slabs(scores, group=None):
    """All-gather per-shard score slabs [Q, n_local] into [Q, n_total] (equal shard sizes)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return scores
    scores = scores.contiguous()
    out = torch.empty((world,) + tuple(scores.shape), dtype=scores.dtype, device=scores.device)
    dist.all_gather(list(out.unbind(0)), scores, group=group)
    return out.permute(1, 0, 2).reshape(scores.shape[0], -1)


class ShardedKeyIndex:
    """The keys of one rank, quantized chunk by chunk into preallocated packed buffers, and top-k
    retrieval over all ranks' keys.

        index = ShardedKeyIndex(quantizer, n_total)        # every rank, same arguments
        for chunk in my_chunks: index.add(chunk)            # device or host arrays, (m, d)
        scores, ids = index.search(queries, k=100)          # identical on every rank
    """

    def __init__(self, quantizer, n_total: int, rank: Optional[int] = None, world: Optional[int] = None,
                 device=None):
        import torch
        import torch.distributed as dist
        self.quantizer = quantizer
        self.world = world if world is not None else (dist.get_world_size() if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank() if dist.is_initialized() else 0)
        self.start, self.stop = shard_range(n_total, self.rank, self.world)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        code_bytes, sign_bytes = quantizer._plans.row_bytes()
        n = self.stop - self.start
        self.codes = torch.empty((n, code_bytes), dtype=torch.uint8, device=self.device)
        self.signs = torch.empty((n, sign_bytes), dtype=torch.uint8, device=self.device)
        self.norms = torch.empty((n,), dtype=torch.float32, device=self.device)
        self.residual_norms = torch.empty((n,), dtype=torch.float32, device=self.device)
        self.filled = 0

    def add(self, keys) -> None:
        """Quantize ``keys`` (m, d) straight into the next m rows of this rank's packed buffers."""
        from .turboquant import _stage
        staged = _stage(keys, self.quantizer.dimension, device=self.device)
        m = int(staged.tensor.shape[0])
        if self.filled + m > self.stop - self.start:
            raise ValueError("more keys than this rank's shard holds")
        s = slice(self.filled, self.filled + m)
        out = {"codes": self.codes[s], "signs": self.signs[s], "norms": self.norms[s],
               "residual_norms": self.residual_norms[s]}
        if all(t.data_ptr() % 16 == 0 for t in out.values()):
            self.quantizer.mse._quantize_staged(staged, self.quantizer._plans, True, out=out)
        else:
            # a chunk that starts off a 16-byte boundary of the norm arrays (row count so far not a multiple
            # of 4): the kernels want aligned outputs, so quantize into fresh buffers and copy
            pk = self.quantizer.mse._quantize_staged(staged, self.quantizer._plans, True)
            out["codes"].copy_(pk.codes)
            out["signs"].copy_(pk.signs)
            out["norms"].copy_(pk.norms)
            out["residual_norms"].copy_(pk.residual_norms)
        self.filled += m

    def encoding(self):
        from .turboquant import TurboQuantProdEncoding, _Packed, _encoding_from_packed
        n = self.filled
        pk = _Packed(self.codes[:n], self.signs[:n], self.norms[:n], self.residual_norms[:n], n, "torch",
                     self.device, self.quantizer._plans)
        return _encoding_from_packed(TurboQuantProdEncoding, pk, (n,))

    def search_start(self, queries, k: int, group=None) -> TopkExchange:
        """Score this rank's keys and enqueue the all-gather of the candidates; ``.finish()`` of the returned
        exchange gives the global (scores, indices).  Work enqueued in between overlaps the collective."""
        from .turboquant import _stage
        q = _stage(queries, self.quantizer.dimension, device=self.device).tensor
        ex = TopkExchange(q.shape[0], k, self.device, group=group)
        self.quantizer.attention_scores(q, self.encoding(), topk=k, index_base=self.start, out=(ex.top_scores, ex.top_idx))
        return ex.start()

    def search(self, queries, k: int, group=None, timeout_s: Optional[float] = None):
        return self.search_start(queries, k, group=group).finish(timeout_s=timeout_s)
