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


def merge_topk_across_ranks(top_scores, top_idx, group=None, merge: Optional[Callable] = None):
    """All-gather every rank's per-query top-k (``top_scores`` float32 [Q, k] descending, ``top_idx``
    int64 [Q, k] global key indices) and merge them into the global top-k, identical on all ranks.
    Ties go to the lower rank, i.e. to the lower global index for contiguous shards.

    ``merge`` replaces the GPU merge kernel; the CPU tests use it to exercise the gather plumbing
    over gloo without a device."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    top_scores = top_scores.contiguous()
    top_idx = top_idx.contiguous()
    if world == 1:
        gathered_s, gathered_i = top_scores[None], top_idx[None]
    else:
        # one collective for both arrays: the score bits ride in an int64 beside the indices
        k = top_scores.shape[-1]
        packed = torch.cat((top_scores.view(torch.int32).to(torch.int64), top_idx), dim=-1)
        gathered = torch.empty((world,) + tuple(packed.shape), dtype=torch.int64, device=packed.device)
        if packed.is_cuda:
            dist.all_gather_into_tensor(gathered, packed, group=group)
        else:  # gloo
            dist.all_gather(list(gathered.unbind(0)), packed, group=group)
        gathered_s = gathered[..., :k].to(torch.int32).view(torch.float32).contiguous()
        gathered_i = gathered[..., k:].contiguous()
    return (merge or _merge_on_gpu)(gathered_s, gathered_i)


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

    def search(self, queries, k: int, group=None):
        top_s, top_i = self.quantizer.attention_scores(queries, self.encoding(), topk=k, index_base=self.start)
        import torch
        if not isinstance(top_s, torch.Tensor):
            top_s, top_i = torch.as_tensor(top_s, device=self.device), torch.as_tensor(top_i, device=self.device)
        return merge_topk_across_ranks(top_s, top_i, group=group)
