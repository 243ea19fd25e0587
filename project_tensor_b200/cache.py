"""A growing packed key cache: the step before decode scoring.

The reference's ``TurboQuantProd.quantize`` (tensor_gpu_v2/_quant.py:297-315) builds a new immutable encoding
from all keys at once.  A decoder adds one key per sequence and head per step and scores against everything so
far; re-quantizing is out of the question and so is allocating per step.  ``PackedKeyCache`` keeps the packed
arrays of ``groups`` (= batch x KV heads) sequences at a fixed capacity and

  * ``append``s new keys with one kernel launch straight into place (``tq_prod_append``: the position is read
    from device memory, so a captured CUDA graph of the step stays valid while the cache grows);
  * ``scores`` queries against the filled part of every group (``tq_score_cache``), optionally top-k only.

Row p of group g holds exactly what ``quantize`` gives for that key: the append kernel is the reference-order
kernel, bit-identical to the oracle.
"""
from __future__ import annotations

from typing import Any, Optional

from . import _native
from . import turboquant as _tq


class PackedKeyCache:
    """Packed TurboQuantProd keys of ``groups`` sequences, ``capacity`` rows each, all of one length."""

    #: appends of at most this many rows go through the one-launch append kernel; larger ones (prefill) through
    #: the bulk quantizer and a copy of the packed rows into place
    SMALL_APPEND_ROWS = 4096

    def __init__(self, quantizer: "_tq.TurboQuantProd", groups: int, capacity: int, device: Any = None):
        if not isinstance(quantizer, _tq.TurboQuantProd):
            raise TypeError("PackedKeyCache holds TurboQuantProd keys")
        if groups < 1 or capacity < 1:
            raise ValueError("groups and capacity must be positive")
        if groups * capacity >= 1 << 32:
            raise ValueError("groups * capacity must stay below 2^32")
        torch = _tq._require_cuda()
        self.quantizer, self.groups, self.capacity = quantizer, int(groups), int(capacity)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._plans = quantizer._plans
        code_bytes, sign_bytes = self._plans.row_bytes()
        rows = self.groups * self.capacity
        dev = self.device
        self.codes = torch.zeros((rows, code_bytes), dtype=torch.uint8, device=dev)
        self.signs = torch.zeros((rows, sign_bytes), dtype=torch.uint8, device=dev)
        self.norms = torch.zeros((rows,), dtype=torch.float32, device=dev)
        self.residual_norms = torch.zeros((rows,), dtype=torch.float32, device=dev)
        self.length_device = torch.zeros((1,), dtype=torch.int64, device=dev)
        self._length = 0     # host mirror; replays of a captured append do not pass through here (see sync_length)

    # ---- length ---------------------------------------------------------------------------------
    def __len__(self) -> int:
        return self._length

    def sync_length(self) -> int:
        """Read the length back from the device (needed after replaying a CUDA graph that appends)."""
        self._length = int(self.length_device.item())
        self._plans.check_status(self.device)
        return self._length

    def reset(self) -> None:
        self.length_device.zero_()
        self._length = 0

    # ---- append ---------------------------------------------------------------------------------
    def append(self, keys: Any) -> None:
        """Add keys of shape (groups, tokens, d), or (groups, d) for one token each, behind the present rows.
        A contiguous float32 CUDA tensor of at most ``SMALL_APPEND_ROWS`` rows is appended with no allocation
        and no host synchronisation (capturable in a CUDA graph)."""
        torch = _tq._torch()
        d = self.quantizer.dimension
        array = _tq._to_array(keys)
        _tq._ensure_last_dim(array, d)
        if array.ndim == 2:
            tokens = 1
        elif array.ndim == 3:
            tokens = int(array.shape[1])
        else:
            raise ValueError(f"expected keys of shape (groups, tokens, {d}) or (groups, {d}), got {tuple(array.shape)}")
        if int(array.shape[0]) != self.groups:
            raise ValueError(f"expected {self.groups} groups of keys, got {int(array.shape[0])}")
        if self._length + tokens > self.capacity:
            raise ValueError(f"cache is full: {self._length} + {tokens} rows exceed the capacity {self.capacity}")
        if tokens == 0:
            return
        staged = _tq._stage(keys, d, device=self.device)
        x = staged.tensor
        lib = _native.load()
        handle = self._plans.handle(self.device)
        rows = self.groups * tokens
        with torch.cuda.device(self.device):
            if rows <= self.SMALL_APPEND_ROWS:
                _native.check(lib.tq_prod_append(handle, x.data_ptr(), self.groups, tokens, self.codes.data_ptr(),
                                                 self.signs.data_ptr(), self.residual_norms.data_ptr(),
                                                 self.norms.data_ptr(), self.capacity, self.length_device.data_ptr(), 1,
                                                 _tq._stream_ptr(self.device)))
            else:
                pk = self.quantizer.mse._quantize_staged(staged, self._plans, True)
                lo, hi = self._length, self._length + tokens
                g, c = self.groups, self.capacity
                self.codes.view(g, c, -1)[:, lo:hi] = pk.codes.view(g, tokens, -1)
                self.signs.view(g, c, -1)[:, lo:hi] = pk.signs.view(g, tokens, -1)
                self.norms.view(g, c)[:, lo:hi] = pk.norms.view(g, tokens)
                self.residual_norms.view(g, c)[:, lo:hi] = pk.residual_norms.view(g, tokens)
                self.length_device.add_(tokens)
        self._length += tokens

    # ---- scoring --------------------------------------------------------------------------------
    def scores(self, queries: Any, *, topk: Optional[int] = None, return_matrix: Optional[bool] = None):
        """Score ``queries`` of shape (groups, q_per_group, d) (or (groups, d)) against the filled rows of their
        group.  Returns the scores, shape (groups, q_per_group, len(self)); with ``topk=k`` returns
        ``(top_scores, top_positions)`` of shape (groups, q_per_group, k), descending, positions counted inside
        the group (-1 and -inf fill slots beyond the length); ``return_matrix=True`` adds the matrix."""
        torch = _tq._torch()
        d = self.quantizer.dimension
        array = _tq._to_array(queries)
        _tq._ensure_last_dim(array, d)
        if array.ndim not in (2, 3) or int(array.shape[0]) != self.groups:
            raise ValueError(f"expected queries of shape ({self.groups}, q_per_group, {d}), got {tuple(array.shape)}")
        qpg = 1 if array.ndim == 2 else int(array.shape[1])
        staged = _tq._stage(queries, d, device=self.device)
        q = staged.tensor
        k = int(topk) if topk else 0
        want_matrix = (k == 0) if return_matrix is None else bool(return_matrix)
        if k == 0 and not want_matrix:
            raise ValueError("nothing to compute: no top-k requested and return_matrix is False")
        n = self._length
        lib = _native.load()
        handle = self._plans.handle(self.device)
        dev = self.device
        with torch.cuda.device(dev):
            mat = torch.empty((self.groups, qpg, n), dtype=torch.float32, device=dev) if want_matrix else None
            top_s = torch.empty((self.groups, qpg, k), dtype=torch.float32, device=dev) if k else None
            top_i = torch.empty((self.groups, qpg, k), dtype=torch.int64, device=dev) if k else None
            if n == 0:
                # nothing to score yet: a matrix without columns, top-k slots at their fill values
                if k:
                    top_s.fill_(float("-inf"))
                    top_i.fill_(-1)
                if k == 0:
                    return _tq._deliver(mat, staged.kind, self._plans)
                result = (_tq._deliver(top_s, staged.kind, self._plans), _tq._deliver(top_i, staged.kind))
                return result + (_tq._deliver(mat, staged.kind, self._plans),) if want_matrix else result
            need = int(lib.tq_topk_scratch_bytes(handle, self.groups, qpg, n, k))
            scratch = torch.empty((max(need, 16),), dtype=torch.uint8, device=dev)
            _native.check(lib.tq_score_cache(handle, q.data_ptr(), self.groups, qpg, self.codes.data_ptr(),
                                             self.signs.data_ptr(), self.residual_norms.data_ptr(),
                                             self.norms.data_ptr(), n, self.capacity, _tq._ptr(mat), k,
                                             _tq._ptr(top_s), _tq._ptr(top_i), 0, scratch.data_ptr(), scratch.numel(),
                                             _tq._stream_ptr(dev)))
            if k:
                # rows of the arrays -> positions inside the group; empty slots stay -1
                base = (torch.arange(self.groups, device=dev, dtype=torch.int64) * self.capacity).view(-1, 1, 1)
                top_i = torch.where(top_i >= 0, top_i - base, top_i)
        if k == 0:
            return _tq._deliver(mat, staged.kind, self._plans)
        result = (_tq._deliver(top_s, staged.kind, self._plans), _tq._deliver(top_i, staged.kind))
        return result + (_tq._deliver(mat, staged.kind, self._plans),) if want_matrix else result

    # ---- views ----------------------------------------------------------------------------------
    def encoding(self, group: int):
        """The filled rows of one group as a TurboQuantProdEncoding (a view of the cache, no copy)."""
        if not 0 <= group < self.groups:
            raise IndexError(f"group {group} outside [0, {self.groups})")
        lo, n = group * self.capacity, self._length
        pk = _tq._Packed(self.codes[lo:lo + n], self.signs[lo:lo + n], self.norms[lo:lo + n],
                         self.residual_norms[lo:lo + n], n, "torch", self.device, self._plans)
        return _tq._encoding_from_packed(_tq.TurboQuantProdEncoding, pk, (n,))


class PackedKVCache:
    """Packed keys (TurboQuantProd) and values (TurboQuantMSE) of ``groups`` sequences/heads, ``capacity`` rows
    each, and decode attention over them without materialising scores or dequantized values.

    ``attend(queries)`` returns ``softmax(scale * attention_score(q, keys)) @ dequantize(values)`` per group --
    the reference's ``scaled_dot_product_attention`` (tensor_gpu_v2/_core.py:1606-1683, no mask, no dropout)
    with the key product replaced by ``TurboQuantProd.attention_score`` (_quant.py:334-358) and the values by
    ``TurboQuantMSE.dequantize`` (_quant.py:251-254) -- computed by ``tq_decode_attention`` in one pass over
    the packed rows (d = 64 or 128, at most 4 code bits for keys and values)."""

    def __init__(self, key_quantizer: "_tq.TurboQuantProd", value_quantizer: "_tq.TurboQuantMSE", groups: int,
                 capacity: int, device: Any = None):
        if not isinstance(value_quantizer, _tq.TurboQuantMSE):
            raise TypeError("PackedKVCache holds TurboQuantMSE values")
        if value_quantizer.dimension != key_quantizer.dimension:
            raise ValueError(f"keys have dimension {key_quantizer.dimension}, values {value_quantizer.dimension}")
        self.keys = PackedKeyCache(key_quantizer, groups, capacity, device)
        torch = _tq._torch()
        self.value_quantizer = value_quantizer
        self.groups, self.capacity, self.device = self.keys.groups, self.keys.capacity, self.keys.device
        self._vplans = value_quantizer._plans
        rows = self.groups * self.capacity
        self.value_codes = torch.zeros((rows, self._vplans.row_bytes()[0]), dtype=torch.uint8, device=self.device)
        self.value_norms = torch.zeros((rows,), dtype=torch.float32, device=self.device)

    def __len__(self) -> int:
        return len(self.keys)

    def sync_length(self) -> int:
        return self.keys.sync_length()

    def reset(self) -> None:
        self.keys.reset()

    def append(self, keys: Any, values: Any) -> None:
        """Add one key and one value per token: both of shape (groups, tokens, d) or (groups, d).  The values
        are written at the position the keys take; the shared length advances once."""
        torch = _tq._torch()
        d = self.value_quantizer.dimension
        karr, varr = _tq._to_array(keys), _tq._to_array(values)
        _tq._ensure_last_dim(varr, d)
        if tuple(karr.shape) != tuple(varr.shape):
            raise ValueError(f"keys {tuple(karr.shape)} and values {tuple(varr.shape)} differ in shape")
        if varr.ndim not in (2, 3) or int(varr.shape[0]) != self.groups:
            raise ValueError(f"expected values of shape ({self.groups}, tokens, {d}) or ({self.groups}, {d}), "
                             f"got {tuple(varr.shape)}")
        tokens = 1 if varr.ndim == 2 else int(varr.shape[1])
        lo = len(self.keys)
        if lo + tokens > self.capacity:
            raise ValueError(f"cache is full: {lo} + {tokens} rows exceed the capacity {self.capacity}")
        if tokens == 0:
            return
        staged = _tq._stage(values, d, device=self.device)
        with torch.cuda.device(self.device):
            if self.groups * tokens <= PackedKeyCache.SMALL_APPEND_ROWS:
                # the values first, without advancing: the key append that follows reads the same length
                _native.check(_native.load().tq_mse_append(
                    self._vplans.handle(self.device), staged.tensor.data_ptr(), self.groups, tokens,
                    self.value_codes.data_ptr(), self.value_norms.data_ptr(), self.capacity,
                    self.keys.length_device.data_ptr(), 0, _tq._stream_ptr(self.device)))
            else:
                pk = self.value_quantizer._quantize_staged(staged, self._vplans, False)
                g, c = self.groups, self.capacity
                self.value_codes.view(g, c, -1)[:, lo:lo + tokens] = pk.codes.view(g, tokens, -1)
                self.value_norms.view(g, c)[:, lo:lo + tokens] = pk.norms.view(g, tokens)
        self.keys.append(keys)

    def attend(self, queries: Any, *, scale: Optional[float] = None, use_device_length: bool = False):
        """``queries`` of shape (groups, q_per_group, d) or (groups, d) -> attention output of the same shape.
        ``scale`` defaults to d ** -0.5.  ``use_device_length=True`` makes the kernel read the number of keys from
        the device-side counter (up to the capacity) instead of the host's mirror, for a step that is replayed from
        a CUDA graph while the cache grows."""
        torch = _tq._torch()
        d = self.value_quantizer.dimension
        array = _tq._to_array(queries)
        _tq._ensure_last_dim(array, d)
        if array.ndim not in (2, 3) or int(array.shape[0]) != self.groups:
            raise ValueError(f"expected queries of shape ({self.groups}, q_per_group, {d}), got {tuple(array.shape)}")
        qpg = 1 if array.ndim == 2 else int(array.shape[1])
        staged = _tq._stage(queries, d, device=self.device)
        n = self.capacity if use_device_length else len(self.keys)
        lib = _native.load()
        kc, dev = self.keys, self.device
        kh, vh = kc._plans.handle(dev), self._vplans.handle(dev)
        with torch.cuda.device(dev):
            out = torch.empty((self.groups, qpg, d), dtype=torch.float32, device=dev)
            need = int(lib.tq_decode_attention_scratch_bytes(kh, self.groups, qpg, n))
            scratch = torch.empty((max(need, 16),), dtype=torch.uint8, device=dev)
            _native.check(lib.tq_decode_attention(
                kh, vh, staged.tensor.data_ptr(), self.groups, qpg, kc.codes.data_ptr(), kc.signs.data_ptr(),
                kc.residual_norms.data_ptr(), kc.norms.data_ptr(), self.value_codes.data_ptr(),
                self.value_norms.data_ptr(), n, self.capacity,
                kc.length_device.data_ptr() if use_device_length else None, float(scale or 0.0), out.data_ptr(),
                scratch.data_ptr(), scratch.numel(), _tq._stream_ptr(dev)))
        out = _tq._deliver(out, staged.kind)
        return out.reshape(tuple(array.shape))

    def value_encoding(self, group: int):
        """The filled value rows of one group as a TurboQuantMSEEncoding (a view of the cache)."""
        if not 0 <= group < self.groups:
            raise IndexError(f"group {group} outside [0, {self.groups})")
        lo, n = group * self.capacity, len(self.keys)
        pk = _tq._Packed(self.value_codes[lo:lo + n], None, self.value_norms[lo:lo + n], None, n, "torch", self.device,
                         self._vplans)
        return _tq._encoding_from_packed(_tq.TurboQuantMSEEncoding, pk, (n,))
