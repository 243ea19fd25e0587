"""TurboQuant quantizers with the public surface of Project-Tensor's ``tensor_gpu_v2/_quant.py``
and all array arithmetic in hand-written sm_100a kernels (libtq_sm100.so, called through ctypes).

Same names, constructor keywords, method names, encoding field names and ``ValueError`` texts as
the reference (``TurboQuantMSE`` _quant.py:172-254, ``TurboQuantProd`` :257-358, encodings
:156-169, helpers :361-374).  What differs, on purpose:

* Inputs may be NumPy arrays, anything exposing ``__cuda_array_interface__`` (CuPy arrays, torch
  CUDA tensors, ...) or a ``Tensor``-like wrapper whose ``.data`` is one of those.  Every input is
  computed on the GPU; NumPy callers get NumPy results back, device callers get device arrays.
  There is no CPU path: without a CUDA device (or without the built library) calls raise.
* Arithmetic is float32, like the reference's documented use; other float dtypes are cast.
* Encodings keep bit-packed device buffers (``d*bits/8`` bytes of codes and ``d/8`` bytes of QJL
  signs per vector).  ``encoding.indices`` / ``encoding.qjl`` unpack on first access into the
  reference's ``uint8 (N, d)`` / ``int8 (N, d)`` arrays.
* ``bits`` above 8 for the MSE stage and ``dimension`` above 1024 are rejected.
* ``TurboQuantProd.attention_scores`` (plural) is an addition: many queries against shared keys
  in one pass, optionally with a fused per-query top-k.  The reference's users obtain the same
  matrix by calling ``attention_score`` once per query.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

import numpy as np

from . import _native
from .codebook import (_build_lloyd_max_codebook, _random_orthogonal_matrix,
                       _random_projection_matrix)

_MAX_BITS = 8
_MAX_DIM = 1024


# ------------------------------------------------------------------------------------------------
# small host helpers
# ------------------------------------------------------------------------------------------------
class Tensor:
    """Minimal stand-in for the reference's ``Tensor``: a holder whose ``.data`` is the array.
    The quantizers only ever read ``.data`` (_quant.py:27-34); no autograd lives here."""

    def __init__(self, data, requires_grad: bool = False):
        self.data = data
        self.requires_grad = bool(requires_grad)

    @property
    def shape(self):
        return self.data.shape


def _torch():
    import torch  # imported lazily: constructing a quantizer needs NumPy only
    return torch


def _is_device_array(obj: Any) -> bool:
    return hasattr(obj, "__cuda_array_interface__")


def _to_array(data: Any):
    """Unwrap a ``Tensor``-like object; leave arrays alone (_quant.py:31-34)."""
    if isinstance(data, np.ndarray) or _is_device_array(data):
        return data
    torch = _torch_if_loaded()
    if torch is not None and isinstance(data, torch.Tensor):
        return data
    if isinstance(data, Tensor) or (hasattr(data, "data") and hasattr(data, "requires_grad")):
        return data.data
    return np.asarray(data)


def _torch_if_loaded():
    import sys
    return sys.modules.get("torch")


def _ensure_last_dim(array, dim: int) -> None:
    if array.ndim == 0 or array.shape[-1] != dim:
        raise ValueError(
            f"expected input with trailing dimension {dim}, got shape {tuple(array.shape)}"
        )


def _quant_index_dtype(bits: int):
    if bits <= 8:
        return np.uint8
    if bits <= 16:
        return np.uint16
    return np.int32


class _Staged:
    """An input brought to the GPU as a contiguous float32 (N, d) torch tensor, remembering what
    kind of array the caller used so that results can be handed back in the same kind."""

    __slots__ = ("tensor", "prefix", "kind", "device")

    def __init__(self, tensor, prefix, kind, device):
        self.tensor, self.prefix, self.kind, self.device = tensor, prefix, kind, device


def _require_cuda():
    torch = _torch()
    if not torch.cuda.is_available():
        raise _native.TurboQuantNativeError(
            "TurboQuant needs a CUDA device (B200, sm_100a); there is no CPU fallback")
    return torch


def _stage(data: Any, dim: int, device=None) -> _Staged:
    array = _to_array(data)
    _ensure_last_dim(array, dim)
    prefix = tuple(array.shape[:-1])
    torch = _require_cuda()
    if isinstance(array, np.ndarray):
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        host = np.ascontiguousarray(array.reshape(-1, dim), dtype=np.float32)
        t = torch.from_numpy(host)
        return _Staged(t.to(dev, non_blocking=t.is_pinned()), prefix, "numpy", dev)
    if isinstance(array, torch.Tensor):
        if array.is_cuda:
            t = array.reshape(-1, dim).to(torch.float32).contiguous()
            return _Staged(t, prefix, "torch", array.device)
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        t = array.reshape(-1, dim).to(torch.float32).contiguous()
        return _Staged(t.to(dev), prefix, "torch_cpu", dev)
    # CuPy or any other __cuda_array_interface__ producer: zero-copy view
    t = torch.as_tensor(array, device="cuda")
    kind = "cupy" if type(array).__module__.split(".")[0] == "cupy" else "torch"
    return _Staged(t.reshape(-1, dim).to(torch.float32).contiguous(), prefix, kind, t.device)


def _deliver(tensor, kind: str, plans: "Optional[_PlanSet]" = None):
    """Hand a device tensor back in the caller's kind of array.  A result that goes to host memory synchronises
    anyway; with ``plans`` the status word of the kernels is read at that point, so that the output of a kernel
    that gave up on a bounded wait is never handed out as if it were complete."""
    if plans is not None and kind in ("numpy", "torch_cpu"):
        plans.check_status(tensor.device)
    if kind == "numpy":
        return _to_host(tensor).numpy()
    if kind == "torch_cpu":
        return _to_host(tensor)
    if kind == "cupy":
        try:
            import cupy
            return cupy.asarray(tensor)
        except ImportError:  # CuPy-like producer without CuPy importable: give the torch view
            return tensor
    return tensor


_PINNED_FROM_BYTES = 1 << 20


def _to_host(tensor):
    """Device tensor -> CPU tensor.  Results of a megabyte and more land in page-locked memory from torch's caching host
    allocator (the block goes back to that cache when the array that wraps it dies): a copy into pageable memory runs at
    a few GB/s, so that the 128 MiB score matrix of 32 queries x 1,048,576 keys took 62 ms to hand back, against 3 ms
    at the rate of the link."""
    torch = _torch()
    if tensor.device.type != "cuda" or tensor.numel() * tensor.element_size() < _PINNED_FROM_BYTES:
        return tensor.cpu()
    host = torch.empty(tensor.shape, dtype=tensor.dtype, pin_memory=True)
    host.copy_(tensor, non_blocking=True)
    torch.cuda.current_stream(tensor.device).synchronize()
    return host


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _stream_ptr(device) -> int:
    return _torch().cuda.current_stream(device).cuda_stream


# ------------------------------------------------------------------------------------------------
# plans: one set of device constants per (quantizer, GPU)
# ------------------------------------------------------------------------------------------------
class _PlanSet:
    """Lazily created tq_plan handles of one quantizer, one per CUDA device index."""

    def __init__(self, dimension, bits_mse, rotation, codebook, projection):
        self.dimension, self.bits_mse = dimension, bits_mse
        self._rotation = np.ascontiguousarray(rotation, dtype=np.float32)
        self._codebook = np.ascontiguousarray(codebook, dtype=np.float32)
        self._projection = None if projection is None else np.ascontiguousarray(projection, dtype=np.float32)
        self._plans: Dict[int, int] = {}
        self._geometry: Optional[Tuple[int, int]] = None
        self._path = _native.TQ_PATH_AUTO

    def handle(self, device) -> int:
        idx = device.index if device.index is not None else _torch().cuda.current_device()
        h = self._plans.get(idx)
        if h is None:
            lib = _native.load()
            out = ctypes.c_void_p()
            proj = None if self._projection is None else self._projection.ctypes.data
            _native.check(lib.tq_plan_create(self.dimension, self.bits_mse, self._rotation.ctypes.data,
                                             self._codebook.ctypes.data, proj, idx, ctypes.byref(out)))
            h = out.value
            if self._path != _native.TQ_PATH_AUTO:
                _native.check(lib.tq_plan_set_path(h, self._path))
            self._plans[idx] = h
        return h

    def check_status(self, device) -> None:
        """Raise if a tensor-core kernel of this quantizer gave up on a bounded wait on ``device`` since the last
        check (synchronises the current stream of that device)."""
        idx = device.index if device.index is not None else _torch().cuda.current_device()
        h = self._plans.get(idx)
        if h is None:
            return
        status = ctypes.c_int64(0)
        with _torch().cuda.device(idx):
            _native.check(_native.load().tq_plan_status(h, _stream_ptr(device), ctypes.byref(status)))
        if status.value:
            what = {1: "quantize", 2: "scoring", 3: "dequantize"}.get(status.value, "tensor-core")
            raise _native.TurboQuantNativeError(
                f"a {what} kernel gave up on a bounded wait (status {status.value}); the results of the calls "
                f"since the last check are incomplete")

    def set_wait_limit(self, cycles: int) -> None:
        """Limit of one bounded wait inside the tensor-core kernels, in GPU cycles, for plans that exist already."""
        for h in self._plans.values():
            _native.check(_native.load().tq_plan_set_wait_limit(h, int(cycles)))

    def set_path(self, path: int) -> None:
        self._path = path
        lib = _native.load()
        for h in self._plans.values():
            _native.check(lib.tq_plan_set_path(h, path))

    def row_bytes(self) -> Tuple[int, int]:
        """(code row bytes, sign row bytes); same formula as the library, usable without a GPU."""
        return 4 * ((self.dimension * self.bits_mse + 31) // 32), 4 * ((self.dimension + 31) // 32)

    def __del__(self):
        try:
            lib = _native.load()
            for h in self._plans.values():
                lib.tq_plan_destroy(h)
        except Exception:
            pass


# ------------------------------------------------------------------------------------------------
# encodings
# ------------------------------------------------------------------------------------------------
class _Packed:
    """Device-resident form of an encoding: bit-packed rows plus per-row float32 scalars."""

    __slots__ = ("codes", "signs", "norms", "residual_norms", "n", "kind", "device", "plans")

    def __init__(self, codes, signs, norms, residual_norms, n, kind, device, plans):
        self.codes, self.signs, self.norms, self.residual_norms = codes, signs, norms, residual_norms
        self.n, self.kind, self.device, self.plans = n, kind, device, plans


def _lazy_field(name: str, make):
    slot = "_" + name

    def getter(self):
        value = self.__dict__.get(slot)
        if value is None and self.__dict__.get("_packed") is not None:
            value = make(self.__dict__["_packed"])
            self.__dict__[slot] = value
        return value

    def setter(self, value):
        self.__dict__[slot] = value

    return property(getter, setter)


def _unpack_codes(pk: _Packed):
    torch = _torch()
    out = torch.empty((pk.n, pk.plans.dimension), dtype=torch.uint8, device=pk.device)
    if pk.n:
        with torch.cuda.device(pk.device):
            _native.check(_native.load().tq_unpack_codes(pk.plans.handle(pk.device), _ptr(pk.codes), pk.n,
                                                         _ptr(out), _stream_ptr(pk.device)))
    return _deliver(out, pk.kind, pk.plans)


def _unpack_signs(pk: _Packed):
    torch = _torch()
    out = torch.empty((pk.n, pk.plans.dimension), dtype=torch.int8, device=pk.device)
    if pk.n:
        with torch.cuda.device(pk.device):
            _native.check(_native.load().tq_unpack_signs(pk.plans.handle(pk.device), _ptr(pk.signs), pk.n,
                                                         _ptr(out), _stream_ptr(pk.device)))
    return _deliver(out, pk.kind, pk.plans)


@dataclass
class TurboQuantMSEEncoding:
    indices: Any
    norms: Any
    prefix_shape: Tuple[int, ...]


@dataclass
class TurboQuantProdEncoding:
    indices: Any
    qjl: Any
    residual_norms: Any
    norms: Any
    prefix_shape: Tuple[int, ...]


# The dataclass fields above stay what ``dataclasses.fields`` reports; the array-valued ones are
# served by properties so that encodings produced here can keep packed device buffers and only
# materialise the reference-shaped arrays when somebody reads them.
for _cls in (TurboQuantMSEEncoding, TurboQuantProdEncoding):
    _cls.indices = _lazy_field("indices", _unpack_codes)
    _cls.norms = _lazy_field("norms", lambda pk: _deliver(pk.norms, pk.kind, pk.plans))
TurboQuantProdEncoding.qjl = _lazy_field("qjl", _unpack_signs)
TurboQuantProdEncoding.residual_norms = _lazy_field(
    "residual_norms", lambda pk: _deliver(pk.residual_norms, pk.kind, pk.plans))


def _encoding_from_packed(cls, pk: _Packed, prefix):
    enc = cls.__new__(cls)
    enc.__dict__["_packed"] = pk
    enc.__dict__["prefix_shape"] = tuple(prefix)
    return enc


def packed_buffers(encoding) -> Dict[str, Any]:
    """The device buffers behind an encoding produced by this package, as torch tensors:
    ``codes`` uint8 (N, code_row_bytes), ``signs`` uint8 (N, sign_row_bytes) or None, ``norms``
    and ``residual_norms`` float32 (N,).  Raises for encodings built by hand from arrays."""
    pk = encoding.__dict__.get("_packed")
    if pk is None:
        raise ValueError("this encoding holds plain arrays, not packed device buffers")
    return {"codes": pk.codes, "signs": pk.signs, "norms": pk.norms, "residual_norms": pk.residual_norms}


def packed_to_host(encoding, out: Optional[Dict[str, Any]] = None, wait: bool = True) -> Dict[str, Any]:
    """Copy the packed buffers of an encoding into page-locked host tensors (same keys as
    ``packed_buffers``).  ``out`` may be the dict returned by an earlier call for an encoding of the
    same shape; its tensors are reused, which avoids allocating (and faulting in) fresh host memory for
    every batch -- a device-to-host copy into new pageable memory runs far below the link rate.  The
    copies are enqueued on the current stream; with ``wait=False`` the caller synchronises."""
    torch = _require_cuda()
    bufs = packed_buffers(encoding)
    host: Dict[str, Any] = {} if out is None else out
    for name, dev_t in bufs.items():
        if dev_t is None:
            host[name] = None
            continue
        dst = host.get(name)
        if dst is None or dst.shape != dev_t.shape or dst.dtype != dev_t.dtype or not dst.is_pinned():
            dst = torch.empty(dev_t.shape, dtype=dev_t.dtype, pin_memory=True)
            host[name] = dst
        dst.copy_(dev_t, non_blocking=True)
    if wait:
        pk = encoding.__dict__["_packed"]
        pk.plans.check_status(pk.device)     # synchronises the stream, and refuses results of a kernel that gave up
    return host


def quantize_to_host(quantizer, keys, chunk_rows: int = 131072, out: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    """Quantize host-resident keys and leave the packed encoding in page-locked host tensors, for key sets
    that do not stay on the GPU (``quantizer`` is a TurboQuantMSE or TurboQuantProd, ``keys`` a NumPy
    array of shape (..., d), best page-locked).  The keys go up in chunks of ``chunk_rows`` on one stream
    while the previous chunk is quantized on a second and the chunk before that is copied back on a third,
    so the call takes about as long as the host-to-device copy alone.  Returns the dict described under
    ``packed_buffers`` (``out`` may be the dict of an earlier call of the same size: its tensors are
    reused)."""
    torch = _require_cuda()
    prod = isinstance(quantizer, TurboQuantProd)
    mseq = quantizer.mse if prod else quantizer
    plans = quantizer._plans
    d = quantizer.dimension
    array = _to_array(keys)
    if not isinstance(array, np.ndarray):
        raise TypeError("quantize_to_host expects host (NumPy) keys; use quantize() for device arrays")
    _ensure_last_dim(array, d)
    flat = torch.from_numpy(np.ascontiguousarray(array.reshape(-1, d), dtype=np.float32))
    n = flat.shape[0]
    device = torch.device("cuda", torch.cuda.current_device())
    code_bytes, sign_bytes = plans.row_bytes()
    shapes = {"codes": ((n, code_bytes), torch.uint8), "norms": ((n,), torch.float32)}
    if prod:
        shapes.update({"signs": ((n, sign_bytes), torch.uint8), "residual_norms": ((n,), torch.float32)})
    host: Dict[str, Any] = {} if out is None else out
    for name, (shape, dtype) in shapes.items():
        t = host.get(name)
        if t is None or tuple(t.shape) != shape or t.dtype != dtype or not t.is_pinned():
            host[name] = torch.empty(shape, dtype=dtype, pin_memory=True)
    if not prod:
        host["signs"] = host["residual_norms"] = None
    if n == 0:
        return host
    chunk_rows = max(1, min(int(chunk_rows), n))
    with torch.cuda.device(device):
        s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        for s_ in (s_in, s_run, s_out):
            s_.wait_stream(torch.cuda.current_stream())
        bufs = [torch.empty((chunk_rows, d), dtype=torch.float32, device=device) for _ in range(2)]
        ran = [None, None]          # event: the kernels that read bufs[b] have finished
        alive = []                  # chunk results stay allocated until the copies back are done
        for i, start in enumerate(range(0, n, chunk_rows)):
            m = min(chunk_rows, n - start)
            b = i & 1
            with torch.cuda.stream(s_in):
                if ran[b] is not None:
                    s_in.wait_event(ran[b])
                bufs[b][:m].copy_(flat[start:start + m], non_blocking=True)
                up = torch.cuda.Event()
                up.record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(up)
                pk = mseq._quantize_staged(_Staged(bufs[b][:m], (m,), "torch", device), plans, prod)
                ran[b] = torch.cuda.Event()
                ran[b].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ran[b])
                host["codes"][start:start + m].copy_(pk.codes, non_blocking=True)
                host["norms"][start:start + m].copy_(pk.norms, non_blocking=True)
                if prod:
                    host["signs"][start:start + m].copy_(pk.signs, non_blocking=True)
                    host["residual_norms"][start:start + m].copy_(pk.residual_norms, non_blocking=True)
            alive.append(pk)
        s_out.synchronize()
        torch.cuda.current_stream().wait_stream(s_run)
        plans.check_status(device)     # a chunk whose kernel gave up on a bounded wait must not pass as quantized
    return host


def _as_packed(encoding, plans: _PlanSet, need_signs: bool) -> _Packed:
    """Packed device form of ``encoding``: its own buffers when it came from this quantizer's
    geometry, else packed now from the reference-style array fields."""
    pk = encoding.__dict__.get("_packed")
    if pk is not None and pk.plans.dimension == plans.dimension and pk.plans.bits_mse == plans.bits_mse:
        if pk.plans is not plans:
            pk = _Packed(pk.codes, pk.signs, pk.norms, pk.residual_norms, pk.n, pk.kind, pk.device, plans)
        return pk
    torch = _require_cuda()
    lib = _native.load()
    indices = _to_array(encoding.indices)
    d = plans.dimension
    if isinstance(indices, np.ndarray):
        kind = "numpy"
        device = torch.device("cuda", torch.cuda.current_device())
        to_dev = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).to(device).to(dt).contiguous()
    else:
        kind = "torch"
        first = torch.as_tensor(indices, device="cuda") if not isinstance(indices, torch.Tensor) else indices
        device = first.device if first.is_cuda else torch.device("cuda", torch.cuda.current_device())
        kind = "torch" if first.is_cuda else "torch_cpu"
        to_dev = lambda a, dt: (a if isinstance(a, torch.Tensor) else torch.as_tensor(a, device="cuda")).to(device).to(dt).contiguous()
    idx = to_dev(indices, torch.uint8)
    if idx.ndim != 2 or idx.shape[1] != d:
        raise ValueError(f"expected indices of shape (N, {d}), got {tuple(idx.shape)}")
    n = idx.shape[0]
    code_bytes, sign_bytes = plans.row_bytes()
    handle = plans.handle(device)
    codes = torch.empty((n, code_bytes), dtype=torch.uint8, device=device)
    norms = to_dev(_to_array(encoding.norms), torch.float32).reshape(-1)
    signs = rnorms = None
    with torch.cuda.device(device):
        st = _stream_ptr(device)
        if n:
            _native.check(lib.tq_pack_codes(handle, _ptr(idx), n, _ptr(codes), st))
        if need_signs:
            qjl = to_dev(_to_array(encoding.qjl), torch.int8)
            signs = torch.empty((n, sign_bytes), dtype=torch.uint8, device=device)
            rnorms = to_dev(_to_array(encoding.residual_norms), torch.float32).reshape(-1)
            if n:
                _native.check(lib.tq_pack_signs(handle, _ptr(qjl), n, _ptr(signs), st))
    return _Packed(codes, signs, norms, rnorms, n, kind, device, plans)


# ------------------------------------------------------------------------------------------------
# quantizers
# ------------------------------------------------------------------------------------------------
class TurboQuantMSE:
    """TurboQuant variant optimized for MSE reconstruction (GPU kernels behind the reference API)."""

    def __init__(self, dimension: int, bits: int, *, seed: Optional[int] = None, grid_size: int = 16385,
                 max_iter: int = 200, rotation: Optional[np.ndarray] = None,
                 codebook: Optional[np.ndarray] = None):
        if dimension < 2:
            raise ValueError("dimension must be >= 2")
        if bits < 1:
            raise ValueError("bits must be >= 1")
        if bits > _MAX_BITS:
            raise ValueError(f"bits must be <= {_MAX_BITS} on the B200 path")
        if dimension > _MAX_DIM:
            raise ValueError(f"dimension must be <= {_MAX_DIM} on the B200 path")
        self.dimension = int(dimension)
        self.bits = int(bits)
        if rotation is not None:
            self.rotation = np.asarray(rotation, dtype=np.float32)
        else:
            self.rotation = _random_orthogonal_matrix(self.dimension, seed)
        if self.rotation.shape != (self.dimension, self.dimension):
            raise ValueError(
                f"rotation must have shape {(self.dimension, self.dimension)}, got {self.rotation.shape}"
            )
        if codebook is not None:
            self.codebook = np.asarray(codebook, dtype=np.float32)
        else:
            self.codebook = _build_lloyd_max_codebook(
                self.dimension, self.bits, grid_size=grid_size, max_iter=max_iter).astype(np.float32)
        if self.codebook.ndim != 1 or self.codebook.shape[0] != (1 << self.bits):
            raise ValueError("codebook shape does not match bit-width")
        self.boundaries = 0.5 * (self.codebook[:-1] + self.codebook[1:])
        self.index_dtype = _quant_index_dtype(self.bits)
        self._plans = _PlanSet(self.dimension, self.bits, self.rotation, self.codebook, None)

    # The tensor-core kernels are used when they exist for (dimension, bits); tests and
    # benchmarks can pin either arithmetic.
    def set_kernel_path(self, path: str) -> None:
        """'auto' | 'exact' | 'tensor' (see TQ_PATH_* in include/tq_b200.h)."""
        self._plans.set_path({"auto": _native.TQ_PATH_AUTO, "exact": _native.TQ_PATH_EXACT,
                              "tensor": _native.TQ_PATH_TENSOR}[path])

    def _quantize_staged(self, staged: _Staged, plans: _PlanSet, prod: bool, out: Optional[Dict[str, Any]] = None) -> _Packed:
        """``out``: contiguous device tensors {codes, norms[, signs, residual_norms]} of n rows to write into
        (e.g. slices of a preallocated index) instead of fresh ones."""
        torch = _torch()
        lib = _native.load()
        x, device = staged.tensor, staged.device
        n = x.shape[0]
        code_bytes, sign_bytes = plans.row_bytes()
        handle = plans.handle(device)
        with torch.cuda.device(device):
            codes = out["codes"] if out else torch.empty((n, code_bytes), dtype=torch.uint8, device=device)
            norms = out["norms"] if out else torch.empty((n,), dtype=torch.float32, device=device)
            scratch = torch.empty((max(int(lib.tq_quantize_scratch_bytes(handle, n)), 16),),
                                  dtype=torch.uint8, device=device)
            st = _stream_ptr(device)
            if prod:
                signs = out["signs"] if out else torch.empty((n, sign_bytes), dtype=torch.uint8, device=device)
                rnorms = out["residual_norms"] if out else torch.empty((n,), dtype=torch.float32, device=device)
                _native.check(lib.tq_prod_quantize(handle, _ptr(x), n, _ptr(codes), _ptr(signs), _ptr(rnorms),
                                                   _ptr(norms), _ptr(scratch), scratch.numel(), st))
            else:
                signs = rnorms = None
                _native.check(lib.tq_mse_quantize(handle, _ptr(x), n, _ptr(codes), _ptr(norms), _ptr(scratch),
                                                  scratch.numel(), st))
        return _Packed(codes, signs, norms, rnorms, n, staged.kind, device, plans)

    def quantize(self, vectors: Any) -> TurboQuantMSEEncoding:
        staged = _stage(vectors, self.dimension)
        pk = self._quantize_staged(staged, self._plans, prod=False)
        return _encoding_from_packed(TurboQuantMSEEncoding, pk, staged.prefix)

    def dequantize(self, encoding: TurboQuantMSEEncoding):
        pk = _as_packed(encoding, self._plans, need_signs=False)
        torch = _torch()
        out = torch.empty((pk.n, self.dimension), dtype=torch.float32, device=pk.device)
        with torch.cuda.device(pk.device):
            _native.check(_native.load().tq_mse_dequantize(self._plans.handle(pk.device), _ptr(pk.codes),
                                                           _ptr(pk.norms), pk.n, _ptr(out),
                                                           _stream_ptr(pk.device)))
        return _deliver(out, pk.kind, pk.plans).reshape(tuple(encoding.prefix_shape) + (self.dimension,))


class TurboQuantProd:
    """TurboQuant variant optimized for unbiased inner-product estimation (GPU kernels behind the
    reference API)."""

    def __init__(self, dimension: int, bits: int, *, seed: Optional[int] = None, grid_size: int = 16385,
                 max_iter: int = 200, rotation: Optional[np.ndarray] = None,
                 projection: Optional[np.ndarray] = None):
        if bits < 1:
            raise ValueError("bits must be >= 1")
        self.dimension = int(dimension)
        self.bits = int(bits)
        self.mse = TurboQuantMSE(dimension, max(bits - 1, 1), seed=seed, grid_size=grid_size,
                                 max_iter=max_iter, rotation=rotation)
        if projection is not None:
            self.projection = np.asarray(projection, dtype=np.float32)
        else:
            self.projection = _random_projection_matrix(self.dimension, None if seed is None else seed + 1)
        if self.projection.shape != (self.dimension, self.dimension):
            raise ValueError(
                f"projection must have shape {(self.dimension, self.dimension)}, got {self.projection.shape}"
            )
        self._plans = _PlanSet(self.dimension, self.mse.bits, self.mse.rotation, self.mse.codebook,
                               self.projection)

    def set_kernel_path(self, path: str) -> None:
        self._plans.set_path({"auto": _native.TQ_PATH_AUTO, "exact": _native.TQ_PATH_EXACT,
                              "tensor": _native.TQ_PATH_TENSOR}[path])

    def quantize(self, vectors: Any) -> TurboQuantProdEncoding:
        staged = _stage(vectors, self.dimension)
        pk = self.mse._quantize_staged(staged, self._plans, prod=True)
        return _encoding_from_packed(TurboQuantProdEncoding, pk, staged.prefix)

    def dequantize(self, encoding: TurboQuantProdEncoding):
        pk = _as_packed(encoding, self._plans, need_signs=True)
        torch = _torch()
        out = torch.empty((pk.n, self.dimension), dtype=torch.float32, device=pk.device)
        with torch.cuda.device(pk.device):
            _native.check(_native.load().tq_prod_dequantize(
                self._plans.handle(pk.device), _ptr(pk.codes), _ptr(pk.signs), _ptr(pk.residual_norms),
                _ptr(pk.norms), pk.n, _ptr(out), _stream_ptr(pk.device)))
        return _deliver(out, pk.kind, pk.plans).reshape(tuple(encoding.prefix_shape) + (self.dimension,))

    def attention_score(self, query: Any, encoding: TurboQuantProdEncoding):
        """One query row broadcast over all keys, or one query row per key (_quant.py:334-358)."""
        pk = _as_packed(encoding, self._plans, need_signs=True)
        staged = _stage(query, self.dimension, device=pk.device)
        q = staged.tensor
        if q.device != pk.device:
            q = q.to(pk.device)
        num_codes = pk.n
        q_prefix = staged.prefix
        broadcast = q.shape[0] == 1 and num_codes > 1
        if broadcast:
            q_prefix = tuple(encoding.prefix_shape)
        elif q.shape[0] != num_codes:
            raise ValueError(
                f"query batch size {q.shape[0]} does not match encoding batch size {num_codes}"
            )
        torch = _torch()
        lib = _native.load()
        scores = torch.empty((num_codes,), dtype=torch.float32, device=pk.device)
        handle = self._plans.handle(pk.device)
        with torch.cuda.device(pk.device):
            if broadcast and self._plans._path == _native.TQ_PATH_AUTO:
                # one query against all keys: the entry point that needs no scratch buffer
                _native.check(lib.tq_score_broadcast(handle, _ptr(q), _ptr(pk.codes), _ptr(pk.signs),
                                                     _ptr(pk.residual_norms), _ptr(pk.norms), num_codes,
                                                     _ptr(scores), _stream_ptr(pk.device)))
            elif broadcast:
                # a forced kernel path: the one-row case of the batched entry point
                need =int(lib.tq_topk_scratch_bytes(handle, 1, 1, num_codes, 0))
                scratch = torch.empty((max(need, 16),), dtype=torch.uint8, device=pk.device)
                _native.check(lib.tq_score_batched(handle, _ptr(q), 1, 1, _ptr(pk.codes), _ptr(pk.signs),
                                                   _ptr(pk.residual_norms), _ptr(pk.norms), num_codes,
                                                   _ptr(scores), 0, None, None, 0, _ptr(scratch),
                                                   scratch.numel(), _stream_ptr(pk.device)))
            else:
                _native.check(lib.tq_score_pairwise(handle, _ptr(q), _ptr(pk.codes), _ptr(pk.signs),
                                                    _ptr(pk.residual_norms), _ptr(pk.norms), num_codes,
                                                    _ptr(scores), _stream_ptr(pk.device)))
        shape = q_prefix if (broadcast or q.shape[0] != 1) else tuple(encoding.prefix_shape)
        return _deliver(scores, staged.kind, self._plans).reshape(shape)

    def attention_scores(self, queries: Any, encoding: TurboQuantProdEncoding, *, topk: Optional[int] = None,
                         groups: int = 1, return_matrix: Optional[bool] = None, index_base: int = 0,
                         out: Optional[Tuple[Any, Any]] = None):
        """Score many queries against shared keys in one pass over the packed keys.

        ``queries`` has shape (..., d) and flattens to Q rows; the N keys are split into ``groups``
        equal consecutive blocks and the Q rows into ``groups`` equal blocks; query block g meets
        key block g only (``groups=1``: every query meets every key; larger values give the
        per-sequence / per-head batching of a KV cache).  Row i of the result equals
        ``attention_score(queries[i], keys of its block)``.

        Returns the score matrix of shape (Q, N // groups) when ``topk`` is None; with ``topk=k``
        returns ``(top_scores, top_indices)`` of shape (Q, k), descending, indices counted over
        all N keys plus ``index_base`` (set ``return_matrix=True`` to get the matrix as a third
        element as well).  ``out=(top_scores, top_indices)``: contiguous device tensors of shape (Q, k), float32 and
        int64, that receive the top-k instead of fresh ones (e.g. the send block of ``sharded.TopkExchange``, so
        that the candidates need no repacking before the collective).
        """
        pk = _as_packed(encoding, self._plans, need_signs=True)
        staged = _stage(queries, self.dimension, device=pk.device)
        q = staged.tensor
        if q.device != pk.device:
            q = q.to(pk.device)
        nq, n = q.shape[0], pk.n
        if groups < 1 or nq % groups or n % groups:
            raise ValueError(f"groups={groups} must divide both the query count {nq} and the key count {n}")
        qpg, kpg = nq // groups, n // groups
        k = int(topk) if topk else 0
        want_matrix = (k == 0) if return_matrix is None else bool(return_matrix)
        if k == 0 and not want_matrix:
            raise ValueError("nothing to compute: no top-k requested and return_matrix is False")
        torch = _torch()
        lib = _native.load()
        handle = self._plans.handle(pk.device)
        with torch.cuda.device(pk.device):
            scores = torch.empty((nq, kpg), dtype=torch.float32, device=pk.device) if want_matrix else None
            if out is not None and k:
                top_s, top_i = out
                if (tuple(top_s.shape) != (nq, k) or tuple(top_i.shape) != (nq, k) or top_s.dtype != torch.float32
                        or top_i.dtype != torch.int64 or not top_s.is_contiguous() or not top_i.is_contiguous()
                        or top_s.device != pk.device or top_i.device != pk.device):
                    raise ValueError(f"out must be contiguous float32 / int64 tensors of shape ({nq}, {k}) on {pk.device}")
            else:
                top_s = torch.empty((nq, k), dtype=torch.float32, device=pk.device) if k else None
                top_i = torch.empty((nq, k), dtype=torch.int64, device=pk.device) if k else None
            need = int(lib.tq_topk_scratch_bytes(handle, groups, qpg, kpg, k))
            scratch = torch.empty((max(need, 16),), dtype=torch.uint8, device=pk.device)
            _native.check(lib.tq_score_batched(handle, _ptr(q), groups, qpg, _ptr(pk.codes), _ptr(pk.signs),
                                               _ptr(pk.residual_norms), _ptr(pk.norms), kpg, _ptr(scores), k,
                                               _ptr(top_s), _ptr(top_i), int(index_base), _ptr(scratch),
                                               scratch.numel(), _stream_ptr(pk.device)))
        if k == 0:
            return _deliver(scores, staged.kind, self._plans)
        result = (_deliver(top_s, staged.kind, self._plans), _deliver(top_i, staged.kind))
        return result + (_deliver(scores, staged.kind),) if want_matrix else result


def turboquant_mse(vectors: Any, bits: int, *, seed: Optional[int] = None) -> Tuple[TurboQuantMSE, TurboQuantMSEEncoding]:
    """Convenience helper that instantiates and applies `TurboQuantMSE`."""
    array = _to_array(vectors)
    quantizer = TurboQuantMSE(array.shape[-1], bits, seed=seed)
    return quantizer, quantizer.quantize(vectors)


def turboquant_prod(vectors: Any, bits: int, *, seed: Optional[int] = None) -> Tuple[TurboQuantProd, TurboQuantProdEncoding]:
    """Convenience helper that instantiates and applies `TurboQuantProd`."""
    array = _to_array(vectors)
    quantizer = TurboQuantProd(array.shape[-1], bits, seed=seed)
    return quantizer, quantizer.quantize(vectors)
