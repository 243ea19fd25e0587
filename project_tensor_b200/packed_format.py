"""On-disk / wire format of packed TurboQuant encodings.

The reference keeps encodings only as in-memory dataclasses of unpacked arrays
(tensor_gpu_v2/_quant.py:156-169: one byte per code, one int8 per QJL sign); its only file format is the
model checkpoint of tensor_gpu_v2/_training.py:19-139.  A quantized key set that outlives its process -- a
persistent KV cache, a vector index, a shard handed to another rank -- needs a format of its own; this is it.

File layout (all integers little-endian):

    offset 0    8 bytes   magic  b"TQPACKED"
    offset 8    u32       format version (2)
    offset 12   u32       length H of the header text
    offset 16   H bytes   header, UTF-8 JSON (see ``_header``)
    offset 16+H u32       CRC-32 of the H header bytes
    ...         padding with zero bytes to a multiple of 64
    sections              the arrays named in header["sections"], each starting on a multiple of 64 bytes
                          counted from the start of the file, raw little-endian, C order

The header names the quantizer by content, not by seed: SHA-256 of the float32 codebook, rotation and
projection, so that a reader refuses to interpret codes with other constants than the writer's.  The header and
every section carry a CRC-32 of their bytes, and a reader checks the header against itself before it trusts it:
the sections must be exactly those of the quantizer's kind, with the row count, row widths and dtypes the header's
own dimension and bit width imply (the kernels index the arrays by these numbers, so a header that overstates
them would send them past the end of the buffers).

Bit layout of the rows (the same as the device buffers, csrc/tq_common.cuh):
  * codes: coordinate j occupies bits [j*b, (j+1)*b) of the row read as a little-endian bit stream, rows padded
    to whole 32-bit words (b = bits of the MSE stage);
  * signs: one bit per coordinate (1 = +1), 32 coordinates per 32-bit word; inside a word the even coordinates
    fill bits 0..15 and the odd ones bits 16..31.

The NumPy packers here are the CPU statement of that layout: they let a process without a GPU read a file back
into the reference's array fields, and the tests hold the GPU packers to them.
"""
from __future__ import annotations

import hashlib
import json
import struct
import zlib
from typing import Any, Dict, Tuple

import numpy as np

MAGIC = b"TQPACKED"
VERSION = 2
_ALIGN = 64
_SECTION_DTYPES = {"codes": "<u1", "signs": "<u1", "norms": "<f4", "residual_norms": "<f4"}


class PackedFormatError(ValueError):
    """The bytes are not a packed-encoding file, are damaged, or belong to another quantizer."""


# ------------------------------------------------------------------------------------------------
# row layout on the CPU
# ------------------------------------------------------------------------------------------------
def code_row_bytes(d: int, bits: int) -> int:
    return 4 * ((d * bits + 31) // 32)


def sign_row_bytes(d: int) -> int:
    return 4 * ((d + 31) // 32)


def pack_codes_numpy(indices: np.ndarray, bits: int) -> np.ndarray:
    """(N, d) codes in [0, 2^bits) -> (N, code_row_bytes) uint8."""
    idx = np.ascontiguousarray(indices).astype(np.uint8, copy=False)
    n, d = idx.shape
    # bit k of code j is bit j*bits + k of the stream; numpy's "little" bit order puts stream bit 8m + i
    # into bit i of byte m, which for little-endian 32-bit words is the same stream
    bit_planes = ((idx[:, :, None] >> np.arange(bits, dtype=np.uint8)) & 1).reshape(n, d * bits)
    row_bits = 8 * code_row_bytes(d, bits)
    padded = np.zeros((n, row_bits), dtype=np.uint8)
    padded[:, : d * bits] = bit_planes
    return np.packbits(padded, axis=1, bitorder="little")


def unpack_codes_numpy(codes: np.ndarray, d: int, bits: int) -> np.ndarray:
    """(N, code_row_bytes) uint8 -> (N, d) uint8 codes."""
    rows = np.ascontiguousarray(codes, dtype=np.uint8)
    n = rows.shape[0]
    stream = np.unpackbits(rows, axis=1, bitorder="little")[:, : d * bits].reshape(n, d, bits)
    weights = (1 << np.arange(bits, dtype=np.uint16)).astype(np.uint16)
    return (stream.astype(np.uint16) * weights).sum(axis=2).astype(np.uint8)


def _sign_bit_positions(d: int) -> np.ndarray:
    j = np.arange(d)
    return 32 * (j // 32) + ((j % 32) // 2) + 16 * (j % 2)


def pack_signs_numpy(qjl: np.ndarray) -> np.ndarray:
    """(N, d) values of +-1 (anything >= 0 counts as +1, _quant.py:67-70) -> (N, sign_row_bytes) uint8."""
    q = np.asarray(qjl)
    n, d = q.shape
    padded = np.zeros((n, 8 * sign_row_bytes(d)), dtype=np.uint8)
    padded[:, _sign_bit_positions(d)] = (q >= 0).astype(np.uint8)
    return np.packbits(padded, axis=1, bitorder="little")


def unpack_signs_numpy(signs: np.ndarray, d: int) -> np.ndarray:
    """(N, sign_row_bytes) uint8 -> (N, d) int8 of +-1."""
    rows = np.ascontiguousarray(signs, dtype=np.uint8)
    stream = np.unpackbits(rows, axis=1, bitorder="little")
    return (2 * stream[:, _sign_bit_positions(d)].astype(np.int8) - 1).astype(np.int8)


# ------------------------------------------------------------------------------------------------
# quantizer identity
# ------------------------------------------------------------------------------------------------
def _sha(array) -> str:
    return hashlib.sha256(np.ascontiguousarray(array, dtype="<f4").tobytes()).hexdigest()


def quantizer_fingerprint(quantizer) -> Dict[str, Any]:
    """What a reader must share with the writer for the codes to mean the same vectors.  Works for the
    quantizers of this package and for the reference's (same attribute names, _quant.py:175-213, 260-292)."""
    inner = getattr(quantizer, "mse", None)
    prod = inner is not None
    mse = inner if prod else quantizer
    out = {
        "kind": "prod" if prod else "mse",
        "dimension": int(quantizer.dimension),
        "bits": int(quantizer.bits),
        "bits_mse": int(mse.bits),
        "codebook_sha256": _sha(mse.codebook),
        "rotation_sha256": _sha(mse.rotation),
        "projection_sha256": _sha(quantizer.projection) if prod else None,
    }
    return out


# ------------------------------------------------------------------------------------------------
# writing and reading
# ------------------------------------------------------------------------------------------------
def _pad(n: int) -> int:
    return (-n) % _ALIGN


def _raw(a: np.ndarray):
    """The bytes of a C-contiguous array (an empty array has none to view)."""
    return memoryview(a).cast("B") if a.size else b""


def _header(fingerprint: Dict[str, Any], prefix_shape, n: int, sections) -> bytes:
    d, b = fingerprint["dimension"], fingerprint["bits_mse"]
    doc = {
        "format": "turboquant-packed",
        "version": VERSION,
        "quantizer": fingerprint,
        "rows": int(n),
        "prefix_shape": [int(s) for s in prefix_shape],
        "layout": {"code_row_bytes": code_row_bytes(d, b), "sign_row_bytes": sign_row_bytes(d),
                   "code_bit_order": "little-endian stream, coordinate-major",
                   "sign_bit_order": "even coordinates of each 32 in bits 0-15, odd in bits 16-31"},
        "sections": sections,
    }
    return json.dumps(doc, sort_keys=True).encode("utf-8")


def write_packed(target, fingerprint: Dict[str, Any], prefix_shape: Tuple[int, ...], buffers: Dict[str, Any]) -> int:
    """Write host buffers (NumPy arrays or anything ``np.asarray`` takes: ``codes`` (N, code_row_bytes) uint8,
    ``norms`` (N,) float32 and for TurboQuantProd ``signs`` and ``residual_norms``) to ``target``, a path or a
    binary file object.  Returns the number of bytes written."""
    prod = fingerprint["kind"] == "prod"
    names = ["codes", "norms"] + (["signs", "residual_norms"] if prod else [])
    d, b = fingerprint["dimension"], fingerprint["bits_mse"]
    arrays = {}
    for name in names:
        if buffers.get(name) is None:
            raise PackedFormatError(f"buffer {name!r} is missing")
        arrays[name] = np.ascontiguousarray(np.asarray(buffers[name]), dtype=_SECTION_DTYPES[name])
    n = arrays["norms"].shape[0]
    want = {"codes": (n, code_row_bytes(d, b)), "norms": (n,), "signs": (n, sign_row_bytes(d)), "residual_norms": (n,)}
    for name in names:
        if tuple(arrays[name].shape) != want[name]:
            raise PackedFormatError(f"buffer {name!r} has shape {tuple(arrays[name].shape)}, expected {want[name]}")
    if int(np.prod(prefix_shape, dtype=np.int64)) != n:
        raise PackedFormatError(f"prefix_shape {tuple(prefix_shape)} does not describe {n} rows")

    # two passes: the header's length decides where the sections start, and the header names those offsets;
    # offsets are written with a fixed width so that the length does not depend on their values
    def layout(header_len: int):
        pos = 16 + header_len + 4
        pos += _pad(pos)
        secs = []
        for name in names:
            a = arrays[name]
            secs.append({"name": name, "dtype": _SECTION_DTYPES[name], "shape": list(a.shape),
                         "offset": f"{pos:020d}", "nbytes": f"{a.nbytes:020d}",
                         "crc32": f"{zlib.crc32(_raw(a)) & 0xFFFFFFFF:08x}"})
            pos += a.nbytes
            pos += _pad(pos)
        return secs, pos

    secs, _ = layout(0)
    header = _header(fingerprint, prefix_shape, n, secs)
    secs, total = layout(len(header))
    header2 = _header(fingerprint, prefix_shape, n, secs)
    assert len(header2) == len(header)

    own = isinstance(target, (str, bytes)) or hasattr(target, "__fspath__")
    f = open(target, "wb") if own else target
    try:
        f.write(MAGIC + struct.pack("<II", VERSION, len(header2)) + header2 + struct.pack("<I", zlib.crc32(header2) & 0xFFFFFFFF))
        pos = 16 + len(header2) + 4
        f.write(b"\0" * _pad(pos))
        pos += _pad(pos)
        for name in names:
            a = arrays[name]
            f.write(_raw(a))
            pos += a.nbytes
            f.write(b"\0" * _pad(pos))
            pos += _pad(pos)
    finally:
        if own:
            f.close()
    return total


class PackedFile:
    """A file read back: ``quantizer`` (the writer's fingerprint), ``rows``, ``prefix_shape`` and ``buffers``
    (NumPy arrays by section name; memory-mapped when the file was opened with ``mmap=True``)."""

    def __init__(self, header: Dict[str, Any], buffers: Dict[str, np.ndarray]):
        self.header = header
        self.quantizer: Dict[str, Any] = header["quantizer"]
        self.rows: int = header["rows"]
        self.prefix_shape: Tuple[int, ...] = tuple(header["prefix_shape"])
        self.buffers = buffers

    def indices(self) -> np.ndarray:
        """The reference's ``indices`` field, (N, d) uint8, unpacked on the CPU."""
        q = self.quantizer
        return unpack_codes_numpy(self.buffers["codes"], q["dimension"], q["bits_mse"])

    def qjl(self) -> np.ndarray:
        """The reference's ``qjl`` field, (N, d) int8 of +-1, unpacked on the CPU."""
        if "signs" not in self.buffers:
            raise PackedFormatError("a TurboQuantMSE file has no sign bits")
        return unpack_signs_numpy(self.buffers["signs"], self.quantizer["dimension"])


def read_packed(source, *, mmap: bool = False, verify: bool = True) -> PackedFile:
    """Read a file written by ``write_packed`` from a path, ``bytes`` or a binary file object.  ``mmap=True``
    (paths only) maps the sections instead of reading them; ``verify`` checks every section's CRC-32 (which
    touches every byte, also of a mapped file)."""
    if isinstance(source, (bytes, bytearray, memoryview)):
        data = bytes(source)
        path = None
    elif isinstance(source, str) or hasattr(source, "__fspath__"):
        path = source
        data = None
    else:
        data = source.read()
        path = None
    if mmap and path is None:
        raise PackedFormatError("mmap=True needs a file path")
    if path is not None:
        with open(path, "rb") as f:
            head = f.read(16)
            hlen = struct.unpack("<II", head[8:16])[1] if len(head) == 16 else 0
            header_bytes = f.read(hlen)
            header_crc = f.read(4)
            if not mmap:
                f.seek(0)
                data = f.read()
    else:
        head = data[:16]
        hlen = struct.unpack("<II", head[8:16])[1] if len(head) == 16 else 0
        header_bytes = data[16:16 + hlen]
        header_crc = data[16 + hlen:16 + hlen + 4]
    if len(head) != 16 or head[:8] != MAGIC:
        raise PackedFormatError("not a packed TurboQuant encoding (bad magic)")
    version = struct.unpack("<II", head[8:16])[0]
    if version != VERSION:
        raise PackedFormatError(f"format version {version} is not supported (this reader knows {VERSION})")
    if len(header_bytes) != hlen or len(header_crc) != 4:
        raise PackedFormatError("file ends inside the header")
    if struct.unpack("<I", header_crc)[0] != (zlib.crc32(header_bytes) & 0xFFFFFFFF):
        raise PackedFormatError("header CRC-32 mismatch (file damaged or edited)")
    try:
        header = json.loads(header_bytes.decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise PackedFormatError(f"unreadable header: {e}") from None
    _check_header(header)
    buffers: Dict[str, np.ndarray] = {}
    for sec in header["sections"]:
        off, nbytes = int(sec["offset"]), int(sec["nbytes"])
        dtype, shape = np.dtype(sec["dtype"]), tuple(sec["shape"])
        if int(np.prod(shape, dtype=np.int64)) * dtype.itemsize != nbytes or off % _ALIGN:
            raise PackedFormatError(f"section {sec['name']!r}: inconsistent shape, size or offset")
        if mmap:
            arr = np.memmap(path, dtype=dtype, mode="r", offset=off, shape=shape) if nbytes else np.empty(shape, dtype)
        else:
            if off + nbytes > len(data):
                raise PackedFormatError(f"file ends inside section {sec['name']!r}")
            arr = np.frombuffer(data, dtype=dtype, count=nbytes // dtype.itemsize, offset=off).reshape(shape)
        if verify and nbytes:
            crc = zlib.crc32(_raw(np.ascontiguousarray(arr))) & 0xFFFFFFFF
            if f"{crc:08x}" != sec["crc32"]:
                raise PackedFormatError(f"section {sec['name']!r}: CRC-32 mismatch (file damaged)")
        buffers[sec["name"]] = arr
    return PackedFile(header, buffers)


def _check_header(header: Dict[str, Any]) -> None:
    """The header against itself: kind -> section names, (dimension, bits) -> row widths, rows -> every section's
    first extent and the prefix shape.  A reader indexes the arrays by these numbers."""
    try:
        q = header["quantizer"]
        kind, d, b = q["kind"], int(q["dimension"]), int(q["bits_mse"])
        rows = int(header["rows"])
        prefix = [int(v) for v in header["prefix_shape"]]
        secs = {sec["name"]: sec for sec in header["sections"]}
        if len(secs) != len(header["sections"]):
            raise PackedFormatError("a section is listed twice")
        if kind not in ("mse", "prod") or d < 2 or b < 1 or rows < 0 or any(v < 0 for v in prefix):
            raise PackedFormatError("header values out of range")
        names = ["codes", "norms"] + (["signs", "residual_norms"] if kind == "prod" else [])
        if sorted(secs) != sorted(names):
            raise PackedFormatError(f"a {kind} file must hold the sections {names}, found {sorted(secs)}")
        want = {"codes": [rows, code_row_bytes(d, b)], "norms": [rows], "signs": [rows, sign_row_bytes(d)],
                "residual_norms": [rows]}
        for name in names:
            sec = secs[name]
            if [int(v) for v in sec["shape"]] != want[name]:
                raise PackedFormatError(f"section {name!r} has shape {sec['shape']}, the header's own numbers "
                                        f"({rows} rows, d = {d}, {b} code bits) require {want[name]}")
            if sec["dtype"] != _SECTION_DTYPES[name]:
                raise PackedFormatError(f"section {name!r} has dtype {sec['dtype']!r}, expected {_SECTION_DTYPES[name]!r}")
        if int(np.prod(prefix, dtype=np.int64)) != rows:
            raise PackedFormatError(f"prefix_shape {prefix} does not describe {rows} rows")
    except (KeyError, TypeError, ValueError) as e:
        if isinstance(e, PackedFormatError):
            raise
        raise PackedFormatError(f"malformed header: {e!r}") from None


def check_same_quantizer(file_fingerprint: Dict[str, Any], quantizer) -> None:
    mine = quantizer_fingerprint(quantizer)
    for key, value in mine.items():
        if file_fingerprint.get(key) != value:
            raise PackedFormatError(
                f"the file was written by another quantizer: {key} is {file_fingerprint.get(key)!r} in the file, "
                f"{value!r} here")


# ------------------------------------------------------------------------------------------------
# encodings of this package <-> files
# ------------------------------------------------------------------------------------------------
def save_encoding(target, quantizer, encoding) -> int:
    """Write ``encoding`` (of ``quantizer``) to ``target``.  An encoding produced by this package is copied from
    its packed device buffers; one that holds the reference's plain arrays (``indices``, ``qjl``, ...) is
    packed on the CPU, so encodings made by the reference itself can be written too, without a GPU."""
    fp = quantizer_fingerprint(quantizer)
    prod = fp["kind"] == "prod"
    if encoding.__dict__.get("_packed") is not None:
        from . import turboquant as _tq
        host = _tq.packed_to_host(encoding)
        buffers = {k: (None if v is None else v.numpy()) for k, v in host.items()}
    else:
        d = fp["dimension"]
        indices = np.asarray(encoding.indices).reshape(-1, d)
        buffers = {"codes": pack_codes_numpy(indices, fp["bits_mse"]),
                   "norms": np.asarray(encoding.norms, dtype=np.float32).reshape(-1)}
        if prod:
            buffers["signs"] = pack_signs_numpy(np.asarray(encoding.qjl).reshape(-1, d))
            buffers["residual_norms"] = np.asarray(encoding.residual_norms, dtype=np.float32).reshape(-1)
    return write_packed(target, fp, tuple(encoding.prefix_shape), buffers)


def load_encoding(source, quantizer, *, device=None, mmap: bool = False):
    """Read a file back into an encoding of ``quantizer`` with its packed buffers on ``device`` (default: the
    current CUDA device).  Raises ``PackedFormatError`` when the file was written with other constants."""
    from . import turboquant as _tq
    pf = read_packed(source, mmap=mmap)
    check_same_quantizer(pf.quantizer, quantizer)
    torch = _tq._require_cuda()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    up = {}
    for name in ("codes", "signs", "norms", "residual_norms"):
        a = pf.buffers.get(name)
        up[name] = None if a is None else torch.from_numpy(np.array(a, copy=True)).to(dev)
    pk = _tq._Packed(up["codes"], up["signs"], up["norms"], up["residual_norms"], pf.rows, "torch", dev,
                     quantizer._plans)
    cls = _tq.TurboQuantProdEncoding if pf.quantizer["kind"] == "prod" else _tq.TurboQuantMSEEncoding
    return _tq._encoding_from_packed(cls, pk, pf.prefix_shape)
