"""The file format of packed encodings: CPU round trips, damage and mismatch detection, files written from the
oracle's (reference-shaped) arrays; on the GPU, the device packers against the NumPy statement of the bit
layout and a save -> load -> score round trip."""
import io
import types

import numpy as np
import pytest

import project_tensor_b200 as tg
from project_tensor_b200 import packed_format as pf
from oracle import turboquant_oracle as orc


def _oracle_prod_encoding(d, bits, n, seed=2026):
    p = orc.prod_params(d, bits, seed=seed)
    x = np.random.default_rng(7).standard_normal((n, d)).astype(np.float32)
    codes, qjl, rn, norms = orc.prod_quantize(p, x)[:4]
    enc = types.SimpleNamespace(indices=codes, qjl=qjl, residual_norms=rn, norms=norms, prefix_shape=(n,))
    return p, x, enc


@pytest.mark.parametrize("d,bits", [(64, 1), (64, 3), (128, 2), (128, 3), (128, 4), (96, 5), (256, 8)])
def test_numpy_packers_round_trip(d, bits):
    rng = np.random.default_rng(d * 10 + bits)
    idx = rng.integers(0, 1 << bits, (53, d)).astype(np.uint8)
    packed = pf.pack_codes_numpy(idx, bits)
    assert packed.shape == (53, pf.code_row_bytes(d, bits)) and packed.dtype == np.uint8
    assert np.array_equal(pf.unpack_codes_numpy(packed, d, bits), idx)
    # coordinate j sits at bits [j*bits, (j+1)*bits) of the little-endian stream
    words = packed.view("<u4")
    for j in (0, 1, d // 2, d - 1):
        bit = j * bits
        v = int(words[5, bit // 32]) >> (bit % 32)
        if bit % 32 + bits > 32:
            v |= int(words[5, bit // 32 + 1]) << (32 - bit % 32)
        assert v & ((1 << bits) - 1) == idx[5, j]
    q = (rng.integers(0, 2, (53, d)) * 2 - 1).astype(np.int8)
    s = pf.pack_signs_numpy(q)
    assert s.shape == (53, pf.sign_row_bytes(d))
    assert np.array_equal(pf.unpack_signs_numpy(s, d), q)
    sw = s.view("<u4")
    for j in (0, 1, 2, 31, d - 1):
        pos = (j % 32) // 2 + 16 * (j % 2)
        assert (int(sw[9, j // 32]) >> pos) & 1 == (1 if q[9, j] > 0 else 0)


def test_file_round_trip_from_reference_shaped_arrays(tmp_path):
    quant = tg.TurboQuantProd(128, 4, seed=2026)
    p, x, enc = _oracle_prod_encoding(128, 4, 300)
    # the package's host constants are the oracle's (and the reference's): same fingerprint
    fake = types.SimpleNamespace(dimension=128, bits=4, projection=p.projection,
                                 mse=types.SimpleNamespace(bits=3, codebook=p.mse.codebook, rotation=p.mse.rotation))
    assert pf.quantizer_fingerprint(fake) == pf.quantizer_fingerprint(quant)
    enc.prefix_shape = (3, 100)
    path = tmp_path / "keys.tqp"
    nbytes = pf.save_encoding(path, quant, enc)
    assert path.stat().st_size == nbytes
    for mmap in (False, True):
        back = pf.read_packed(path, mmap=mmap)
        assert back.rows == 300 and back.prefix_shape == (3, 100)
        assert back.quantizer["kind"] == "prod" and back.quantizer["bits_mse"] == 3
        assert np.array_equal(back.indices(), enc.indices)
        assert np.array_equal(back.qjl(), enc.qjl)
        assert np.array_equal(back.buffers["norms"], enc.norms)
        assert np.array_equal(back.buffers["residual_norms"], enc.residual_norms)
        for sec in back.header["sections"]:
            assert int(sec["offset"]) % 64 == 0
    # the unpacked file gives the oracle's scores again
    q = np.random.default_rng(3).standard_normal(128).astype(np.float32)
    want = orc.prod_attention_score(p, q, enc.indices, enc.qjl, enc.residual_norms, enc.norms, (300,))
    got = orc.prod_attention_score(p, q, back.indices(), back.qjl(), back.buffers["residual_norms"],
                                   back.buffers["norms"], (300,))
    assert np.array_equal(want, got)


def test_mse_file_and_file_objects():
    quant = tg.TurboQuantMSE(64, 3, seed=11)
    p = orc.mse_params(64, 3, seed=11)
    x = np.random.default_rng(1).standard_normal((17, 64)).astype(np.float32)
    codes, norms = orc.mse_quantize(p, x)[:2]
    enc = types.SimpleNamespace(indices=codes, norms=norms, prefix_shape=(17,))
    buf = io.BytesIO()
    pf.save_encoding(buf, quant, enc)
    back = pf.read_packed(buf.getvalue())
    assert set(back.buffers) == {"codes", "norms"}
    assert np.array_equal(back.indices(), codes)
    with pytest.raises(pf.PackedFormatError):
        back.qjl()
    buf.seek(0)
    assert pf.read_packed(buf).rows == 17
    # empty encodings are files too
    empty = types.SimpleNamespace(indices=np.zeros((0, 64), np.uint8), norms=np.zeros((0,), np.float32), prefix_shape=(0,))
    out = io.BytesIO()
    pf.save_encoding(out, quant, empty)
    assert pf.read_packed(out.getvalue()).rows == 0


def test_damage_and_mismatch_are_refused():
    quant = tg.TurboQuantProd(64, 3, seed=5)
    _, _, enc = _oracle_prod_encoding(64, 3, 40, seed=5)
    buf = io.BytesIO()
    pf.save_encoding(buf, quant, enc)
    data = bytearray(buf.getvalue())
    with pytest.raises(pf.PackedFormatError, match="magic"):
        pf.read_packed(b"NOTAFILE" + bytes(data[8:]))
    bad_version = bytearray(data)
    bad_version[8] = 9
    with pytest.raises(pf.PackedFormatError, match="version"):
        pf.read_packed(bytes(bad_version))
    flipped = bytearray(data)
    flipped[-70] ^= 0x10
    with pytest.raises(pf.PackedFormatError, match="CRC"):
        pf.read_packed(bytes(flipped))
    with pytest.raises(pf.PackedFormatError, match="ends inside"):
        pf.read_packed(bytes(data[: len(data) // 2]))
    other = tg.TurboQuantProd(64, 3, seed=6)
    with pytest.raises(pf.PackedFormatError, match="another quantizer"):
        pf.check_same_quantizer(pf.read_packed(bytes(data)).quantizer, other)
    with pytest.raises(pf.PackedFormatError, match="shape"):
        pf.write_packed(io.BytesIO(), pf.quantizer_fingerprint(quant), (40,),
                        {"codes": np.zeros((40, 3), np.uint8), "norms": np.zeros(40, np.float32),
                         "signs": np.zeros((40, 8), np.uint8), "residual_norms": np.zeros(40, np.float32)})


def _rewrite_header(data: bytes, edit) -> bytes:
    """The same file with its JSON header changed by `edit` (a hand edit or a damaged header that happens to
    parse); `fix_crc` decides whether the header's own checksum is recomputed, as a careful editor would."""
    import json
    import struct
    import zlib
    hlen = struct.unpack("<II", data[8:16])[1]
    doc = json.loads(data[16:16 + hlen].decode())
    edit(doc)
    first = min(int(sec["offset"]) for sec in json.loads(data[16:16 + hlen].decode())["sections"])
    new = json.dumps(doc, sort_keys=True).encode()
    head = data[:8] + struct.pack("<II", struct.unpack("<II", data[8:16])[0], len(new)) + new + struct.pack("<I", zlib.crc32(new) & 0xFFFFFFFF)
    assert len(head) <= first, "the edits below keep the sections where they are"
    return head + b"\0" * (first - len(head)) + data[first:]


def test_a_header_that_contradicts_itself_is_refused():
    """rows, shapes, section set and prefix shape are what the kernels index by: a header whose numbers do not
    agree with each other must not reach the device, whether or not its checksum was fixed up."""
    quant = tg.TurboQuantProd(64, 3, seed=5)
    _, _, enc = _oracle_prod_encoding(64, 3, 40, seed=5)
    buf = io.BytesIO()
    pf.save_encoding(buf, quant, enc)
    data = buf.getvalue()
    assert pf.read_packed(data).rows == 40
    # a header edited without fixing its checksum
    import struct
    hlen = struct.unpack("<II", data[8:16])[1]
    raw = bytearray(data)
    at = data.index(b'"rows": 40')
    raw[at + 8:at + 10] = b"99"
    with pytest.raises(pf.PackedFormatError, match="header CRC"):
        pf.read_packed(bytes(raw))

    def rows_up(doc): doc["rows"] = 99                                   # more rows than the sections hold
    def codes_wide(doc): [sec for sec in doc["sections"] if sec["name"] == "codes"][0]["shape"][1] = 99
    def signs_gone(doc):
        for sec in doc["sections"]:
            if sec["name"] == "signs":
                sec["name"] = "sigma"
    def prefix_off(doc): doc["prefix_shape"] = [41]
    def kind_mse(doc): doc["quantizer"]["kind"] = "mse"                  # four sections in an MSE file
    def dtype_off(doc): [sec for sec in doc["sections"] if sec["name"] == "norms"][0]["dtype"] = "<i4"
    for edit, what in ((rows_up, "require"), (codes_wide, "require|inconsistent"), (signs_gone, "must hold"),
                       (prefix_off, "prefix_shape"), (kind_mse, "must hold"), (dtype_off, "dtype")):
        with pytest.raises(pf.PackedFormatError, match=what):
            pf.read_packed(_rewrite_header(data, edit))


@pytest.mark.gpu
@pytest.mark.parametrize("d,bits", [(128, 4), (64, 3), (256, 2)])
def test_gpu_buffers_follow_the_numpy_layout(d, bits):
    quant = tg.TurboQuantProd(d, bits, seed=2026)
    x = np.random.default_rng(4).standard_normal((1000, d)).astype(np.float32)
    enc = quant.quantize(x)
    host = tg.packed_to_host(enc)
    assert np.array_equal(host["codes"].numpy(), pf.pack_codes_numpy(np.asarray(enc.indices), max(bits - 1, 1)))
    assert np.array_equal(host["signs"].numpy(), pf.pack_signs_numpy(np.asarray(enc.qjl)))


@pytest.mark.gpu
def test_gpu_save_load_round_trip(tmp_path):
    import torch
    quant = tg.TurboQuantProd(128, 4, seed=2026)
    keys = torch.randn(4, 2500, 128, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    enc = quant.quantize(keys)
    path = tmp_path / "cache.tqp"
    pf.save_encoding(path, quant, enc)
    back = pf.load_encoding(path, quant)
    assert back.prefix_shape == (4, 2500)
    a, b = tg.packed_buffers(enc), tg.packed_buffers(back)
    for name in a:
        assert torch.equal(a[name], b[name])
    q = torch.randn(128, device="cuda", generator=torch.Generator("cuda").manual_seed(2))
    assert torch.equal(quant.attention_score(q, enc), quant.attention_score(q, back))
    assert torch.equal(quant.dequantize(enc), quant.dequantize(back))
    with pytest.raises(pf.PackedFormatError):
        pf.load_encoding(path, tg.TurboQuantProd(128, 4, seed=1))
    # a file written on the CPU from reference-shaped arrays loads the same way
    cpu_file = tmp_path / "cpu.tqp"
    plain = types.SimpleNamespace(indices=enc.indices.cpu().numpy().reshape(-1, 128), qjl=enc.qjl.cpu().numpy().reshape(-1, 128),
                                  residual_norms=enc.residual_norms.cpu().numpy().reshape(-1),
                                  norms=enc.norms.cpu().numpy().reshape(-1), prefix_shape=(4, 2500))
    pf.save_encoding(cpu_file, quant, plain)
    again = pf.load_encoding(cpu_file, quant)
    for name in a:
        assert torch.equal(a[name], tg.packed_buffers(again)[name])
