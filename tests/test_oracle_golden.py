"""CPU suite: the NumPy oracle must reproduce every fixture recorded from the unmodified
reference, bit for bit; the shipped host code (codebook solver, argument checks) must agree
with both; the C ABI library must build, load and export every declared symbol."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import CASES, CASE_IDS, ROOT, golden_case, golden_codebooks, golden_manifest
from oracle import turboquant_oracle as orc


def _params(case, g):
    kw = case["kwargs"]
    mp = orc.mse_params(case["dimension"], case["bits"], seed=case["seed"], **kw)
    pp = orc.prod_params(case["dimension"], case["bits"], seed=case["seed"], **kw)
    return mp, pp


@pytest.mark.parametrize("case", CASES, ids=CASE_IDS)
def test_oracle_constants_match_reference(case):
    g = golden_case(case["name"])
    mp, pp = _params(case, g)
    # codebook / boundaries are pure NumPy arithmetic: identical everywhere
    assert np.array_equal(mp.codebook, g["mse_codebook"])
    assert np.array_equal(mp.boundaries, g["mse_boundaries"])
    assert np.array_equal(pp.mse.codebook, g["prod_codebook"])
    assert np.array_equal(pp.projection, g["prod_projection"])
    # the rotation goes through LAPACK's QR: identical on the build that recorded the fixture,
    # and within float32 rounding on any other
    np.testing.assert_allclose(mp.rotation, g["mse_rotation"], rtol=0, atol=2e-6)


@pytest.mark.parametrize("case", CASES, ids=CASE_IDS)
def test_oracle_outputs_match_reference(case):
    g = golden_case(case["name"])
    d, bits = case["dimension"], case["bits"]
    mp = orc.mse_params(d, bits, rotation=g["mse_rotation"], codebook=g["mse_codebook"])
    codes, norms, prefix = orc.mse_quantize(mp, g["x"])
    assert np.array_equal(codes, g["mse_indices"])
    assert np.array_equal(norms, g["mse_norms"], equal_nan=True)
    assert np.array_equal(orc.mse_dequantize(mp, codes, norms, prefix), g["mse_recon"], equal_nan=True)

    inner = orc.mse_params(d, max(bits - 1, 1), rotation=g["prod_rotation"], codebook=g["prod_codebook"])
    pp = orc.ProdParams(d, bits, inner, g["prod_projection"])
    enc = orc.prod_quantize(pp, g["x"])
    assert np.array_equal(enc[0], g["prod_indices"])
    assert np.array_equal(enc[1], g["prod_qjl"])
    assert np.array_equal(enc[2], g["prod_residual_norms"])
    assert np.array_equal(enc[3], g["prod_norms"])
    assert np.array_equal(orc.prod_dequantize(pp, *enc), g["prod_recon"])
    for q, want in zip(g["queries"], g["scores_broadcast"]):
        assert np.array_equal(orc.prod_attention_score(pp, q, *enc), want)
    assert np.array_equal(orc.prod_attention_score(pp, g["pair_queries"], *enc), g["scores_pairwise"])


def test_codebooks_oracle_and_product_match_reference():
    from project_tensor_b200.codebook import _build_lloyd_max_codebook
    books = golden_codebooks()
    for d, b, grid, iters in golden_manifest()["codebooks"]:
        want = books[f"d{d}_b{b}_g{grid}_i{iters}"]
        assert np.array_equal(orc.lloyd_max_codebook(d, b, grid_size=grid, max_iter=iters), want)
        assert np.array_equal(_build_lloyd_max_codebook(d, b, grid_size=grid, max_iter=iters), want)


def test_codebook_is_not_symmetric_and_middle_boundary_is_negative():
    # property of the reference's discretisation that a "cleaner" solver would lose
    cb = orc.lloyd_max_codebook(128, 4).astype(np.float32)
    bd = 0.5 * (cb[:-1] + cb[1:])
    assert cb[0] != -cb[-1]
    assert bd[7] < 0 and abs(bd[7]) < 1e-3


def test_product_host_constants_match_oracle():
    import project_tensor_b200 as tg
    for d, bits, seed in [(128, 4, 2026), (64, 2, 7), (16, 3, 123)]:
        q = tg.TurboQuantMSE(d, bits, seed=seed)
        p = orc.mse_params(d, bits, seed=seed)
        assert np.array_equal(q.rotation, p.rotation)
        assert np.array_equal(q.codebook, p.codebook)
        assert np.array_equal(q.boundaries, p.boundaries)
        assert q.index_dtype is np.uint8
        pq = tg.TurboQuantProd(d, bits, seed=seed)
        pp = orc.prod_params(d, bits, seed=seed)
        assert pq.mse.bits == max(bits - 1, 1)
        assert np.array_equal(pq.projection, pp.projection)
        assert np.array_equal(pq.mse.codebook, pp.mse.codebook)


def test_reference_error_messages():
    import project_tensor_b200 as tg
    with pytest.raises(ValueError, match="dimension must be >= 2"):
        tg.TurboQuantMSE(1, 2)
    with pytest.raises(ValueError, match="bits must be >= 1"):
        tg.TurboQuantMSE(8, 0)
    with pytest.raises(ValueError, match="bits must be >= 1"):
        tg.TurboQuantProd(8, 0)
    with pytest.raises(ValueError, match=r"rotation must have shape \(8, 8\), got \(4, 4\)"):
        tg.TurboQuantMSE(8, 2, rotation=np.eye(4))
    with pytest.raises(ValueError, match="codebook shape does not match bit-width"):
        tg.TurboQuantMSE(8, 2, rotation=np.eye(8), codebook=np.zeros(3))
    with pytest.raises(ValueError, match=r"projection must have shape \(8, 8\), got \(8, 4\)"):
        tg.TurboQuantProd(8, 2, seed=1, projection=np.zeros((8, 4)))
    quant = tg.TurboQuantMSE(8, 2, seed=1, grid_size=513, max_iter=8)
    with pytest.raises(ValueError, match=r"expected input with trailing dimension 8, got shape \(3, 7\)"):
        quant.quantize(np.zeros((3, 7), np.float32))
    with pytest.raises(ValueError, match="expected input with trailing dimension 8"):
        quant.quantize(np.float32(1.0))


def test_encoding_dataclasses_keep_reference_fields():
    import dataclasses
    import project_tensor_b200 as tg
    assert [f.name for f in dataclasses.fields(tg.TurboQuantMSEEncoding)] == ["indices", "norms", "prefix_shape"]
    assert [f.name for f in dataclasses.fields(tg.TurboQuantProdEncoding)] == [
        "indices", "qjl", "residual_norms", "norms", "prefix_shape"]
    e = tg.TurboQuantProdEncoding(indices=np.zeros((2, 4), np.uint8), qjl=np.ones((2, 4), np.int8),
                                  residual_norms=np.ones(2, np.float32), norms=np.ones(2, np.float32),
                                  prefix_shape=(2,))
    assert e.qjl.dtype == np.int8 and e.indices.shape == (2, 4) and e.prefix_shape == (2,)


def test_library_builds_loads_and_exports_every_declared_symbol(lib_built):
    header = open(os.path.join(ROOT, "include", "tq_b200.h")).read()
    declared = set(re.findall(r"\b(tq_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 20
    lib = ctypes.CDLL(lib_built)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/tq_b200.h but not exported"
    from project_tensor_b200 import _native
    assert set(_native.SIGNATURES) == declared
    assert _native.load().tq_version() == 100


def test_no_cpu_fallback_without_a_device(lib_built):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import project_tensor_b200 as tg
    from project_tensor_b200._native import TurboQuantNativeError
    quant = tg.TurboQuantMSE(8, 2, seed=1, grid_size=513, max_iter=8)
    with pytest.raises(TurboQuantNativeError):
        quant.quantize(np.zeros((3, 8), np.float32))
    # the caches hold device memory from the start: they refuse to exist without a device, and argument
    # errors still come first
    prod = tg.TurboQuantProd(8, 2, seed=1, grid_size=513, max_iter=8)
    with pytest.raises(TurboQuantNativeError):
        tg.PackedKeyCache(prod, 2, 16)
    with pytest.raises(TurboQuantNativeError):
        tg.PackedKVCache(prod, quant, 2, 16)
    with pytest.raises(TypeError):
        tg.PackedKeyCache(quant, 2, 16)
    with pytest.raises(ValueError):
        tg.PackedKeyCache(prod, 0, 16)


@pytest.mark.parametrize("name", ["d128_b4", "d64_b2", "d128_b1"])
def test_oracle_decode_attention_on_reference_scores_and_values(name):
    """decode_attention = softmax(scale * scores) @ values.  The scores and the dequantized values inside are the
    reference's own recorded outputs (fixtures); the softmax and the weighted sum around them are recomputed
    here in float64 from the formula of Tensor.softmax / scaled_dot_product_attention."""
    case = next(c for c in CASES if c["name"] == name)
    g = golden_case(name)
    if g["x"].ndim != 2:
        pytest.skip("flat cases only")
    d, bits = case["dimension"], case["bits"]
    mp = orc.mse_params(d, bits, rotation=g["mse_rotation"], codebook=g["mse_codebook"])
    inner = orc.mse_params(d, max(bits - 1, 1), rotation=g["prod_rotation"], codebook=g["prod_codebook"])
    pp = orc.ProdParams(d, bits, inner, g["prod_projection"])
    finite = np.isfinite(g["mse_recon"]).all(axis=1) & np.isfinite(g["scores_broadcast"]).all(axis=0)
    rows = np.nonzero(finite)[0]
    kenc = tuple(g[k][rows] for k in ("prod_indices", "prod_qjl", "prod_residual_norms", "prod_norms"))
    for scale in (None, 0.5):
        got = orc.decode_attention(pp, mp, g["queries"], kenc, g["mse_indices"][rows], g["mse_norms"][rows], scale)
        s = g["scores_broadcast"][:, rows].astype(np.float64) * np.float64(np.float32(scale or d ** -0.5))
        w = np.exp(s - s.max(axis=1, keepdims=True))
        w /= w.sum(axis=1, keepdims=True)
        want = w @ g["mse_recon"][rows].astype(np.float64)
        assert got.dtype == np.float32 and got.shape == (g["queries"].shape[0], d)
        np.testing.assert_allclose(got, want, rtol=0, atol=2e-6 * np.abs(want).max() + 1e-7)
