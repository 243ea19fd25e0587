"""The reference's own TurboQuant tests (Project-Tensor test_turboquant.py:7-123), restated
against this package with the same shapes, seeds, settings and tolerances."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tg(lib_built):
    import project_tensor_b200 as tg
    return tg


def test_mse_roundtrip_shape_and_scale(tg):                       # test_turboquant.py:7-22
    tg.set_device("cpu")
    x = np.random.default_rng(7).standard_normal((5, 16)).astype(np.float32) * 3.0
    quant = tg.TurboQuantMSE(16, 3, seed=123, grid_size=4097, max_iter=64)
    enc = quant.quantize(x)
    recon = quant.dequantize(enc)
    assert enc.indices.shape == x.shape
    assert enc.norms.shape == (5,)
    assert recon.shape == x.shape
    np.testing.assert_allclose(np.linalg.norm(recon, axis=1), np.linalg.norm(x, axis=1), rtol=0.15, atol=1e-3)


def test_mse_accepts_tensor_input(tg):                            # :25-35
    x = tg.Tensor(np.random.default_rng(11).standard_normal((3, 8)).astype(np.float32), requires_grad=False)
    quant = tg.TurboQuantMSE(8, 2, seed=99, grid_size=2049, max_iter=48)
    enc = quant.quantize(x)
    assert enc.indices.shape == (3, 8)
    assert quant.dequantize(enc).shape == (3, 8)


def test_prod_attention_score_matches_explicit_dequant(tg):       # :38-51
    rng = np.random.default_rng(21)
    q = rng.standard_normal((4, 12)).astype(np.float32)
    k = rng.standard_normal((4, 12)).astype(np.float32)
    quant = tg.TurboQuantProd(12, 3, seed=314, grid_size=4097, max_iter=64)
    enc = quant.quantize(k)
    recon = quant.dequantize(enc)
    np.testing.assert_allclose(quant.attention_score(q, enc), np.sum(q * recon, axis=1), rtol=1e-5, atol=1e-5)


def test_prod_single_query_broadcasts_over_many_keys(tg):         # :54-67
    rng = np.random.default_rng(29)
    q = rng.standard_normal((10,)).astype(np.float32)
    k = rng.standard_normal((6, 10)).astype(np.float32)
    quant = tg.TurboQuantProd(10, 3, seed=2026, grid_size=2049, max_iter=48)
    enc = quant.quantize(k)
    recon = quant.dequantize(enc)
    np.testing.assert_allclose(quant.attention_score(q, enc), recon @ q, rtol=1e-5, atol=1e-5)


def test_mse_rotation_is_orthogonal(tg):                          # :70-75
    quant = tg.TurboQuantMSE(16, 3, seed=123)
    np.testing.assert_allclose(quant.rotation.T @ quant.rotation, np.eye(16, dtype=np.float32), rtol=1e-5, atol=1e-5)


def test_lloyd_max_codebook_is_sorted_and_bounded(tg):            # :78-83
    codebook = tg._build_lloyd_max_codebook(32, 3, grid_size=2049, max_iter=64)
    assert np.all(np.diff(codebook) >= 0.0)
    assert codebook.min() >= -1.0 - 1e-6
    assert codebook.max() <= 1.0 + 1e-6


def test_mse_reconstruction_improves_with_more_bits(tg):          # :86-101
    x = np.random.default_rng(101).standard_normal((128, 24)).astype(np.float32)
    x /= np.linalg.norm(x, axis=1, keepdims=True) + 1e-12
    low = tg.TurboQuantMSE(24, 2, seed=77, grid_size=2049, max_iter=64)
    high = tg.TurboQuantMSE(24, 5, seed=77, grid_size=2049, max_iter=64)
    low_mse = float(np.mean((x - low.dequantize(low.quantize(x))) ** 2))
    high_mse = float(np.mean((x - high.dequantize(high.quantize(x))) ** 2))
    assert high_mse < low_mse


def test_prod_dot_error_improves_with_more_bits(tg):              # :104-123
    rng = np.random.default_rng(303)
    q = rng.standard_normal((16, 20)).astype(np.float32)
    k = rng.standard_normal((32, 20)).astype(np.float32)
    low = tg.TurboQuantProd(20, 3, seed=88, grid_size=2049, max_iter=64)
    high = tg.TurboQuantProd(20, 6, seed=88, grid_size=2049, max_iter=64)
    low_enc, high_enc = low.quantize(k), high.quantize(k)
    exact = q @ k.T
    low_scores = np.stack([low.attention_score(query, low_enc) for query in q], axis=0)
    high_scores = np.stack([high.attention_score(query, high_enc) for query in q], axis=0)
    assert float(np.mean(np.abs(exact - high_scores))) < float(np.mean(np.abs(exact - low_scores)))
