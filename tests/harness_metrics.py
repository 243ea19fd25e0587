"""The quality metrics of the reference's validation harness (validate_turboquant.py:22-31, 58-70, 73-119),
restated: same seeded inputs, same definitions, for any object with the quantizers' interface."""
import numpy as np


def harness_inputs(dimension, bits, base_seed=2026, vector_count=256, query_count=32):
    seed = base_seed + dimension * 10 + bits
    keys = (np.random.default_rng(seed + 1).standard_normal((vector_count, dimension)) * 3.0).astype(np.float32)
    queries = (np.random.default_rng(seed + 2).standard_normal((query_count, dimension)) * 1.5).astype(np.float32)
    return seed, keys, queries


def recall_at(exact, approx, k):
    hits = []
    for e, a in zip(np.argpartition(-exact, kth=k - 1, axis=1)[:, :k], np.argpartition(-approx, kth=k - 1, axis=1)[:, :k]):
        hits.append(len(set(e.tolist()) & set(a.tolist())) / k)
    return float(np.mean(hits))


def harness_metrics(make_mse, make_prod, dimension, bits):
    """make_mse / make_prod(dimension, bits, seed=, grid_size=, max_iter=) build the quantizers."""
    seed, keys, queries = harness_inputs(dimension, bits)
    mse_q = make_mse(dimension, bits, seed=seed, grid_size=4097, max_iter=96)
    prod_q = make_prod(dimension, bits, seed=seed, grid_size=4097, max_iter=96)
    recon = np.asarray(mse_q.dequantize(mse_q.quantize(keys)))
    enc = prod_q.quantize(keys)
    approx = np.stack([np.asarray(prod_q.attention_score(q, enc)) for q in queries], axis=0)
    exact = queries @ keys.T
    dots = np.sum(keys * recon, axis=1)
    norms = np.linalg.norm(keys, axis=1) * np.linalg.norm(recon, axis=1)
    return {
        "mse_mse": float(np.mean((keys - recon) ** 2)),
        "mean_cosine_similarity": float(np.mean(dots / np.where(norms > 0.0, norms, 1.0))),
        "prod_dot_mae": float(np.mean(np.abs(exact - approx))),
        "prod_recall_at_10": recall_at(exact, approx, 10),
    }


def assert_matches_table(got, want):
    assert abs(got["mse_mse"] - want["mse_mse"]) <= 2e-6 + 1e-5 * want["mse_mse"], (got, want)
    assert abs(got["mean_cosine_similarity"] - want["mean_cosine_similarity"]) <= 1e-4, (got, want)
    assert abs(got["prod_dot_mae"] - want["prod_dot_mae"]) <= 1e-5 + 1e-5 * want["prod_dot_mae"], (got, want)
    assert abs(got["prod_recall_at_10"] - want["prod_recall_at_10"]) <= 1.0 / 320 + 6e-4, (got, want)
