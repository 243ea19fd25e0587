"""The reference's validation harness prints quality metrics for seeded inputs; the table recorded from the
unmodified reference is a known-answer test for the whole path: the oracle must reproduce it on CPU, the CUDA
path on a GPU (every metric to the printed precision; recall@10 within one swapped neighbour)."""
import json
import os

import numpy as np
import pytest

import harness_metrics as hm

TABLE = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "harness_table.json")))["rows"]
IDS = [f"d{r['dimension']}_b{r['bits']}" for r in TABLE]


class _OracleMSE:
    def __init__(self, d, bits, seed, grid_size, max_iter):
        from oracle import turboquant_oracle as orc
        self.orc, self.p = orc, orc.mse_params(d, bits, seed=seed, grid_size=grid_size, max_iter=max_iter)

    def quantize(self, x):
        return self.orc.mse_quantize(self.p, x)

    def dequantize(self, enc):
        return self.orc.mse_dequantize(self.p, *enc)


class _OracleProd:
    def __init__(self, d, bits, seed, grid_size, max_iter):
        from oracle import turboquant_oracle as orc
        self.orc, self.p = orc, orc.prod_params(d, bits, seed=seed, grid_size=grid_size, max_iter=max_iter)

    def quantize(self, x):
        return self.orc.prod_quantize(self.p, x)

    def attention_score(self, q, enc):
        return self.orc.prod_attention_score(self.p, q, *enc)


@pytest.mark.parametrize("row", TABLE, ids=IDS)
def test_oracle_reproduces_the_harness_table(row):
    got = hm.harness_metrics(lambda d, b, **kw: _OracleMSE(d, b, **kw), lambda d, b, **kw: _OracleProd(d, b, **kw),
                             row["dimension"], row["bits"])
    hm.assert_matches_table(got, row)


@pytest.mark.gpu
@pytest.mark.parametrize("row", TABLE, ids=IDS)
def test_cuda_path_reproduces_the_harness_table(row, lib_built):
    import project_tensor_b200 as tg
    got = hm.harness_metrics(tg.TurboQuantMSE, tg.TurboQuantProd, row["dimension"], row["bits"])
    hm.assert_matches_table(got, row)


@pytest.mark.gpu
@pytest.mark.parametrize("row", TABLE, ids=IDS)
def test_device_side_quality_report_reproduces_the_harness_table(row, lib_built):
    """quality_report computes the harness's metrics on the device, chunk by chunk, with the device top-k for the
    recall; on the harness's own 256 vectors (walked in chunks of 100 to exercise the merging) it must print the
    table of the unmodified reference."""
    import project_tensor_b200 as tg
    d, bits = row["dimension"], row["bits"]
    seed, keys, queries = hm.harness_inputs(d, bits)
    mse_q = tg.TurboQuantMSE(d, bits, seed=seed, grid_size=4097, max_iter=96)
    prod_q = tg.TurboQuantProd(d, bits, seed=seed, grid_size=4097, max_iter=96)
    got = tg.quality_report(mse_q, prod_q, keys, queries, ks=(1, 5, 10), chunk_rows=100)
    assert got["keys"] == 256 and got["queries"] == 32
    hm.assert_matches_table(got, row)
    # the score equals the dot product with the explicit reconstruction (test_turboquant.py:38-67 in the reference)
    assert got["prod_vs_explicit_gap"] <= 1e-4 * max(1.0, got["prod_dot_mae"])
    assert 0.0 <= got["prod_recall_at_1"] <= 1.0 and got["prod_dot_rmse"] >= got["prod_dot_mae"]


@pytest.mark.gpu
def test_quality_report_at_scale_from_a_generator(lib_built):
    """2,097,152 keys that never exist at once (a callable yields them chunk by chunk): the metrics must sit where the
    harness's small-sample values for d = 128, bits = 4 sit, and recall must grow with k."""
    import torch
    import project_tensor_b200 as tg
    d, bits, n, chunk = 128, 4, 1 << 21, 1 << 19
    def keys(off, rows):
        if off >= n:
            return None
        gen = torch.Generator(device="cuda").manual_seed(1000 + off // chunk)
        return torch.randn((min(rows, n - off), d), generator=gen, device="cuda") * 3.0
    queries = torch.randn((16, d), generator=torch.Generator(device="cuda").manual_seed(5), device="cuda") * 1.5
    got = tg.quality_report(tg.TurboQuantMSE(d, bits, seed=2026), tg.TurboQuantProd(d, bits, seed=2026), keys, queries,
                            ks=(1, 10, 100), chunk_rows=chunk)
    assert got["keys"] == n
    assert abs(got["mse_mse"] - 0.083) < 0.004 and got["mean_cosine_similarity"] > 0.995
    assert 8.0 < got["prod_dot_mae"] < 10.5
    assert 0.0 < got["prod_recall_at_1"] <= 1.0 and got["prod_recall_at_10"] > 0.3 and got["prod_recall_at_100"] > 0.4
