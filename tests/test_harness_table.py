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
