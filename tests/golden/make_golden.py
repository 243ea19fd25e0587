#!/usr/bin/env python3
"""Regenerate the golden fixtures in this directory from the unmodified reference.

Usage (only where a checkout of Project-Tensor is available):

    python tests/golden/make_golden.py --reference /path/to/Project-Tensor

The reference package imports cupy unconditionally, but its TurboQuant module
(``tensor_gpu_v2/_quant.py``) only needs ``cupy.ndarray`` for an isinstance test
and ``Tensor`` for input unwrapping, so that one file is executed as shipped
behind two stub modules.  Everything stored here is an output of that file's
NumPy path; nothing is computed by this repository's own code.

The fixtures carry the rotation / projection / codebook that the reference
built, so that consumers can pass them back in (``rotation=``, ``codebook=``,
``projection=``) and are not exposed to last-bit differences between LAPACK
builds when the QR factorisation is repeated on another host.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference_quant(root: str):
    cupy = types.ModuleType("cupy")
    cupy.ndarray = type("ndarray", (), {})
    sys.modules.setdefault("cupy", cupy)
    pkg = types.ModuleType("tensor_gpu_v2")
    pkg.__path__ = []
    core = types.ModuleType("tensor_gpu_v2._core")

    class Tensor:  # stand-in: the quantizers only read ``.data``
        def __init__(self, data, requires_grad=False):
            self.data = data

    core.Tensor = Tensor
    sys.modules["tensor_gpu_v2"] = pkg
    sys.modules["tensor_gpu_v2._core"] = core
    spec = importlib.util.spec_from_file_location(
        "tensor_gpu_v2._quant", os.path.join(root, "tensor_gpu_v2", "_quant.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["tensor_gpu_v2._quant"] = mod
    spec.loader.exec_module(mod)
    return mod


def normal32(seed, shape):
    return np.random.default_rng(seed).standard_normal(shape).astype(np.float32)


# (name, dimension, bits, quantizer seed, leading shape, ctor kwargs, input recipe)
CASES = [
    ("d128_b4", 128, 4, 2026, (256,), {}, "edge"),
    ("d128_b3", 128, 3, 2026, (2, 96), {}, "outlier"),
    ("d64_b2", 64, 2, 2026, (160,), {}, "edge"),
    ("d256_b4", 256, 4, 2026, (96,), {}, "plain"),
    ("d128_b1", 128, 1, 2026, (64,), {}, "plain"),
    ("d12_b3", 12, 3, 314, (2, 3), {"grid_size": 4097, "max_iter": 64}, "plain"),
    ("d20_b6", 20, 6, 88, (33,), {"grid_size": 2049, "max_iter": 64}, "plain"),
]

CODEBOOK_SETTINGS = (
    [(d, b, 16385, 200) for d in (64, 128, 256) for b in (1, 2, 3, 4)]
    + [(16, 3, 4097, 64), (8, 2, 2049, 48), (12, 2, 4097, 64), (10, 2, 2049, 48),
       (32, 3, 2049, 64), (24, 2, 2049, 64), (24, 5, 2049, 64), (20, 2, 2049, 64),
       (20, 5, 2049, 64), (128, 5, 16385, 200), (64, 8, 4097, 96)]
)


def make_inputs(name, d, lead, recipe):
    seed = 20260 + sum(map(ord, name))
    x = normal32(seed, tuple(lead) + (d,))
    flat = x.reshape(-1, d)
    if recipe == "edge":
        flat[0] = 0.0                       # zero row: norm 0, code of zero
        flat[1] *= 1e-3                     # small and large scales
        flat[2] *= 1e3
        flat[3] = 0.0
        flat[3, 5] = 2.5                    # axis-aligned row
        flat[4] = flat[5]                   # duplicate rows
    elif recipe == "outlier":
        ch = np.random.default_rng(20280).choice(d, 4, replace=False)
        flat[:, ch] *= 10.0                 # fixed outlier channels (KV-cache-like)
    return x


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a Project-Tensor checkout")
    args = ap.parse_args()
    rq = load_reference_quant(args.reference)
    manifest = {"numpy": np.__version__, "cases": [], "codebooks": []}

    books = {}
    for d, b, g, it in CODEBOOK_SETTINGS:
        books[f"d{d}_b{b}_g{g}_i{it}"] = rq._build_lloyd_max_codebook(d, b, grid_size=g, max_iter=it)
        manifest["codebooks"].append([d, b, g, it])
    np.savez_compressed(os.path.join(HERE, "codebooks.npz"), **books)

    for name, d, bits, seed, lead, kw, recipe in CASES:
        x = make_inputs(name, d, lead, recipe)
        n = int(np.prod(lead))
        out = {"x": x}
        mse = rq.TurboQuantMSE(d, bits, seed=seed, **kw)
        enc = mse.quantize(x)
        out.update(mse_rotation=mse.rotation, mse_codebook=mse.codebook,
                   mse_boundaries=mse.boundaries, mse_indices=enc.indices,
                   mse_norms=enc.norms, mse_recon=mse.dequantize(enc))
        prod = rq.TurboQuantProd(d, bits, seed=seed, **kw)
        penc = prod.quantize(x)
        queries = normal32(20270 + d + bits, (4, d))
        pair_q = normal32(20275 + d + bits, tuple(lead) + (d,))
        out.update(prod_rotation=prod.mse.rotation, prod_codebook=prod.mse.codebook,
                   prod_boundaries=prod.mse.boundaries, prod_projection=prod.projection,
                   prod_indices=penc.indices, prod_qjl=penc.qjl,
                   prod_residual_norms=penc.residual_norms, prod_norms=penc.norms,
                   prod_recon=prod.dequantize(penc),
                   queries=queries, pair_queries=pair_q,
                   scores_broadcast=np.stack([prod.attention_score(q, penc) for q in queries]),
                   scores_pairwise=prod.attention_score(pair_q, penc))
        np.savez_compressed(os.path.join(HERE, f"case_{name}.npz"), **out)
        manifest["cases"].append({"name": name, "dimension": d, "bits": bits, "seed": seed,
                                  "lead": list(lead), "kwargs": kw, "n": n})
    with open(os.path.join(HERE, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1)
    print("wrote", len(CASES), "cases and", len(books), "codebooks to", HERE)


if __name__ == "__main__":
    main()
