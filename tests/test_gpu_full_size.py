"""GPU suite at the sizes the benchmark configurations name.

The headline configuration (TurboQuantProd d=128 bits=4 seed=2026, 1,048,576 keys, 32 queries) is compared
with the NumPy oracle on this host at its full size: packed codes and QJL signs (differences counted, each
must lie within 1e-5 of its decision point, rate <= 1e-6), norms and residual norms (1e-5 relative) and
scores (1e-4 of |q||k|/sqrt(d)).  The tensor-core and the reference-order kernels are compared byte for byte
on the same 1,048,576 rows for both quantizers, the KV-cache configuration runs at its shape on a sample of
(batch, head) groups, and the twelve (dimension, bits) settings of the sweep run quantize, dequantize and
16-query scoring for both classes.
"""
import numpy as np
import pytest

from oracle import turboquant_oracle as orc
import parity

pytestmark = pytest.mark.gpu

REL_RECON = 1e-5
REL_SCORE = 1e-4


@pytest.fixture(scope="module")
def tg(lib_built):
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import project_tensor_b200 as tg
    return tg


def _prod_params(prod, d, bits):
    inner = orc.mse_params(d, max(bits - 1, 1), rotation=prod.mse.rotation, codebook=prod.mse.codebook)
    return orc.ProdParams(d, bits, inner, prod.projection)


def _sign_window_violations(x, want, prod, rows, cols):
    """|residual . S_j| in float64 for the listed (row, coordinate) pairs, residual from the reference's codes."""
    if len(rows) == 0:
        return 0
    x64 = x[rows].astype(np.float64)
    n = np.linalg.norm(x64, axis=1)
    unit = np.where(n[:, None] > 0, x64 / np.where(n > 0, n, 1.0)[:, None], 0.0)
    recon = prod.mse.codebook.astype(np.float64)[want[0][rows]] @ prod.mse.rotation.astype(np.float64)
    proj = np.einsum("rk,rk->r", unit - recon, prod.projection.astype(np.float64)[cols])
    return int((np.abs(proj) > parity.WINDOW).sum())


@pytest.mark.parametrize("path", ["auto", "exact"])
def test_config2_full_size_against_oracle(tg, path):
    """1,048,576 keys: every packed code, sign bit, norm and residual norm against the oracle, and the
    scores of two of the 32 queries (the reference scores one query per call)."""
    d, bits, n = 128, 4, 1 << 20
    x = np.random.default_rng(20262).standard_normal((n, d)).astype(np.float32)
    queries = np.random.default_rng(20272).standard_normal((32, d)).astype(np.float32)
    prod = tg.TurboQuantProd(d, bits, seed=2026)
    prod.set_kernel_path(path)
    pp = _prod_params(prod, d, bits)
    want = orc.prod_quantize(pp, x)
    enc = prod.quantize(x)
    codes, qjl = enc.indices, enc.qjl
    f, o, t = parity.code_flip_report(codes, want[0], prod.mse.rotation, prod.mse.boundaries, x)
    parity.assert_discrete_parity(f, o, t, f"config 2 codes ({path})")
    same_row = ~np.any(codes != want[0], axis=1)
    sdiff = (qjl != want[1]) & same_row[:, None]
    rows, cols = np.nonzero(sdiff)
    outside = _sign_window_violations(x, want, prod, rows, cols)
    sf = int(sdiff.sum())
    print(f"config 2 ({path}): {f} code differences ({o} outside the window), {sf} sign differences "
          f"({outside} outside) in {t} coordinates")
    parity.assert_discrete_parity(sf, outside, t, f"config 2 signs ({path})")
    assert parity.max_rel_scalar(enc.norms, want[3]) <= REL_RECON
    assert parity.max_rel_scalar(enc.residual_norms[same_row], want[2][same_row]) <= REL_RECON
    got = prod.attention_scores(queries, enc)
    for qi in (0, 31):
        ref = orc.prod_attention_score(pp, queries[qi], *want)
        err = parity.max_score_err(got[qi][same_row], ref[same_row], np.linalg.norm(queries[qi]), want[3][same_row], d)
        assert err <= REL_SCORE, (qi, err)


@pytest.mark.parametrize("cls_name,bits,d", [("TurboQuantProd", 4, 128), ("TurboQuantProd", 3, 128), ("TurboQuantMSE", 4, 128),
                                             ("TurboQuantMSE", 4, 256), ("TurboQuantMSE", 1, 256), ("TurboQuantProd", 4, 256)])
def test_tensor_and_exact_kernels_agree_byte_for_byte_at_full_size(tg, cls_name, bits, d):
    """The tensor-core pass plus its exact second stage must leave the same packed bytes as the
    reference-order kernels on all 1,048,576 rows (d = 256, where the rotation streams through shared memory:
    524,288 rows), run after run, and the same norms within 1e-5."""
    import torch
    from project_tensor_b200 import packed_buffers
    n = (1 << 20) * 128 // d
    gen = torch.Generator(device="cuda").manual_seed(20262 + bits)
    x = torch.randn((n, d), generator=gen, device="cuda", dtype=torch.float32)
    q = getattr(tg, cls_name)(d, bits, seed=2026)
    q.set_kernel_path("exact")
    ref = packed_buffers(q.quantize(x))
    q.set_kernel_path("auto")
    for rep in range(3):
        got = packed_buffers(q.quantize(x))
        for name in ("codes", "signs"):
            if ref[name] is not None:
                bad = int((got[name] != ref[name]).any(dim=1).sum())
                assert bad == 0, f"{cls_name} bits={bits} run {rep}: {bad} rows with different {name}"
        for name in ("norms", "residual_norms"):
            if ref[name] is not None:
                rel = float(((got[name] - ref[name]).abs() / ref[name].abs().clamp_min(1e-30)).max())
                assert rel <= REL_RECON, f"{cls_name} bits={bits} run {rep}: {name} off by {rel:.2e}"


def test_config3_kv_cache_shape_on_sampled_groups(tg):
    """batch 8 x 8 KV heads x 32,768 tokens x 128, four outlier channels per head scaled x10, bits = 3, 32 query
    heads (4 per KV head), one new token: three (batch, head) groups at their full length against the oracle."""
    d, bits, tokens, heads = 128, 3, 32768, 8
    picks = [(0, 0), (3, 5), (7, 7)]
    out_rng = np.random.default_rng(20280)
    outliers = [out_rng.choice(d, 4, replace=False) for _ in range(heads)]
    prod = tg.TurboQuantProd(d, bits, seed=2026)
    pp = _prod_params(prod, d, bits)
    keys = np.empty((len(picks), tokens, d), np.float32)
    queries = np.empty((len(picks), 4, d), np.float32)
    for gi, (b, h) in enumerate(picks):
        keys[gi] = np.random.default_rng(20263 * 1000 + b * heads + h).standard_normal((tokens, d)).astype(np.float32)
        keys[gi][:, outliers[h]] *= 10.0
        queries[gi] = np.random.default_rng(20273 * 1000 + b * heads + h).standard_normal((4, d)).astype(np.float32)
    enc = prod.quantize(keys)
    assert enc.prefix_shape == (len(picks), tokens)
    got = prod.attention_scores(queries.reshape(-1, d), enc, groups=len(picks))
    codes = enc.indices.reshape(len(picks), tokens, d)
    qjl = enc.qjl.reshape(len(picks), tokens, d)
    norms = enc.norms.reshape(len(picks), tokens)
    for gi in range(len(picks)):
        want = orc.prod_quantize(pp, keys[gi])
        f, o, t = parity.code_flip_report(codes[gi], want[0], prod.mse.rotation, prod.mse.boundaries, keys[gi])
        parity.assert_discrete_parity(f, o, t, f"config 3 group {picks[gi]} codes")
        same = ~np.any(codes[gi] != want[0], axis=1)
        sdiff = (qjl[gi] != want[1]) & same[:, None]
        rows, cols = np.nonzero(sdiff)
        parity.assert_discrete_parity(int(sdiff.sum()), _sign_window_violations(keys[gi], want, prod, rows, cols), t,
                                      f"config 3 group {picks[gi]} signs")
        assert parity.max_rel_scalar(norms[gi], want[3]) <= REL_RECON
        for qi in range(4):
            ref = orc.prod_attention_score(pp, queries[gi, qi], *want)
            err = parity.max_score_err(got[gi * 4 + qi][same], ref[same], np.linalg.norm(queries[gi, qi]), want[3][same], d)
            assert err <= REL_SCORE, (picks[gi], qi, err)


@pytest.mark.parametrize("bits", [1, 2, 3, 4])
@pytest.mark.parametrize("d", [64, 128, 256])
def test_config4_sweep_every_setting(tg, d, bits):
    """bits in {1..4} x dimension in {64,128,256}, both classes: quantize, dequantize and 16-query scores
    against the oracle (the oracle's size, 8,192 rows; the full 4,194,304 rows run in the benchmark)."""
    n = 8192
    x = np.random.default_rng(20264 * 100 + d + bits).standard_normal((n, d)).astype(np.float32)
    queries = np.random.default_rng(20274).standard_normal((16, d)).astype(np.float32)
    mse = tg.TurboQuantMSE(d, bits, seed=2026)
    mp = orc.mse_params(d, bits, rotation=mse.rotation, codebook=mse.codebook)
    codes, norms, prefix = orc.mse_quantize(mp, x)
    enc = mse.quantize(x)
    f, o, t = parity.code_flip_report(enc.indices, codes, mse.rotation, mse.boundaries, x)
    parity.assert_discrete_parity(f, o, t, f"MSE codes d={d} bits={bits}")
    assert parity.max_rel_scalar(enc.norms, norms) <= REL_RECON
    ref_enc = tg.TurboQuantMSEEncoding(indices=codes, norms=norms, prefix_shape=prefix)
    assert parity.max_rel_rows(mse.dequantize(ref_enc), orc.mse_dequantize(mp, codes, norms, prefix)) <= REL_RECON

    prod = tg.TurboQuantProd(d, bits, seed=2026)
    pp = _prod_params(prod, d, bits)
    want = orc.prod_quantize(pp, x)
    penc = prod.quantize(x)
    f, o, t = parity.code_flip_report(penc.indices, want[0], prod.mse.rotation, prod.mse.boundaries, x)
    parity.assert_discrete_parity(f, o, t, f"Prod codes d={d} bits={bits}")
    same = ~np.any(penc.indices != want[0], axis=1)
    sdiff = (penc.qjl != want[1]) & same[:, None]
    rows, cols = np.nonzero(sdiff)
    parity.assert_discrete_parity(int(sdiff.sum()), _sign_window_violations(x, want, prod, rows, cols), t,
                                  f"Prod signs d={d} bits={bits}")
    assert parity.max_rel_scalar(penc.norms, want[3]) <= REL_RECON
    assert parity.max_rel_scalar(penc.residual_norms[same], want[2][same]) <= REL_RECON
    ref_penc = tg.TurboQuantProdEncoding(indices=want[0], qjl=want[1], residual_norms=want[2], norms=want[3],
                                         prefix_shape=(n,))
    assert parity.max_rel_rows(prod.dequantize(ref_penc), orc.prod_dequantize(pp, *want)) <= REL_RECON
    ref = np.stack([orc.prod_attention_score(pp, q, *want) for q in queries])
    got = prod.attention_scores(queries, ref_penc)
    assert parity.max_score_err(got, ref, np.linalg.norm(queries, axis=1)[:, None], want[3][None, :], d) <= REL_SCORE
