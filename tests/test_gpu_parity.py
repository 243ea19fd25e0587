"""GPU suite: the CUDA path (through the public Python API, which calls the C ABI) against the
fixtures recorded from the unmodified reference and against the NumPy oracle run on the same host.

Tolerances (see parity.py): codes / sign bits equal except within 1e-5 of a decision point, at a
rate <= 1e-6; norms and reconstructions within 1e-5 relative; scores within 1e-4 relative.
"""
import numpy as np
import pytest

from conftest import CASES, CASE_IDS, golden_case
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


def _quantizers(tg, case, g, path, need=("mse", "prod")):
    """Both quantizers of a fixture case on `path`; the test is skipped when a quantizer it needs (`need`) has no
    tensor-core kernel for the case's geometry (d = 256 has one for TurboQuantMSE only)."""
    d, bits = case["dimension"], case["bits"]
    mse = tg.TurboQuantMSE(d, bits, rotation=g["mse_rotation"], codebook=g["mse_codebook"])
    prod = tg.TurboQuantProd(d, bits, rotation=g["prod_rotation"], projection=g["prod_projection"],
                             **case["kwargs"])
    assert np.array_equal(prod.mse.codebook, g["prod_codebook"])
    for name, q in (("mse", mse), ("prod", prod)):
        if name not in need:
            continue
        if path == "tensor":
            from project_tensor_b200 import _native
            import torch
            if not _native.load().tq_plan_has_tensor_path(q._plans.handle(torch.device("cuda", 0))):
                pytest.skip("no tensor-core kernel for this (d, bits)")
        q.set_kernel_path(path)
    return mse, prod


def _proj_values(g, d):
    """float64 residual . S^T of the reference's own codes, to locate near-zero projections."""
    x = g["x"].reshape(-1, d).astype(np.float64)
    n = np.linalg.norm(x, axis=1)
    unit = np.where(n[:, None] > 0, x / np.where(n > 0, n, 1.0)[:, None], 0.0)
    recon = g["prod_codebook"].astype(np.float64)[g["prod_indices"]] @ g["prod_rotation"].astype(np.float64)
    return (unit - recon) @ g["prod_projection"].astype(np.float64).T


@pytest.mark.parametrize("path", ["exact", "tensor"])
@pytest.mark.parametrize("case", CASES, ids=CASE_IDS)
def test_mse_matches_reference_fixture(tg, case, path):
    g = golden_case(case["name"])
    d = case["dimension"]
    mse, _ = _quantizers(tg, case, g, path, need=("mse",))
    enc = mse.quantize(g["x"])
    assert enc.prefix_shape == tuple(case["lead"])
    assert enc.indices.shape == g["mse_indices"].shape and enc.indices.dtype == np.uint8
    flips, outside, total = parity.code_flip_report(enc.indices, g["mse_indices"], g["mse_rotation"],
                                                    g["mse_boundaries"], g["x"])
    parity.assert_discrete_parity(flips, outside, total, "MSE codes")
    assert parity.max_rel_scalar(enc.norms, g["mse_norms"]) <= REL_RECON
    # dequantize the REFERENCE's encoding, so that a tolerated code flip cannot hide an error here
    ref_enc = tg.TurboQuantMSEEncoding(indices=g["mse_indices"], norms=g["mse_norms"],
                                       prefix_shape=tuple(case["lead"]))
    recon = mse.dequantize(ref_enc)
    assert recon.shape == g["mse_recon"].shape and recon.dtype == np.float32
    assert parity.max_rel_rows(recon, g["mse_recon"]) <= REL_RECON
    # and our own encoding round-trips to the same thing when no code differs
    if flips == 0:
        assert parity.max_rel_rows(mse.dequantize(enc), g["mse_recon"]) <= REL_RECON


@pytest.mark.parametrize("path", ["exact", "tensor"])
@pytest.mark.parametrize("case", CASES, ids=CASE_IDS)
def test_prod_matches_reference_fixture(tg, case, path):
    g = golden_case(case["name"])
    d = case["dimension"]
    _, prod = _quantizers(tg, case, g, path, need=("prod",))
    enc = prod.quantize(g["x"])
    flips, outside, total = parity.code_flip_report(enc.indices, g["prod_indices"], g["prod_rotation"],
                                                    g["prod_boundaries"], g["x"])
    parity.assert_discrete_parity(flips, outside, total, "Prod codes")
    assert enc.qjl.dtype == np.int8 and set(np.unique(enc.qjl)) <= {-1, 1}
    rows_same = ~np.any(enc.indices != g["prod_indices"], axis=1)
    sflips, soutside, stotal = parity.sign_flip_report(enc.qjl[rows_same], g["prod_qjl"][rows_same],
                                                       _proj_values(g, d)[rows_same])
    parity.assert_discrete_parity(sflips, soutside, stotal, "QJL signs")
    assert parity.max_rel_scalar(enc.norms, g["prod_norms"]) <= REL_RECON
    assert parity.max_rel_scalar(enc.residual_norms[rows_same], g["prod_residual_norms"][rows_same]) <= REL_RECON

    ref_enc = tg.TurboQuantProdEncoding(indices=g["prod_indices"], qjl=g["prod_qjl"],
                                        residual_norms=g["prod_residual_norms"], norms=g["prod_norms"],
                                        prefix_shape=tuple(case["lead"]))
    recon = prod.dequantize(ref_enc)
    assert recon.shape == g["prod_recon"].shape
    assert parity.max_rel_rows(recon, g["prod_recon"]) <= REL_RECON

    knorm = g["prod_norms"].reshape(case["lead"])
    for q, want in zip(g["queries"], g["scores_broadcast"]):
        got = prod.attention_score(q, ref_enc)
        assert got.shape == want.shape
        assert parity.max_score_err(got, want, np.linalg.norm(q), knorm, d) <= REL_SCORE
    got = prod.attention_score(g["pair_queries"], ref_enc)
    assert got.shape == g["scores_pairwise"].shape
    qn = np.linalg.norm(g["pair_queries"], axis=-1)
    assert parity.max_score_err(got, g["scores_pairwise"], qn, knorm, d) <= REL_SCORE

    # batched entry point == the reference's loop over queries
    mat = prod.attention_scores(g["queries"], ref_enc)
    want = g["scores_broadcast"].reshape(len(g["queries"]), -1)
    assert mat.shape == want.shape
    assert parity.max_score_err(mat, want, np.linalg.norm(g["queries"], axis=1)[:, None],
                                g["prod_norms"][None, :], d) <= REL_SCORE
    k = min(5, want.shape[1])
    top_s, top_i = prod.attention_scores(g["queries"], ref_enc, topk=k)
    for r in range(want.shape[0]):
        order = np.lexsort((np.arange(want.shape[1]), -mat[r]))[:k]
        assert np.array_equal(top_i[r], order)
        assert np.array_equal(top_s[r], mat[r][order])


@pytest.mark.parametrize("n", [0, 1, 2, 31, 32, 33, 127, 128, 129, 1000])
@pytest.mark.parametrize("path", ["exact", "auto"])
def test_ragged_sizes_against_live_oracle(tg, n, path):
    d, bits = 128, 4
    x = np.random.default_rng(100 + n).standard_normal((n, d)).astype(np.float32)
    prod = tg.TurboQuantProd(d, bits, seed=2026)
    prod.set_kernel_path(path)
    pp = orc.ProdParams(d, bits, orc.mse_params(d, bits - 1, rotation=prod.mse.rotation,
                                                codebook=prod.mse.codebook), prod.projection)
    enc = prod.quantize(x)
    want = orc.prod_quantize(pp, x)
    assert enc.indices.shape == (n, d) and enc.qjl.shape == (n, d)
    assert enc.norms.shape == (n,) and enc.residual_norms.shape == (n,)
    f, o, t = parity.code_flip_report(enc.indices, want[0], prod.mse.rotation, prod.mse.boundaries, x)
    assert o == 0 and f <= 1
    if f == 0:
        assert int((enc.qjl != want[1]).sum()) <= 1
        if n:
            assert parity.max_rel_scalar(enc.residual_norms, want[2]) <= REL_RECON
    if n:
        assert parity.max_rel_scalar(enc.norms, want[3]) <= REL_RECON
        assert parity.max_rel_rows(prod.dequantize(enc), orc.prod_dequantize(pp, np.asarray(enc.indices), np.asarray(enc.qjl), np.asarray(enc.residual_norms), np.asarray(enc.norms), (n,))) <= REL_RECON
    assert prod.dequantize(enc).shape == (n, d)


def test_special_rows(tg):
    """Zero rows, a NaN row and an Inf row follow the reference's where() rules (_quant.py:227-229)."""
    d, bits = 64, 3
    x = np.random.default_rng(5).standard_normal((8, d)).astype(np.float32)
    x[1] = 0.0
    x[2, 7] = np.nan
    x[3] *= 1e-20
    x[4] *= 1e18
    mse = tg.TurboQuantMSE(d, bits, seed=11)
    mp = orc.mse_params(d, bits, rotation=mse.rotation, codebook=mse.codebook)
    with np.errstate(all="ignore"):
        codes, norms, _ = orc.mse_quantize(mp, x)
    for path in ("exact", "auto"):
        mse.set_kernel_path(path)
        enc = mse.quantize(x)
        assert np.array_equal(enc.indices, codes)
        got = np.asarray(enc.norms)
        if path == "exact":
            assert np.array_equal(got, norms, equal_nan=True)
        else:   # the tensor-core path sums the squares in another order: within 1e-5, special values alike
            assert np.array_equal(np.isnan(got), np.isnan(norms)) and np.array_equal(np.isinf(got), np.isinf(norms))
            fin = np.isfinite(norms)
            assert np.array_equal(got[fin] == 0, norms[fin] == 0)
            assert parity.max_rel_scalar(got[fin], norms[fin]) <= REL_RECON
        assert np.all(enc.indices[1] == np.searchsorted(mse.boundaries, 0.0, side="left"))


def test_input_kinds_and_shapes(tg):
    import torch
    d = 32
    x = np.random.default_rng(9).standard_normal((2, 3, 5, d)).astype(np.float32)
    prod = tg.TurboQuantProd(d, 3, seed=4)
    enc_np = prod.quantize(x)
    assert enc_np.indices.shape == (30, d) and enc_np.prefix_shape == (2, 3, 5)
    assert isinstance(enc_np.norms, np.ndarray)
    assert prod.dequantize(enc_np).shape == x.shape
    q = np.random.default_rng(10).standard_normal(d).astype(np.float32)
    s_np = prod.attention_score(q, enc_np)
    assert s_np.shape == (2, 3, 5)

    xt = torch.from_numpy(x).cuda()
    enc_t = prod.quantize(xt)                      # __cuda_array_interface__ / torch CUDA input
    assert isinstance(enc_t.indices, torch.Tensor) and enc_t.indices.is_cuda
    assert np.array_equal(enc_t.indices.cpu().numpy(), enc_np.indices)
    assert np.array_equal(enc_t.qjl.cpu().numpy(), enc_np.qjl)
    s_t = prod.attention_score(torch.from_numpy(q).cuda(), enc_t)
    assert s_t.is_cuda and np.array_equal(s_t.cpu().numpy(), s_np)

    class Cai:                                     # any __cuda_array_interface__ producer
        def __init__(self, t):
            self._t = t
            self.__cuda_array_interface__ = t.__cuda_array_interface__
            self.shape, self.ndim = tuple(t.shape), t.ndim
    enc_c = prod.quantize(Cai(xt))
    assert np.array_equal(enc_c.indices.cpu().numpy(), enc_np.indices)

    wrapped = tg.Tensor(x, requires_grad=False)    # Tensor-like wrapper
    assert np.array_equal(prod.quantize(wrapped).indices, enc_np.indices)
    enc64 = prod.quantize(x.astype(np.float64))    # other float dtypes are cast to float32
    assert np.array_equal(enc64.indices, enc_np.indices)

    with pytest.raises(ValueError, match="query batch size 7 does not match encoding batch size 30"):
        prod.attention_score(np.zeros((7, d), np.float32), enc_np)
    quant, enc = tg.turboquant_prod(x, 3, seed=4)
    assert np.array_equal(enc.indices, enc_np.indices)
    quant, enc = tg.turboquant_mse(x, 2, seed=4)
    assert enc.indices.shape == (30, d)


@pytest.mark.parametrize("d,bits", [(64, 1), (64, 4), (128, 2), (256, 3), (256, 1), (96, 5), (40, 8)])
def test_sweep_against_live_oracle(tg, d, bits):
    n = 4096
    x = np.random.default_rng(d * 10 + bits).standard_normal((n, d)).astype(np.float32)
    mse = tg.TurboQuantMSE(d, bits, seed=2026)
    prod = tg.TurboQuantProd(d, bits, seed=2026)
    mp = orc.mse_params(d, bits, rotation=mse.rotation, codebook=mse.codebook)
    pp = orc.ProdParams(d, bits, orc.mse_params(d, max(bits - 1, 1), rotation=prod.mse.rotation,
                                                codebook=prod.mse.codebook), prod.projection)
    codes, norms, _ = orc.mse_quantize(mp, x)
    enc = mse.quantize(x)
    f, o, t = parity.code_flip_report(enc.indices, codes, mse.rotation, mse.boundaries, x)
    parity.assert_discrete_parity(f, o, t, f"MSE codes d={d} bits={bits}")
    assert parity.max_rel_scalar(enc.norms, norms) <= REL_RECON
    want = orc.prod_quantize(pp, x)
    penc = prod.quantize(x)
    f, o, t = parity.code_flip_report(penc.indices, want[0], prod.mse.rotation, prod.mse.boundaries, x)
    parity.assert_discrete_parity(f, o, t, f"Prod codes d={d} bits={bits}")
    same = ~np.any(penc.indices != want[0], axis=1)
    assert int((penc.qjl[same] != want[1][same]).sum()) <= max(1, int(1e-6 * same.sum() * d))
    queries = np.random.default_rng(3).standard_normal((16, d)).astype(np.float32)
    ref = np.stack([orc.prod_attention_score(pp, q, *want) for q in queries])
    ref_enc = tg.TurboQuantProdEncoding(indices=want[0], qjl=want[1], residual_norms=want[2],
                                        norms=want[3], prefix_shape=(n,))
    got = prod.attention_scores(queries, ref_enc)
    assert parity.max_score_err(got, ref, np.linalg.norm(queries, axis=1)[:, None], want[3][None, :], d) <= REL_SCORE


def test_config1_full_size_codes_norms_mse(tg):
    """TurboQuantMSE d=128 bits=4 seed=2026 over N=65,536 N(0,1) vectors: codes, norms and
    reconstruction MSE against the oracle run on this host."""
    d, bits, n = 128, 4, 65536
    x = np.random.default_rng(20261).standard_normal((n, d)).astype(np.float32)
    mse = tg.TurboQuantMSE(d, bits, seed=2026)
    mp = orc.mse_params(d, bits, rotation=mse.rotation, codebook=mse.codebook)
    codes, norms, prefix = orc.mse_quantize(mp, x)
    enc = mse.quantize(x)
    f, o, t = parity.code_flip_report(enc.indices, codes, mse.rotation, mse.boundaries, x)
    print(f"config 1: {f} code differences in {t} ({f / t:.2e}), {o} outside the window")
    parity.assert_discrete_parity(f, o, t, "config 1 codes")
    assert parity.max_rel_scalar(enc.norms, norms) <= REL_RECON
    recon = mse.dequantize(enc)
    ref = orc.mse_dequantize(mp, codes, norms, prefix)
    ours_mse, ref_mse = float(np.mean((x - recon) ** 2)), float(np.mean((x - ref) ** 2))
    assert abs(ours_mse - ref_mse) <= 1e-5 * ref_mse
    if f == 0:
        assert parity.max_rel_rows(recon, ref) <= REL_RECON


def test_round_trip_properties_at_scale(tg):
    """Size-independent properties on device-resident data (1,048,576 keys): score == q . dequantize,
    reconstruction error bounded, idempotence of re-quantising a reconstruction's codes."""
    import torch
    d, bits, n = 128, 4, 1 << 20
    gen = torch.Generator(device="cuda").manual_seed(20262)
    x = torch.randn((n, d), generator=gen, device="cuda", dtype=torch.float32)
    prod = tg.TurboQuantProd(d, bits, seed=2026)
    enc = prod.quantize(x)
    recon = prod.dequantize(enc)
    q = torch.randn((d,), generator=gen, device="cuda", dtype=torch.float32)
    s = prod.attention_score(q, enc)
    explicit = recon @ q
    scale = torch.linalg.norm(q) * enc.norms / d ** 0.5
    assert float(torch.max(torch.abs(s - explicit) / scale)) <= REL_SCORE
    cos = torch.nn.functional.cosine_similarity(recon, x, dim=1)
    assert float(cos.mean()) > 0.95
    mse = tg.TurboQuantMSE(d, bits, seed=2026)
    e1 = mse.quantize(x)
    e2 = mse.quantize(mse.dequantize(e1))
    same = (e1.indices == e2.indices).float().mean()
    assert float(same) > 0.999          # centroids sit mid-cell: re-quantising keeps the code
    # checksum of checksums: packed buffers are a pure function of the input
    from project_tensor_b200 import packed_buffers
    again = packed_buffers(prod.quantize(x))
    first = packed_buffers(enc)
    assert torch.equal(first["codes"], again["codes"]) and torch.equal(first["signs"], again["signs"])


@pytest.mark.parametrize("cls_name,bits", [("TurboQuantMSE", 4), ("TurboQuantMSE", 3), ("TurboQuantMSE", 1),
                                           ("TurboQuantProd", 4), ("TurboQuantProd", 2)])
@pytest.mark.parametrize("n", [1, 127, 129, 40000])
def test_tensor_dequantize_matches_exact_dequantize(tg, cls_name, bits, n):
    """The tensor-core dequantize kernel against the exact kernel (which reproduces the reference's float32
    arithmetic bit for bit) on ragged sizes, with a zero row and rows of very different norms."""
    import torch
    d = 128
    gen = torch.Generator(device="cuda").manual_seed(20290 + n)
    x = torch.randn((n, d), generator=gen, device="cuda", dtype=torch.float32)
    x *= torch.logspace(-6, 6, n, device="cuda")[:, None]
    if n > 3:
        x[3] = 0
    quant = getattr(tg, cls_name)(d, bits, seed=2026)
    enc = quant.quantize(x)
    quant.set_kernel_path("exact")
    ref = quant.dequantize(enc).cpu().numpy()
    quant.set_kernel_path("tensor")
    got = quant.dequantize(enc).cpu().numpy()
    assert got.shape == ref.shape == (n, d)
    assert parity.max_rel_rows(got, ref) <= REL_RECON
    if n > 3:
        assert not got[3].any()


@pytest.mark.parametrize("cls_name", ["TurboQuantMSE", "TurboQuantProd"])
def test_quantize_to_host_equals_quantize(tg, cls_name):
    """The chunked host-to-host path gives the same packed bytes as one device call, for a size that is not
    a multiple of the chunk, with pageable and with page-locked input, and when its output is reused."""
    import torch
    from project_tensor_b200 import packed_buffers, quantize_to_host
    d, n = 128, 70001
    x = np.random.default_rng(20291).standard_normal((n, d)).astype(np.float32)
    quant = getattr(tg, cls_name)(d, 4, seed=2026)
    ref = packed_buffers(quant.quantize(torch.from_numpy(x).cuda()))
    pinned = torch.from_numpy(x).pin_memory().numpy()
    out = None
    for keys in (x, pinned, pinned):
        out = quantize_to_host(quant, keys, chunk_rows=16384, out=out)
        for name, dev_t in ref.items():
            if dev_t is None:
                assert out[name] is None
            else:
                assert torch.equal(out[name], dev_t.cpu()), name


@pytest.mark.parametrize("bits", [4, 3, 1])
@pytest.mark.parametrize("n", [1, 129, 38405])
def test_d64_tensor_paths_match_exact_paths(tg, bits, n):
    """d = 64 runs on the tensor-core kernels in the layouts of d = 128 with the upper half absent.  Packed
    codes and sign bits must equal the exact kernels', norms, reconstructions and scores agree within the
    bounds, for odd and ragged sizes too (rows of 8 and 24 bytes end a tile off a 16-byte boundary)."""
    import torch
    from project_tensor_b200 import packed_buffers
    d = 64
    gen = torch.Generator(device="cuda").manual_seed(20292 + n + bits)
    x = torch.randn((n, d), generator=gen, device="cuda", dtype=torch.float32)
    x *= torch.logspace(-3, 3, n, device="cuda")[:, None]
    q = torch.randn((5, d), generator=gen, device="cuda", dtype=torch.float32)
    for cls_name in ("TurboQuantMSE", "TurboQuantProd"):
        quant = getattr(tg, cls_name)(d, bits, seed=2026)
        quant.set_kernel_path("exact")
        ref = quant.quantize(x)
        ref_bufs = packed_buffers(ref)
        ref_recon = quant.dequantize(ref).cpu().numpy()
        quant.set_kernel_path("tensor")
        got_bufs = packed_buffers(quant.quantize(x))
        assert torch.equal(got_bufs["codes"], ref_bufs["codes"])
        assert parity.max_rel_scalar(got_bufs["norms"].cpu().numpy(), ref_bufs["norms"].cpu().numpy()) <= REL_RECON
        assert parity.max_rel_rows(quant.dequantize(ref).cpu().numpy(), ref_recon) <= REL_RECON
        if cls_name == "TurboQuantProd":
            assert torch.equal(got_bufs["signs"], ref_bufs["signs"])
            assert parity.max_rel_scalar(got_bufs["residual_norms"].cpu().numpy(),
                                         ref_bufs["residual_norms"].cpu().numpy()) <= REL_RECON
            got_s = quant.attention_scores(q, ref).cpu().numpy()
            quant.set_kernel_path("exact")
            ref_s = quant.attention_scores(q, ref).cpu().numpy()
            scale = np.linalg.norm(q.cpu().numpy(), axis=1)[:, None]
            assert parity.max_score_err(got_s, ref_s, scale, ref_bufs["norms"].cpu().numpy()[None, :], d) <= REL_SCORE


def test_a_wait_that_runs_out_is_reported_not_hidden(tg):
    """Every wait inside the tensor-core kernels is bounded.  With the limit set to 0 the first wait that finds its
    barrier unfinished counts as run out (at the start of a kernel every consumer is in that position): the kernel must
    come back (all roles leave their loops, copies and tensor instructions in flight are waited for), the plan's status
    word must say so, the Python layer must raise at its next synchronisation point instead of handing the encoding
    out, and the next call with the normal limit must be correct again on the same context."""
    import torch
    from project_tensor_b200 import _native
    x = torch.randn((65536, 128), device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
    quant = tg.TurboQuantProd(128, 4, seed=2026)
    good = quant.quantize(x)
    torch.cuda.synchronize()
    quant._plans.check_status(x.device)                 # nothing to report so far
    quant._plans.set_wait_limit(0)
    enc = quant.quantize(x)
    with pytest.raises(_native.TurboQuantNativeError, match="gave up on a bounded wait"):
        quant._plans.check_status(x.device)
    quant._plans.check_status(x.device)                 # reported once, then clear
    quant._plans.set_wait_limit(4_000_000_000)
    again = quant.quantize(x)
    from project_tensor_b200 import packed_buffers
    a, b = packed_buffers(again), packed_buffers(good)
    assert torch.equal(a["codes"], b["codes"]) and torch.equal(a["signs"], b["signs"])
    quant._plans.check_status(x.device)
    del enc
