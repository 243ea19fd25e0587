"""GPU suite for batched scoring: query groups (one block of queries per block of keys, as the heads of a KV
cache), per-query top-k, index offsets, key sets that span several scratch chunks.  The oracle scores one
query at a time, exactly as the reference's callers do (validate_turboquant.py:92-95)."""
import numpy as np
import pytest

from oracle import turboquant_oracle as orc
import parity

pytestmark = pytest.mark.gpu

REL_SCORE = 1e-4


@pytest.fixture(scope="module")
def tg(lib_built):
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import project_tensor_b200 as tg
    return tg


def _oracle_params(prod):
    d, bits = prod.dimension, prod.bits
    return orc.ProdParams(d, bits, orc.mse_params(d, max(bits - 1, 1), rotation=prod.mse.rotation,
                                                  codebook=prod.mse.codebook), prod.projection)


@pytest.mark.parametrize("path", ["exact", "tensor"])
def test_grouped_queries_with_outlier_channels_against_oracle(tg, path):
    """Six key groups (KV heads) of 4096 keys with four channels per head scaled by 10, four queries per
    group, TurboQuantProd(128, 3): every query meets the keys of its own group only."""
    d, bits, groups, kpg, qpg = 128, 3, 6, 4096, 4
    rng = np.random.default_rng(20263)
    keys = rng.standard_normal((groups, kpg, d)).astype(np.float32)
    for h in range(groups):
        keys[h][:, np.random.default_rng(20280 + h).choice(d, 4, replace=False)] *= 10.0
    queries = np.random.default_rng(20273).standard_normal((groups, qpg, d)).astype(np.float32)
    prod = tg.TurboQuantProd(d, bits, seed=2026)
    prod.set_kernel_path(path)
    pp = _oracle_params(prod)
    flat = keys.reshape(-1, d)
    want = orc.prod_quantize(pp, flat)
    ref_enc = tg.TurboQuantProdEncoding(indices=want[0], qjl=want[1], residual_norms=want[2], norms=want[3],
                                        prefix_shape=(groups * kpg,))
    got = prod.attention_scores(queries.reshape(-1, d), ref_enc, groups=groups)
    assert got.shape == (groups * qpg, kpg)
    for g in range(groups):
        sl = slice(g * kpg, (g + 1) * kpg)
        part = (want[0][sl], want[1][sl], want[2][sl], want[3][sl], (kpg,))
        ref = np.stack([orc.prod_attention_score(pp, q, *part) for q in queries[g]])
        err = parity.max_score_err(got[g * qpg:(g + 1) * qpg], ref, np.linalg.norm(queries[g], axis=1)[:, None],
                                   want[3][sl][None, :], d)
        assert err <= REL_SCORE, (g, err)
    # top-k of the same call: global key indices, descending scores, equal to the matrix they come from
    k = 10
    top_s, top_i, mat = prod.attention_scores(queries.reshape(-1, d), ref_enc, groups=groups, topk=k, return_matrix=True,
                                              index_base=1000)
    assert np.array_equal(mat, got)
    for r in range(groups * qpg):
        g = r // qpg
        order = np.argsort(-got[r], kind="stable")[:k]
        assert np.array_equal(top_s[r], got[r][order])
        assert np.array_equal(top_i[r], order + g * kpg + 1000)


@pytest.mark.parametrize("path", ["exact", "tensor"])
@pytest.mark.parametrize("n,nq,k", [(1000, 4, 10), (70000, 40, 100), (38405, 32, 300), (257, 3, 500)])
def test_topk_equals_sorted_matrix(tg, path, n, nq, k):
    """Per-query top-k, with and without the matrix, against a stable sort of the matrix of the same kernels:
    ragged key counts, more than 32 queries (two passes), k above 128 and k above the number of keys."""
    import torch
    d = 128
    gen = torch.Generator(device="cuda").manual_seed(20264 + n)
    x = torch.randn((n, d), generator=gen, device="cuda", dtype=torch.float32)
    q = torch.randn((nq, d), generator=gen, device="cuda", dtype=torch.float32)
    prod = tg.TurboQuantProd(d, 4, seed=2026)
    prod.set_kernel_path(path)
    enc = prod.quantize(x)
    mat = prod.attention_scores(q, enc)
    top_s, top_i = prod.attention_scores(q, enc, topk=k)
    top_s2, top_i2, mat2 = prod.attention_scores(q, enc, topk=k, return_matrix=True)
    assert torch.equal(mat, mat2) and torch.equal(top_s, top_s2) and torch.equal(top_i, top_i2)
    kk = min(k, n)
    srt = torch.sort(mat, dim=1, descending=True, stable=True)
    assert torch.equal(top_s[:, :kk], srt.values[:, :kk])
    assert torch.equal(top_i[:, :kk], srt.indices[:, :kk])
    if k > n:   # the slots beyond the last key are marked empty
        assert bool((top_i[:, n:] == -1).all()) and bool(torch.isinf(top_s[:, n:]).all())


def test_topk_over_several_scratch_chunks(tg):
    """9,000,000 keys: without a matrix from the caller the keys are scored in chunks of 2^21 (four full ones and a
    ragged fifth) with only the scores above each query's running threshold kept; the result must be the same
    top-100 as a sort of the full matrix."""
    import torch
    d, n, nq, k = 128, 9_000_000, 8, 100
    gen = torch.Generator(device="cuda").manual_seed(20265)
    x = torch.randn((n, d), generator=gen, device="cuda", dtype=torch.float32)
    q = torch.randn((nq, d), generator=gen, device="cuda", dtype=torch.float32)
    prod = tg.TurboQuantProd(d, 4, seed=2026)
    enc = prod.quantize(x)
    del x
    mat = prod.attention_scores(q, enc)
    top_s, top_i = prod.attention_scores(q, enc, topk=k, index_base=7)
    srt = torch.sort(mat, dim=1, descending=True, stable=True)
    assert torch.equal(top_s, srt.values[:, :k])
    assert torch.equal(top_i, srt.indices[:, :k] + 7)


def _sorted_topk(mat, k):
    import torch
    srt = torch.sort(mat, dim=1, descending=True, stable=True)
    return srt.values[:, :k], srt.indices[:, :k]


def test_topk_without_matrix_when_every_key_beats_the_threshold(tg):
    """Above 4,194,304 keys per group the top-k comes from candidate lists filled by the scoring kernel (scores that
    reach the query's running threshold) instead of a scratch matrix.  Worst cases for that scheme, 4,500,003 keys:
    query 0 meets keys whose scores rise with the index (every key passes the threshold of its moment, so the lists
    fill to their capacity), query 1 the same keys falling (nothing passes after the sampled pass), long runs of
    identical keys tie exactly (ties go to the lower index), and 38 random queries make a second pass of queries.
    The result must equal a stable sort of the full matrix, for k = 100 and k = 300."""
    import torch
    d, n, nq = 128, 4_500_003, 40
    gen = torch.Generator(device="cuda").manual_seed(20266)
    u = torch.randn((d,), generator=gen, device="cuda", dtype=torch.float32)
    scale = 0.5 + (torch.arange(n, device="cuda", dtype=torch.float32) // 1000) * (1000.0 / n)   # runs of 1000 equal keys
    x = scale[:, None] * u[None, :]
    x[n // 2:n // 2 + 200_000] = torch.randn((200_000, d), generator=gen, device="cuda")
    q = torch.randn((nq, d), generator=gen, device="cuda", dtype=torch.float32)
    q[0] = u
    q[1] = -u
    prod = tg.TurboQuantProd(d, 4, seed=2026)
    enc = prod.quantize(x)
    del x, scale
    mat = prod.attention_scores(q, enc)
    for k in (100, 300):
        top_s, top_i = prod.attention_scores(q, enc, topk=k)
        want_s, want_i = _sorted_topk(mat, k)
        assert torch.equal(top_s, want_s), k
        assert torch.equal(top_i, want_i), k


def test_topk_without_matrix_is_the_same_call_after_call(tg):
    """Candidate mode lets the epilogue warps of the scoring kernel run free of each other, and a query that every key
    passes (query 0 below) keeps its warps microseconds behind the rest.  Values read from a ring stage must then have
    been read when the warp releases the stage: with plain loads the compiler had moved the read of a key's norm behind
    the release, and about one call in three returned a score computed with the norm of a key eight tiles on.  Thirty
    calls on the data of the worst-case test, 40 queries (one pass of 64), each equal to a stable sort of the
    matrix."""
    import torch
    d, n, nq, k = 128, 4_500_003, 40, 300
    gen = torch.Generator(device="cuda").manual_seed(20266)
    u = torch.randn((d,), generator=gen, device="cuda", dtype=torch.float32)
    scale = 0.5 + (torch.arange(n, device="cuda", dtype=torch.float32) // 1000) * (1000.0 / n)
    x = scale[:, None] * u[None, :]
    x[n // 2:n // 2 + 200_000] = torch.randn((200_000, d), generator=gen, device="cuda")
    q = torch.randn((nq, d), generator=gen, device="cuda", dtype=torch.float32)
    q[0] = u
    q[1] = -u
    prod = tg.TurboQuantProd(d, 4, seed=2026)
    enc = prod.quantize(x)
    del x, scale
    want_s, want_i = _sorted_topk(prod.attention_scores(q, enc), k)
    for rep in range(30):
        top_s, top_i = prod.attention_scores(q, enc, topk=k)
        assert torch.equal(top_s, want_s), rep
        assert torch.equal(top_i, want_i), rep


@pytest.mark.parametrize("kpg", [4_300_000, 4_200_003])
def test_topk_without_matrix_for_query_groups(tg, kpg):
    """Two key groups of 4,300,000 keys (ragged last tile and last chunk), three queries per group, k = 64: the
    candidate lists are per query of every group and the indices count from the start of the group's keys.  With
    4,200,003 keys per group the second group's tiles start off a 16-byte boundary in the norm arrays, so the norms
    come by plain loads instead of riding with the packed rows."""
    import torch
    d, groups, qpg, k = 64, 2, 3, 64
    gen = torch.Generator(device="cuda").manual_seed(20267)
    x = torch.randn((groups * kpg, d), generator=gen, device="cuda", dtype=torch.float32)
    q = torch.randn((groups * qpg, d), generator=gen, device="cuda", dtype=torch.float32)
    prod = tg.TurboQuantProd(d, 3, seed=2026)
    enc = prod.quantize(x)
    del x
    mat = prod.attention_scores(q, enc, groups=groups)
    assert mat.shape == (groups * qpg, kpg)
    top_s, top_i = prod.attention_scores(q, enc, groups=groups, topk=k, index_base=5)
    want_s, want_i = _sorted_topk(mat, k)
    assert torch.equal(top_s, want_s)
    for r in range(groups * qpg):
        assert torch.equal(top_i[r], want_i[r] + (r // qpg) * kpg + 5)


@pytest.mark.parametrize("d,bits", [(128, 4), (128, 1), (64, 3)])
@pytest.mark.parametrize("groups,qpg", [(1, 64), (1, 33), (3, 40), (1, 100)])
def test_passes_of_up_to_64_queries(tg, d, bits, groups, qpg):
    """From 33 queries per group on a scoring launch takes up to 64 queries (one operand buffer in tensor memory, 256
    accumulator columns, two blocks of 16 queries per epilogue thread, one group's prepared queries resident):
    33, 40 (three groups, so the prepared queries change inside a block's tile range), 64 and 100 (64 + 36) queries
    against 5,003 keys per group.  The matrix within the fp32 tolerance of the kernels that accumulate in the
    reference's order; the top-k equal to a stable sort of the matrix."""
    import torch
    kpg, k = 5003, 50
    gen = torch.Generator(device="cuda").manual_seed(20293 + qpg)
    x = torch.randn((groups * kpg, d), generator=gen, device="cuda", dtype=torch.float32)
    q = torch.randn((groups * qpg, d), generator=gen, device="cuda", dtype=torch.float32)
    prod = tg.TurboQuantProd(d, bits, seed=2026)
    enc = prod.quantize(x)
    mat = prod.attention_scores(q, enc, groups=groups)
    prod.set_kernel_path("exact")
    ref = prod.attention_scores(q, enc, groups=groups)
    prod.set_kernel_path("auto")
    norms = tg.packed_buffers(enc)["norms"].view(groups, 1, kpg)
    scale = (q.norm(dim=1).view(groups, qpg, 1) * norms / d ** 0.5).reshape(groups * qpg, kpg)
    assert float(((mat - ref).abs() / scale).max()) <= REL_SCORE
    top_s, top_i = prod.attention_scores(q, enc, groups=groups, topk=k)
    want_s, want_i = _sorted_topk(mat, k)
    assert torch.equal(top_s, want_s)
    for r in range(groups * qpg):
        assert torch.equal(top_i[r], want_i[r] + (r // qpg) * kpg)


@pytest.mark.parametrize("bits,kpg", [(2, 1000), (3, 1001), (4, 1000)])
def test_d256_query_groups_on_the_tensor_core_kernel_against_oracle(tg, bits, kpg):
    """d = 256 passes every tile of keys through the operand buffers in two halves of 128 coordinates, and only one
    group's prepared queries are resident at a time.  Three groups of 1,000 keys (ragged last tile, a change of group
    inside a block's tile range), five queries per group, against the oracle's one-query-at-a-time scores; then the
    top-k of the same call against the matrix.  With 1,001 keys per group the groups start off a 16-byte boundary in
    the norm arrays (norms by plain loads) and the matrix rows off one too (plain stores instead of tile stores)."""
    d, groups, qpg = 256, 3, 5
    rng = np.random.default_rng(20290 + bits)
    keys = (rng.standard_normal((groups, kpg, d)) * rng.uniform(0.1, 5.0, (groups, kpg, 1))).astype(np.float32)
    queries = rng.standard_normal((groups, qpg, d)).astype(np.float32)
    prod = tg.TurboQuantProd(d, bits, seed=2026)
    prod.set_kernel_path("tensor")
    pp = _oracle_params(prod)
    want = orc.prod_quantize(pp, keys.reshape(-1, d))
    ref_enc = tg.TurboQuantProdEncoding(indices=want[0], qjl=want[1], residual_norms=want[2], norms=want[3],
                                        prefix_shape=(groups * kpg,))
    got = prod.attention_scores(queries.reshape(-1, d), ref_enc, groups=groups)
    assert got.shape == (groups * qpg, kpg)
    for g in range(groups):
        sl = slice(g * kpg, (g + 1) * kpg)
        part = (want[0][sl], want[1][sl], want[2][sl], want[3][sl], (kpg,))
        ref = np.stack([orc.prod_attention_score(pp, q, *part) for q in queries[g]])
        err = parity.max_score_err(got[g * qpg:(g + 1) * qpg], ref, np.linalg.norm(queries[g], axis=1)[:, None],
                                   want[3][sl][None, :], d)
        assert err <= REL_SCORE, (g, err)
    k = 7
    top_s, top_i = prod.attention_scores(queries.reshape(-1, d), ref_enc, groups=groups, topk=k, index_base=3)
    for r in range(groups * qpg):
        order = np.argsort(-got[r], kind="stable")[:k]
        assert np.array_equal(top_s[r], got[r][order])
        assert np.array_equal(top_i[r], order + (r // qpg) * kpg + 3)


@pytest.mark.parametrize("bits,n,nq,k", [(4, 70000, 40, 100), (2, 38405, 32, 300), (1, 257, 3, 500), (3, 20000, 16, 64)])
def test_d256_topk_equals_sorted_matrix_and_matches_the_exact_kernels(tg, bits, n, nq, k):
    """d = 256 through the default dispatch (tensor-core kernel from two queries on): the score matrix within the
    fp32 tolerance of the kernels that accumulate in the reference's order, the top-k equal to a stable sort of the
    matrix (ragged key counts, two passes of queries, k above 128 and above the number of keys)."""
    import torch
    d = 256
    gen = torch.Generator(device="cuda").manual_seed(20291 + n)
    x = torch.randn((n, d), generator=gen, device="cuda", dtype=torch.float32)
    q = torch.randn((nq, d), generator=gen, device="cuda", dtype=torch.float32)
    prod = tg.TurboQuantProd(d, bits, seed=2026)
    enc = prod.quantize(x)
    mat = prod.attention_scores(q, enc)
    prod.set_kernel_path("exact")
    ref = prod.attention_scores(q, enc)
    prod.set_kernel_path("auto")
    norms = tg.packed_buffers(enc)["norms"]
    scale = q.norm(dim=1)[:, None] * norms[None, :] / d ** 0.5
    assert float(((mat - ref).abs() / scale).max()) <= REL_SCORE
    top_s, top_i = prod.attention_scores(q, enc, topk=k)
    kk = min(k, n)
    want_s, want_i = _sorted_topk(mat, kk)
    assert torch.equal(top_s[:, :kk], want_s)
    assert torch.equal(top_i[:, :kk], want_i)
    if k > n:
        assert bool((top_i[:, n:] == -1).all()) and bool(torch.isinf(top_s[:, n:]).all())


def test_d256_topk_without_matrix_over_several_chunks(tg):
    """4,200,003 keys of d = 256 in one group: top-64 from the candidate lists (three chunks, the last ragged) equals
    a stable sort of the full matrix."""
    import torch
    d, n, nq, k = 256, 4_200_003, 5, 64
    gen = torch.Generator(device="cuda").manual_seed(20292)
    prod = tg.TurboQuantProd(d, 2, seed=2026)
    x = torch.randn((n, d), generator=gen, device="cuda", dtype=torch.float32)
    q = torch.randn((nq, d), generator=gen, device="cuda", dtype=torch.float32)
    enc = prod.quantize(x)
    del x
    mat = prod.attention_scores(q, enc)
    top_s, top_i = prod.attention_scores(q, enc, topk=k, index_base=11)
    want_s, want_i = _sorted_topk(mat, k)
    assert torch.equal(top_s, want_s)
    assert torch.equal(top_i, want_i + 11)


def test_sharded_index_matches_single_index(tg):
    """ShardedKeyIndex filled chunk by chunk (device and host chunks) and searched, and two shards of the same
    keys searched one after the other and merged with tq_topk_merge as the ranks of a job would after the
    all-gather: both give the top-k of one index over all keys."""
    import torch
    from project_tensor_b200.sharded import ShardedKeyIndex, _merge_on_gpu, shard_range
    d, n, nq, k = 128, 150_001, 5, 50
    gen = torch.Generator(device="cuda").manual_seed(20266)
    x = torch.randn((n, d), generator=gen, device="cuda", dtype=torch.float32)
    q = torch.randn((nq, d), generator=gen, device="cuda", dtype=torch.float32)
    prod = tg.TurboQuantProd(d, 4, seed=2026)
    whole = ShardedKeyIndex(prod, n, rank=0, world=1)
    whole.add(x[:60_000])
    whole.add(x[60_000:60_007].cpu().numpy())
    whole.add(x[60_007:])
    with pytest.raises(ValueError):
        whole.add(x[:1])
    ref_s, ref_i = prod.attention_scores(q, prod.quantize(x), topk=k)
    got_s, got_i = whole.search(q, k)
    assert torch.equal(got_s, ref_s) and torch.equal(got_i, ref_i)
    parts = []
    for rank in range(2):
        lo, hi = shard_range(n, rank, 2)
        shard = ShardedKeyIndex(prod, n, rank=rank, world=2)
        shard.add(x[lo:hi])
        assert (shard.start, shard.stop) == (lo, hi)
        parts.append(prod.attention_scores(q, shard.encoding(), topk=k, index_base=lo))
    merged_s, merged_i = _merge_on_gpu(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]))
    assert torch.equal(merged_s, ref_s) and torch.equal(merged_i, ref_i)


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("bits", [2, 4, 5])
def test_one_and_two_queries_on_every_path(tg, d, bits):
    """The reference's own call -- one query broadcast over all keys -- runs on a streaming lookup-table kernel
    by default; it, the tensor-core kernel and the exact kernel must agree within the score bound, for one
    query, for two, and for one query per group of keys; and the default path must match the oracle."""
    import torch
    n = 30_006
    rng = np.random.default_rng(20267 + d + bits)
    x = rng.standard_normal((n, d)).astype(np.float32) * rng.uniform(0.2, 5.0, (n, 1)).astype(np.float32)
    prod = tg.TurboQuantProd(d, bits, seed=2026)
    pp = _oracle_params(prod)
    want = orc.prod_quantize(pp, x)
    enc = tg.TurboQuantProdEncoding(indices=want[0], qjl=want[1], residual_norms=want[2], norms=want[3], prefix_shape=(n,))
    for nq, groups in ((1, 1), (2, 1), (6, 6), (12, 6)):
        q = rng.standard_normal((nq, d)).astype(np.float32)
        res = {}
        for path in ("exact", "tensor", "auto"):
            prod.set_kernel_path(path)
            res[path] = np.asarray(prod.attention_scores(q, enc, groups=groups))
        kpg = n // groups
        qn = np.linalg.norm(q, axis=1)[:, None]
        kn = want[3].reshape(groups, kpg).repeat(nq // groups, axis=0)
        for path in ("tensor", "auto"):
            assert parity.max_score_err(res[path], res["exact"], qn, kn, d) <= REL_SCORE, (path, nq, groups)
    prod.set_kernel_path("auto")
    q1 = rng.standard_normal((d,)).astype(np.float32)
    got = prod.attention_score(q1, enc)
    ref = orc.prod_attention_score(pp, q1, *want)
    assert got.shape == ref.shape == (n,)
    assert parity.max_score_err(got[None, :], ref[None, :], np.linalg.norm(q1), want[3][None, :], d) <= REL_SCORE


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("qpg", [3, 4])
def test_three_and_four_queries_per_group_on_every_path(tg, bits, qpg):
    """Grouped-query decode scoring -- 3 or 4 queries per group of keys, d = 128, up to 3 code bits -- runs on the
    lane-interleaved lookup-table kernel by default: it must agree with the exact and the tensor-core kernels
    within the score bound (ragged group length, several groups, a single group), and with the oracle."""
    groups, kpg, d = 5, 4_099, 128
    n = groups * kpg
    rng = np.random.default_rng(20269 + bits + qpg)
    x = rng.standard_normal((n, d)).astype(np.float32) * rng.uniform(0.2, 5.0, (n, 1)).astype(np.float32)
    prod = tg.TurboQuantProd(d, bits, seed=2026)
    pp = _oracle_params(prod)
    want = orc.prod_quantize(pp, x)
    enc = tg.TurboQuantProdEncoding(indices=want[0], qjl=want[1], residual_norms=want[2], norms=want[3], prefix_shape=(n,))
    for nq, grp in ((qpg * groups, groups), (qpg, 1)):
        q = rng.standard_normal((nq, d)).astype(np.float32)
        res = {}
        for path in ("exact", "tensor", "auto"):
            prod.set_kernel_path(path)
            res[path] = np.asarray(prod.attention_scores(q, enc, groups=grp))
        prod.set_kernel_path("auto")
        per = n // grp
        assert res["auto"].shape == (nq, per)
        qn = np.linalg.norm(q, axis=1)[:, None]
        kn = want[3].reshape(grp, per).repeat(nq // grp, axis=0)
        for path in ("tensor", "auto"):
            assert parity.max_score_err(res[path], res["exact"], qn, kn, d) <= REL_SCORE, (path, nq, grp)
        # the oracle, one broadcast call per query as the reference's users do, on the first and the last query
        for a in (0, nq - 1):
            g = a // (nq // grp)
            rows = slice(g * per, (g + 1) * per)
            ref = orc.prod_attention_score(pp, q[a], *(w[rows] for w in want[:4]), (per,))
            assert parity.max_score_err(res["auto"][a][None, :], ref[None, :], qn[a], want[3][rows][None, :], d) <= REL_SCORE


@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("n", [1, 129, 20_003])
def test_one_query_per_key_on_both_paths(tg, d, bits, n):
    """attention_score with a query row per key (_quant.py:342-358): the tensor-core kernel (the dequantize
    contraction with a dot product in its epilogue) against the exact kernel and against the oracle."""
    rng = np.random.default_rng(20268 + d + bits + n)
    x = rng.standard_normal((n, d)).astype(np.float32) * rng.uniform(0.2, 5.0, (n, 1)).astype(np.float32)
    q = rng.standard_normal((n, d)).astype(np.float32)
    prod = tg.TurboQuantProd(d, bits, seed=2026)
    pp = _oracle_params(prod)
    want = orc.prod_quantize(pp, x)
    enc = tg.TurboQuantProdEncoding(indices=want[0], qjl=want[1], residual_norms=want[2], norms=want[3], prefix_shape=(n,))
    ref = orc.prod_attention_score(pp, q, *want)
    qn = np.linalg.norm(q, axis=1)
    for path in ("exact", "tensor"):
        prod.set_kernel_path(path)
        got = np.asarray(prod.attention_score(q, enc))
        assert got.shape == (n,)
        assert parity.max_score_err(got, ref, qn, want[3], d) <= REL_SCORE, path


@pytest.mark.parametrize("d,bits", [(128, 4), (64, 3), (256, 4)])
def test_c_abi_broadcast_entry_point(tg, d, bits):
    """tq_score_broadcast called directly (no scratch argument): one query against all keys, equal to the
    batched entry point the Python class uses, on the tensor geometries and on one without tensor kernels."""
    import torch
    from project_tensor_b200 import _native, packed_buffers
    lib = _native.load()
    n = 10_007
    gen = torch.Generator(device="cuda").manual_seed(20269 + d)
    x = torch.randn((n, d), generator=gen, device="cuda", dtype=torch.float32)
    q = torch.randn((d,), generator=gen, device="cuda", dtype=torch.float32)
    prod = tg.TurboQuantProd(d, bits, seed=2026)
    enc = prod.quantize(x)
    bufs = packed_buffers(enc)
    want = prod.attention_score(q, enc)
    out = torch.empty((n,), dtype=torch.float32, device="cuda")
    handle = prod._plans.handle(torch.device("cuda", torch.cuda.current_device()))
    _native.check(lib.tq_score_broadcast(handle, q.data_ptr(), bufs["codes"].data_ptr(), bufs["signs"].data_ptr(),
                                         bufs["residual_norms"].data_ptr(), bufs["norms"].data_ptr(), n, out.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(out, want)


def test_c_abi_rejects_grids_beyond_the_launch_limits(tg):
    """A top-k over more than 65,535 (group, query) pairs would need a grid the selection kernels cannot have: the
    entry point must say so before anything is enqueued (not fail halfway with a launch error)."""
    import torch
    from project_tensor_b200 import _native
    lib = _native.load()
    prod = tg.TurboQuantProd(128, 4, seed=2026)
    handle = prod._plans.handle(torch.device("cuda", torch.cuda.current_device()))
    dummy = torch.zeros((64,), dtype=torch.float32, device="cuda")
    p = dummy.data_ptr()
    before = int(lib.tq_kernel_launches())
    rc = lib.tq_score_cache(handle, p, 8192, 16, p, p, p, p, 4, 4, None, 5, p, p, 0, p, 256,
                            torch.cuda.current_stream().cuda_stream)
    assert rc == -1 and b"groups * q_per_group" in lib.tq_last_error()
    assert int(lib.tq_kernel_launches()) == before
    # the merge over gathered blocks checks its block geometry the same way
    rc = lib.tq_topk_merge_gathered(p, 100, 48, 2, 3, 4, p, p, torch.cuda.current_stream().cuda_stream)
    assert rc == -1 and b"does not hold" in lib.tq_last_error()


def test_merge_on_gathered_blocks_equals_merge_on_lists(tg):
    """tq_topk_merge_gathered reads scores and indices out of the per-rank blocks of one all-gather; it must give what
    tq_topk_merge gives on the same lists laid out as two arrays."""
    import torch
    from project_tensor_b200 import _native
    from project_tensor_b200.sharded import TopkExchange
    lib = _native.load()
    lists, q, k = 3, 7, 100
    gen = torch.Generator(device="cuda").manual_seed(11)
    s = torch.randn((lists, q, k), device="cuda", generator=gen).sort(dim=2, descending=True).values.contiguous()
    i = torch.randint(0, 1 << 40, (lists, q, k), device="cuda", generator=gen)
    ex = TopkExchange(q, k, torch.device("cuda", torch.cuda.current_device()))
    gathered = torch.empty((lists, ex.block_bytes), dtype=torch.uint8, device="cuda")
    for l in range(lists):
        gathered[l, :4 * q * k] = s[l].reshape(-1).view(torch.uint8)
        gathered[l, ex.idx_offset:] = i[l].reshape(-1).view(torch.uint8)
    out = [torch.empty((q, k), dtype=torch.float32, device="cuda"), torch.empty((q, k), dtype=torch.int64, device="cuda"),
           torch.empty((q, k), dtype=torch.float32, device="cuda"), torch.empty((q, k), dtype=torch.int64, device="cuda")]
    st = torch.cuda.current_stream().cuda_stream
    _native.check(lib.tq_topk_merge(s.data_ptr(), i.data_ptr(), lists, q, k, out[0].data_ptr(), out[1].data_ptr(), st))
    _native.check(lib.tq_topk_merge_gathered(gathered.data_ptr(), ex.block_bytes, ex.idx_offset, lists, q, k,
                                             out[2].data_ptr(), out[3].data_ptr(), st))
    torch.cuda.synchronize()
    assert torch.equal(out[0], out[2]) and torch.equal(out[1], out[3])
    assert torch.equal(out[0], s.permute(1, 0, 2).reshape(q, -1).sort(dim=1, descending=True).values[:, :k])
