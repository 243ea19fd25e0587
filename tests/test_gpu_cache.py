"""The growing packed key cache: appended rows equal the rows of a one-shot quantize (reference-order kernel,
bit for bit, and the oracle on a sample), scores over the strided cache equal scores over contiguous
encodings on every kernel path, a captured CUDA graph of the append step keeps working as the cache grows,
and a full cache drops rows instead of writing out of bounds."""
import numpy as np
import pytest

import project_tensor_b200 as tg
from project_tensor_b200 import _native
from project_tensor_b200.cache import PackedKeyCache
from oracle import turboquant_oracle as orc

pytestmark = pytest.mark.gpu


def _torch():
    import torch
    return torch


def _keys(groups, tokens, d, seed):
    torch = _torch()
    return torch.randn(groups, tokens, d, device="cuda", generator=torch.Generator("cuda").manual_seed(seed))


def _exact_encoding(quant, keys):
    quant.set_kernel_path("exact")
    try:
        return quant.quantize(keys)
    finally:
        quant.set_kernel_path("auto")


@pytest.mark.parametrize("d,bits", [(128, 4), (64, 3), (256, 2), (96, 5)])
def test_appended_rows_equal_one_shot_quantize(d, bits):
    torch = _torch()
    groups, steps, cap = 6, 9, 16
    quant = tg.TurboQuantProd(d, bits, seed=2026)
    keys = _keys(groups, steps, d, 1)
    cache = PackedKeyCache(quant, groups, cap)
    cache.append(keys[:, :4])              # several tokens at once
    for t in range(4, steps):
        cache.append(keys[:, t])           # then one token per step, shape (groups, d)
    assert len(cache) == steps and cache.sync_length() == steps
    want = tg.packed_buffers(_exact_encoding(quant, keys))
    for g in range(groups):
        got = tg.packed_buffers(cache.encoding(g))
        for name in ("codes", "signs", "norms", "residual_norms"):
            assert torch.equal(got[name], want[name][g * steps:(g + 1) * steps]), (g, name)
    # rows behind the length were never written
    assert int(cache.codes.view(groups, cap, -1)[:, steps:].sum()) == 0
    # and a sample against the oracle
    p = orc.prod_params(d, bits, seed=2026)
    codes, qjl, rn, norms = orc.prod_quantize(p, keys[2].cpu().numpy())[:4]
    enc = cache.encoding(2)
    assert np.array_equal(enc.indices.cpu().numpy(), codes)
    assert np.array_equal(enc.qjl.cpu().numpy(), qjl)
    np.testing.assert_allclose(enc.residual_norms.cpu().numpy(), rn, rtol=1e-5)
    np.testing.assert_allclose(enc.norms.cpu().numpy(), norms, rtol=1e-5)


@pytest.mark.parametrize("d,bits,qpg", [(128, 4, 4), (128, 3, 1), (64, 3, 2), (64, 4, 8), (256, 2, 3)])
def test_scores_over_the_cache_equal_scores_over_encodings(d, bits, qpg):
    torch = _torch()
    groups, n, cap = 5, 700, 1000
    quant = tg.TurboQuantProd(d, bits, seed=2026)
    keys = _keys(groups, n, d, 2)
    cache = PackedKeyCache(quant, groups, cap)
    cache.append(keys)                     # 3500 rows: the one-launch kernel
    queries = _keys(groups, qpg, d, 3)
    got = cache.scores(queries)
    assert got.shape == (groups, qpg, n)
    k = 10
    top_s, top_p, mat = cache.scores(queries, topk=k, return_matrix=True)
    top_s2, top_p2 = cache.scores(queries, topk=k)
    # one or two queries without top-k take the streaming kernel, with top-k the tensor-core one: two
    # summation orders of the same float32 score, held to the scoring tolerance
    assert float((mat - got).abs().max()) <= 1e-4 * float(got.abs().max())
    for g in range(groups):
        want = quant.attention_scores(queries[g], cache.encoding(g))
        scale = float(want.abs().max())
        assert float((got[g] - want).abs().max()) <= 1e-4 * scale
        # top-k: positions inside the group, scores descending and equal to the matrix at those positions
        for a in range(qpg):
            assert bool((top_p[g, a] >= 0).all()) and bool((top_p[g, a] < n).all())
            assert torch.equal(mat[g, a][top_p[g, a]], top_s[g, a])
            assert bool((top_s[g, a][:-1] >= top_s[g, a][1:]).all())
            kth = torch.sort(mat[g, a], descending=True).values[k - 1]
            assert float(top_s[g, a][-1]) == float(kth)
            assert float((top_s2[g, a] - top_s[g, a]).abs().max()) <= 1e-4 * scale
    # oracle on one group and query
    p = orc.prod_params(d, bits, seed=2026)
    codes, qjl, rn, norms = orc.prod_quantize(p, keys[1].cpu().numpy())[:4]
    want = orc.prod_attention_score(p, queries[1, 0].cpu().numpy(), codes, qjl, rn, norms, (n,))
    np.testing.assert_allclose(got[1, 0].cpu().numpy(), want, rtol=0, atol=1e-4 * np.abs(want).max())


def test_prefill_then_decode_and_kernel_paths():
    torch = _torch()
    groups, prefill, cap = 4, 3000, 3072          # 12000 rows at once: the bulk quantizer, copied into place
    quant = tg.TurboQuantProd(128, 4, seed=2026)
    keys = _keys(groups, prefill + 3, 128, 4)
    cache = PackedKeyCache(quant, groups, cap)
    cache.append(keys[:, :prefill])
    for t in range(3):
        cache.append(keys[:, prefill + t])
    assert len(cache) == prefill + 3 == cache.sync_length()
    whole = tg.packed_buffers(quant.quantize(keys))
    n = prefill + 3
    for g in range(groups):
        got = tg.packed_buffers(cache.encoding(g))
        # the bulk quantizer may differ from the reference-order kernel on knife-edge coordinates only
        diff = (got["codes"] != whole["codes"][g * n:(g + 1) * n]).any(dim=1).float().mean()
        assert float(diff) < 1e-3
        assert torch.allclose(got["norms"], whole["norms"][g * n:(g + 1) * n], rtol=1e-5)
    queries = _keys(groups, 32, 128, 5)
    ref = cache.scores(queries)
    scale = float(ref.abs().max())
    for path in ("exact", "tensor", "auto"):
        quant.set_kernel_path(path)
        try:
            got = cache.scores(queries)
        finally:
            quant.set_kernel_path("auto")
        assert float((got - ref).abs().max()) <= 1e-4 * scale, path


def test_append_step_in_a_cuda_graph():
    torch = _torch()
    groups, cap, d = 8, 64, 128
    quant = tg.TurboQuantProd(d, 4, seed=2026)
    cache = PackedKeyCache(quant, groups, cap)
    step_in = torch.zeros(groups, 1, d, device="cuda")
    keys = _keys(groups, 12, d, 6)
    # warm up outside the capture (plan creation, function attributes), then start from an empty cache
    cache.append(step_in)
    cache.reset()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            cache.append(step_in)
    cache.reset()                                   # capture does not execute; the host mirror counted one
    for t in range(12):
        step_in.copy_(keys[:, t:t + 1])
        graph.replay()
    torch.cuda.synchronize()
    assert cache.sync_length() == 12
    want = tg.packed_buffers(_exact_encoding(quant, keys))
    for g in range(groups):
        got = tg.packed_buffers(cache.encoding(g))
        for name in ("codes", "signs", "norms", "residual_norms"):
            assert torch.equal(got[name], want[name][g * 12:(g + 1) * 12]), (g, name)


def test_full_cache_refuses_and_the_c_entry_drops_rows():
    torch = _torch()
    groups, cap, d = 3, 5, 64
    quant = tg.TurboQuantProd(d, 3, seed=2026)
    cache = PackedKeyCache(quant, groups, cap)
    keys = _keys(groups, 6, d, 7)
    cache.append(keys[:, :4])
    with pytest.raises(ValueError, match="full"):
        cache.append(keys[:, 4:6])
    with pytest.raises(ValueError, match="groups"):
        cache.append(keys[:2, 4])
    # the C entry point itself: two tokens into one free row -> the first lands, the second is dropped,
    # the length stops at the capacity, nothing outside the arrays is touched
    lib = _native.load()
    handle = quant._plans.handle(cache.device)
    x = keys[:, 4:6].contiguous()
    before = cache.codes.clone()
    _native.check(lib.tq_prod_append(handle, x.data_ptr(), groups, 2, cache.codes.data_ptr(), cache.signs.data_ptr(),
                                     cache.residual_norms.data_ptr(), cache.norms.data_ptr(), cap,
                                     cache.length_device.data_ptr(), 1, torch.cuda.current_stream().cuda_stream))
    assert cache.sync_length() == cap
    want = tg.packed_buffers(_exact_encoding(quant, keys[:, :5]))
    for g in range(groups):
        assert torch.equal(tg.packed_buffers(cache.encoding(g))["codes"], want["codes"][g * 5:(g + 1) * 5])
        assert torch.equal(cache.codes.view(groups, cap, -1)[g, :4], before.view(groups, cap, -1)[g, :4])
    # argument checks of the entry point
    assert lib.tq_prod_append(handle, x.data_ptr(), groups, 9, cache.codes.data_ptr(), cache.signs.data_ptr(),
                              cache.residual_norms.data_ptr(), cache.norms.data_ptr(), cap,
                              cache.length_device.data_ptr(), 1, 0) == -1   # TQ_ERR_INVALID_ARGUMENT
    assert lib.tq_prod_append(handle, x.data_ptr(), groups, 1, cache.codes.data_ptr(), cache.signs.data_ptr(),
                              cache.residual_norms.data_ptr(), cache.norms.data_ptr(), cap, None, 1, 0) != 0


def test_empty_cache_scores():
    torch = _torch()
    quant = tg.TurboQuantProd(128, 4, seed=2026)
    cache = PackedKeyCache(quant, 2, 8)
    q = _keys(2, 3, 128, 8)
    assert cache.scores(q).shape == (2, 3, 0)
    s, p = cache.scores(q, topk=4)
    assert bool((p == -1).all()) and bool(torch.isinf(s).all())
