"""Decode attention over the packed key/value cache: tq_decode_attention (scores, softmax and the weighted sum
of values in one pass over the packed rows) against the oracle's restatement of the reference's
scaled_dot_product_attention over attention_score and dequantize, and against the composition of this
package's own scoring and dequantize kernels; ragged lengths, several key splits, several query passes, the
device-side length, an empty cache, argument checks."""
import numpy as np
import pytest

import project_tensor_b200 as tg
from project_tensor_b200 import _native
from project_tensor_b200.cache import PackedKVCache
from oracle import turboquant_oracle as orc

pytestmark = pytest.mark.gpu

TOL = 1e-4    # of the largest output magnitude; the scoring tolerance of the path carried through the softmax


def _torch():
    import torch
    return torch


def _randn(shape, seed, scale=1.0):
    torch = _torch()
    return scale * torch.randn(*shape, device="cuda", generator=torch.Generator("cuda").manual_seed(seed))


def _filled(d, kbits, vbits, groups, n, cap, seed, key_scale=1.0):
    kq = tg.TurboQuantProd(d, kbits, seed=2026)
    vq = tg.TurboQuantMSE(d, vbits, seed=77)            # its own rotation and codebook
    cache = PackedKVCache(kq, vq, groups, cap)
    keys, values = _randn((groups, n, d), seed, key_scale), _randn((groups, n, d), seed + 1)
    cache.append(keys, values)
    return kq, vq, cache, keys, values


def _composed(kq, vq, cache, queries, scale):
    """softmax(scale * scores) @ dequantize(values) from the package's own kernels, float64 softmax."""
    torch = _torch()
    out = []
    for g in range(cache.groups):
        s = kq.attention_scores(queries[g], cache.keys.encoding(g)).double() * scale
        w = torch.softmax(s, dim=-1)
        v = vq.dequantize(cache.value_encoding(g)).double()
        out.append(w @ v)
    return torch.stack(out).float()


@pytest.mark.parametrize("d,kbits,vbits,qpg,n", [
    (128, 4, 4, 4, 1500),     # the cache of cfg 3's kind: 3-bit codes + signs, 4 queries per group
    (128, 3, 2, 1, 700),      # one query per group
    (128, 5, 3, 3, 1100),     # 4 code bits: two queries per pass, two passes, the second half empty
    (128, 2, 1, 6, 513),      # 1 code bit; a tile with a single key
    (64, 4, 4, 4, 1301),      # d = 64: 24-byte code rows, 8-byte sign rows
    (64, 3, 3, 1, 37),
])
def test_attend_against_oracle_and_composition(d, kbits, vbits, qpg, n):
    torch = _torch()
    groups, cap = 3, 1600
    kq, vq, cache, keys, values = _filled(d, kbits, vbits, groups, n, cap, seed=11)
    queries = _randn((groups, qpg, d), 13)
    scale = d ** -0.5
    got = cache.attend(queries)
    assert got.shape == (groups, qpg, d)
    want = _composed(kq, vq, cache, queries, scale)
    peak = float(want.abs().max())
    assert float((got - want).abs().max()) <= TOL * peak
    # oracle on one group: its own quantize of the same keys and values, its scores, softmax and dequantize
    kp, vp = orc.prod_params(d, kbits, seed=2026), orc.mse_params(d, vbits, seed=77)
    g = 1
    kenc = orc.prod_quantize(kp, keys[g].cpu().numpy())[:4]
    vcodes, vnorms, _ = orc.mse_quantize(vp, values[g].cpu().numpy())
    ref = orc.decode_attention(kp, vp, queries[g].cpu().numpy(), kenc, vcodes, vnorms)
    np.testing.assert_allclose(got[g].cpu().numpy(), ref, rtol=0, atol=TOL * np.abs(ref).max())


def test_peaked_softmax_and_explicit_scale():
    """Large scores (keys of norm ~ 60, scale 1): the softmax concentrates on a few keys; the running maximum
    has to carry it."""
    torch = _torch()
    d, groups, n = 128, 2, 2000
    kq, vq, cache, keys, values = _filled(d, 4, 4, groups, n, 2048, seed=21, key_scale=5.0)
    queries = _randn((groups, 4, d), 23)
    got = cache.attend(queries, scale=1.0)
    want = _composed(kq, vq, cache, queries, 1.0)
    assert bool(torch.isfinite(got).all())
    assert float((got - want).abs().max()) <= 2e-3 * float(want.abs().max())   # e^(1e-4 * |s|max ~ 20) on the weights


def test_many_keys_many_splits_and_groups():
    """32,768 keys per group (64 tiles, several splits per group) and 16 groups of 4 queries."""
    torch = _torch()
    d, groups, n = 128, 16, 32768
    kq, vq, cache, keys, values = _filled(d, 3, 4, groups, n, n, seed=31)
    queries = _randn((groups, 4, d), 33)
    got = cache.attend(queries)
    want = _composed(kq, vq, cache, queries, d ** -0.5)
    assert float((got - want).abs().max()) <= TOL * float(want.abs().max())


def test_length_from_the_device_counter_and_growth():
    torch = _torch()
    d, groups, cap = 128, 4, 1024
    kq, vq, cache, keys, values = _filled(d, 4, 4, groups, 600, cap, seed=41)
    queries = _randn((groups, 4, d), 43)
    a = cache.attend(queries)
    b = cache.attend(queries, use_device_length=True)
    assert torch.equal(a, b) or float((a - b).abs().max()) <= 1e-6 * float(a.abs().max())
    # one more token changes the result, and both ways of passing the length agree again
    cache.append(_randn((groups, d), 45), _randn((groups, d), 46))
    a2 = cache.attend(queries)
    b2 = cache.attend(queries, use_device_length=True)
    assert float((a2 - b2).abs().max()) <= 1e-6 * float(a2.abs().max())
    assert float((a2 - a).abs().max()) > 0


def test_empty_cache_gives_zeros_and_argument_checks():
    torch = _torch()
    kq, vq = tg.TurboQuantProd(128, 4, seed=2026), tg.TurboQuantMSE(128, 4, seed=77)
    cache = PackedKVCache(kq, vq, 2, 8)
    q = _randn((2, 3, 128), 51)
    out = cache.attend(q, use_device_length=True)
    assert out.shape == (2, 3, 128) and bool((out == 0).all())
    with pytest.raises(ValueError, match="differ in shape"):
        cache.append(_randn((2, 128), 1), _randn((2, 2, 128), 2))
    with pytest.raises(ValueError, match="dimension"):
        PackedKVCache(kq, tg.TurboQuantMSE(64, 4, seed=1), 2, 8)
    # unsupported geometry is refused by the library, not computed some other way
    kq256, vq256 = tg.TurboQuantProd(256, 3, seed=1), tg.TurboQuantMSE(256, 3, seed=2)
    big = PackedKVCache(kq256, vq256, 1, 8)
    big.append(_randn((1, 4, 256), 3), _randn((1, 4, 256), 4))
    with pytest.raises(_native.TurboQuantNativeError, match="decode attention covers"):
        big.attend(_randn((1, 256), 5))
    # scratch too small
    cache.append(_randn((2, 4, 128), 6), _randn((2, 4, 128), 7))
    lib = _native.load()
    kh, vh = kq._plans.handle(cache.device), vq._plans.handle(cache.device)
    out = torch.empty(2, 3, 128, device="cuda")
    tiny = torch.empty(16, dtype=torch.uint8, device="cuda")
    kc = cache.keys
    rc = lib.tq_decode_attention(kh, vh, q.data_ptr(), 2, 3, kc.codes.data_ptr(), kc.signs.data_ptr(),
                                 kc.residual_norms.data_ptr(), kc.norms.data_ptr(), cache.value_codes.data_ptr(),
                                 cache.value_norms.data_ptr(), 4, 8, None, 0.0, out.data_ptr(), tiny.data_ptr(), 16, 0)
    assert rc == -4   # TQ_ERR_SCRATCH_TOO_SMALL


def test_decode_step_replayed_from_a_cuda_graph():
    """One captured decode step -- append the new key and value of every group, attend with the length read on
    the device -- replayed while the cache grows, against the same steps run eagerly on a second cache."""
    torch = _torch()
    d, groups, qpg, cap, steps = 128, 8, 4, 640, 6
    kq, vq = tg.TurboQuantProd(d, 4, seed=2026), tg.TurboQuantMSE(d, 4, seed=77)
    prefill_k, prefill_v = _randn((groups, 500, d), 61), _randn((groups, 500, d), 62)
    new_k, new_v = _randn((groups, steps, d), 63), _randn((groups, steps, d), 64)
    queries = _randn((steps, groups, qpg, d), 65)
    eager, graphed = PackedKVCache(kq, vq, groups, cap), PackedKVCache(kq, vq, groups, cap)
    for cache in (eager, graphed):
        cache.append(prefill_k, prefill_v)
    k_in, v_in, q_in = torch.zeros(groups, 1, d, device="cuda"), torch.zeros(groups, 1, d, device="cuda"), \
        torch.zeros(groups, qpg, d, device="cuda")
    # warm up outside the capture on a scratch cache (function attributes, plans), then capture one step
    scratch = PackedKVCache(kq, vq, groups, cap)
    scratch.append(k_in, v_in)
    scratch.attend(q_in, use_device_length=True)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            graphed.append(k_in, v_in)
            out = graphed.attend(q_in, use_device_length=True)
    torch.cuda.current_stream().wait_stream(stream)
    assert graphed.sync_length() == 500          # capturing executed nothing
    for t in range(steps):
        k_in.copy_(new_k[:, t:t + 1])
        v_in.copy_(new_v[:, t:t + 1])
        q_in.copy_(queries[t])
        graph.replay()
        eager.append(new_k[:, t], new_v[:, t])
        want = eager.attend(queries[t])
        torch.cuda.synchronize()
        assert float((out - want).abs().max()) <= 1e-6 * float(want.abs().max()), t
    assert graphed.sync_length() == 500 + steps
