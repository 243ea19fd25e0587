"""Bytes behind the outputs.  Every entry point writes into caller-owned buffers of exactly the documented size; the
kernels tile rows by 128 and write 16-byte pieces, so a ragged row count is where a stray store would go.  Each output
here is a slice of a larger allocation with 256 canary bytes on either side; after the call, for row counts around the
tile and warp sizes, the canaries must be untouched (a memory checker's job, done by hand through the C ABI)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GUARD = 256
SIZES = [1, 31, 33, 127, 129, 1000]


class Guarded:
    """A device buffer of `nbytes` between two canary zones (16-byte aligned start)."""

    def __init__(self, torch, nbytes, dev):
        self.torch = torch
        self.nbytes = int(nbytes)
        pad = (-self.nbytes) % 16
        self.raw = torch.full((GUARD + self.nbytes + pad + GUARD,), 0xC5, dtype=torch.uint8, device=dev)
        self.body = self.raw[GUARD:GUARD + self.nbytes]

    def ptr(self):
        return self.body.data_ptr() if self.nbytes else self.raw[GUARD:].data_ptr()

    def intact(self):
        front = bool((self.raw[:GUARD] == 0xC5).all())
        back = bool((self.raw[GUARD + self.nbytes:] == 0xC5).all())
        return front and back

    def view(self, dtype, shape):
        return self.body.view(dtype).view(*shape)


@pytest.fixture(scope="module")
def env(lib_built):
    import torch
    assert torch.cuda.is_available()
    import project_tensor_b200 as tg
    from project_tensor_b200 import _native
    return torch, tg, _native, _native.load(), torch.device("cuda", torch.cuda.current_device())


@pytest.mark.parametrize("path", ["auto", "exact"])
@pytest.mark.parametrize("d,bits", [(128, 4), (128, 3), (64, 3), (64, 2)])
def test_quantize_dequantize_and_scores_stay_inside_their_buffers(env, d, bits, path):
    torch, tg, _native, lib, dev = env
    st = torch.cuda.current_stream(dev).cuda_stream
    prod = tg.TurboQuantProd(d, bits, seed=2026)
    mse = tg.TurboQuantMSE(d, bits, seed=2026)
    prod.set_kernel_path(path)
    mse.set_kernel_path(path)
    hp, hm = prod._plans.handle(dev), mse._plans.handle(dev)
    cbp, sbp = int(lib.tq_code_row_bytes(hp)), int(lib.tq_sign_row_bytes(hp))
    cbm = int(lib.tq_code_row_bytes(hm))
    gen = torch.Generator(device=dev).manual_seed(d * 10 + bits)
    for n in SIZES:
        x = torch.randn((n, d), generator=gen, device=dev)
        q1 = torch.randn((d,), generator=gen, device=dev)
        qn = torch.randn((n, d), generator=gen, device=dev)
        q5 = torch.randn((5, d), generator=gen, device=dev)
        G = lambda nbytes: Guarded(torch, nbytes, dev)
        codes, signs, rn, nr = G(n * cbp), G(n * sbp), G(4 * n), G(4 * n)
        scratch = G(max(int(lib.tq_quantize_scratch_bytes(hp, n)), 16))
        _native.check(lib.tq_prod_quantize(hp, x.data_ptr(), n, codes.ptr(), signs.ptr(), rn.ptr(), nr.ptr(), scratch.ptr(),
                                           scratch.nbytes, st))
        mcodes, mnr = G(n * cbm), G(4 * n)
        mscratch = G(max(int(lib.tq_quantize_scratch_bytes(hm, n)), 16))
        _native.check(lib.tq_mse_quantize(hm, x.data_ptr(), n, mcodes.ptr(), mnr.ptr(), mscratch.ptr(), mscratch.nbytes, st))
        out_p, out_m = G(4 * n * d), G(4 * n * d)
        _native.check(lib.tq_prod_dequantize(hp, codes.ptr(), signs.ptr(), rn.ptr(), nr.ptr(), n, out_p.ptr(), st))
        _native.check(lib.tq_mse_dequantize(hm, mcodes.ptr(), mnr.ptr(), n, out_m.ptr(), st))
        s_b, s_p = G(4 * n), G(4 * n)
        _native.check(lib.tq_score_broadcast(hp, q1.data_ptr(), codes.ptr(), signs.ptr(), rn.ptr(), nr.ptr(), n, s_b.ptr(), st))
        _native.check(lib.tq_score_pairwise(hp, qn.data_ptr(), codes.ptr(), signs.ptr(), rn.ptr(), nr.ptr(), n, s_p.ptr(), st))
        k = min(7, n)
        mat, ts, ti = G(4 * 5 * n), G(4 * 5 * k), G(8 * 5 * k)
        need = int(lib.tq_topk_scratch_bytes(hp, 1, 5, n, k))
        tscr = G(max(need, 16))
        _native.check(lib.tq_score_batched(hp, q5.data_ptr(), 1, 5, codes.ptr(), signs.ptr(), rn.ptr(), nr.ptr(), n, mat.ptr(),
                                           k, ts.ptr(), ti.ptr(), 0, tscr.ptr(), tscr.nbytes, st))
        idx8, qjl8 = G(n * d), G(n * d)
        _native.check(lib.tq_unpack_codes(hp, codes.ptr(), n, idx8.ptr(), st))
        _native.check(lib.tq_unpack_signs(hp, signs.ptr(), n, qjl8.ptr(), st))
        recodes, resigns = G(n * cbp), G(n * sbp)
        _native.check(lib.tq_pack_codes(hp, idx8.ptr(), n, recodes.ptr(), st))
        _native.check(lib.tq_pack_signs(hp, qjl8.ptr(), n, resigns.ptr(), st))
        torch.cuda.synchronize()
        named = dict(codes=codes, signs=signs, residual_norms=rn, norms=nr, quantize_scratch=scratch, mse_codes=mcodes,
                     mse_norms=mnr, mse_scratch=mscratch, prod_recon=out_p, mse_recon=out_m, broadcast_scores=s_b,
                     pairwise_scores=s_p, score_matrix=mat, top_scores=ts, top_idx=ti, topk_scratch=tscr, indices=idx8,
                     qjl=qjl8, repacked_codes=recodes, repacked_signs=resigns)
        for name, g in named.items():
            assert g.intact(), f"d={d} bits={bits} path={path} n={n}: bytes around {name} were written"
        # and the round trips are what they should be, so the calls really ran on these buffers
        assert torch.equal(recodes.body, codes.body) and torch.equal(resigns.body, signs.body)
        assert torch.isfinite(mat.view(torch.float32, (5, n))).all()
        top = ts.view(torch.float32, (5, k))
        assert bool((top[:, :-1] >= top[:, 1:]).all())
        prod._plans.check_status(dev)


@pytest.mark.parametrize("n", SIZES)
def test_append_and_decode_attention_stay_inside_their_buffers(env, n):
    """Cache arrays at exactly groups x capacity rows with canaries behind them; `n` rows filled by appends of ragged
    sizes, then scores of the filled part and decode attention over it."""
    torch, tg, _native, lib, dev = env
    st = torch.cuda.current_stream(dev).cuda_stream
    d, groups, cap = 128, 3, n
    prod, mse = tg.TurboQuantProd(d, 4, seed=2026), tg.TurboQuantMSE(d, 4, seed=2026)
    hp, hm = prod._plans.handle(dev), mse._plans.handle(dev)
    cbp, sbp, cbm = int(lib.tq_code_row_bytes(hp)), int(lib.tq_sign_row_bytes(hp)), int(lib.tq_code_row_bytes(hm))
    rows = groups * cap
    G = lambda nbytes: Guarded(torch, nbytes, dev)
    codes, signs, rn, nr = G(rows * cbp), G(rows * sbp), G(4 * rows), G(4 * rows)
    vcodes, vnr = G(rows * cbm), G(4 * rows)
    length = torch.zeros((2,), dtype=torch.int64, device=dev)
    gen = torch.Generator(device=dev).manual_seed(n)
    done = 0
    for step in (max(1, n // 3), n):        # a first append, then the rest; the last one ends exactly at the capacity
        t = min(step, n - done)
        if t <= 0:
            continue
        xk = torch.randn((groups, t, d), generator=gen, device=dev)
        xv = torch.randn((groups, t, d), generator=gen, device=dev)
        _native.check(lib.tq_prod_append(hp, xk.data_ptr(), groups, t, codes.ptr(), signs.ptr(), rn.ptr(), nr.ptr(), cap,
                                         length.data_ptr(), 0, st))
        _native.check(lib.tq_mse_append(hm, xv.data_ptr(), groups, t, vcodes.ptr(), vnr.ptr(), cap, length.data_ptr(), 1, st))
        done += t
    assert int(length[0].item()) == n
    q = torch.randn((groups, 4, d), generator=gen, device=dev)
    mat = G(4 * groups * 4 * n)
    need = int(lib.tq_topk_scratch_bytes(hp, groups, 4, n, 0))
    scr = G(max(need, 16))
    _native.check(lib.tq_score_cache(hp, q.data_ptr(), groups, 4, codes.ptr(), signs.ptr(), rn.ptr(), nr.ptr(), n, cap, mat.ptr(),
                                     0, None, None, 0, scr.ptr(), scr.nbytes, st))
    out = G(4 * groups * 4 * d)
    need = int(lib.tq_decode_attention_scratch_bytes(hp, groups, 4, n))
    dscr = G(max(need, 16))
    _native.check(lib.tq_decode_attention(hp, hm, q.data_ptr(), groups, 4, codes.ptr(), signs.ptr(), rn.ptr(), nr.ptr(),
                                          vcodes.ptr(), vnr.ptr(), n, cap, None, 0.0, out.ptr(), dscr.ptr(), dscr.nbytes, st))
    torch.cuda.synchronize()
    for name, g in dict(codes=codes, signs=signs, residual_norms=rn, norms=nr, value_codes=vcodes, value_norms=vnr,
                        score_matrix=mat, score_scratch=scr, attention_out=out, attention_scratch=dscr).items():
        assert g.intact(), f"n={n}: bytes around {name} were written"
    assert torch.isfinite(out.view(torch.float32, (groups, 4, d))).all()
