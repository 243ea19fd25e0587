"""Quality metrics of a quantizer pair on device-resident data, at any scale.

The reference validates TurboQuant with a harness that works on a few hundred NumPy vectors
(validate_turboquant.py:65-71 ``topk_recall``, :74-125 ``collect_metrics``): reconstruction MSE and cosine of
``TurboQuantMSE``, mean absolute / RMS error of ``TurboQuantProd.attention_score`` against the exact dot products,
the gap between the score and the dot product with the explicit reconstruction, and recall@k of the approximate
ranking.  ``quality_report`` computes the same quantities for key sets of 10^6 .. 10^8 rows without ever holding an
(N, d) reconstruction or a (Q, N) score matrix: the keys are walked in chunks, every chunk goes through the CUDA
quantize / dequantize / scoring kernels of this package, sums are accumulated in float64 on the device, and the
recall compares the device top-k of the approximate scores (``attention_scores(topk=k)``) with the top-k of the exact
float32 products of the same chunked walk.  Only the exact products ``queries @ keys.T`` -- the yardstick, not the
path -- come from a torch matmul.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, Optional, Sequence

from . import turboquant as _tq


def _chunks(keys: Any, chunk_rows: int, device) -> Iterable:
    """(offset, float32 device tensor) pairs over the rows of ``keys`` (NumPy, torch, or a callable
    ``keys(offset, rows) -> array`` for sets that are generated rather than stored)."""
    torch = _tq._require_cuda()
    if callable(keys):
        off = 0
        while True:
            part = keys(off, chunk_rows)
            if part is None or len(part) == 0:
                return
            t = torch.as_tensor(part, dtype=torch.float32, device=device)
            yield off, t
            off += t.shape[0]
    else:
        n = keys.shape[0]
        for off in range(0, n, chunk_rows):
            yield off, torch.as_tensor(keys[off:off + chunk_rows], dtype=torch.float32, device=device).contiguous()


def quality_report(mse_quantizer: Optional["_tq.TurboQuantMSE"], prod_quantizer: Optional["_tq.TurboQuantProd"], keys: Any,
                   queries: Any, ks: Sequence[int] = (1, 5, 10), chunk_rows: int = 1 << 20, device: Any = None) -> Dict[str, float]:
    """The harness's metrics (validate_turboquant.py:96-121) for ``keys`` (N, d) and ``queries`` (Q, d).

    Returns ``mse_mse``, ``mean_cosine_similarity`` (TurboQuantMSE round trip), ``prod_dot_mae``, ``prod_dot_rmse``,
    ``prod_vs_explicit_gap`` and ``prod_recall_at_<k>`` for every k in ``ks`` (TurboQuantProd), plus ``keys`` and
    ``queries`` counts.  Either quantizer may be None; its metrics are left out.  Ties in a top-k are broken towards
    the lower key index on both sides.
    """
    torch = _tq._require_cuda()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    q = torch.as_tensor(queries, dtype=torch.float32, device=dev).reshape(-1, queries.shape[-1]).contiguous()
    nq, d = q.shape
    kmax = max(ks) if ks else 0
    f64 = dict(dtype=torch.float64, device=dev)
    sq_err = torch.zeros((), **f64)
    cos_sum = torch.zeros((), **f64)
    abs_err = torch.zeros((), **f64)
    sq_score_err = torch.zeros((), **f64)
    gap = torch.zeros((), **f64)
    n = 0
    exact_s, exact_i, approx_s, approx_i = [], [], [], []
    with torch.cuda.device(dev):
        for off, x in _chunks(keys, chunk_rows, dev):
            m = x.shape[0]
            if mse_quantizer is not None:
                recon = mse_quantizer.dequantize(mse_quantizer.quantize(x))
                sq_err += ((x - recon).double() ** 2).sum()
                dots = (x * recon).sum(dim=1)
                norms = torch.linalg.norm(x, dim=1) * torch.linalg.norm(recon, dim=1)
                cos_sum += (dots / torch.where(norms > 0, norms, torch.ones_like(norms))).double().sum()
                del recon
            if prod_quantizer is not None:
                enc = prod_quantizer.quantize(x)
                exact = q @ x.T                                     # the yardstick: float32 products
                k_here = min(kmax, m)
                if k_here:
                    # the approximate ranking never leaves the scoring kernels: device top-k, no matrix
                    ts, ti = prod_quantizer.attention_scores(q, enc, topk=k_here, index_base=off)
                    approx_s.append(ts)
                    approx_i.append(ti)
                    es, ei = torch.topk(exact, k_here, dim=1)
                    exact_s.append(es)
                    exact_i.append(ei + off)
                approx = prod_quantizer.attention_scores(q, enc)
                diff = (exact - approx).double()
                abs_err += diff.abs().sum()
                sq_score_err += (diff ** 2).sum()
                explicit = q @ prod_quantizer.dequantize(enc).T
                gap += (approx - explicit).double().abs().sum()
                del enc, exact, approx, explicit, diff
            n += m
    out: Dict[str, float] = {"keys": n, "queries": nq, "dimension": d}
    if n == 0:
        return out
    if mse_quantizer is not None:
        out["mse_mse"] = float(sq_err / (n * d))
        out["mean_cosine_similarity"] = float(cos_sum / n)
    if prod_quantizer is not None:
        out["prod_dot_mae"] = float(abs_err / (n * nq))
        out["prod_dot_rmse"] = float(torch.sqrt(sq_score_err / (n * nq)))
        out["prod_vs_explicit_gap"] = float(gap / (n * nq))
        if kmax and approx_s:
            def best(scores, idx, k):
                s, i = torch.cat(scores, dim=1), torch.cat(idx, dim=1)
                # descending by score, ties to the lower index: sort by index first, then stably by score
                order = torch.argsort(i, dim=1, stable=True)
                s, i = torch.gather(s, 1, order), torch.gather(i, 1, order)
                order = torch.argsort(s, dim=1, descending=True, stable=True)[:, :k]
                return torch.gather(i, 1, order)
            for k in ks:
                kk = min(k, n)
                a, e = best(approx_s, approx_i, kk), best(exact_s, exact_i, kk)
                hits = (a[:, :, None] == e[:, None, :]).any(dim=2).double().sum(dim=1) / kk
                out[f"prod_recall_at_{k}"] = float(hits.mean())
    return out
