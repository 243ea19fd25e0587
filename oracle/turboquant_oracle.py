"""CPU oracle for the TurboQuant path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

A plain NumPy restatement of the reference algorithm in
``tensor_gpu_v2/_quant.py`` (Project-Tensor).  It exists so that the CUDA
kernels can be checked against the reference's arithmetic on a machine where
the reference itself is not present.  Only the test-suite, the smoke check and
the CPU-baseline leg of the benchmark may import this module; the shipped
package never does.

Parity pin: ``tests/golden/make_golden.py`` runs the unmodified reference file
and stores its outputs as fixtures; ``tests/test_oracle_golden.py`` requires
this restatement to reproduce every one of them bit for bit.

Every function names the reference lines it restates.  The array expressions
are kept in the reference's order (normalise -> rotate -> search; gather ->
rotate back; residual in the un-rotated domain) because float32 results depend
on that order.
"""
from __future__ import annotations

import math
from typing import NamedTuple, Optional, Tuple

import numpy as np

_ALPHA_NUM = math.sqrt(math.pi / 2.0)


# --------------------------------------------------------------------------
# host constants
# --------------------------------------------------------------------------
def sphere_coordinate_density(d: int, t: np.ndarray) -> np.ndarray:
    """Density of one coordinate of a uniform point on S^(d-1).

    Restates ``_beta_coordinate_pdf`` (_quant.py:73-83):
    Gamma(d/2) / (sqrt(pi) Gamma((d-1)/2)) * (1 - t^2)^((d-3)/2).
    """
    if d < 2:
        raise ValueError("TurboQuant requires dimension >= 2")
    log_c = math.lgamma(d / 2) - 0.5 * math.log(math.pi) - math.lgamma((d - 1) / 2)
    body = np.maximum(0.0, 1.0 - t * t) ** (0.5 * (d - 3))
    return np.exp(log_c) * body


def lloyd_max_codebook(d: int, bits: int, *, grid_size: int = 16385,
                       max_iter: int = 200, tol: float = 1e-8) -> np.ndarray:
    """Lloyd-Max scalar codebook (float64, sorted) for the density above.

    Restates ``_build_lloyd_max_codebook`` (_quant.py:93-138) including its
    discretisation: trapezoid end weights (:107-112), start from weighted
    quantiles (:114-116, helper :86-90), assignment by
    ``searchsorted(..., side="left")`` (:121), the empty-cell rules (:127-132),
    sort+clip every sweep (:133) and the max-move stopping test (:134).
    """
    levels = 1 << bits
    t = np.linspace(-1.0, 1.0, grid_size, dtype=np.float64)
    w = sphere_coordinate_density(d, t) * (t[1] - t[0])
    w[0] *= 0.5
    w[-1] *= 0.5

    mass = np.cumsum(w)
    want = np.clip((np.arange(levels, dtype=np.float64) + 0.5) / levels, 0.0, 1.0) * mass[-1]
    c = np.clip(np.sort(np.interp(want, mass, t)), -1.0, 1.0)

    for _ in range(max_iter):
        prev = c.copy()
        cuts = 0.5 * (c[:-1] + c[1:])
        cell = np.searchsorted(cuts, t, side="left")
        for k in range(levels):
            sel = cell == k
            m = w[sel].sum()
            if m > 0:
                c[k] = float(np.sum(t[sel] * w[sel]) / m)
            elif k == 0:
                c[k] = -1.0
            elif k == levels - 1:
                c[k] = 1.0
            else:
                c[k] = 0.5 * (c[k - 1] + c[k + 1])
        c = np.clip(np.sort(c), -1.0, 1.0)
        if np.max(np.abs(c - prev)) < tol:
            break
    return c


def seeded_rotation(d: int, seed: Optional[int]) -> np.ndarray:
    """Sign-fixed Q of a seeded Gaussian's QR, float32 (_quant.py:141-148)."""
    g = np.random.default_rng(seed).standard_normal((d, d))
    q, r = np.linalg.qr(g)
    s = np.sign(np.diag(r))
    s[s == 0] = 1.0
    return (q * s).astype(np.float32)


def seeded_projection(d: int, seed: Optional[int]) -> np.ndarray:
    """d x d standard-normal sketch matrix, float32 (_quant.py:151-153)."""
    return np.random.default_rng(seed).standard_normal((d, d)).astype(np.float32)


class MSEParams(NamedTuple):
    d: int
    bits: int
    rotation: np.ndarray      # (d, d) float32
    codebook: np.ndarray      # (2**bits,) float32
    boundaries: np.ndarray    # (2**bits - 1,) float32


class ProdParams(NamedTuple):
    d: int
    bits: int
    mse: MSEParams            # stage with max(bits-1, 1) bits
    projection: np.ndarray    # (d, d) float32


def mse_params(d: int, bits: int, *, seed: Optional[int] = None, grid_size: int = 16385,
               max_iter: int = 200, rotation=None, codebook=None) -> MSEParams:
    """Constants of ``TurboQuantMSE.__init__`` (_quant.py:175-213)."""
    if d < 2:
        raise ValueError("dimension must be >= 2")
    if bits < 1:
        raise ValueError("bits must be >= 1")
    rot = np.asarray(rotation, dtype=np.float32) if rotation is not None else seeded_rotation(d, seed)
    if rot.shape != (d, d):
        raise ValueError(f"rotation must have shape {(d, d)}, got {rot.shape}")
    if codebook is not None:
        cb = np.asarray(codebook, dtype=np.float32)
    else:
        cb = lloyd_max_codebook(d, bits, grid_size=grid_size, max_iter=max_iter).astype(np.float32)
    if cb.ndim != 1 or cb.shape[0] != (1 << bits):
        raise ValueError("codebook shape does not match bit-width")
    return MSEParams(int(d), int(bits), rot, cb, 0.5 * (cb[:-1] + cb[1:]))


def prod_params(d: int, bits: int, *, seed: Optional[int] = None, grid_size: int = 16385,
                max_iter: int = 200, rotation=None, projection=None) -> ProdParams:
    """Constants of ``TurboQuantProd.__init__`` (_quant.py:260-292): the MSE
    stage has max(bits-1, 1) bits (:277) and the sketch uses seed+1 (:283)."""
    if bits < 1:
        raise ValueError("bits must be >= 1")
    inner = mse_params(d, max(bits - 1, 1), seed=seed, grid_size=grid_size,
                       max_iter=max_iter, rotation=rotation)
    if projection is not None:
        proj = np.asarray(projection, dtype=np.float32)
    else:
        proj = seeded_projection(int(d), None if seed is None else seed + 1)
    if proj.shape != (int(d), int(d)):
        raise ValueError(f"projection must have shape {(int(d), int(d))}, got {proj.shape}")
    return ProdParams(int(d), int(bits), inner, proj)


# --------------------------------------------------------------------------
# array path
# --------------------------------------------------------------------------
def _rows(a: np.ndarray, d: int) -> Tuple[np.ndarray, Tuple[int, ...]]:
    """(..., d) -> (N, d) plus the leading shape (_quant.py:43-52)."""
    if a.ndim == 0 or a.shape[-1] != d:
        raise ValueError(f"expected input with trailing dimension {d}, got shape {a.shape}")
    return a.reshape(-1, d), a.shape[:-1]


def unit_rows(x: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Row norms and unit rows; rows whose norm is not > 0 become zeros
    (_quant.py:224-230)."""
    n = np.linalg.norm(x, axis=1)
    ok = n > 0
    u = x / np.where(ok, n, np.ones_like(n))[:, None]
    return np.where(ok[:, None], u, np.zeros_like(u)), n


def rotate_and_search(p: MSEParams, u: np.ndarray) -> np.ndarray:
    """codes = #boundaries strictly below (u R^T) (_quant.py:232-236)."""
    y = u @ p.rotation.T
    return np.searchsorted(p.boundaries, y, side="left").astype(np.uint8 if p.bits <= 8 else np.uint16)


def gather_and_unrotate(p: MSEParams, codes: np.ndarray) -> np.ndarray:
    """codebook[codes] R (_quant.py:238-242)."""
    return p.codebook[codes] @ p.rotation


def mse_quantize(p: MSEParams, vectors: np.ndarray):
    """``TurboQuantMSE.quantize`` (_quant.py:244-249) -> (codes, norms, prefix)."""
    x, prefix = _rows(np.asarray(vectors), p.d)
    u, n = unit_rows(x)
    return rotate_and_search(p, u), n, prefix


def mse_dequantize(p: MSEParams, codes, norms, prefix) -> np.ndarray:
    """``TurboQuantMSE.dequantize`` (_quant.py:251-254)."""
    r = gather_and_unrotate(p, codes) * norms[:, None]
    return r.reshape(tuple(prefix) + (r.shape[-1],))


def prod_quantize(p: ProdParams, vectors: np.ndarray):
    """``TurboQuantProd.quantize`` (_quant.py:297-315) ->
    (codes, qjl(+1/-1 int8), residual_norms, norms, prefix)."""
    x, prefix = _rows(np.asarray(vectors), p.d)
    u, n = unit_rows(x)
    codes = rotate_and_search(p.mse, u)
    resid = u - gather_and_unrotate(p.mse, codes)
    rn = np.linalg.norm(resid, axis=1)
    z = resid @ p.projection.T
    one = np.ones_like(z, dtype=np.int8)
    return codes, np.where(z >= 0, one, -one), rn, n, prefix


def prod_dequantize(p: ProdParams, codes, qjl, residual_norms, norms, prefix) -> np.ndarray:
    """``TurboQuantProd.dequantize`` (_quant.py:317-332)."""
    corr = (qjl @ p.projection) * (_ALPHA_NUM / p.d)
    u = gather_and_unrotate(p.mse, codes) + corr * residual_norms[:, None]
    r = u * norms[:, None]
    return r.reshape(tuple(prefix) + (r.shape[-1],))


def prod_attention_score(p: ProdParams, query, codes, qjl, residual_norms, norms, prefix) -> np.ndarray:
    """``TurboQuantProd.attention_score`` (_quant.py:334-358): one query row
    broadcast over all keys, or one query row per key."""
    q, q_prefix = _rows(np.asarray(query), p.d)
    n_keys = codes.shape[0]
    single = q.shape[0] == 1
    if single and n_keys > 1:
        q = np.broadcast_to(q, (n_keys, p.d))
        q_prefix = prefix
    elif q.shape[0] != n_keys:
        raise ValueError(f"query batch size {q.shape[0]} does not match encoding batch size {n_keys}")
    s1 = np.sum(q * gather_and_unrotate(p.mse, codes), axis=1)
    s2 = _ALPHA_NUM / p.d * residual_norms * np.sum((q @ p.projection.T) * qjl, axis=1)
    out = norms * (s1 + s2)
    return out.reshape(tuple(q_prefix) if q.shape[0] != 1 else tuple(prefix))


# --------------------------------------------------------------------------
# caller side of attention_score: scale -> softmax -> weighted sum of values
# --------------------------------------------------------------------------
def softmax_rows(x: np.ndarray) -> np.ndarray:
    """``Tensor.softmax`` over the last axis (_core.py:1286-1291)."""
    shifted = x - np.max(x, axis=-1, keepdims=True)
    e = np.exp(shifted)
    return e / np.sum(e, axis=-1, keepdims=True)


def decode_attention(kp: ProdParams, vp: MSEParams, queries, key_encoding, value_codes, value_norms,
                     scale: Optional[float] = None) -> np.ndarray:
    """``scaled_dot_product_attention`` (_core.py:1606-1683; no mask, no dropout) for one group of keys, with
    ``query @ key.T`` replaced by ``TurboQuantProd.attention_score`` over the packed keys (one broadcast call
    per query, as the reference's users loop it) and ``value`` by ``TurboQuantMSE.dequantize`` of the packed
    values.  queries: (Q, d); key_encoding: (codes, qjl, residual_norms, norms) of N keys; returns (Q, d)."""
    codes, qjl, rn, norms = key_encoding
    q = np.asarray(queries, dtype=np.float32).reshape(-1, kp.d)
    n = codes.shape[0]
    scale = scale or (kp.d ** -0.5)
    scores = np.stack([prod_attention_score(kp, q[a], codes, qjl, rn, norms, (n,)) for a in range(q.shape[0])])
    scores = scores * np.float32(scale)
    weights = softmax_rows(scores)
    values = mse_dequantize(vp, value_codes, value_norms, (n,))
    return weights @ values
