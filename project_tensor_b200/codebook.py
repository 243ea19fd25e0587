"""Host-side constants of a TurboQuant quantizer: the Lloyd-Max codebook, the seeded rotation and
the seeded QJL projection.

These are small (at most a few hundred KB), built once per quantizer and uploaded to the GPU as a
plan; they stay on the host by design.  They have to agree with Project-Tensor's
``tensor_gpu_v2/_quant.py`` to the last float32 bit, because the packed codes can only match the
reference's when the decision boundaries and the rotation do:

* codebook: ``_build_lloyd_max_codebook`` (_quant.py:93-138) on the density of
  ``_beta_coordinate_pdf`` (:73-83).  The solver works on a fixed grid and its discretisation is
  part of the result (the codebook is *not* symmetric: for d=128, 4 bits the middle boundary is
  about -6e-5, not 0), so the same grid, weights, starting point, assignment rule
  (``searchsorted(..., side="left")``), empty-cell rules and stopping test are used.  Because the
  grid is sorted, each cell is a contiguous slice of it; summing the slice gives the same float64
  result as the reference's boolean-mask sums (same elements, same order, same pairwise scheme)
  at a fraction of the cost.
* rotation: ``_random_orthogonal_matrix`` (:141-148); projection: ``_random_projection_matrix``
  (:151-153).
"""
from __future__ import annotations

import math
import threading
from typing import Dict, Optional, Tuple

import numpy as np

_cache: Dict[Tuple[int, int, int, int, float], np.ndarray] = {}
_cache_lock = threading.Lock()


def _coordinate_weights(dimension: int, grid_size: int) -> Tuple[np.ndarray, np.ndarray]:
    """Grid on [-1, 1] and trapezoid weights of the density of one coordinate of a point drawn
    uniformly from the unit sphere in ``dimension`` dimensions."""
    if dimension < 2:
        raise ValueError("TurboQuant requires dimension >= 2")
    grid = np.linspace(-1.0, 1.0, grid_size, dtype=np.float64)
    log_norm = (math.lgamma(dimension / 2) - 0.5 * math.log(math.pi)
                - math.lgamma((dimension - 1) / 2))
    pdf = np.exp(log_norm) * np.maximum(0.0, 1.0 - grid * grid) ** (0.5 * (dimension - 3))
    weights = pdf * (grid[1] - grid[0])
    weights[0] *= 0.5
    weights[-1] *= 0.5
    return grid, weights


def _build_lloyd_max_codebook(dimension: int, bits: int, *, grid_size: int = 16385,
                              max_iter: int = 200, tol: float = 1e-8) -> np.ndarray:
    """float64 Lloyd-Max centroids (sorted, inside [-1, 1]); cached per argument tuple."""
    key = (int(dimension), int(bits), int(grid_size), int(max_iter), float(tol))
    with _cache_lock:
        hit = _cache.get(key)
    if hit is not None:
        return hit.copy()

    levels = 1 << bits
    grid, weights = _coordinate_weights(dimension, grid_size)
    moments = grid * weights  # first-moment integrand; elementwise, so slice sums see the same terms

    cdf = np.cumsum(weights)
    targets = np.clip((np.arange(levels, dtype=np.float64) + 0.5) / levels, 0.0, 1.0) * cdf[-1]
    centroids = np.clip(np.sort(np.interp(targets, cdf, grid)), -1.0, 1.0)

    for _ in range(max_iter):
        previous = centroids.copy()
        boundaries = 0.5 * (centroids[:-1] + centroids[1:])
        # grid point g belongs to cell k = #boundaries strictly below g, so cell k starts at the
        # first grid point above boundary k-1
        edges = np.concatenate(([0], np.searchsorted(grid, boundaries, side="right"), [grid_size]))
        for k in range(levels):
            lo, hi = int(edges[k]), int(edges[k + 1])
            mass = weights[lo:hi].sum() if hi > lo else 0.0
            if mass > 0:
                centroids[k] = float(np.sum(moments[lo:hi]) / mass)
            elif k == 0:
                centroids[k] = -1.0
            elif k == levels - 1:
                centroids[k] = 1.0
            else:
                centroids[k] = 0.5 * (centroids[k - 1] + centroids[k + 1])
        centroids = np.clip(np.sort(centroids), -1.0, 1.0)
        if np.max(np.abs(centroids - previous)) < tol:
            break

    with _cache_lock:
        _cache[key] = centroids.copy()
    return centroids


def _random_orthogonal_matrix(dimension: int, seed: Optional[int]) -> np.ndarray:
    """float32 rotation: Q of the QR factorisation of a seeded Gaussian, columns flipped so that
    diag(R) is non-negative."""
    gaussian = np.random.default_rng(seed).standard_normal((dimension, dimension))
    q, r = np.linalg.qr(gaussian)
    flip = np.sign(np.diag(r))
    flip[flip == 0] = 1.0
    return (q * flip).astype(np.float32)


def _random_projection_matrix(dimension: int, seed: Optional[int]) -> np.ndarray:
    """float32 d x d standard-normal QJL sketch."""
    return np.random.default_rng(seed).standard_normal((dimension, dimension)).astype(np.float32)
