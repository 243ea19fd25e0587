"""Parity measures shared by the GPU tests.

Acceptance for discrete outputs: packed codes and QJL signs must equal the reference's except
where the deciding quantity lies within 1e-5 of its decision point, and the overall rate of such
differences must not exceed 1e-6.  For float outputs: 1e-5 relative for norms and
reconstructions, 1e-4 relative for scores; "relative" is taken against the natural scale of the
row (its largest magnitude, or |q||k|/sqrt(d) for scores, which cross zero).
"""
import numpy as np

WINDOW = 1e-5
MAX_FLIP_RATE = 1e-6


def code_flip_report(ours, ref, rotation, boundaries, x):
    """Compare code arrays; returns (flips, flips_outside_window, total)."""
    ours = np.asarray(ours)
    ref = np.asarray(ref)
    assert ours.shape == ref.shape and ours.dtype == ref.dtype
    diff = ours != ref
    flips = int(diff.sum())
    outside = 0
    if flips:
        x64 = x.reshape(-1, x.shape[-1]).astype(np.float64)
        n = np.linalg.norm(x64, axis=1)
        unit = np.where(n[:, None] > 0, x64 / np.where(n > 0, n, 1.0)[:, None], 0.0)
        rot = unit @ rotation.astype(np.float64).T
        rows, cols = np.nonzero(diff)
        dist = np.min(np.abs(rot[rows, cols][:, None] - boundaries.astype(np.float64)[None, :]), axis=1)
        outside = int((dist > WINDOW).sum())
    return flips, outside, ref.size


def sign_flip_report(ours, ref, proj_values=None):
    ours = np.asarray(ours)
    ref = np.asarray(ref)
    assert ours.shape == ref.shape
    diff = ours != ref
    flips = int(diff.sum())
    outside = 0
    if flips and proj_values is not None:
        outside = int((np.abs(proj_values[diff]) > WINDOW).sum())
    return flips, outside, ref.size


def assert_discrete_parity(flips, outside, total, what):
    assert outside == 0, f"{what}: {outside} differences lie outside the {WINDOW} window"
    # small arrays: a single in-window difference must not fail the rate test by itself
    allowed = max(int(np.floor(MAX_FLIP_RATE * total)), 1 if total < 1 / MAX_FLIP_RATE else 0)
    assert flips <= allowed, f"{what}: {flips} differences in {total} (rate {flips / total:.2e})"


def max_rel_rows(ours, ref):
    """max over rows of max|ours - ref| / max|ref| (rows of zeros compare absolutely)."""
    ours = np.asarray(ours, dtype=np.float64).reshape(-1, ref.shape[-1])
    ref2 = np.asarray(ref, dtype=np.float64).reshape(-1, ref.shape[-1])
    scale = np.max(np.abs(ref2), axis=1)
    err = np.max(np.abs(ours - ref2), axis=1)
    return float(np.max(err / np.where(scale > 0, scale, 1.0)))


def max_rel_scalar(ours, ref):
    ours = np.asarray(ours, dtype=np.float64).ravel()
    ref = np.asarray(ref, dtype=np.float64).ravel()
    return float(np.max(np.abs(ours - ref) / np.where(ref != 0, np.abs(ref), 1.0))) if ref.size else 0.0


def max_score_err(ours, ref, q_norms, k_norms, d):
    """max |ours - ref| / (|q| |k| / sqrt(d)) with q_norms, k_norms broadcastable to the scores."""
    ours = np.asarray(ours, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    scale = np.asarray(q_norms, np.float64) * np.asarray(k_norms, np.float64) / np.sqrt(d)
    scale = np.broadcast_to(scale, ref.shape)
    return float(np.max(np.abs(ours - ref) / np.where(scale > 0, scale, 1.0))) if ref.size else 0.0
