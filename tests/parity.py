"""Tolerance rules shared by the GPU parity tests.

Per-row predictions: |gpu - ref| <= 1e-5 * |ref| + 1e-6 (float32), NaN and Inf masks
identical.  A row whose float32 reference value is itself not reproducible to that
precision -- the same program evaluated by the oracle on inputs perturbed by one ulp moves
by more than the tolerance -- is ill-conditioned: there the bound is widened to eight times
that observed sensitivity.  Sums of squared errors: 1e-4 relative against the oracle's
float64-accumulated sum, widened the same way by the per-row sensitivity.
"""
import numpy as np

ROW_RTOL, ROW_ATOL = 1e-5, 1e-6
SSE_RTOL = 1e-4


def row_mismatches(gpu, ref, sensitivity=None):
    """Boolean mask of rows that violate the per-row rule."""
    gpu = np.asarray(gpu, dtype=np.float32)
    ref = np.asarray(ref, dtype=np.float32)
    bad = np.isnan(gpu) != np.isnan(ref)
    bad |= np.isinf(gpu) != np.isinf(ref)
    both_inf = np.isinf(gpu) & np.isinf(ref)
    bad |= both_inf & (np.sign(gpu) != np.sign(ref))
    finite = np.isfinite(gpu) & np.isfinite(ref)
    with np.errstate(invalid="ignore", over="ignore"):
        tol = ROW_RTOL * np.abs(ref.astype(np.float64)) + ROW_ATOL
        if sensitivity is not None:
            tol = np.maximum(tol, 8.0 * np.nan_to_num(sensitivity.astype(np.float64), nan=np.inf, posinf=np.inf))
        diff = np.abs(gpu.astype(np.float64) - ref.astype(np.float64))
    bad |= finite & (diff > tol)
    return bad


def sse_mismatches(gpu, ref64, slack=None):
    """Bins violating the SSE rule.  Bins whose slack is infinite (a row changes between finite
    and non-finite under a 2-ulp shift of the math library) are not comparable and are skipped;
    callers bound how many such bins a test may have with ill_conditioned_fraction()."""
    gpu = np.asarray(gpu, dtype=np.float64)
    ref64 = np.asarray(ref64, dtype=np.float64)
    bad = np.isnan(gpu) != np.isnan(ref64)
    # float32 sums overflow to inf where the float64 oracle sum is finite but above FLT_MAX
    ref_inf = np.isinf(ref64) | (np.abs(ref64) > 3.0e38)
    bad |= np.isinf(gpu) != ref_inf
    finite = np.isfinite(gpu) & ~ref_inf & ~np.isnan(ref64)
    with np.errstate(invalid="ignore", over="ignore"):
        tol = SSE_RTOL * np.abs(ref64) + 1e-30
        if slack is not None:
            tol = tol + slack
        bad |= finite & (np.abs(gpu - ref64) > tol)
    if slack is not None:
        bad &= np.isfinite(slack)
    return bad


def ill_conditioned_fraction(slack):
    return float(np.mean(~np.isfinite(slack)))
