"""Shared test helpers: the error metric and device round trips."""
import numpy as np

REL_TOL = 2e-3  # matvec / attention outputs: max relative error against the oracle


def rel_err(got, ref) -> float:
    """max_i |got_i - ref_i| / max(|ref_i|, rms(ref)/8).

    A plain relative error is undefined where an output crosses zero; the floor of one eighth
    of the output RMS keeps the metric relative for ordinary elements and bounds the absolute
    error of near-zero ones (two correct fp32 summation orders already differ there by about
    1e-4 of the RMS)."""
    got = np.asarray(got, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    floor = np.sqrt(np.mean(ref * ref)) / 8.0
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), max(floor, 1e-30))))


def inf_err(got, ref) -> float:
    """max_i |got_i - ref_i| / max_i |ref_i|: never larger than rel_err (whose denominators are
    at most the largest |ref_i|), asserted beside it with a tighter bound so that the slack the
    floor in rel_err gives near-zero outputs is visible."""
    got = np.asarray(got, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    return float(np.max(np.abs(got - ref)) / max(float(np.max(np.abs(ref))), 1e-30))


INF_TOL = 1e-3  # matvec / attention outputs: largest absolute error over the largest |output|
# The reference's D256 split-K attention pair hands its partial outputs from the first record to the
# second as fp16 (Resources/Shaders/attention.metal:1140): every partial carries a 2^-11 relative
# rounding, which for outputs an eighth of the RMS (the floor of rel_err) is up to 8 * 2^-11 = 4e-3
# per block before the blocks are combined.  The pair is therefore held to INF_TOL on the
# largest-output scale and to this looser bound under rel_err.
TWO_PASS_REL_TOL = 8e-3


def ulp_diff_f16(a, b) -> np.ndarray:
    """Distance in fp16 ulps (monotone integer mapping of the bit patterns)."""
    def key(x):
        u = np.asarray(x, np.float16).view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(a) - key(b))


def add_rel_err(got, ref, summand) -> float:
    """Error metric for y = half(half(acc) + residual): where acc and the residual cancel, the
    fp16 rounding of acc (|acc| 2^-11) is large next to |y|, so the error is measured against
    max(|y|, |acc|) with the same floor as rel_err.  summand: the oracle's acc as fp16."""
    got = np.asarray(got, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    acc = np.asarray(summand, np.float64).reshape(-1)
    floor = np.sqrt(np.mean(ref * ref)) / 8.0
    return float(np.max(np.abs(got - ref) / np.maximum(np.maximum(np.abs(ref), np.abs(acc)), max(floor, 1e-30))))
