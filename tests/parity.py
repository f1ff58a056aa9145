"""Parity gates shared by the tests.

Floating-point gate for matmul / attention outputs against the double-accumulate
oracle:  |a - b| <= RTOL*|b| + RTOL*rms(b)  element-wise with RTOL = 1e-3 (f32
accumulation).  The reference's own comparison formula
(tools/lib/q4k-projection-reference.js:211-250) is reported next to it.
"""
import numpy as np

RTOL = 1e-3


def stats(actual, expected):
    a = np.asarray(actual, np.float64).ravel()
    b = np.asarray(expected, np.float64).ravel()
    diff = np.abs(a - b)
    denom = np.maximum(np.maximum(np.abs(a), np.abs(b)), 1e-12)
    rms = float(np.sqrt(np.mean(b * b))) if b.size else 0.0
    cos = float(a @ b / max(np.sqrt((a @ a) * (b @ b)), 1e-30)) if b.size else 1.0
    return {
        "max_abs": float(diff.max()) if b.size else 0.0,
        "max_rel_ref_formula": float((diff / denom).max()) if b.size else 0.0,
        "rmse": float(np.sqrt(np.mean(diff * diff))) if b.size else 0.0,
        "rms_expected": rms,
        "cosine": cos,
        "worst_gate_ratio": float((diff / (RTOL * np.abs(b) + RTOL * rms + 1e-300)).max()) if b.size else 0.0,
    }


def assert_close(actual, expected, what, rtol=RTOL):
    a = np.asarray(actual, np.float64).ravel()
    b = np.asarray(expected, np.float64).ravel()
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    assert np.all(np.isfinite(a)), f"{what}: non-finite output"
    rms = float(np.sqrt(np.mean(b * b))) if b.size else 0.0
    bad = np.abs(a - b) > rtol * np.abs(b) + rtol * rms
    s = stats(a, b)
    print(f"[parity] {what}: " + ", ".join(f"{k}={v:.3e}" for k, v in s.items()))
    assert not bad.any(), f"{what}: {int(bad.sum())}/{b.size} elements outside |a-b| <= {rtol}*|b| + {rtol}*rms(b); {s}"
