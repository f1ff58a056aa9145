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


# ---- the reference's 9B gate_proj receipt (tests/golden/receipt_9b_gate_headers.npz) ----------
def receipt_headers():
    """Block headers of the real [12288, 4096] Q4_K gate_proj tensor the reference's receipt
    reports/qwen-3-5-9b-metal/2026-07-12/layer0-ffn-gate-oracle.json was taken on: f16 d / dmin
    bits, the eight 6-bit scale and min codes of every block, and the sha256 digests the
    reference recorded for ITS decoded scales f32(d*sc) and minima f32(dmin*m)."""
    import os

    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "receipt_9b_gate_headers.npz"))
    return z


def pack_q4k_headers(d_f16_bits, dmin_f16_bits, scale_codes, min_codes, nibble_byte):
    """144-byte super-blocks from header fields, by the layout rule of
    src/converter/quantizer.js:137-153 (reader: fused_matmul_q4.wgsl:65-80): bytes 0-1 d, 2-3 dmin,
    b[4+i] = sc_i | (sc_{i+4} >> 4) << 6, b[8+i] = m_i | (m_{i+4} >> 4) << 6,
    b[12+i] = (sc_{i+4} & 15) | (m_{i+4} & 15) << 4; every quant byte = nibble_byte."""
    nb = d_f16_bits.size
    sc = np.asarray(scale_codes, np.uint8).reshape(nb, 8)
    mn = np.asarray(min_codes, np.uint8).reshape(nb, 8)
    blocks = np.empty((nb, 144), np.uint8)
    blocks[:, 0:2] = np.asarray(d_f16_bits, "<u2").reshape(nb, 1).view(np.uint8)
    blocks[:, 2:4] = np.asarray(dmin_f16_bits, "<u2").reshape(nb, 1).view(np.uint8)
    blocks[:, 4:8] = sc[:, 0:4] | ((sc[:, 4:8] >> 4) << 6)
    blocks[:, 8:12] = mn[:, 0:4] | ((mn[:, 4:8] >> 4) << 6)
    blocks[:, 12:16] = (sc[:, 4:8] & 15) | ((mn[:, 4:8] & 15) << 4)
    blocks[:, 16:] = nibble_byte
    return blocks.reshape(-1)


def receipt_probe_blocks():
    """Two block arrays built from the receipt's headers: with every nibble 0 a dequantised weight
    is 0 - f32(dmin*m) (the negated minimum of its sub-block); with the min codes cleared and every
    nibble 1 it is f32(d*sc)*1 - 0 (the scale).  Returns (blocks_for_minima, blocks_for_scales)."""
    z = receipt_headers()
    zeros = np.zeros_like(z["min_codes"])
    return (pack_q4k_headers(z["d_f16"], z["dmin_f16"], z["scale_codes"], z["min_codes"], 0x00),
            pack_q4k_headers(z["d_f16"], z["dmin_f16"], z["scale_codes"], zeros, 0x11))


def sha256_f32(a):
    import hashlib

    return hashlib.sha256(np.ascontiguousarray(a, "<f4").tobytes()).hexdigest()
