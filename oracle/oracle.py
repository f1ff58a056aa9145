"""ctypes/numpy front end of the CPU oracle (``doppler_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
benchmark's CPU-baseline leg.  The shipped package never imports this module.

The shared object is built on demand with ``make`` (gcc) next to this file.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")

QK_K = 256
Q4K_BLOCK_BYTES = 144


def build(force: bool = False) -> str:
    src = [os.path.join(_HERE, f) for f in ("doppler_oracle.c", "doppler_oracle.h")]
    stale = (not os.path.exists(_SO)) or any(os.path.getmtime(s) > os.path.getmtime(_SO) for s in src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _declare(_lib)
    return _lib


def _p(a, t=None):
    return a.ctypes.data_as(C.c_void_p)


class ModelCfg(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim",
                                        "inter", "vocab", "max_seq")] + [("eps", C.c_float), ("rope_theta", C.c_float)]


class LayerWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown",
                                           "in_norm", "post_norm", "q_norm", "k_norm")]


def _declare(L):
    vp, sz, u32, u64, dbl, flt, i32 = C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint64, C.c_double, C.c_float, C.c_int
    sig = {
        "orc_f32_to_f16_trunc": (C.c_uint16, [dbl]),
        "orc_f16_to_f32": (flt, [C.c_uint16]),
        "orc_f32_to_f16_kvhost": (C.c_uint16, [flt]),
        "orc_f32_to_f16_rne": (C.c_uint16, [flt]),
        "orc_lcg_test_data": (None, [vp, sz, u32, dbl, dbl]),
        "orc_prng1664525": (None, [vp, sz, u32]),
        "orc_q4k_quantize_block": (None, [vp, i32, vp]),
        "orc_q4k_quantize_flat": (sz, [vp, sz, vp]),
        "orc_q4k_quantize_rowwise": (sz, [vp, sz, sz, vp]),
        "orc_q4k_dequant_block": (None, [vp, vp]),
        "orc_q4k_dequant_flat": (None, [vp, sz, sz, vp]),
        "orc_q4k_dequant_rowwise": (None, [vp, sz, sz, vp]),
        "orc_q4k_decode_header": (None, [vp, vp, vp, vp, vp]),
        "orc_q4k_gemv": (None, [vp, sz, sz, vp, flt, vp]),
        "orc_q4k_gemm": (None, [vp, sz, sz, vp, sz, flt, vp]),
        "orc_q4k_gemm_f16_weights": (None, [vp, sz, sz, vp, sz, flt, vp]),
        "orc_f16_gemv": (None, [vp, sz, sz, vp, vp]),
        "orc_attention": (None, [vp, vp, vp, i32, i32, i32, i32, i32, vp, dbl, vp]),
        "orc_attention_f16kv": (None, [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, dbl, vp]),
        "orc_rmsnorm": (None, [vp, vp, i32, i32, dbl, vp]),
        "orc_rope_tables": (None, [dbl, i32, i32, vp, vp]),
        "orc_rope": (None, [vp, vp, vp, i32, i32, i32, i32]),
        "orc_silu_gated": (None, [vp, vp, sz, vp]),
        "orc_silu_gated_clamped": (None, [vp, vp, sz, vp]),
        "orc_residual_add": (None, [vp, vp, sz, flt, vp]),
        "orc_gather_f16": (None, [vp, vp, i32, i32, vp]),
        "orc_argmax": (i32, [vp, i32, i32]),
        "orc_model_create": (vp, [vp, vp, vp, vp, vp]),
        "orc_model_destroy": (None, [vp]),
        "orc_model_reset": (None, [vp]),
        "orc_model_forward": (i32, [vp, vp, i32, vp, vp]),
        "orc_model_seq_len": (i32, [vp]),
        "orc_model_last_hidden": (vp, [vp]),
        "orc_num_threads": (i32, []),
        "orc_set_num_threads": (None, [i32]),
        "orc_synth_key": (u64, [u64, u64]),
        "orc_synth_normal_f32": (None, [u64, u64, sz, flt, flt, vp]),
        "orc_synth_normal_f16": (None, [u64, u64, sz, flt, vp]),
        "orc_synth_q4k_blocks": (None, [u64, u64, sz, vp]),
        "orc_synth_tokens": (None, [u64, sz, i32, vp]),
        "orc_model_fill_kv": (i32, [vp, i32, u64]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ---- f16 ---------------------------------------------------------------------
def f32_to_f16_trunc(v: float) -> int:
    return lib().orc_f32_to_f16_trunc(float(v))


def f16_to_f32(h: int) -> float:
    return lib().orc_f16_to_f32(int(h))


def f32_to_f16_kvhost(v: float) -> int:
    return lib().orc_f32_to_f16_kvhost(float(v))


def f32_to_f16_rne(v: float) -> int:
    return lib().orc_f32_to_f16_rne(float(v))


# ---- harness data --------------------------------------------------------------
def lcg_test_data(n: int, seed: int = 42, lo: float = -1.0, hi: float = 1.0) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().orc_lcg_test_data(_p(out), n, seed, lo, hi)
    return out


def prng1664525(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, np.float64)
    lib().orc_prng1664525(_p(out), n, seed)
    return out


# ---- Q4_K ----------------------------------------------------------------------
def q4k_quantize_block(data, valid_len: int = QK_K) -> np.ndarray:
    d = np.zeros(QK_K, np.float32)
    src = _f32(data)
    d[: min(QK_K, src.size)] = src[:QK_K]
    out = np.empty(Q4K_BLOCK_BYTES, np.uint8)
    lib().orc_q4k_quantize_block(_p(d), valid_len, _p(out))
    return out


def q4k_quantize_flat(data) -> np.ndarray:
    d = _f32(data).ravel()
    nb = (d.size + QK_K - 1) // QK_K
    out = np.empty(nb * Q4K_BLOCK_BYTES, np.uint8)
    lib().orc_q4k_quantize_flat(_p(d), d.size, _p(out))
    return out


def q4k_quantize_rowwise(data, rows: int, cols: int) -> np.ndarray:
    d = _f32(data).ravel()
    assert d.size == rows * cols
    bpr = (cols + QK_K - 1) // QK_K
    out = np.empty(rows * bpr * Q4K_BLOCK_BYTES, np.uint8)
    lib().orc_q4k_quantize_rowwise(_p(d), rows, cols, _p(out))
    return out


def q4k_dequant_block(block) -> np.ndarray:
    b = np.ascontiguousarray(block, np.uint8)
    out = np.empty(QK_K, np.float32)
    lib().orc_q4k_dequant_block(_p(b), _p(out))
    return out


def q4k_dequant_flat(q, n: int) -> np.ndarray:
    b = np.ascontiguousarray(q, np.uint8)
    out = np.zeros(n, np.float32)
    lib().orc_q4k_dequant_flat(_p(b), b.size // Q4K_BLOCK_BYTES, n, _p(out))
    return out


def q4k_dequant_rowwise(q, rows: int, cols: int) -> np.ndarray:
    b = np.ascontiguousarray(q, np.uint8)
    out = np.zeros((rows, cols), np.float32)
    lib().orc_q4k_dequant_rowwise(_p(b), rows, cols, _p(out))
    return out


def q4k_decode_header(block):
    b = np.ascontiguousarray(block, np.uint8)
    sc, mn = np.empty(8, np.uint8), np.empty(8, np.uint8)
    d, dm = C.c_float(), C.c_float()
    lib().orc_q4k_decode_header(_p(b), _p(sc), _p(mn), C.byref(d), C.byref(dm))
    return sc, mn, d.value, dm.value


def q4k_gemv(w, rows: int, cols: int, x, alpha: float = 1.0) -> np.ndarray:
    wb, xv = np.ascontiguousarray(w, np.uint8), _f32(x)
    y = np.empty(rows, np.float32)
    lib().orc_q4k_gemv(_p(wb), rows, cols, _p(xv), alpha, _p(y))
    return y


def q4k_gemm(w, n: int, k: int, a, m: int, alpha: float = 1.0) -> np.ndarray:
    wb, av = np.ascontiguousarray(w, np.uint8), _f32(a)
    c = np.empty((m, n), np.float32)
    lib().orc_q4k_gemm(_p(wb), n, k, _p(av), m, alpha, _p(c))
    return c


def q4k_gemm_f16_weights(w, n: int, k: int, a, m: int, alpha: float = 1.0) -> np.ndarray:
    """The opt-in tiled prefill kernel's product: dequantised weights rounded to f16 first."""
    wb, av = np.ascontiguousarray(w, np.uint8), _f32(a)
    c = np.empty((m, n), np.float32)
    lib().orc_q4k_gemm_f16_weights(_p(wb), n, k, _p(av), m, alpha, _p(c))
    return c


def f16_gemv(w_f16, rows: int, cols: int, x) -> np.ndarray:
    wv, xv = np.ascontiguousarray(w_f16).view(np.uint16), _f32(x)
    y = np.empty(rows, np.float32)
    lib().orc_f16_gemv(_p(wv), rows, cols, _p(xv), _p(y))
    return y


# ---- attention -------------------------------------------------------------------
def attention(q, k, v, seq_len, kv_len, num_heads, num_kv_heads, head_dim, mask=None, scale=-1.0):
    qv, kv_, vv = _f32(q), _f32(k), _f32(v)
    out = np.empty(seq_len * num_heads * head_dim, np.float32)
    mp = _p(_f32(mask)) if mask is not None else None
    lib().orc_attention(_p(qv), _p(kv_), _p(vv), seq_len, kv_len, num_heads, num_kv_heads, head_dim, mp, scale, _p(out))
    return out


def attention_f16kv(q, k_f16, v_f16, seq_len, kv_len, num_heads, num_kv_heads, head_dim,
                    causal=True, start_pos=0, scale=-1.0):
    qv = _f32(q)
    kk = np.ascontiguousarray(k_f16).view(np.uint16)
    vv = np.ascontiguousarray(v_f16).view(np.uint16)
    out = np.empty(seq_len * num_heads * head_dim, np.float32)
    lib().orc_attention_f16kv(_p(qv), _p(kk), _p(vv), seq_len, kv_len, num_heads, num_kv_heads, head_dim,
                              1 if causal else 0, start_pos, scale, _p(out))
    return out


# ---- small ops ---------------------------------------------------------------------
def rmsnorm(x, w, rows, size, eps=1e-6):
    xv, wv = _f32(x), _f32(w)
    y = np.empty(rows * size, np.float32)
    lib().orc_rmsnorm(_p(xv), _p(wv), rows, size, eps, _p(y))
    return y


def rope_tables(theta, rotary_dim, max_seq):
    c = np.empty((max_seq, rotary_dim // 2), np.float32)
    s = np.empty((max_seq, rotary_dim // 2), np.float32)
    lib().orc_rope_tables(theta, rotary_dim, max_seq, _p(c), _p(s))
    return c, s


def rope(x, cos_t, sin_t, seq_len, num_heads, head_dim, start_pos=0):
    xv = _f32(x).copy()
    lib().orc_rope(_p(xv), _p(_f32(cos_t)), _p(_f32(sin_t)), seq_len, num_heads, head_dim, start_pos)
    return xv


def silu_gated(gate, up, clamped=False):
    g, u = _f32(gate), _f32(up)
    out = np.empty(g.size, np.float32)
    (lib().orc_silu_gated_clamped if clamped else lib().orc_silu_gated)(_p(g), _p(u), g.size, _p(out))
    return out


def residual_add(a, b, scale=1.0):
    av, bv = _f32(a), _f32(b)
    out = np.empty(av.size, np.float32)
    lib().orc_residual_add(_p(av), _p(bv), av.size, scale, _p(out))
    return out


def gather_f16(table_f16, ids, hidden):
    t = np.ascontiguousarray(table_f16).view(np.uint16)
    i = np.ascontiguousarray(ids, np.int32)
    out = np.empty((i.size, hidden), np.float32)
    lib().orc_gather_f16(_p(t), _p(i), i.size, hidden, _p(out))
    return out


def argmax(logits, pad_id=-1):
    lv = _f32(logits)
    return lib().orc_argmax(_p(lv), lv.size, pad_id)


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(int(n))


class SynthBackend:
    """The oracle's restatement of the library's seeded input generators, shaped like the handle
    doppler_b200.synthetic.Generator wraps (same five primitives), so the CPU baseline can build
    the benchmark model without loading the CUDA library."""

    def dp_synth_key(self, seed, tensor_id):
        return lib().orc_synth_key(seed, tensor_id)

    def dp_synth_normal_f32(self, key, first, n, sigma, mean, out):
        lib().orc_synth_normal_f32(key, first, n, sigma, mean, out)

    def dp_synth_normal_f16(self, key, first, n, sigma, out):
        lib().orc_synth_normal_f16(key, first, n, sigma, out)

    def dp_synth_q4k_blocks(self, key, first_block, n_blocks, out):
        lib().orc_synth_q4k_blocks(key, first_block, n_blocks, out)

    def dp_synth_tokens(self, key, n, vocab, out):
        lib().orc_synth_tokens(key, n, vocab, out)


def num_threads() -> int:
    return lib().orc_num_threads()


# ---- whole model --------------------------------------------------------------------------
class OracleModel:
    """Dense Qwen3-shaped decoder evaluated by the oracle.  ``weights`` is the dict
    produced by ``doppler_b200.synthetic.make_model_weights`` (numpy arrays)."""

    def __init__(self, cfg: dict, weights: dict):
        self._keep = weights
        c = ModelCfg(cfg["n_layers"], cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"],
                     cfg["inter"], cfg["vocab"], cfg["max_seq"], cfg.get("eps", 1e-6), cfg.get("rope_theta", 1e6))
        arr = (LayerWeights * cfg["n_layers"])()
        for i, lw in enumerate(weights["layers"]):
            for name in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown", "in_norm", "post_norm", "q_norm", "k_norm"):
                setattr(arr[i], name, lw[name].ctypes.data)
        self.cfg = cfg
        self._h = lib().orc_model_create(C.byref(c), arr, _p(weights["embed"].view(np.uint16)),
                                         _p(weights["lm_head"].view(np.uint16)), _p(weights["final_norm"]))

    def forward(self, tokens, want_logits=False):
        t = np.ascontiguousarray(tokens, np.int32)
        margin = C.c_float()
        logits = np.empty(self.cfg["vocab"], np.float32) if want_logits else None
        tok = lib().orc_model_forward(self._h, _p(t), t.size, C.byref(margin), _p(logits) if want_logits else None)
        if tok < 0:
            raise RuntimeError("oracle model: sequence exceeds max_seq")
        return (tok, margin.value, logits) if want_logits else (tok, margin.value)

    def last_hidden(self, n):
        ptr = lib().orc_model_last_hidden(self._h)
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_float)), shape=(n, self.cfg["hidden"])).copy()

    def reset(self):
        lib().orc_model_reset(self._h)

    def fill_kv(self, n: int, key: int = 1):
        """Benchmark helper: synthetic f16 K/V for positions [0, n), sequence position = n."""
        if lib().orc_model_fill_kv(self._h, n, key) != 0:
            raise RuntimeError("oracle model: context exceeds max_seq")

    def __del__(self):
        try:
            lib().orc_model_destroy(self._h)
        except Exception:
            pass
