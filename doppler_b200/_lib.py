"""ctypes binding of ``libdoppler_b200.so`` (the C ABI in ``include/doppler_b200.h``).

There is no fallback: if the shared library is missing, or no CUDA device can be
opened, importing callers get an exception.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdoppler_b200.so")

# status codes / dtypes of include/doppler_b200.h
OK, ERR_INVALID, ERR_CUDA, ERR_OOM, ERR_UNSUPPORTED, ERR_TIMEOUT, ERR_STATE, ERR_COMM = range(8)
STATUS_NAMES = ["ok", "invalid", "cuda", "oom", "unsupported", "timeout", "state", "comm"]
F32, F16, Q4K, I32 = 0, 1, 2, 3
DTYPE_CODES = {"f32": F32, "f16": F16, "q4k": Q4K, "i32": I32}
DTYPE_NAMES = {v: k for k, v in DTYPE_CODES.items()}
DTYPE_BYTES = {"f32": 4, "f16": 2, "i32": 4}

W_Q, W_K, W_V, W_O, W_GATE, W_UP, W_DOWN, W_IN_NORM, W_POST_NORM, W_Q_NORM, W_K_NORM = range(11)


class DopplerError(RuntimeError):
    """Raised for every non-OK status (the reference throws ``Error``)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"[{STATUS_NAMES[status] if 0 <= status < 8 else status}] {message}")
        self.status = status


class TensorS(C.Structure):
    _fields_ = [("buf", C.c_void_p), ("offset", C.c_size_t), ("dtype", C.c_int), ("ndim", C.c_int),
                ("shape", C.c_int64 * 4)]


class WeightS(C.Structure):
    _fields_ = [("buf", C.c_void_p), ("offset", C.c_size_t), ("dtype", C.c_int), ("layout", C.c_int),
                ("shape", C.c_int64 * 2)]


class MatmulOpts(C.Structure):
    _fields_ = [("alpha", C.c_float), ("out_dtype", C.c_int), ("a_off", C.c_size_t), ("b_off", C.c_size_t),
                ("c_off", C.c_size_t), ("out_buf", C.c_void_p), ("transpose_b", C.c_int), ("exact_weights", C.c_int), ("f16_weights", C.c_int)]


class AttnOpts(C.Structure):
    _fields_ = [("seq_len", C.c_int), ("kv_len", C.c_int), ("num_kv_heads", C.c_int), ("scale", C.c_float),
                ("causal", C.c_int), ("start_pos", C.c_int), ("sliding_window", C.c_int), ("attn_softcap", C.c_float),
                ("kv_start", C.c_int), ("batch", C.c_int), ("kv_batch_stride", C.c_size_t), ("kv_lens", C.c_void_p),
                ("out_buf", C.c_void_p)]


class RmsNormOpts(C.Structure):
    _fields_ = [("batch_size", C.c_int), ("hidden_size", C.c_int), ("residual", C.POINTER(TensorS)),
                ("pre_residual", C.c_int), ("residual_sum_output", C.c_void_p), ("weight_offset", C.c_int),
                ("output_scale", C.c_float), ("out_buf", C.c_void_p)]


class FfnOpts(C.Structure):
    _fields_ = [("batch_size", C.c_int), ("alpha", C.c_float), ("swiglu_limit", C.c_float), ("out_buf", C.c_void_p)]


class RopeOpts(C.Structure):
    _fields_ = [("num_heads", C.c_int), ("head_dim", C.c_int), ("rotary_dim", C.c_int), ("pair_span_dim", C.c_int),
                ("interleaved", C.c_int), ("start_pos", C.c_int)]


class PoolStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("allocations", "reuses", "releases", "bytes_allocated", "bytes_in_use",
                                          "bytes_pooled", "peak_bytes_allocated")]


class ModelCfg(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "inter", "vocab",
                                        "max_seq")] + [("eps", C.c_float), ("rope_theta", C.c_float),
                                                       ("max_batch", C.c_int), ("tp_rank", C.c_int), ("tp_size", C.c_int)]


_vp, _sz, _i, _f, _u32, _u64, _dbl = C.c_void_p, C.c_size_t, C.c_int, C.c_float, C.c_uint32, C.c_uint64, C.c_double
_T = C.POINTER(TensorS)

# name -> (restype, argtypes); every symbol declared in include/doppler_b200.h
SIGNATURES = {
    "dp_ctx_create": (_i, [_i, C.POINTER(_vp)]),
    "dp_ctx_destroy": (None, [_vp]),
    "dp_last_error": (C.c_char_p, [_vp]),
    "dp_ctx_sync": (_i, [_vp]),
    "dp_ctx_stream": (_vp, [_vp]),
    "dp_ctx_device": (_i, [_vp]),
    "dp_ctx_launch_count": (_u64, [_vp]),
    "dp_version": (C.c_char_p, []),
    "dp_buf_acquire": (_i, [_vp, _sz, C.c_char_p, C.POINTER(_vp)]),
    "dp_buf_release": (_i, [_vp, _vp]),
    "dp_buf_upload": (_i, [_vp, _vp, _vp, _sz, _sz]),
    "dp_buf_read": (_i, [_vp, _vp, _vp, _sz, _sz]),
    "dp_buf_fill": (_i, [_vp, _vp, _i, _sz, _sz]),
    "dp_buf_device_ptr": (_vp, [_vp]),
    "dp_buf_size": (_sz, [_vp]),
    "dp_buf_capacity": (_sz, [_vp]),
    "dp_pool_bucket_size": (_sz, [_sz]),
    "dp_pool_get_stats": (_i, [_vp, C.POINTER(PoolStats)]),
    "dp_pool_trim": (_i, [_vp]),
    "dp_recorder_begin": (_i, [_vp, C.c_char_p, _i, C.POINTER(_vp)]),
    "dp_recorder_track_temporary": (_i, [_vp, _vp]),
    "dp_recorder_submit": (_i, [_vp]),
    "dp_recorder_submit_and_wait": (_i, [_vp]),
    "dp_recorder_abort": (_i, [_vp]),
    "dp_recorder_finish_graph": (_i, [_vp, C.POINTER(_vp)]),
    "dp_graph_launch": (_i, [_vp]),
    "dp_ctx_set_wait_limit": (_i, [_vp, C.c_uint]),
    "dp_tp_init_loopback": (_i, [_vp, _i, _i]),
    "dp_graph_launch_timed": (_i, [_vp, _i, C.POINTER(_dbl)]),
    "dp_graph_destroy": (None, [_vp]),
    "dp_recorder_op_count": (_u32, [_vp]),
    "dp_matmul_opts_default": (None, [C.POINTER(MatmulOpts)]),
    "dp_matmul": (_i, [_vp, _vp, _T, C.POINTER(WeightS), _i, _i, _i, C.POINTER(MatmulOpts), _T]),
    "dp_dequant_q4k": (_i, [_vp, _vp, _vp, _sz, _u32, _i, _sz, _vp, _T]),
    "dp_dequant_q4k_rowwise": (_i, [_vp, _vp, _vp, _sz, _i, _i, _i, _vp, _T]),
    "dp_attn_opts_default": (None, [C.POINTER(AttnOpts)]),
    "dp_attention": (_i, [_vp, _vp, _T, _T, _T, _i, _i, C.POINTER(AttnOpts), _T]),
    "dp_attention_decode_static": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _sz, _f]),
    "dp_attention_decode_static_error": (C.c_char_p, []),
    "dp_attention_decode_static_max_scratch": (_sz, []),
    "dp_rmsnorm_opts_default": (None, [C.POINTER(RmsNormOpts)]),
    "dp_rmsnorm": (_i, [_vp, _vp, _T, _T, _f, C.POINTER(RmsNormOpts), _T]),
    "dp_rmsnorm_qk": (_i, [_vp, _vp, _T, _T, _T, _T, _i, _i, _i, _f, _i]),
    "dp_rope": (_i, [_vp, _vp, _T, _T, _T, _i, C.POINTER(RopeOpts)]),
    "dp_rope_tables": (_i, [_dbl, _i, _i, _vp, _vp]),
    "dp_silu_mul": (_i, [_vp, _vp, _T, _T, _sz, _f, _vp, _T]),
    "dp_residual_add": (_i, [_vp, _vp, _T, _T, _sz, _f, _vp, _T]),
    "dp_gather_f16": (_i, [_vp, _vp, _T, _T, _i, _i, _vp, _T]),
    "dp_kv_write_f32_to_f16": (_i, [_vp, _vp, _T, _vp, _sz, _sz]),
    "dp_argmax": (_i, [_vp, _vp, _T, _i, _i, _vp, _i]),
    "dp_quantize_q4k": (_i, [_vp, _vp, _T, C.c_int64, C.c_int64, _i, _vp, C.POINTER(WeightS)]),
    "dp_ffn_opts_default": (None, [C.POINTER(FfnOpts)]),
    "dp_fused_ffn": (_i, [_vp, _vp, _T, C.POINTER(WeightS), C.POINTER(WeightS), _i, _i, C.POINTER(FfnOpts), _T]),
    "dp_matmul_residual": (_i, [_vp, _vp, _T, C.POINTER(WeightS), _T, _i, _i, _f, _vp, _T]),
    "dp_matmul_rmsnorm": (_i, [_vp, _vp, _T, C.POINTER(WeightS), _T, _i, _i, _f, _T, _i, _vp, _T]),
    "dp_lm_head_argmax": (_i, [_vp, _vp, _T, C.POINTER(WeightS), _i, _i, _i, _vp, _i]),
    "dp_kv_cache_create": (_i, [_vp, _i, _i, _i, _i, _i, C.POINTER(_vp)]),
    "dp_kv_cache_destroy": (None, [_vp]),
    "dp_kv_layer": (_i, [_vp, _i, C.POINTER(_vp), C.POINTER(_vp)]),
    "dp_kv_seq_len": (_i, [_vp]),
    "dp_kv_set_seq_len": (_i, [_vp, _i]),
    "dp_kv_truncate": (_i, [_vp, _i]),
    "dp_kv_clone": (_i, [_vp, C.POINTER(_vp)]),
    "dp_kv_bytes": (_sz, [_vp]),
    "dp_model_create": (_i, [_vp, C.POINTER(ModelCfg), C.POINTER(_vp)]),
    "dp_model_destroy": (None, [_vp]),
    "dp_model_load_q4k": (_i, [_vp, _i, _i, _vp, _i, _i]),
    "dp_model_load_norm": (_i, [_vp, _i, _i, _vp, _i]),
    "dp_model_load_final_norm": (_i, [_vp, _vp, _i]),
    "dp_model_load_embed": (_i, [_vp, _vp, _i, _i]),
    "dp_model_load_lm_head": (_i, [_vp, _vp, _i, _i]),
    "dp_model_reset": (_i, [_vp]),
    "dp_model_prefill": (_i, [_vp, _i, _vp, _i, C.POINTER(C.c_int32)]),
    "dp_model_decode": (_i, [_vp, _i, _vp, _i, _vp]),
    "dp_model_last_decode_ms": (_dbl, [_vp]),
    "dp_model_read_logits": (_i, [_vp, _vp, _i]),
    "dp_model_read_hidden": (_i, [_vp, _vp, _i]),
    "dp_model_weight_bytes": (_sz, [_vp]),
    "dp_model_seq_len": (_i, [_vp, _i]),
    "dp_model_set_allreduce_mode": (_i, [_vp, _i]),
    "dp_model_bench_gemv": (_i, [_vp, _i, C.POINTER(_dbl), C.POINTER(_u64), C.POINTER(_u64)]),
    "dp_tp_unique_id": (_i, [_vp]),
    "dp_tp_init": (_i, [_vp, _i, _i, _vp]),
    "dp_tp_allreduce_f32": (_i, [_vp, _vp, _vp, _sz, _sz]),
    "dp_tp_ipc_export": (_i, [_vp, _vp]),
    "dp_tp_ipc_attach": (_i, [_vp, _vp]),
    "dp_tp_destroy": (_i, [_vp]),
    "dp_synth_key": (_u64, [_u64, _u64]),
    "dp_synth_normal_f32": (None, [_u64, _u64, _sz, _f, _f, _vp]),
    "dp_synth_normal_f16": (None, [_u64, _u64, _sz, _f, _vp]),
    "dp_synth_q4k_blocks": (None, [_u64, _u64, _sz, _vp]),
    "dp_synth_tokens": (None, [_u64, _sz, _i, _vp]),
}

_lib = None


def load():
    """Load the shared library and declare every entry point.  Raises if the library
    has not been built (``python -m doppler_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m doppler_b200.build` "
                          "(there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
