"""Decode / prefill runner for a dense Qwen3-shaped Q4_K model.

Host mirror of the scheduling slice of the reference text pipeline
(``decodeStep`` src/inference/pipelines/text/generator-steps.js:588,
``processLayerGPU`` layer.js:682, weight upload ``loadQ4KFused``
src/loader/tensors/tensor-loader.js:540-558).  The schedule itself (kernel
order, CUDA-graph capture, KV allocation) lives in the C++ library; this class
only feeds it weights and token ids.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import _lib as L
from . import synthetic
from .ops import Device

_Q4K_IDS = {"wq": L.W_Q, "wk": L.W_K, "wv": L.W_V, "wo": L.W_O, "wgate": L.W_GATE, "wup": L.W_UP, "wdown": L.W_DOWN}
_NORM_IDS = {"in_norm": L.W_IN_NORM, "post_norm": L.W_POST_NORM, "q_norm": L.W_Q_NORM, "k_norm": L.W_K_NORM}


class DecoderModel:
    def __init__(self, device: Device, cfg: dict, max_seq: int, max_batch: int = 1, tp_rank: int = 0, tp_size: int = 1):
        self.device, self.cfg = device, dict(cfg)
        self.cfg["max_seq"] = max_seq
        c = L.ModelCfg(cfg["n_layers"], cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["inter"],
                       cfg["vocab"], max_seq, cfg.get("eps", 1e-6), cfg.get("rope_theta", 1e6), max_batch, tp_rank, tp_size)
        h = C.c_void_p()
        device.check(device.lib.dp_model_create(device.h, C.byref(c), C.byref(h)))
        self.h = h
        self.max_batch, self.tp_rank, self.tp_size = max_batch, tp_rank, tp_size

    # -- weights ------------------------------------------------------------------
    def load_layer(self, layer: int, weights: dict):
        shapes = synthetic.layer_shapes(self.cfg)
        lib, dev = self.device.lib, self.device
        for name, wid in _Q4K_IDS.items():
            a = np.ascontiguousarray(weights[name], np.uint8)
            n, k = shapes[name]
            dev.check(lib.dp_model_load_q4k(self.h, layer, wid, a.ctypes.data_as(C.c_void_p), n, k))
        for name, wid in _NORM_IDS.items():
            a = np.ascontiguousarray(weights[name], np.float32)
            dev.check(lib.dp_model_load_norm(self.h, layer, wid, a.ctypes.data_as(C.c_void_p), a.size))

    def load_embed(self, rows_f16: np.ndarray, row0: int = 0):
        a = np.ascontiguousarray(rows_f16)
        self.device.check(self.device.lib.dp_model_load_embed(self.h, a.ctypes.data_as(C.c_void_p), row0, a.shape[0]))

    def load_lm_head(self, rows_f16: np.ndarray, row0: int = 0):
        a = np.ascontiguousarray(rows_f16)
        self.device.check(self.device.lib.dp_model_load_lm_head(self.h, a.ctypes.data_as(C.c_void_p), row0, a.shape[0]))

    def load_final_norm(self, w: np.ndarray):
        a = np.ascontiguousarray(w, np.float32)
        self.device.check(self.device.lib.dp_model_load_final_norm(self.h, a.ctypes.data_as(C.c_void_p), a.size))

    def load_all(self, weights: dict):
        for i, lw in enumerate(weights["layers"]):
            self.load_layer(i, lw)
        self.load_embed(weights["embed"])
        self.load_lm_head(weights["lm_head"])
        self.load_final_norm(weights["final_norm"])

    def load_synthetic(self, seed: int = synthetic.DEFAULT_SEED, chunk_rows: int = 16384):
        """Generate and upload the seeded random-init model layer by layer (bounded host memory)."""
        for i in range(self.cfg["n_layers"]):
            self.load_layer(i, synthetic.make_layer_weights(self.cfg, i, seed))
        v = self.cfg["vocab"]
        shard = v // self.tp_size
        for r0 in range(0, v, chunk_rows):
            rows = min(chunk_rows, v - r0)
            self.load_embed(synthetic.make_embed(self.cfg, seed, r0, rows), r0)
            lo, hi = max(r0, shard * self.tp_rank), min(r0 + rows, shard * (self.tp_rank + 1))
            if hi > lo:
                self.load_lm_head(synthetic.make_lm_head(self.cfg, seed, lo, hi - lo), lo)
        self.load_final_norm(synthetic.make_final_norm(self.cfg, seed))

    # -- running ---------------------------------------------------------------------
    def reset(self):
        self.device.check(self.device.lib.dp_model_reset(self.h))

    def prefill(self, tokens, seq: int = 0) -> int:
        t = np.ascontiguousarray(tokens, np.int32)
        nxt = C.c_int32()
        self.device.check(self.device.lib.dp_model_prefill(self.h, seq, t.ctypes.data_as(C.c_void_p), t.size, C.byref(nxt)))
        return int(nxt.value)

    def decode(self, first_tokens, steps: int) -> np.ndarray:
        """Greedy decode; returns int32 [steps, batch]."""
        ft = np.ascontiguousarray(np.atleast_1d(first_tokens), np.int32)
        out = np.empty((steps, ft.size), np.int32)
        self.device.check(self.device.lib.dp_model_decode(self.h, ft.size, ft.ctypes.data_as(C.c_void_p), steps,
                                                          out.ctypes.data_as(C.c_void_p)))
        return out

    @property
    def last_decode_ms(self) -> float:
        return float(self.device.lib.dp_model_last_decode_ms(self.h))

    @property
    def weight_bytes(self) -> int:
        return int(self.device.lib.dp_model_weight_bytes(self.h))

    def seq_len(self, seq: int = 0) -> int:
        return int(self.device.lib.dp_model_seq_len(self.h, seq))

    def read_logits(self, n: Optional[int] = None) -> np.ndarray:
        n = n or self.cfg["vocab"] // self.tp_size
        out = np.empty(n, np.float32)
        self.device.check(self.device.lib.dp_model_read_logits(self.h, out.ctypes.data_as(C.c_void_p), n))
        return out

    def read_hidden(self, rows: int = 1) -> np.ndarray:
        out = np.empty((rows, self.cfg["hidden"]), np.float32)
        self.device.check(self.device.lib.dp_model_read_hidden(self.h, out.ctypes.data_as(C.c_void_p), out.size))
        return out

    def set_allreduce_mode(self, mode: int):
        """0: NCCL allreduce + residual add; 1: one-shot peer-memory exchange fused with the residual
        add and the next RMSNorm (single-token decode; needs tp.export_exchange + tp.attach_exchange)."""
        self.device.check(self.device.lib.dp_model_set_allreduce_mode(self.h, mode))

    def bench_gemv(self, reps: int = 1) -> dict:
        """Device time of all Q4_K decode GEMVs of the model, back to back (CUDA events)."""
        ms, n, b = C.c_double(), C.c_uint64(), C.c_uint64()
        self.device.check(self.device.lib.dp_model_bench_gemv(self.h, reps, C.byref(ms), C.byref(n), C.byref(b)))
        return {"ms": ms.value, "launches": int(n.value), "bytes": int(b.value)}

    def destroy(self):
        if self.h:
            self.device.lib.dp_model_destroy(self.h)
            self.h = None
