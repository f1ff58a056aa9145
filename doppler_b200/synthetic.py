"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (they stand in for real checkpoints, which are not available offline).

Generation happens in the library's host-side utilities (``dp_synth_*``), counter
based: element i of a tensor depends only on (seed, tensor id, i).  Importing this module
does not load the CUDA library; the first call of a default-generator function does.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L

QK_K = 256
Q4K_BLOCK_BYTES = 144
DEFAULT_SEED = 0xD0771E00

# tensor ids inside one model
_T_EMBED, _T_LMHEAD, _T_FINAL_NORM, _T_TOKENS = 1, 2, 3, 4
_LAYER_BASE = 1000
_W_NAMES = ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown", "in_norm", "post_norm", "q_norm", "k_norm")


class Generator:
    """The five primitive streams, produced by whatever object exports the ``dp_synth_*`` entry
    points: the CUDA library's host utilities by default.  (A benchmark's CPU leg may pass its own
    restatement of the same functions, so that it does not have to load the CUDA library.)"""

    def __init__(self, backend=None):
        self._backend = backend

    @property
    def lib(self):
        if self._backend is None:
            self._backend = L.load()
        return self._backend

    def key(self, seed: int, tensor_id: int) -> int:
        return int(self.lib.dp_synth_key(seed & 0xFFFFFFFFFFFFFFFF, tensor_id))

    def normal_f32(self, k: int, n: int, sigma: float = 1.0, mean: float = 0.0, first: int = 0) -> np.ndarray:
        out = np.empty(n, np.float32)
        self.lib.dp_synth_normal_f32(k, first, n, sigma, mean, out.ctypes.data_as(C.c_void_p))
        return out

    def normal_f16(self, k: int, n: int, sigma: float = 1.0, first: int = 0) -> np.ndarray:
        out = np.empty(n, np.float16)
        self.lib.dp_synth_normal_f16(k, first, n, sigma, out.ctypes.data_as(C.c_void_p))
        return out

    def q4k_blocks(self, k: int, n_blocks: int, first_block: int = 0) -> np.ndarray:
        out = np.empty(n_blocks * Q4K_BLOCK_BYTES, np.uint8)
        self.lib.dp_synth_q4k_blocks(k, first_block, n_blocks, out.ctypes.data_as(C.c_void_p))
        return out

    def tokens(self, k: int, n: int, vocab: int) -> np.ndarray:
        out = np.empty(n, np.int32)
        self.lib.dp_synth_tokens(k, n, vocab, out.ctypes.data_as(C.c_void_p))
        return out


_default = Generator()


def _gen(gen):
    return gen if gen is not None else _default


def key(seed: int, tensor_id: int, gen=None) -> int:
    return _gen(gen).key(seed, tensor_id)


def normal_f32(k: int, n: int, sigma: float = 1.0, mean: float = 0.0, first: int = 0, gen=None) -> np.ndarray:
    return _gen(gen).normal_f32(k, n, sigma, mean, first)


def normal_f16(k: int, n: int, sigma: float = 1.0, first: int = 0, gen=None) -> np.ndarray:
    return _gen(gen).normal_f16(k, n, sigma, first)


def q4k_blocks(k: int, n_blocks: int, first_block: int = 0, gen=None) -> np.ndarray:
    return _gen(gen).q4k_blocks(k, n_blocks, first_block)


def q4k_matrix(k: int, n: int, kdim: int, gen=None) -> np.ndarray:
    """Packed [n, kdim] Q4_K matrix, row-major along K (ceil(kdim/256) blocks per row)."""
    return q4k_blocks(k, n * ((kdim + QK_K - 1) // QK_K), gen=gen)


def tokens(k: int, n: int, vocab: int, gen=None) -> np.ndarray:
    return _gen(gen).tokens(k, n, vocab)


MODEL_CONFIGS = {
    # BASELINE config 3: Qwen3-0.6B-shaped
    "qwen3-0.6b": dict(n_layers=28, hidden=1024, n_heads=16, n_kv_heads=8, head_dim=128, inter=3072, vocab=151936,
                       eps=1e-6, rope_theta=1e6),
    # BASELINE config 4: 9B-shaped
    "9b": dict(n_layers=36, hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128, inter=12288, vocab=151936,
               eps=1e-6, rope_theta=1e6),
    # small shapes for tests
    "tiny": dict(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, inter=512, vocab=512,
                 eps=1e-6, rope_theta=1e6),
    "small": dict(n_layers=3, hidden=1024, n_heads=16, n_kv_heads=8, head_dim=128, inter=3072, vocab=4096,
                  eps=1e-6, rope_theta=1e6),
}


def layer_shapes(cfg: dict) -> dict:
    qd, kvd, h, i = cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"], cfg["hidden"], cfg["inter"]
    return {"wq": (qd, h), "wk": (kvd, h), "wv": (kvd, h), "wo": (h, qd), "wgate": (i, h), "wup": (i, h), "wdown": (h, i)}


def make_layer_weights(cfg: dict, layer: int, seed: int = DEFAULT_SEED, gen=None) -> dict:
    out = {}
    shapes = layer_shapes(cfg)
    for j, name in enumerate(_W_NAMES):
        k = key(seed, _LAYER_BASE + layer * 16 + j, gen)
        if name in shapes:
            n, kd = shapes[name]
            out[name] = q4k_matrix(k, n, kd, gen)
        else:
            size = cfg["head_dim"] if name in ("q_norm", "k_norm") else cfg["hidden"]
            out[name] = normal_f32(k, size, 0.1, 1.0, gen=gen)
    return out


def make_embed(cfg: dict, seed: int = DEFAULT_SEED, row0: int = 0, rows=None, gen=None) -> np.ndarray:
    rows = cfg["vocab"] - row0 if rows is None else rows
    return normal_f16(key(seed, _T_EMBED, gen), rows * cfg["hidden"], 0.02, first=row0 * cfg["hidden"], gen=gen).reshape(rows, cfg["hidden"])


def make_lm_head(cfg: dict, seed: int = DEFAULT_SEED, row0: int = 0, rows=None, gen=None) -> np.ndarray:
    rows = cfg["vocab"] - row0 if rows is None else rows
    return normal_f16(key(seed, _T_LMHEAD, gen), rows * cfg["hidden"], 0.02, first=row0 * cfg["hidden"], gen=gen).reshape(rows, cfg["hidden"])


def make_final_norm(cfg: dict, seed: int = DEFAULT_SEED, gen=None) -> np.ndarray:
    return normal_f32(key(seed, _T_FINAL_NORM, gen), cfg["hidden"], 0.1, 1.0, gen=gen)


def make_prompt(cfg: dict, n: int, seed: int = DEFAULT_SEED, seq: int = 0, gen=None) -> np.ndarray:
    return tokens(key(seed, _T_TOKENS + 100 * seq, gen), n, cfg["vocab"], gen)


def make_model_weights(cfg: dict, seed: int = DEFAULT_SEED, gen=None) -> dict:
    """Whole model in host memory (only sensible for the small configurations)."""
    return {
        "layers": [make_layer_weights(cfg, l, seed, gen) for l in range(cfg["n_layers"])],
        "embed": make_embed(cfg, seed, gen=gen),
        "lm_head": make_lm_head(cfg, seed, gen=gen),
        "final_norm": make_final_norm(cfg, seed, gen=gen),
    }
