"""Tensor-parallel plumbing for the decoder runner (one process per GPU).

The reference has no collective backend; this is the column/row-parallel split of the dense
decoder: q/k/v/gate/up are split by output rows, o/down by 256-element super-block columns (so
every shard is still a valid row-major Q4_K matrix), the KV cache by KV head, the LM head by
vocabulary rows.  After o_proj and down_proj the partial [hidden] vectors are summed over ranks.

`shard_plan` and the two slicing helpers restate on the host what the C++ loader does
(dp_model_load_q4k), so the split can be checked without a GPU.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import _lib as L

QK_K, BLOCK = 256, 144


def shard_plan(cfg: dict, size: int, rank: int) -> dict:
    """Row / super-block ranges this rank keeps of every matrix (raises if the model does not divide)."""
    qd, kvd, hid, inter, vocab = (cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"], cfg["hidden"],
                                  cfg["inter"], cfg["vocab"])
    if cfg["n_heads"] % size or cfg["n_kv_heads"] % size:
        raise ValueError(f"heads ({cfg['n_heads']}/{cfg['n_kv_heads']}) do not divide over {size} ranks")
    if qd % (size * QK_K) or inter % (size * QK_K):
        raise ValueError("row-parallel matrices must split on 256-element super-blocks")
    if vocab % size:
        raise ValueError("vocabulary does not divide over the ranks")

    def rows(n):
        return (rank * n // size, (rank + 1) * n // size)

    def blocks(k):
        b = k // QK_K
        return (rank * b // size, (rank + 1) * b // size)

    return {"wq": {"rows": rows(qd)}, "wk": {"rows": rows(kvd)}, "wv": {"rows": rows(kvd)},
            "wgate": {"rows": rows(inter)}, "wup": {"rows": rows(inter)},
            "wo": {"blocks": blocks(qd)}, "wdown": {"blocks": blocks(inter)},
            "lm_head": {"rows": rows(vocab)}, "q_heads": rows(cfg["n_heads"]), "kv_heads": rows(cfg["n_kv_heads"])}


def slice_q4k_rows(w: np.ndarray, n: int, k: int, r0: int, r1: int) -> np.ndarray:
    """Rows [r0, r1) of a packed [n, k] matrix: a contiguous byte range."""
    rb = ((k + QK_K - 1) // QK_K) * BLOCK
    return np.ascontiguousarray(w.reshape(n, rb)[r0:r1]).ravel()


def slice_q4k_blocks(w: np.ndarray, n: int, k: int, b0: int, b1: int) -> np.ndarray:
    """Super-block columns [b0, b1) of every row, re-packed densely: a [n, (b1-b0)*256] Q4_K matrix."""
    bpr = (k + QK_K - 1) // QK_K
    return np.ascontiguousarray(w.reshape(n, bpr, BLOCK)[:, b0:b1]).ravel()


def merge_argmax(pairs):
    """Vocabulary-sharded greedy pick: the largest value wins, ties go to the lower global index
    (src/gpu/kernels/sample.wgsl:45-53).  `pairs` = [(best value, global index)] per rank."""
    best_v, best_i = -np.inf, 2**31 - 1
    for v, i in pairs:
        if v > best_v or (v == best_v and i < best_i):
            best_v, best_i = v, i
    return best_i


def init_group(dev, rank: int, world: int):
    """Create the NCCL group of the context: rank 0 makes the unique id, torch.distributed (any
    backend, e.g. gloo) carries it to the other ranks."""
    import torch
    import torch.distributed as dist

    uid = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        buf = (C.c_uint8 * 128)()
        if dev.lib.dp_tp_unique_id(buf) != L.OK:
            raise RuntimeError("cannot create the NCCL unique id (libnccl not loadable?)")
        uid = torch.tensor(list(buf), dtype=torch.uint8)
    dist.broadcast(uid, 0)
    ub = (C.c_uint8 * 128)(*uid.tolist())
    dev.check(dev.lib.dp_tp_init(dev.h, rank, world, ub))


def setup_exchange(dev, rank: int, world: int):
    """Map every rank's peer-memory exchange area into this process (CUDA IPC handles travel over
    torch.distributed).  Needed for the one-shot allreduce (DecoderModel.set_allreduce_mode(1))."""
    import torch
    import torch.distributed as dist

    mine = (C.c_uint8 * 64)()
    dev.check(dev.lib.dp_tp_ipc_export(dev.h, mine))
    t = torch.tensor(list(mine), dtype=torch.uint8)
    allh = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(allh, t)
    flat = (C.c_uint8 * (64 * world))(*[int(b) for h in allh for b in h.tolist()])
    dev.check(dev.lib.dp_tp_ipc_attach(dev.h, flat))
    dist.barrier()  # nobody pushes before every rank has mapped every area
