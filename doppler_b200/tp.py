"""Tensor-parallel plumbing for the decoder runner (one process per GPU).

The reference has no collective backend; this is the column/row-parallel split of the dense
decoder: q/k/v/gate/up are split by output rows, o/down by 256-element super-block columns (so
every shard is still a valid row-major Q4_K matrix), the KV cache by KV head, the LM head by
vocabulary rows.  After o_proj and down_proj the partial [hidden] vectors are summed over ranks.

`shard_plan` and the two slicing helpers restate on the host what the C++ loader does
(dp_model_load_q4k), so the split can be checked without a GPU.

Rendezvous is the caller's: the library only makes and consumes the bytes (a 128-byte NCCL
unique id, one 64-byte CUDA IPC handle per rank); how they travel between the processes is up
to the launcher (the tests and the benchmark use a torch.distributed gloo group).
"""
from __future__ import annotations

import ctypes as C

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


def make_unique_id(dev) -> bytes:
    """128-byte NCCL unique id, made by ONE rank; the caller carries it to the others by whatever
    channel it has (a launcher's store, MPI, a file) and every rank passes it to init_group."""
    buf = (C.c_uint8 * 128)()
    if dev.lib.dp_tp_unique_id(buf) != L.OK:
        raise RuntimeError("cannot create the NCCL unique id (libnccl not loadable?)")
    return bytes(buf)


def init_group(dev, rank: int, world: int, unique_id: bytes):
    """Create the NCCL group of the context from the id rank 0 made (make_unique_id)."""
    if len(unique_id) != 128:
        raise ValueError("the NCCL unique id is 128 bytes")
    dev.check(dev.lib.dp_tp_init(dev.h, rank, world, (C.c_uint8 * 128).from_buffer_copy(unique_id)))


def export_exchange(dev) -> bytes:
    """64-byte CUDA IPC handle of this rank's peer-memory exchange area (allocated on first use)."""
    mine = (C.c_uint8 * 64)()
    dev.check(dev.lib.dp_tp_ipc_export(dev.h, mine))
    return bytes(mine)


def attach_exchange(dev, handles_by_rank):
    """Map every rank's exchange area into this process.  `handles_by_rank[r]` is what rank r got
    from export_exchange.  All ranks must have attached (a barrier of the caller's) before any of
    them decodes: a rank pushes into its peers' areas.  Needed for the one-shot exchange
    (DecoderModel.set_allreduce_mode(1))."""
    flat = b"".join(bytes(h) for h in handles_by_rank)
    if len(flat) % 64:
        raise ValueError("IPC handles are 64 bytes each")
    dev.check(dev.lib.dp_tp_ipc_attach(dev.h, (C.c_uint8 * len(flat)).from_buffer_copy(flat)))
