"""Tensor-parallel split, checked on CPU with two gloo ranks: every rank computes its partial
result with the oracle on ITS shard, the partials are summed with a gloo allreduce, and the sum must
match the full-matrix oracle.  The greedy pick over a vocabulary-sharded LM head must match too."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from doppler_b200 import synthetic, tp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
sys.path.insert(0, os.environ["DP_ROOT"]); sys.path.insert(0, os.path.join(os.environ["DP_ROOT"], "tests"))
import numpy as np, torch, torch.distributed as dist
from doppler_b200 import synthetic, tp
from oracle import oracle as O
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
cfg = dict(synthetic.MODEL_CONFIGS["small"])
plan = tp.shard_plan(cfg, world, rank)
lw = synthetic.make_layer_weights(cfg, 0, seed=77)
H, I = cfg["hidden"], cfg["inter"]
x = synthetic.normal_f32(synthetic.key(77, 9), H)
# column parallel gate/up -> silu -> row parallel down, then the sum over ranks
r0, r1 = plan["wgate"]["rows"]
g = O.q4k_gemv(tp.slice_q4k_rows(lw["wgate"], I, H, r0, r1), r1 - r0, H, x)
u = O.q4k_gemv(tp.slice_q4k_rows(lw["wup"], I, H, r0, r1), r1 - r0, H, x)
a = O.silu_gated(g, u, clamped=True)
b0, b1 = plan["wdown"]["blocks"]
part = O.q4k_gemv(tp.slice_q4k_blocks(lw["wdown"], H, I, b0, b1), H, (b1 - b0) * 256, a)
t = torch.from_numpy(part.astype(np.float64)); dist.all_reduce(t)
gf = O.q4k_gemv(lw["wgate"], I, H, x); uf = O.q4k_gemv(lw["wup"], I, H, x)
full = O.q4k_gemv(lw["wdown"], H, I, O.silu_gated(gf, uf, clamped=True))
err = np.abs(t.numpy() - full).max() / np.sqrt(np.mean(full.astype(np.float64) ** 2))
assert np.array_equal(g, gf[r0:r1]), "column-parallel rows differ from the full matrix rows"
assert err < 1e-5, err
# vocabulary-sharded greedy pick
head = synthetic.make_lm_head(cfg, seed=77)
v0, v1 = plan["lm_head"]["rows"]
logits = O.f16_gemv(head[v0:v1], v1 - v0, H, x)
logits[0] = logits.max() if rank == 1 else logits[0]  # force a cross-rank tie candidate
li = int(O.argmax(logits)); pair = torch.tensor([float(logits[li]), float(li + v0)], dtype=torch.float64)
allp = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]; dist.all_gather(allp, pair)
pick = tp.merge_argmax([(float(p[0]), int(p[1])) for p in allp])
fl = [torch.zeros(v1 - v0, dtype=torch.float32) for _ in range(world)]; dist.all_gather(fl, torch.from_numpy(logits))
assert pick == int(O.argmax(np.concatenate([f.numpy() for f in fl]))), "sharded argmax differs from the full argmax"
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok")
'''


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def test_two_rank_split_matches_full_model_on_cpu(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = str(_free_port())
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=port, DP_ROOT=ROOT,
                   OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{o}"


def test_shard_plan_and_slicing():
    cfg = dict(synthetic.MODEL_CONFIGS["9b"])
    for size in (1, 2, 4, 8):
        seen = []
        for r in range(size):
            p = tp.shard_plan(cfg, size, r)
            seen.append(p["wo"]["blocks"])
            assert p["wq"]["rows"][1] - p["wq"]["rows"][0] == 4096 // size
            assert p["kv_heads"][1] - p["kv_heads"][0] == 8 // size
        assert seen[0][0] == 0 and seen[-1][1] == 16 and all(seen[i][1] == seen[i + 1][0] for i in range(size - 1))
    with pytest.raises(ValueError):
        tp.shard_plan(cfg, 16, 0)  # 8 KV heads do not divide over 16 ranks
    with pytest.raises(ValueError):
        tp.shard_plan(dict(cfg, inter=12288 + 256), 8, 0)
    w = synthetic.q4k_matrix(synthetic.key(3, 3), 8, 1024)
    assert np.array_equal(tp.slice_q4k_rows(w, 8, 1024, 2, 4), w[2 * 576:4 * 576])
    cols = tp.slice_q4k_blocks(w, 8, 1024, 1, 3).reshape(8, 2, 144)
    assert np.array_equal(cols[5, 1], w.reshape(8, 4, 144)[5, 2])
    assert tp.merge_argmax([(1.0, 7), (1.0, 3), (0.5, 1)]) == 3
