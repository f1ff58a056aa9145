"""Benchmark of the Q4_K quantized-inference hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload 9b|0.6b|small]

Workload (BASELINE config 4): a 9B-shaped dense decoder, random init (seeded synthetic Q4_K
blocks, f16 embedding / LM head), batch 1, a 1024-token prompt already in the f16 KV cache,
greedy decode.  One "step" is one decode step (one token through all layers, LM head and
argmax).  With N > 1 the weight matrices are tensor-parallel over N GPUs (one process per GPU,
launched by torch.distributed.run), so the total work is fixed: scaling is "strong".

value     tokens/s with everything resident in HBM: K decode steps as K CUDA-graph launches
          back to back inside one library call, device time, max over ranks.
e2e       tokens/s through the public C-ABI call per token with HOST buffers: every step
          uploads the token/position state from host memory, runs the step and reads the
          sampled token back (host<->device copies and the synchronisation inside the timing).
roofline  the dominant kernel (the Q4_K decode GEMV): algorithmic bytes / device time of all
          of the model's GEMVs launched back to back (distinct matrices, 3.9 GB >> L2),
          against the measured HBM copy peak of MEASURED_PEAKS.json.
cpu_baseline / --impl reference
          the CPU restatement of the reference's math (oracle/), OpenMP over all host cores,
          on a bounded sample (a 2-layer slice of the same model + the full LM head) scaled
          to the full depth.  The reference itself (JavaScript + WGSL) cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOADS = {"9b": ("9b", 1024), "0.6b": ("qwen3-0.6b", 512), "small": ("small", 64)}
HBM_FALLBACK_GBS = 6650.0
# DRAM bytes moved per algorithmic byte by the TMA-fed Q4_K GEMV, from one ncu capture of the same
# kernel on a [12288,4096] matrix (dram__bytes_read.sum + dram__bytes_write.sum = 28.347 MB for
# 28.377 MB of weights, activations and output: profiles/gemv_q4k_tma__12288x4096.md).  Traffic grows
# with the weight bytes, so the bench scales it to its own average launch.
GEMV_TRAFFIC_PER_ALGORITHMIC_BYTE = 28.3469 / 28.3771


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return HBM_FALLBACK_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc, self.idx = None, gpu_index
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------
# CPU baseline (oracle port): bounded sample scaled to the full model
# ----------------------------------------------------------------------------------------
def cpu_decode_tokens_per_s(cfg: dict, context: int, reps: int = 3):
    """Oracle decode step on the host cores: a 2-layer slice of the model plus the full LM head is
    timed, the head alone is timed, and the per-layer time is scaled to the model's depth."""
    from doppler_b200 import synthetic
    from oracle import oracle as O

    nl = 2
    c = dict(cfg, n_layers=nl, max_seq=16 + 2 * reps)
    head = synthetic.make_lm_head(cfg)
    w = {"layers": [synthetic.make_layer_weights(cfg, l) for l in range(nl)], "embed": synthetic.make_embed(cfg, rows=1024),
         "lm_head": head, "final_norm": synthetic.make_final_norm(cfg)}
    om = O.OracleModel(c, w)
    tok, _ = om.forward(np.array([1], np.int32))  # warm-up (page in, build tables)
    t0 = time.perf_counter()
    for _ in range(reps):
        tok, _ = om.forward(np.array([tok % 1024], np.int32))
    t_model = (time.perf_counter() - t0) / reps
    x = synthetic.normal_f32(synthetic.key(1, 1), cfg["hidden"])
    O.f16_gemv(head, cfg["vocab"], cfg["hidden"], x)
    t0 = time.perf_counter()
    for _ in range(reps):
        O.f16_gemv(head, cfg["vocab"], cfg["hidden"], x)
    t_head = (time.perf_counter() - t0) / reps
    per_layer = max(t_model - t_head, 1e-9) / nl
    total = t_head + per_layer * cfg["n_layers"]
    sample = (f"{reps} oracle decode steps of a {nl}-layer slice of the model + full LM head ({t_model * 1e3:.1f} ms each), "
              f"LM head alone {t_head * 1e3:.1f} ms; per-layer time x {cfg['n_layers']} + head; short context "
              f"(attention is < 3 % of the step's bytes)")
    return 1.0 / total, O.num_threads(), sample


def reference_arm(args, cfg, context):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # warm-up + K "steps": each step is one bounded sample
    vals = []
    # each bounded sample already holds its own warm-up pass; K is capped to keep the run short
    for _ in range(max(1, min(args.steps, 2))):
        v, cores, sample = cpu_decode_tokens_per_s(cfg, context, reps=3)
        vals.append(v)
    value = statistics.median(vals)
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 / value, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(args, cfg, context),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference's math (the JavaScript/WGSL reference cannot run on this box)",
    }
    print(json.dumps(line), flush=True)


def bench_config(args, cfg, context):
    return {"workload": f"{args.workload}-shaped Q4_K decoder, batch 1, greedy decode at context {context}",
            "layers": cfg["n_layers"], "hidden": cfg["hidden"], "heads": f"{cfg['n_heads']}q/{cfg['n_kv_heads']}kv",
            "head_dim": cfg["head_dim"], "mlp": cfg["inter"], "vocab": cfg["vocab"], "prompt": context, "batch": 1,
            "parallelism": f"tp{args.gpus}" + (f" ({args.allreduce} allreduce)" if args.gpus > 1 else ""), "l2": "inputs larger than L2 (weights 3.9 GB + LM head 1.2 GB per step at 9b)"}



# ----------------------------------------------------------------------------------------
# single-kernel cases (secondary metrics and profiler targets)
# ----------------------------------------------------------------------------------------
def _graph_time(dev, ops, record, n_ops, reps):
    """Record `record(rec)` (n_ops launches of the op over distinct inputs) into one CUDA graph and time
    `reps` replays with the host clock around a synchronise (the graph keeps the GPU busy back to back)."""
    rec = ops.CommandRecorder(dev, "case", capture_graph=True)
    record(rec)
    g = rec.finish_graph()
    for _ in range(3):
        g.launch()
    dev.sync()
    t0 = time.perf_counter()
    for _ in range(reps):
        g.launch()
    dev.sync()
    dt = (time.perf_counter() - t0) / (reps * n_ops)
    g.destroy()
    return dt


def kernel_case(args):
    from doppler_b200 import ops, synthetic
    dev = ops.Device(0)
    peak, peak_src = measured_peaks()
    out_lines = []
    if args.case == "gemv":
        shapes = [tuple(int(v) for v in args.shape.split(","))] if args.shape else [(3072, 1024), (12288, 4096), (4096, 12288), (24576, 4096)]
        for N, K in shapes:
            wbytes = N * ((K + 255) // 256) * 144
            copies = args.copies or max(4, int(300e6 / wbytes))
            ws = [dev.weight_from(synthetic.q4k_matrix(synthetic.key(5, i), N, K), "q4k", [N, K]) for i in range(copies)]
            x = dev.tensor_from(synthetic.normal_f32(synthetic.key(5, 100), K).reshape(1, K))
            out = dev.acquire_buffer(N * 4, "y")
            dt = _graph_time(dev, ops, lambda rec: [ops.record_matmul(rec, x, w, 1, N, K, output_dtype="f32", output_buffer=out) for w in ws],
                             copies, max(args.steps // 8, 3))
            b = wbytes + 4 * K + 4 * N
            out_lines.append({"case": "q4k_gemv", "shape": [1, N, K], "us_per_call": dt * 1e6, "GBps": b / dt / 1e9, "frac_of_measured_hbm": b / dt / 1e9 / peak,
                              "algorithmic_bytes": b, "distinct_weight_copies": copies,
                              "note": "one call = activation digit pre-pass + GEMV kernel, graph of `copies` calls over distinct matrices"})
            for w in ws:
                dev.release_buffer(w.buffer)
            dev.release_buffer(x.buffer); dev.release_buffer(out); dev.pool_trim()
    elif args.case == "gemm":
        M, N, K = tuple(int(v) for v in args.shape.split(",")) if args.shape else (512, 12288, 4096)
        copies = args.copies or 4
        ws = [dev.weight_from(synthetic.q4k_matrix(synthetic.key(5, i), N, K), "q4k", [N, K]) for i in range(copies)]
        a = dev.tensor_from(synthetic.normal_f16(synthetic.key(5, 100), M * K).reshape(M, K))
        out = dev.acquire_buffer(M * N * 2, "c")
        dt = _graph_time(dev, ops, lambda rec: [ops.record_matmul(rec, a, w, M, N, K, output_dtype="f16", output_buffer=out) for w in ws],
                         copies, max(args.steps // 8, 3))
        fl = 2.0 * M * N * K
        try:
            pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
            tf_burst, tf_sus = float(pk["bf16_tflops"]), float(pk["bf16_tflops_sustained"])
        except Exception:
            tf_burst, tf_sus = 1590.0, 1400.0
        out_lines.append({"case": "q4k_gemm_tcgen05", "shape": [M, N, K], "us_per_call": dt * 1e6, "TFLOPs": fl / dt / 1e12,
                          "frac_of_measured_burst": fl / dt / 1e12 / tf_burst, "frac_of_measured_sustained": fl / dt / 1e12 / tf_sus,
                          "frac_of_nominal_2250": fl / dt / 1e12 / 2250.0, "dtype": "f16 x q4k->f16, f32 accumulate"})
    elif args.case == "prefill":
        # whole-model prefill of the 9B-shaped decoder (f32 activations, f32-exact product on the tensor cores in
        # three passes; DP_PREFILL_TC=1 one f16 pass, 0 the CUDA-core kernel).  Times model.prefill(), prompt upload
        # and first-token read-back included.
        from doppler_b200.model import DecoderModel
        n = int(args.shape) if args.shape else 1024
        cfg = dict(synthetic.MODEL_CONFIGS["9b"])
        m = DecoderModel(dev, cfg, max_seq=n + 64)
        m.load_synthetic()
        prompt = synthetic.make_prompt(cfg, n)
        m.prefill(prompt); dev.sync(); m.reset()
        reps = 3
        t0 = time.perf_counter()
        for _ in range(reps):
            m.prefill(prompt); dev.sync(); m.reset()
        dt = (time.perf_counter() - t0) / reps
        layer_flops = 2.0 * n * cfg["hidden"] * ((cfg["n_heads"] + 2 * cfg["n_kv_heads"]) * cfg["head_dim"] + cfg["n_heads"] * cfg["head_dim"] + 3 * cfg["inter"])
        out_lines.append({"case": "prefill_9b", "prompt_tokens": n, "ms": dt * 1e3, "tokens_per_s": n / dt,
                          "q4k_gemm_TFLOPs_useful": layer_flops * cfg["n_layers"] / dt / 1e12,
                          "mode": "DP_PREFILL_TC=" + os.environ.get("DP_PREFILL_TC", "3 (default: three tensor-core passes, f32-exact)")})
        m.destroy()
    else:
        B, kv = tuple(int(v) for v in args.shape.split(",")) if args.shape else (32, 8192)
        H, Hkv, D = 32, 8, 128
        s = synthetic.key(synthetic.DEFAULT_SEED, 20)
        q = dev.tensor_from(synthetic.normal_f16(s, B * H * D).astype(np.float32))
        k = dev.tensor_from(synthetic.normal_f16(s + 1, B * kv * Hkv * D))
        v = dev.tensor_from(synthetic.normal_f16(s + 2, B * kv * Hkv * D))
        out = dev.acquire_buffer(B * H * D * 4, "o")
        ops.run_attention(q, k, v, None, H, D, seq_len=1, kv_len=kv, num_kv_heads=Hkv, causal=False, batch=B, kv_batch_stride=kv * Hkv * D, output_buffer=out)
        dt = _graph_time(dev, ops, lambda rec: [ops.record_attention(rec, q, k, v, None, H, D, seq_len=1, kv_len=kv, num_kv_heads=Hkv, causal=False,
                                                                      batch=B, kv_batch_stride=kv * Hkv * D, output_buffer=out)], 1, max(args.steps // 2, 5))
        b = 2 * B * kv * Hkv * D * 2 + B * H * D * 2 + B * H * D * 4
        out_lines.append({"case": "decode_attention_f16kv", "shape": {"batch": B, "heads": H, "kv_heads": Hkv, "head_dim": D, "kv_len": kv},
                          "us_per_call": dt * 1e6, "GBps": b / dt / 1e9, "frac_of_measured_hbm": b / dt / 1e9 / peak, "algorithmic_bytes": b,
                          "note": "KV (1.07 GB at config 2) is larger than L2"})
    for l in out_lines:
        l["peak_source"] = peak_src
        print(json.dumps(l), flush=True)
    dev.close()


# ----------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="9b", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--case", default=None, choices=["gemv", "gemm", "attention", "prefill"],
                    help="time ONE kernel of the path on a BASELINE configuration instead of the decoder "
                         "(gemv: configs 0 and 9B shapes, gemm: config 1, attention: config 2); also the small "
                         "command the profiler captures use")
    ap.add_argument("--shape", default=None, help="--case gemv/gemm: N,K or M,N,K; --case attention: batch,kv_len")
    ap.add_argument("--copies", type=int, default=0, help="--case: distinct weight copies per pass (0 = enough to exceed L2)")
    ap.add_argument("--only-timed", action="store_true",
                    help="stop after the device-resident timed region (used for profiler launch lists)")
    ap.add_argument("--allreduce", default="oneshot", choices=["oneshot", "nccl"],
                    help="N>1: one-shot peer-memory exchange fused into the decode kernels, or NCCL")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    from doppler_b200 import synthetic

    model_name, context = WORKLOADS[args.workload]
    cfg = dict(synthetic.MODEL_CONFIGS[model_name])

    if args.impl == "reference":
        reference_arm(args, cfg, context)
        return
    if args.case:
        kernel_case(args)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs one process per GPU: python -m torch.distributed.run "
                             f"--nproc-per-node {args.gpus} bench.py --gpus {args.gpus}")
        args.gpus = world

    from doppler_b200 import _lib as L
    from doppler_b200.model import DecoderModel
    from doppler_b200.ops import Device
    import ctypes as C

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        dist = dist_mod
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)

    dev = Device(local_rank)
    if world > 1:
        from doppler_b200 import tp
        tp.init_group(dev, rank, world)
        if args.allreduce == "oneshot":
            tp.setup_exchange(dev, rank, world)

    steps_total = args.warmup + args.steps
    max_seq = context + 2 * steps_total + 64
    model = DecoderModel(dev, cfg, max_seq=max_seq, tp_rank=rank, tp_size=world)
    if world > 1 and args.allreduce == "oneshot":
        model.set_allreduce_mode(1)
    model.load_synthetic()
    prompt = synthetic.make_prompt(cfg, context)

    def barrier():
        dev.sync()
        if dist is not None:
            dist.barrier()

    first = model.prefill(prompt)
    barrier()

    # ---- device-resident throughput ---------------------------------------------------
    warm = model.decode([first], args.warmup)
    nxt = int(warm[-1, 0])
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = dev.launch_count
    out = model.decode([nxt], args.steps)
    ms = model.last_decode_ms
    barrier()
    launches = dev.launch_count - launches0
    nxt = int(out[-1, 0])

    if args.only_timed:
        if rank == 0:
            print(json.dumps({"metric": "decode_tokens_per_s", "value": args.steps / (ms / 1000.0), "unit": "tokens/s",
                              "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
                              "gpu_launches": int(launches), "note": "timed region only"}), flush=True)
        if sampler:
            sampler.stop()
        model.destroy()
        dev.close()
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- end to end through the per-token C-ABI call with host buffers -------------------
    model.reset()
    first = model.prefill(prompt)
    e2e_steps = args.steps
    for _ in range(args.warmup):
        first = int(model.decode([first], 1)[0, 0])
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        first = int(model.decode([first], 1)[0, 0])
    dev.sync()
    e2e_s = time.perf_counter() - t0
    barrier()
    clocks = sampler.stop() if sampler else None

    # ---- dominant kernel: all Q4_K GEMVs of the model back to back --------------------------
    model.bench_gemv(1)
    g = model.bench_gemv(3)
    barrier()

    times = [ms, e2e_s * 1000.0, g["ms"]]
    if dist is not None:
        import torch
        t = torch.tensor(times, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times = t.tolist()
    ms, e2e_ms, gemv_ms = times

    if rank == 0:
        peak, peak_src = measured_peaks()
        value = args.steps / (ms / 1000.0)
        gemv_gbs = g["bytes"] / (gemv_ms / 1000.0) / 1e9
        line = {
            "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": bench_config(args, cfg, context),
            "e2e": {"value": e2e_steps / (e2e_ms / 1000.0), "unit": "tokens/s", "h2d_bytes_per_step": 4096 + 0,
                    "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "Q4_K decode GEMV (all matrices of the model, back to back)",
                         "achieved": gemv_gbs, "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                         "frac": gemv_gbs / peak, "frac_of_nominal_8000": gemv_gbs / 8000.0,
                         "launches": g["launches"], "avg_launch_us": gemv_ms * 1000.0 / max(g["launches"], 1),
                         "bytes_per_launch_avg": g["bytes"] / max(g["launches"], 1),
                         "traffic": GEMV_TRAFFIC_PER_ALGORITHMIC_BYTE * g["bytes"] / max(g["launches"], 1),
                         "traffic_source": "ncu capture of a [12288,4096] launch scaled by bytes"},
            "model_weight_bytes_per_gpu": model.weight_bytes,
        }
        if not args.no_cpu_baseline:
            try:
                v, cores, sample = cpu_decode_tokens_per_s(cfg, context, reps=3)
                line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
            except Exception as e:  # the baseline is a reported number, never the product path
                line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
        print(json.dumps(line), flush=True)
    model.destroy()
    dev.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
