"""Benchmark of the Q4_K quantized-inference hot path.

    python bench.py --gpus N --steps K --warmup W [--batch B] [--impl reference] [--workload 9b|0.6b|small]

Workload (BASELINE config 4): a 9B-shaped dense decoder, random init (seeded synthetic Q4_K
blocks, f16 embedding / LM head), a 1024-token prompt per sequence already in the f16 KV cache,
greedy decode, batch 1 (default) or --batch 64.  One "step" is one decode step (one token per
sequence through all layers, LM head and argmax).  With N > 1 the weight matrices are
tensor-parallel over N GPUs (one process per GPU, launched by torch.distributed.run), so the
total work is fixed: scaling is "strong".

value     tokens/s with everything resident in HBM: K decode steps as K CUDA-graph launches back to
          back inside one library call, device time (CUDA events), max over ranks; the K-step
          region is repeated (--regions, default 5) and the MEDIAN is reported with min and max.
e2e       tokens/s through the public C-ABI call per token with HOST buffers: every step uploads
          the token/position state from host memory, runs the step and reads the sampled tokens
          back (host<->device copies and the synchronisation inside the timing).
roofline  the dominant kernels (the Q4_K decode GEMVs as the decode graph launches them):
          algorithmic bytes / device time of all of the model's GEMV launches back to back
          (distinct matrices, 3.9 GB >> L2), against the measured HBM copy peak.
kernels   the other BASELINE configurations, a few ms each through the C ABI: config 0 GEMV (us),
          config 1 GEMM (TFLOP/s, fraction of the measured bf16 burst and sustained peaks),
          config 2 decode attention (GB/s, fraction of measured HBM).  N = 1 only.
tokens_crc  CRC-32 of the tokens of the warm-up and the first timed region; every rank must hold
          the same tokens (checked), and the N = 1 and N = 8 lines can be compared.
cpu_baseline / --impl reference
          the CPU restatement of the reference's math (oracle/), OpenMP over ALL host cores, on
          the FULL-depth model with a synthetic KV context of the same length: each step is one
          real decode step.  The reference itself (JavaScript + WGSL) cannot run here.  This arm
          builds its model with the oracle's own restatement of the seeded generators and does
          not load the CUDA library.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
import zlib

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOADS = {"9b": ("9b", 1024), "0.6b": ("qwen3-0.6b", 512), "small": ("small", 64)}
HBM_FALLBACK_GBS = 6650.0
TENSOR_FALLBACK = (1590.0, 1400.0)
# DRAM bytes moved per algorithmic byte by the TMA-fed Q4_K GEMV, from one ncu capture of the same
# kernel on a [12288,4096] matrix (dram__bytes_read.sum + dram__bytes_write.sum = 28.347 MB for
# 28.377 MB of weights, activations and output: profiles/gemv_q4k_tma__12288x4096.md).  Traffic grows
# with the weight bytes, so the bench scales it to its own average launch.
GEMV_TRAFFIC_PER_ALGORITHMIC_BYTE = 28.3469 / 28.3771


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            pk = json.load(open(path))
            return {"hbm_gbs": float(pk["hbm_gbs"]), "tf_burst": float(pk["bf16_tflops"]),
                    "tf_sustained": float(pk["bf16_tflops_sustained"]), "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": HBM_FALLBACK_GBS, "tf_burst": TENSOR_FALLBACK[0], "tf_sustained": TENSOR_FALLBACK[1], "source": "fallback"}


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


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
# CPU baseline (oracle port).  Nothing in this section touches the CUDA library.
# ----------------------------------------------------------------------------------------
def _oracle(threads: int):
    from oracle import oracle as O

    O.set_num_threads(threads)  # launchers such as torch.distributed.run export OMP_NUM_THREADS=1
    return O


def cpu_full_model(cfg: dict, context: int, steps: int, warmup: int):
    """Decode steps of the FULL-depth oracle model on all host cores.  The KV cache is filled with
    synthetic f16 values for `context` positions (no prompt pass on the CPU), then `warmup` + `steps`
    real greedy steps run; every step is timed on its own.  Returns (tokens/s from the median step,
    list of step times in s, cores, description)."""
    from doppler_b200 import synthetic

    cores = host_cores()
    O = _oracle(cores)
    gen = synthetic.Generator(O.SynthBackend())
    t0 = time.perf_counter()
    w = synthetic.make_model_weights(cfg, gen=gen)
    t_build = time.perf_counter() - t0
    om = O.OracleModel(dict(cfg, max_seq=context + warmup + steps + 1), w)
    om.fill_kv(context, key=synthetic.key(synthetic.DEFAULT_SEED, 77, gen))
    tok = int(synthetic.make_prompt(cfg, 1, gen=gen)[0])
    for _ in range(warmup):
        tok, _ = om.forward(np.array([tok], np.int32))
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        tok, _ = om.forward(np.array([tok], np.int32))
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    sample = (f"{steps} real greedy decode steps (+{warmup} warm-up) of the full {cfg['n_layers']}-layer model, vocabulary "
              f"{cfg['vocab']}, attention over a synthetic f16 KV context of {context} tokens; median step {med * 1e3:.1f} ms "
              f"(min {min(times) * 1e3:.1f}, max {max(times) * 1e3:.1f}); model built in {t_build:.1f} s outside the timing")
    return 1.0 / med, times, cores, sample


def cpu_kernel_baselines():
    """BASELINE configs 0-2 on the host cores (oracle, OpenMP): config 0 whole, configs 1 and 2 on a
    bounded slice (rows / sequences are independent, so time scales with their number)."""
    from doppler_b200 import synthetic

    cores = host_cores()
    O = _oracle(cores)
    gen = synthetic.Generator(O.SynthBackend())
    k = lambda i: synthetic.key(synthetic.DEFAULT_SEED, 300 + i, gen)  # noqa: E731
    out = {"cores": cores, "kind": "port"}
    # config 0: GEMV [1,1024] x [3072,1024]
    N, K = 3072, 1024
    W, x = synthetic.q4k_matrix(k(0), N, K, gen), synthetic.normal_f32(k(1), K, gen=gen)
    O.q4k_gemv(W, N, K, x)
    ts = []
    for _ in range(20):
        t0 = time.perf_counter(); O.q4k_gemv(W, N, K, x); ts.append(time.perf_counter() - t0)
    b = W.nbytes + 4 * K + 4 * N
    out["config0_gemv"] = {"us": statistics.median(ts) * 1e6, "GBps": b / statistics.median(ts) / 1e9, "sample": "whole config, median of 20"}
    # config 1: GEMM [512,4096] x [12288,4096]: 16 of the 512 activation rows
    M, N, K, Ms = 512, 12288, 4096, 16
    W = synthetic.q4k_matrix(k(2), N, K, gen)
    A = synthetic.normal_f16(k(3), Ms * K, gen=gen).astype(np.float32)
    t0 = time.perf_counter(); O.q4k_gemm(W, N, K, A, Ms); dt = time.perf_counter() - t0
    out["config1_gemm"] = {"TFLOPs": 2.0 * Ms * N * K / dt / 1e12, "ms_scaled_to_512_rows": dt * (M / Ms) * 1e3,
                           "sample": f"{Ms} of {M} activation rows, one pass"}
    # config 2: decode attention, batch 32 x ctx 8192: one of the 32 sequences
    H, Hkv, D, kv = 32, 8, 128, 8192
    q = synthetic.normal_f16(k(4), H * D, gen=gen).astype(np.float32)
    k16, v16 = synthetic.normal_f16(k(5), kv * Hkv * D, gen=gen), synthetic.normal_f16(k(6), kv * Hkv * D, gen=gen)
    t0 = time.perf_counter(); O.attention_f16kv(q, k16, v16, 1, kv, H, Hkv, D, causal=False); dt = time.perf_counter() - t0
    b = 2 * kv * Hkv * D * 2 + H * D * 2 + H * D * 4
    out["config2_attention"] = {"GBps": b / dt / 1e9, "ms_scaled_to_batch_32": dt * 32 * 1e3, "sample": "1 of 32 sequences, one pass"}
    return out


def reference_arm(args, cfg, context):
    if int(os.environ.get("RANK", "0")) != 0:
        return  # one CPU, one run: the other ranks of a torchrun launch have nothing to do
    # each step is ~0.3-0.5 s of all host cores on the 9B shape; a few minutes at most
    steps = max(1, min(args.steps, 200))
    warmup = max(1, min(args.warmup, 3))
    value, times, cores, sample = cpu_full_model(cfg, context, steps, warmup)
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": 1000.0 * statistics.median(times), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(args, cfg, context),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "timed_seconds": sum(times),
        "note": "CPU restatement of the reference's math (the JavaScript/WGSL reference cannot run on this box); batch 1",
    }
    print(json.dumps(line), flush=True)


def bench_config(args, cfg, context):
    return {"workload": f"{args.workload}-shaped Q4_K decoder, batch {args.batch}, greedy decode at context {context}",
            "layers": cfg["n_layers"], "hidden": cfg["hidden"], "heads": f"{cfg['n_heads']}q/{cfg['n_kv_heads']}kv",
            "head_dim": cfg["head_dim"], "mlp": cfg["inter"], "vocab": cfg["vocab"], "prompt": context, "batch": args.batch,
            "parallelism": f"tp{args.gpus}" + (f" ({args.allreduce} exchange)" if args.gpus > 1 else ""),
            "l2": "inputs larger than L2 (weights 3.9 GB + LM head 1.2 GB per step at 9b)"}


# ----------------------------------------------------------------------------------------
# single-kernel cases (secondary metrics and profiler targets)
# ----------------------------------------------------------------------------------------
def _graph_time(dev, ops, record, n_ops, reps):
    """Record `record(rec)` (n_ops launches of the op over distinct inputs) into one CUDA graph and time
    `reps` replays with CUDA events on the library's stream; returns seconds per op."""
    rec = ops.CommandRecorder(dev, "case", capture_graph=True)
    record(rec)
    g = rec.finish_graph()
    g.launch_timed(3)
    ms = g.launch_timed(reps)
    g.destroy()
    return ms / 1000.0 / (reps * n_ops)


def gemv_case(dev, ops, synthetic, N, K, copies, reps, peak):
    wbytes = N * ((K + 255) // 256) * 144
    copies = copies or max(4, int(300e6 / wbytes))
    ws = [dev.weight_from(synthetic.q4k_matrix(synthetic.key(5, i), N, K), "q4k", [N, K]) for i in range(copies)]
    x = dev.tensor_from(synthetic.normal_f32(synthetic.key(5, 100), K).reshape(1, K))
    out = dev.acquire_buffer(N * 4, "y")
    dt = _graph_time(dev, ops, lambda rec: [ops.record_matmul(rec, x, w, 1, N, K, output_dtype="f32", output_buffer=out) for w in ws], copies, reps)
    b = wbytes + 4 * K + 4 * N
    for w in ws:
        dev.release_buffer(w.buffer)
    dev.release_buffer(x.buffer); dev.release_buffer(out); dev.pool_trim()
    return {"case": "q4k_gemv", "shape": [1, N, K], "us_per_call": dt * 1e6, "GBps": b / dt / 1e9, "frac_of_measured_hbm": b / dt / 1e9 / peak["hbm_gbs"],
            "algorithmic_bytes": b, "distinct_weight_copies": copies,
            "note": "one call = dp_matmul of one f32 vector (one kernel: the digits are built in its prologue), graph of `copies` calls over distinct matrices"}


def gemm_case(dev, ops, synthetic, M, N, K, copies, reps, peak, variant="default", adtype="f16"):
    copies = copies or 4
    ws = [dev.weight_from(synthetic.q4k_matrix(synthetic.key(5, i), N, K), "q4k", [N, K]) for i in range(copies)]
    if adtype == "f32":  # the runner's case: f32 activations and output, f32-exact product (three tensor-core products)
        a = dev.tensor_from(synthetic.normal_f32(synthetic.key(5, 100), M * K).reshape(M, K))
    else:
        a = dev.tensor_from(synthetic.normal_f16(synthetic.key(5, 100), M * K).reshape(M, K))
    odt = "f32" if adtype == "f32" else "f16"
    out = dev.acquire_buffer(M * N * (4 if adtype == "f32" else 2), "c")
    kw = {"f16_weights": True} if variant == "f16_weights" else {}
    dt = _graph_time(dev, ops, lambda rec: [ops.record_matmul(rec, a, w, M, N, K, output_dtype=odt, output_buffer=out, **kw) for w in ws], copies, reps)
    fl = 2.0 * M * N * K
    for w in ws:
        dev.release_buffer(w.buffer)
    dev.release_buffer(a.buffer); dev.release_buffer(out); dev.pool_trim()
    return {"case": "q4k_gemm_tcgen05", "variant": variant, "shape": [M, N, K], "us_per_call": dt * 1e6, "TFLOPs": fl / dt / 1e12,
            "frac_of_measured_burst": fl / dt / 1e12 / peak["tf_burst"], "frac_of_measured_sustained": fl / dt / 1e12 / peak["tf_sustained"],
            "frac_of_nominal_2250": fl / dt / 1e12 / 2250.0, "dtype": f"{adtype} x q4k -> {odt}, f32 accumulate",
            "weights_per_s": N * K / dt, "q4k_GBps": N * K * 0.5625 / dt / 1e9}


def lm_head_case(dev, ops, synthetic, M, N, K, reps, peak):
    """f16 [N, K] head times M f32 activation rows (the batched decode step's logits matmul); the weights of
    the default shape (311 MB) are larger than L2."""
    w = dev.weight_from(synthetic.normal_f16(synthetic.key(6, 0), N * K, 0.02), "f16", [N, K])
    a = dev.tensor_from(synthetic.normal_f32(synthetic.key(6, 1), M * K).reshape(M, K))
    out = dev.acquire_buffer(M * N * 4, "logits")
    dt = _graph_time(dev, ops, lambda rec: [ops.record_matmul(rec, a, w, M, N, K, output_dtype="f32", output_buffer=out)], 1, reps)
    b = N * K * 2 + M * K * 4 + M * N * 4
    dev.release_buffer(w.buffer); dev.release_buffer(a.buffer); dev.release_buffer(out); dev.pool_trim()
    return {"case": "lm_head_f16w", "shape": [M, N, K], "us_per_call": dt * 1e6, "GBps": b / dt / 1e9, "frac_of_measured_hbm": b / dt / 1e9 / peak["hbm_gbs"],
            "algorithmic_bytes": b, "note": "one call = row scaling pre-pass (M > 1) + kernel"}


def attention_case(dev, ops, synthetic, B, kv, reps, peak):
    H, Hkv, D = 32, 8, 128
    s = synthetic.key(synthetic.DEFAULT_SEED, 20)
    q = dev.tensor_from(synthetic.normal_f16(s, B * H * D).astype(np.float32))
    k = dev.tensor_from(synthetic.normal_f16(s + 1, B * kv * Hkv * D))
    v = dev.tensor_from(synthetic.normal_f16(s + 2, B * kv * Hkv * D))
    out = dev.acquire_buffer(B * H * D * 4, "o")
    ops.run_attention(q, k, v, None, H, D, seq_len=1, kv_len=kv, num_kv_heads=Hkv, causal=False, batch=B, kv_batch_stride=kv * Hkv * D, output_buffer=out)
    dt = _graph_time(dev, ops, lambda rec: [ops.record_attention(rec, q, k, v, None, H, D, seq_len=1, kv_len=kv, num_kv_heads=Hkv, causal=False,
                                                                  batch=B, kv_batch_stride=kv * Hkv * D, output_buffer=out)], 1, reps)
    b = 2 * B * kv * Hkv * D * 2 + B * H * D * 2 + B * H * D * 4
    for t in (q, k, v):
        dev.release_buffer(t.buffer)
    dev.release_buffer(out); dev.pool_trim()
    return {"case": "decode_attention_f16kv", "shape": {"batch": B, "heads": H, "kv_heads": Hkv, "head_dim": D, "kv_len": kv},
            "us_per_call": dt * 1e6, "GBps": b / dt / 1e9, "frac_of_measured_hbm": b / dt / 1e9 / peak["hbm_gbs"], "algorithmic_bytes": b,
            "note": "KV (1.07 GB at config 2) is larger than L2"}


def kernels_record(dev, peak):
    """BASELINE configs 0, 1 and 2 through dp_matmul / dp_attention, a few ms each."""
    from doppler_b200 import ops, synthetic

    g0 = gemv_case(dev, ops, synthetic, 3072, 1024, 0, 5, peak)
    g1 = gemm_case(dev, ops, synthetic, 512, 12288, 4096, 4, 5, peak)
    g1f = gemm_case(dev, ops, synthetic, 512, 12288, 4096, 4, 5, peak, variant="f16_weights")
    a2 = attention_case(dev, ops, synthetic, 32, 8192, 5, peak)
    keep = lambda d, ks: {k: d[k] for k in ks}  # noqa: E731
    return {
        "config0_gemv_3072x1024": keep(g0, ("us_per_call", "GBps", "frac_of_measured_hbm", "note")),
        "config1_gemm_512x12288x4096": dict(keep(g1, ("us_per_call", "TFLOPs", "frac_of_measured_burst", "frac_of_measured_sustained")),
                                            note="default: exact product (dequantised weights kept to f32 accuracy), gate 1e-3"),
        "config1_gemm_f16_weights": dict(keep(g1f, ("us_per_call", "TFLOPs", "frac_of_measured_burst", "frac_of_measured_sustained")),
                                         note="opt-in: weights rounded to f16 as in the reference's tiled f16 prefill kernel"),
        "config2_attention_b32_ctx8192": keep(a2, ("us_per_call", "GBps", "frac_of_measured_hbm")),
    }


def kernel_case(args):
    from doppler_b200 import ops, synthetic
    dev = ops.Device(0)
    peak = measured_peaks()
    out_lines = []
    reps = max(args.steps // 8, 3)
    if args.case == "gemv":
        shapes = [tuple(int(v) for v in args.shape.split(","))] if args.shape else [(3072, 1024), (12288, 4096), (4096, 12288), (24576, 4096)]
        for N, K in shapes:
            out_lines.append(gemv_case(dev, ops, synthetic, N, K, args.copies, reps, peak))
    elif args.case == "gemm":
        M, N, K = tuple(int(v) for v in args.shape.split(",")) if args.shape else (512, 12288, 4096)
        out_lines.append(gemm_case(dev, ops, synthetic, M, N, K, args.copies, reps, peak, variant=args.variant, adtype=args.adtype))
    elif args.case == "lm_head":
        M, N, K = tuple(int(v) for v in args.shape.split(",")) if args.shape else (64, 151936, 4096)
        out_lines.append(lm_head_case(dev, ops, synthetic, M, N, K, max(reps, 5), peak))
    elif args.case == "prefill":
        # whole-model prefill of the 9B-shaped decoder (f32 activations, f32-exact product on the tensor cores).
        # Times model.prefill(), prompt upload and first-token read-back included.
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
                          "q4k_gemm_TFLOPs_useful": layer_flops * cfg["n_layers"] / dt / 1e12})
        m.destroy()
    else:
        B, kv = tuple(int(v) for v in args.shape.split(",")) if args.shape else (32, 8192)
        out_lines.append(attention_case(dev, ops, synthetic, B, kv, max(args.steps // 2, 5), peak))
    for l in out_lines:
        l["peak_source"] = peak["source"]
        print(json.dumps(l), flush=True)
    dev.close()


# ----------------------------------------------------------------------------------------
def kernel_trace(model, dev, tokens, steps, path, barrier, world, batch):
    """One region of `steps` decode steps under torch.profiler's CUDA activity tracing (every rank runs it, rank 0
    writes the table).  Times under a tracer are for SHARES; the bench value never comes from here."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    torch.cuda.init()
    barrier()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        model.decode(tokens, steps)
        dev.sync()
    barrier()
    if path is None:
        return
    rows = []
    for e in prof.key_averages():
        t = float(getattr(e, "device_time_total", 0.0) or getattr(e, "cuda_time_total", 0.0) or 0.0)
        if t > 0.0:
            rows.append((t, int(e.count), str(e.key)))
    rows.sort(reverse=True)
    total = sum(r[0] for r in rows) or 1.0
    with open(path, "w") as f:
        f.write(f"# decode step kernels, rank 0 of {world}, batch {batch}, {steps} steps traced (CUPTI activity records)\n")
        f.write(f"# device time in kernels per step: {total / steps:.1f} us; wall time of the traced region per step: {model.last_decode_ms * 1000.0 / steps:.1f} us\n")
        f.write("share_pct\ttotal_us\tlaunches\tavg_us\tkernel\n")
        for t, c, k in rows:
            f.write(f"{100.0 * t / total:.1f}\t{t:.0f}\t{c}\t{t / max(c, 1):.2f}\t{k[:160]}\n")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1, help="sequences decoded together (BASELINE config 4: 1 and 64)")
    ap.add_argument("--regions", type=int, default=5, help="repeats of the K-step resident region (median reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="9b", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-kernels", action="store_true", help="skip the config 0/1/2 kernel record")
    ap.add_argument("--case", default=None, choices=["gemv", "gemm", "attention", "prefill", "lm_head"],
                    help="time ONE kernel of the path on a BASELINE configuration instead of the decoder "
                         "(gemv: configs 0 and 9B shapes, gemm: config 1, attention: config 2); also the small "
                         "command the profiler captures use")
    ap.add_argument("--shape", default=None, help="--case gemv/gemm: N,K or M,N,K; --case attention: batch,kv_len")
    ap.add_argument("--variant", default="default", choices=["default", "f16_weights"], help="--case gemm: exact product or f16-rounded weights")
    ap.add_argument("--adtype", default="f16", choices=["f16", "f32"], help="--case gemm: activation (and output) dtype")
    ap.add_argument("--copies", type=int, default=0, help="--case: distinct weight copies per pass (0 = enough to exceed L2)")
    ap.add_argument("--only-timed", action="store_true",
                    help="stop after the first device-resident timed region (used for profiler launch lists)")
    ap.add_argument("--kernel-trace", default=None, metavar="FILE",
                    help="with --only-timed: run one more region of --steps decode steps under torch.profiler (CUPTI activity "
                         "records, no kernel replay) and have rank 0 write a per-kernel table (launches, device time, share) to FILE")
    ap.add_argument("--allreduce", default="oneshot", choices=["oneshot", "nccl"],
                    help="N>1: one-shot peer-memory exchange fused into the decode kernels, or NCCL")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    from doppler_b200 import synthetic  # importing does not load the CUDA library

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

    from doppler_b200.model import DecoderModel
    from doppler_b200.ops import Device

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
        # the library makes and consumes the rendezvous bytes; the launcher's gloo group carries them
        from doppler_b200 import tp
        box = [tp.make_unique_id(dev) if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        tp.init_group(dev, rank, world, box[0])
        if args.allreduce == "oneshot":
            handles = [None] * world
            dist.all_gather_object(handles, tp.export_exchange(dev))
            tp.attach_exchange(dev, handles)
            dist.barrier()

    B = args.batch
    regions = max(1, args.regions)
    steps_total = args.warmup + regions * args.steps + args.warmup + args.steps
    max_seq = context + steps_total + 64
    model = DecoderModel(dev, cfg, max_seq=max_seq, max_batch=B, tp_rank=rank, tp_size=world)
    if world > 1 and args.allreduce == "oneshot":
        model.set_allreduce_mode(1)
    model.load_synthetic()
    prompts = [synthetic.make_prompt(cfg, context, seq=b) for b in range(B)]

    def barrier():
        dev.sync()
        if dist is not None:
            dist.barrier()

    def prefill_all():
        model.reset()
        return [model.prefill(prompts[b], seq=b) for b in range(B)]

    firsts = prefill_all()
    barrier()

    # ---- device-resident throughput ---------------------------------------------------
    warm = model.decode(firsts, args.warmup)
    nxt = warm[-1].tolist()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    region_ms, launches, crc_tokens = [], 0, [np.asarray(firsts, np.int32).ravel(), warm.ravel()]
    for r in range(regions):
        launches0 = dev.launch_count
        out = model.decode(nxt, args.steps)
        ms_r = model.last_decode_ms
        barrier()
        if dist is not None:
            import torch
            t = torch.tensor([ms_r], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_r = float(t[0])
        region_ms.append(ms_r)
        launches = dev.launch_count - launches0
        nxt = out[-1].tolist()
        if r == 0:
            crc_tokens.append(out.ravel())
        if args.only_timed:
            break
    ms = statistics.median(region_ms)
    tokens = np.concatenate(crc_tokens).astype("<i4")
    crc = zlib.crc32(tokens.tobytes()) & 0xFFFFFFFF
    if dist is not None:  # every rank must have decoded the same tokens
        all_crc = [None] * world
        dist.all_gather_object(all_crc, crc)
        if len(set(all_crc)) != 1:
            raise SystemExit(f"ranks decoded different tokens: crc per rank {all_crc}")

    if args.only_timed:
        if args.kernel_trace:
            kernel_trace(model, dev, nxt, args.steps, args.kernel_trace if rank == 0 else None, barrier, world, B)
        if rank == 0:
            print(json.dumps({"metric": "decode_tokens_per_s", "value": B * args.steps / (ms / 1000.0), "unit": "tokens/s",
                              "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
                              "gpu_launches": int(launches), "tokens_crc": f"{crc:08x}", "note": "first timed region only"}), flush=True)
        if sampler:
            sampler.stop()
        model.destroy()
        dev.close()
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- end to end through the per-token C-ABI call with host buffers -------------------
    cur = prefill_all()
    for _ in range(args.warmup):
        cur = model.decode(cur, 1)[0].tolist()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cur = model.decode(cur, 1)[0].tolist()
    dev.sync()
    e2e_s = time.perf_counter() - t0
    barrier()
    clocks = sampler.stop() if sampler else None

    # ---- dominant kernels: all Q4_K GEMV launches of the decode graph, back to back -------------
    model.bench_gemv(1)
    g = model.bench_gemv(3)
    barrier()

    times = [e2e_s * 1000.0, g["ms"]]
    if dist is not None:
        import torch
        t = torch.tensor(times, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times = t.tolist()
    e2e_ms, gemv_ms = times

    if rank == 0:
        peak = measured_peaks()
        value = B * args.steps / (ms / 1000.0)
        gemv_gbs = g["bytes"] / (gemv_ms / 1000.0) / 1e9
        kv_bytes_step = 2 * B * (context + args.warmup + args.steps * regions // 2) * (cfg["n_kv_heads"] * cfg["head_dim"] // world) * 2 * cfg["n_layers"]
        line = {
            "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": bench_config(args, cfg, context),
            "regions": {"count": len(region_ms), "ms_per_step_median": ms / args.steps, "ms_per_step_min": min(region_ms) / args.steps,
                        "ms_per_step_max": max(region_ms) / args.steps},
            "e2e": {"value": B * args.steps / (e2e_ms / 1000.0), "unit": "tokens/s", "h2d_bytes_per_step": 4096,
                    "d2h_bytes_per_step": 4 * B},
            "gpu_launches": int(launches),
            "tokens_crc": f"{crc:08x}",
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "Q4_K decode GEMV kernels, the instantiations the decode graph launches (RMSNorm / split-merge / silu*up prologues included), all matrices of the model back to back, each reading its predecessor's output",
                         "achieved": gemv_gbs, "peak": peak["hbm_gbs"], "peak_source": peak["source"], "unit": "GB/s",
                         "frac": gemv_gbs / peak["hbm_gbs"], "frac_of_nominal_8000": gemv_gbs / 8000.0,
                         "launches": g["launches"], "avg_launch_us": gemv_ms * 1000.0 / max(g["launches"], 1),
                         "bytes_per_launch_avg": g["bytes"] / max(g["launches"], 1),
                         "traffic": GEMV_TRAFFIC_PER_ALGORITHMIC_BYTE * g["bytes"] / max(g["launches"], 1),
                         "traffic_source": "ncu capture of a [12288,4096] launch scaled by bytes"},
            "step_hbm": {"kv_read_GBps": kv_bytes_step / (ms / args.steps / 1000.0) / 1e9,
                         "weights_GBps": model.weight_bytes / (ms / args.steps / 1000.0) / 1e9, "per": "GPU"},
            "model_weight_bytes_per_gpu": model.weight_bytes,
        }
        if world == 1 and B == 1 and not args.no_kernels:
            # whole-model prefill of the same prompt on the same model (host clock around the call, prompt upload and
            # first-token read-back included), a secondary figure like the `kernels` record below
            try:
                times_p = []
                for _ in range(3):
                    model.reset()
                    dev.sync()
                    t0 = time.perf_counter()
                    model.prefill(prompts[0], seq=0)
                    dev.sync()
                    times_p.append((time.perf_counter() - t0) * 1e3)
                pms = statistics.median(times_p)
                line["prefill"] = {"prompt_tokens": context, "ms": pms, "tokens_per_s": context / (pms / 1e3),
                                   "note": "f32 activations, f32-exact product (three tensor-core products per K step)"}
            except Exception as e:
                line["prefill"] = {"failed": str(e)}
        model.destroy()
        model = None
        if world == 1 and not args.no_kernels:
            try:
                line["kernels"] = kernels_record(dev, peak)
            except Exception as e:
                line["kernels"] = {"failed": str(e)}
        if world == 1 and not args.no_cpu_baseline:
            try:
                v, times_cpu, cores, sample = cpu_full_model(cfg, context, steps=3, warmup=1)
                line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample,
                                        "batch": 1, "kernels": cpu_kernel_baselines()}
            except Exception as e:  # the baseline is a reported number, never the product path
                line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
        print(json.dumps(line), flush=True)
    if model is not None:
        model.destroy()
    dev.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
