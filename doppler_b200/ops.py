"""Host-side mirror of the reference's kernel-layer op surface.

Same names, argument order and error behaviour as ``src/gpu/kernels/index.js`` of
clocksmith/doppler (``runMatmul`` -> :func:`run_matmul`, ``recordMatmul`` ->
:func:`record_matmul`, ...), with the three data types it passes around
(``Tensor`` src/gpu/tensor.js:7-19, ``WeightBuffer`` src/gpu/weight-buffer.js:78-115
and pooled buffers src/memory/buffer-pool.js:815-869).  Every function is a thin
call into the C ABI; all arithmetic happens in the CUDA library.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

from . import _lib as L
from ._lib import DopplerError

QK_K = 256
Q4K_BLOCK_BYTES = 144


# ------------------------------------------------------------------------------
# device, buffers, tensors
# ------------------------------------------------------------------------------
class Device:
    """One CUDA context + stream + buffer pool (reference: src/gpu/device.js, buffer-pool.js)."""

    def __init__(self, index: int = 0):
        self.lib = L.load()
        h = C.c_void_p()
        st = self.lib.dp_ctx_create(index, C.byref(h))
        if st != L.OK:
            raise DopplerError(st, f"cannot open CUDA device {index} (no CPU fallback exists)")
        self.h = h
        self.index = index

    # -- error plumbing
    def check(self, st: int):
        if st != L.OK:
            raise DopplerError(st, (self.lib.dp_last_error(self.h) or b"").decode())

    def close(self):
        if self.h:
            self.lib.dp_ctx_destroy(self.h)
            self.h = None

    def sync(self):
        self.check(self.lib.dp_ctx_sync(self.h))

    @property
    def launch_count(self) -> int:
        return int(self.lib.dp_ctx_launch_count(self.h))

    @property
    def stream(self) -> int:
        return int(self.lib.dp_ctx_stream(self.h) or 0)

    # -- pool (acquireBuffer / releaseBuffer / uploadData / readBuffer)
    def acquire_buffer(self, size: int, label: str = "pooled_buffer") -> "Buffer":
        h = C.c_void_p()
        self.check(self.lib.dp_buf_acquire(self.h, int(size), label.encode(), C.byref(h)))
        return Buffer(self, h, int(size), label)

    def release_buffer(self, buf: "Buffer"):
        self.check(self.lib.dp_buf_release(self.h, buf.h))

    def upload_data(self, buf: "Buffer", data, offset: int = 0):
        a = np.ascontiguousarray(data)
        self.check(self.lib.dp_buf_upload(self.h, buf.h, a.ctypes.data_as(C.c_void_p), int(offset), a.nbytes))

    def read_buffer(self, buf: "Buffer", size: Optional[int] = None, offset: int = 0) -> np.ndarray:
        n = buf.size - offset if size is None else int(size)
        out = np.empty(n, np.uint8)
        self.check(self.lib.dp_buf_read(self.h, buf.h, out.ctypes.data_as(C.c_void_p), int(offset), n))
        return out

    def pool_stats(self) -> dict:
        s = L.PoolStats()
        self.check(self.lib.dp_pool_get_stats(self.h, C.byref(s)))
        return {n: int(getattr(s, n)) for n, _ in L.PoolStats._fields_}

    def pool_trim(self):
        self.check(self.lib.dp_pool_trim(self.h))

    # -- convenience
    def tensor_from(self, array, dtype: Optional[str] = None, label: str = "tensor") -> "Tensor":
        a = np.ascontiguousarray(array)
        if dtype is None:
            dtype = {np.dtype(np.float32): "f32", np.dtype(np.float16): "f16", np.dtype(np.int32): "i32"}[a.dtype]
        buf = self.acquire_buffer(max(a.nbytes, 4), label)
        if a.nbytes:
            self.upload_data(buf, a)
        return create_tensor(buf, dtype, list(a.shape), label)

    def weight_from(self, array, dtype: str, shape: Sequence[int], label: str = "weight") -> "WeightBuffer":
        a = np.ascontiguousarray(array)
        buf = self.acquire_buffer(max(a.nbytes, 4), label)
        if a.nbytes:
            self.upload_data(buf, a)
        return create_weight_buffer(buf, dtype, "row", list(shape), label)

    def read_tensor(self, t: "Tensor") -> np.ndarray:
        n = int(np.prod(t.shape)) if len(t.shape) else 1
        raw = self.read_buffer(t.buffer, n * L.DTYPE_BYTES[t.dtype], t.offset)
        np_dt = {"f32": np.float32, "f16": np.float16, "i32": np.int32}[t.dtype]
        return raw.view(np_dt).reshape(t.shape)


@dataclass
class Buffer:
    device: Device
    h: C.c_void_p
    size: int
    label: str = ""

    @property
    def capacity(self) -> int:
        return int(self.device.lib.dp_buf_capacity(self.h))

    @property
    def device_ptr(self) -> int:
        return int(self.device.lib.dp_buf_device_ptr(self.h) or 0)


@dataclass
class Tensor:
    buffer: Buffer
    dtype: str
    shape: list
    label: str = ""
    offset: int = 0

    def c(self) -> L.TensorS:
        s = L.TensorS()
        s.buf = self.buffer.h
        s.offset = self.offset
        s.dtype = L.DTYPE_CODES[self.dtype]
        s.ndim = len(self.shape)
        for i, d in enumerate(self.shape[:4]):
            s.shape[i] = int(d)
        return s


@dataclass
class WeightBuffer:
    buffer: Buffer
    dtype: str  # 'q4k' | 'f16' | 'f32'
    layout: str  # 'row' | 'column'
    shape: list  # [N, K]
    label: str = ""
    offset: int = 0
    materializations: dict = field(default_factory=dict)

    def c(self) -> L.WeightS:
        s = L.WeightS()
        s.buf = self.buffer.h
        s.offset = self.offset
        s.dtype = L.DTYPE_CODES[self.dtype]
        s.layout = 0 if self.layout == "row" else 1
        s.shape[0], s.shape[1] = int(self.shape[0]), int(self.shape[1])
        return s


def create_tensor(buffer: Buffer, dtype: str, shape, label: str = "") -> Tensor:
    """reference: createTensor, src/gpu/tensor.js:7"""
    if dtype not in ("f16", "f32", "i32"):
        raise DopplerError(L.ERR_INVALID, f"createTensor: unsupported dtype {dtype}")
    return Tensor(buffer, dtype, list(shape), label)


def create_weight_buffer(buffer: Buffer, dtype: str, layout: str, shape, label: str = "") -> WeightBuffer:
    """reference: createWeightBuffer, src/gpu/weight-buffer.js:78"""
    if dtype not in ("q4k", "f16", "f32"):
        raise DopplerError(L.ERR_INVALID, f"createWeightBuffer: unsupported dtype {dtype}")
    if layout not in ("row", "column"):
        raise DopplerError(L.ERR_INVALID, f"createWeightBuffer: unknown layout {layout}")
    return WeightBuffer(buffer, dtype, layout, list(shape), label)


def _wrap(dev: Device, s: L.TensorS, out_buf: Optional[Buffer], label: str) -> Tensor:
    shape = [int(s.shape[i]) for i in range(s.ndim)]
    dtype = L.DTYPE_NAMES[s.dtype]
    if out_buf is not None:
        buf = out_buf
    else:
        n = int(np.prod(shape)) if shape else 1
        buf = Buffer(dev, C.c_void_p(s.buf), n * L.DTYPE_BYTES[dtype], label)
    return Tensor(buf, dtype, shape, label, int(s.offset))


# ------------------------------------------------------------------------------
# recorder
# ------------------------------------------------------------------------------
class CommandRecorder:
    """reference: CommandRecorder, src/gpu/command-recorder.js:14.  Ops recorded with
    ``record_*`` run in order on the device stream; with ``capture_graph`` the whole
    recording becomes one replayable CUDA graph."""

    def __init__(self, device: Device, label: str = "recorder", capture_graph: bool = False):
        self.device = device
        h = C.c_void_p()
        device.check(device.lib.dp_recorder_begin(device.h, label.encode(), 1 if capture_graph else 0, C.byref(h)))
        self.h = h

    def track_temporary_buffer(self, buf: Buffer):
        self.device.check(self.device.lib.dp_recorder_track_temporary(self.h, buf.h))

    @property
    def op_count(self) -> int:
        return int(self.device.lib.dp_recorder_op_count(self.h))

    def submit(self):
        h, self.h = self.h, None
        self.device.check(self.device.lib.dp_recorder_submit(h))

    def submit_and_wait(self):
        h, self.h = self.h, None
        self.device.check(self.device.lib.dp_recorder_submit_and_wait(h))

    def abort(self):
        h, self.h = self.h, None
        if h:
            self.device.check(self.device.lib.dp_recorder_abort(h))

    def finish_graph(self) -> "Graph":
        h, self.h = self.h, None
        g = C.c_void_p()
        self.device.check(self.device.lib.dp_recorder_finish_graph(h, C.byref(g)))
        return Graph(self.device, g)


class Graph:
    def __init__(self, device: Device, h):
        self.device, self.h = device, h

    def launch(self):
        self.device.check(self.device.lib.dp_graph_launch(self.h))

    def launch_timed(self, reps: int = 1) -> float:
        """Device time in ms of `reps` replays (CUDA events on the context's stream; synchronises)."""
        ms = C.c_double()
        self.device.check(self.device.lib.dp_graph_launch_timed(self.h, reps, C.byref(ms)))
        return float(ms.value)

    def destroy(self):
        if self.h:
            self.device.lib.dp_graph_destroy(self.h)
            self.h = None


def _rec(recorder: Optional[CommandRecorder]):
    return recorder.h if recorder is not None else None


# ------------------------------------------------------------------------------
# ops
# ------------------------------------------------------------------------------
def record_matmul(recorder, A: Tensor, B: WeightBuffer, M: int, N: int, K: int, *, alpha: float = 1.0,
                  output_buffer: Optional[Buffer] = None, transpose_b=True, a_offset: int = 0, b_offset: int = 0,
                  c_offset: int = 0, output_dtype: Optional[str] = None, exact_weights: bool = False, f16_weights: bool = False,
                  **_ignored) -> Tensor:
    """reference: recordMatmul, src/gpu/kernels/matmul.js:664 (options matmul.d.ts:20-87)"""
    dev = A.buffer.device
    if output_dtype is None:
        raise DopplerError(L.ERR_INVALID, "matmul: outputDtype is required ('f16' or 'f32')")
    if output_dtype not in ("f16", "f32"):
        raise DopplerError(L.ERR_INVALID, f"matmul: outputDtype must be 'f16' or 'f32', got {output_dtype}")
    o = L.MatmulOpts()
    dev.lib.dp_matmul_opts_default(C.byref(o))
    o.alpha = alpha
    o.out_dtype = L.DTYPE_CODES[output_dtype]
    o.a_off, o.b_off, o.c_off = a_offset, b_offset, c_offset
    o.out_buf = output_buffer.h if output_buffer is not None else None
    o.transpose_b = 1 if transpose_b in (True, "auto") else 0
    o.exact_weights = 1 if exact_weights else 0
    o.f16_weights = 1 if f16_weights else 0  # opt-in: the reference's tiled f16 prefill kernel's numerics
    a, b, out = A.c(), B.c(), L.TensorS()
    dev.check(dev.lib.dp_matmul(dev.h, _rec(recorder), C.byref(a), C.byref(b), M, N, K, C.byref(o), C.byref(out)))
    return _wrap(dev, out, output_buffer, "matmul_output")


def run_matmul(A, B, M, N, K, **options) -> Tensor:
    """reference: runMatmul, src/gpu/kernels/matmul.js:659"""
    return record_matmul(None, A, B, M, N, K, **options)


def record_dequantize(recorder, quantized: Buffer, num_blocks: int, *, output_offset: int = 0,
                      output_buffer: Optional[Buffer] = None, output_dtype: str = "f32", input_offset: int = 0) -> Tensor:
    """reference: recordDequantize, src/gpu/kernels/dequant.js:455"""
    dev = quantized.device
    out = L.TensorS()
    dev.check(dev.lib.dp_dequant_q4k(dev.h, _rec(recorder), quantized.h, input_offset, num_blocks,
                                     L.DTYPE_CODES[output_dtype], output_offset,
                                     output_buffer.h if output_buffer is not None else None, C.byref(out)))
    return _wrap(dev, out, output_buffer, "dequant_output")


def dequantize(quantized: Buffer, num_blocks: int, **options) -> Tensor:
    """reference: dequantize, src/gpu/kernels/dequant.js:90"""
    return record_dequantize(None, quantized, num_blocks, **options)


def dequantize_rowwise(quantized: Buffer, rows: int, K: int, *, output_buffer: Optional[Buffer] = None,
                       output_dtype: str = "f32", input_offset: int = 0, recorder=None) -> Tensor:
    """reference: dequantizeRowwise, src/gpu/kernels/dequant.js:162"""
    dev = quantized.device
    out = L.TensorS()
    dev.check(dev.lib.dp_dequant_q4k_rowwise(dev.h, _rec(recorder), quantized.h, input_offset, rows, K,
                                             L.DTYPE_CODES[output_dtype],
                                             output_buffer.h if output_buffer is not None else None, C.byref(out)))
    return _wrap(dev, out, output_buffer, "dequant_output")


def record_attention(recorder, Q: Tensor, K: Tensor, V: Tensor, mask, num_heads: int, head_dim: int, *,
                     seq_len: int = 1, kv_len: Optional[int] = None, num_kv_heads: Optional[int] = None,
                     scale: Optional[float] = None, causal: bool = True, start_pos: int = 0, sliding_window: int = 0,
                     attn_softcap: float = 0.0, kv_len_buffer: Optional[Buffer] = None, kv_start: int = 0,
                     kv_layout: str = "contiguous", batch: int = 1, kv_batch_stride: int = 0,
                     output_buffer: Optional[Buffer] = None, **_ignored) -> Tensor:
    """reference: recordAttention, src/gpu/kernels/attention.js:2019 (options attention.d.ts:18-50)"""
    dev = Q.buffer.device
    if mask is not None:
        raise DopplerError(L.ERR_UNSUPPORTED, "attention: explicit mask tensors are outside this path (use causal/startPos)")
    if kv_layout != "contiguous":
        raise DopplerError(L.ERR_UNSUPPORTED, f"attention: kvLayout '{kv_layout}' is outside this path (contiguous f16 only)")
    if kv_len is None:
        raise DopplerError(L.ERR_INVALID, "attention: kvLen is required")
    o = L.AttnOpts()
    dev.lib.dp_attn_opts_default(C.byref(o))
    o.seq_len, o.kv_len = seq_len, kv_len
    o.num_kv_heads = num_kv_heads if num_kv_heads is not None else num_heads
    o.scale = scale if scale is not None else 0.0
    o.causal = 1 if causal else 0
    o.start_pos, o.sliding_window, o.attn_softcap, o.kv_start = start_pos, sliding_window, attn_softcap, kv_start
    o.batch, o.kv_batch_stride = batch, kv_batch_stride
    o.kv_lens = kv_len_buffer.h if kv_len_buffer is not None else None
    o.out_buf = output_buffer.h if output_buffer is not None else None
    q, k, v, out = Q.c(), K.c(), V.c(), L.TensorS()
    dev.check(dev.lib.dp_attention(dev.h, _rec(recorder), C.byref(q), C.byref(k), C.byref(v), num_heads, head_dim,
                                   C.byref(o), C.byref(out)))
    return _wrap(dev, out, output_buffer, "attention_output")


def run_attention(Q, K, V, mask, num_heads, head_dim, **options) -> Tensor:
    """reference: runAttention, src/gpu/kernels/attention.js:2007"""
    return record_attention(None, Q, K, V, mask, num_heads, head_dim, **options)


def record_rmsnorm(recorder, input: Tensor, weight: Tensor, eps: float, *, batch_size: int = 1,
                   hidden_size: Optional[int] = None, residual: Optional[Tensor] = None, pre_residual: bool = False,
                   residual_sum_output: Optional[Buffer] = None, rms_norm_weight_offset: bool = False,
                   output_scale: float = 1.0, output_buffer: Optional[Buffer] = None) -> Tensor:
    """reference: recordRMSNorm, src/gpu/kernels/rmsnorm.js:224"""
    dev = input.buffer.device
    if hidden_size is None:
        raise DopplerError(L.ERR_INVALID, "rmsnorm: hiddenSize is required")
    o = L.RmsNormOpts()
    dev.lib.dp_rmsnorm_opts_default(C.byref(o))
    o.batch_size, o.hidden_size = batch_size, hidden_size
    res_c = residual.c() if residual is not None else None
    o.residual = C.pointer(res_c) if res_c is not None else None
    o.pre_residual = 1 if pre_residual else 0
    o.residual_sum_output = residual_sum_output.h if residual_sum_output is not None else None
    o.weight_offset = 1 if rms_norm_weight_offset else 0
    o.output_scale = output_scale
    o.out_buf = output_buffer.h if output_buffer is not None else None
    i, w, out = input.c(), weight.c(), L.TensorS()
    dev.check(dev.lib.dp_rmsnorm(dev.h, _rec(recorder), C.byref(i), C.byref(w), eps, C.byref(o), C.byref(out)))
    return _wrap(dev, out, output_buffer, "rmsnorm_output")


def run_rmsnorm(input, weight, eps, **options) -> Tensor:
    """reference: runRMSNorm, src/gpu/kernels/rmsnorm.js:146"""
    return record_rmsnorm(None, input, weight, eps, **options)


def run_rmsnorm_qk(q: Tensor, q_weight: Tensor, k: Tensor, k_weight: Tensor, *, q_rows: int, k_rows: int,
                   head_dim: int, eps: float, rms_norm_weight_offset: bool = False, recorder=None):
    """reference: runRMSNormQK, src/gpu/kernels/rmsnorm-qk.js (in place)"""
    dev = q.buffer.device
    qc, qw, kc, kw = q.c(), q_weight.c(), k.c(), k_weight.c()
    dev.check(dev.lib.dp_rmsnorm_qk(dev.h, _rec(recorder), C.byref(qc), C.byref(qw), C.byref(kc), C.byref(kw),
                                    q_rows, k_rows, head_dim, eps, 1 if rms_norm_weight_offset else 0))


def record_rope(recorder, input: Tensor, freqs_cos: Tensor, freqs_sin: Tensor, seq_len: int, *, num_heads: int,
                head_dim: int, rotary_dim: Optional[int] = None, pair_span_dim: Optional[int] = None,
                interleaved: bool = False, start_pos: int = 0):
    """reference: recordRoPE, src/gpu/kernels/rope.js:112 (in place)"""
    dev = input.buffer.device
    o = L.RopeOpts(num_heads, head_dim, rotary_dim or 0, pair_span_dim or 0, 1 if interleaved else 0, start_pos)
    i, c, s = input.c(), freqs_cos.c(), freqs_sin.c()
    dev.check(dev.lib.dp_rope(dev.h, _rec(recorder), C.byref(i), C.byref(c), C.byref(s), seq_len, C.byref(o)))
    return input


def run_rope(input, freqs_cos, freqs_sin, seq_len, **options):
    """reference: runRoPE, src/gpu/kernels/rope.js:108"""
    return record_rope(None, input, freqs_cos, freqs_sin, seq_len, **options)


def rope_tables(theta: float, rotary_dim: int, max_seq: int):
    """reference: computeRoPEFreqsForTheta, src/inference/pipelines/text/init-rope.js:11-134 (no scaling)"""
    lib = L.load()
    c = np.empty((max_seq, rotary_dim // 2), np.float32)
    s = np.empty((max_seq, rotary_dim // 2), np.float32)
    st = lib.dp_rope_tables(theta, rotary_dim, max_seq, c.ctypes.data_as(C.c_void_p), s.ctypes.data_as(C.c_void_p))
    if st != L.OK:
        raise DopplerError(st, "rope tables: invalid arguments")
    return c, s


def run_silu(input: Tensor, *, size: int, gate: Optional[Tensor] = None, swiglu_limit: float = 0.0,
             output_buffer: Optional[Buffer] = None, recorder=None) -> Tensor:
    """reference: runSiLU with a gate tensor, src/gpu/kernels/silu.wgsl:98-104: silu(gate) * input"""
    dev = input.buffer.device
    if gate is None:
        raise DopplerError(L.ERR_UNSUPPORTED, "silu: only the gated form silu(gate)*up is on this path")
    u, g, out = input.c(), gate.c(), L.TensorS()
    dev.check(dev.lib.dp_silu_mul(dev.h, _rec(recorder), C.byref(u), C.byref(g), size, swiglu_limit,
                                  output_buffer.h if output_buffer is not None else None, C.byref(out)))
    return _wrap(dev, out, output_buffer, "silu_output")


def run_residual_add(a: Tensor, b: Tensor, size: int, *, scale: float = 1.0, output_buffer: Optional[Buffer] = None,
                     recorder=None) -> Tensor:
    """reference: runResidualAdd, src/gpu/kernels/residual.wgsl:25-32"""
    dev = a.buffer.device
    ac, bc, out = a.c(), b.c(), L.TensorS()
    dev.check(dev.lib.dp_residual_add(dev.h, _rec(recorder), C.byref(ac), C.byref(bc), size, scale,
                                      output_buffer.h if output_buffer is not None else None, C.byref(out)))
    return _wrap(dev, out, output_buffer, "residual_output")


def run_gather(indices: Tensor, embeddings: Tensor, num_tokens: int, hidden_size: int, *,
               output_buffer: Optional[Buffer] = None, recorder=None) -> Tensor:
    """reference: runGather, src/gpu/kernels/gather_f16.wgsl:35-66"""
    dev = indices.buffer.device
    ic, ec, out = indices.c(), embeddings.c(), L.TensorS()
    dev.check(dev.lib.dp_gather_f16(dev.h, _rec(recorder), C.byref(ic), C.byref(ec), num_tokens, hidden_size,
                                    output_buffer.h if output_buffer is not None else None, C.byref(out)))
    return _wrap(dev, out, output_buffer, "gather_output")


def run_kv_cache_write_f32_to_f16(src: Tensor, dst: Buffer, dst_offset_elems: int, n: int, recorder=None):
    """reference: runKVCacheWriteF32ToF16, src/gpu/kernels/kv_cache_write_f32_to_f16.wgsl:19"""
    dev = src.buffer.device
    sc = src.c()
    dev.check(dev.lib.dp_kv_write_f32_to_f16(dev.h, _rec(recorder), C.byref(sc), dst.h, dst_offset_elems, n))


def run_argmax(logits: Tensor, vocab_size: int, *, pad_token_id: int = -1, output_buffer: Optional[Buffer] = None,
               output_index: int = 0, recorder=None) -> Buffer:
    """reference: runArgmax, src/gpu/kernels/sample.wgsl:311-408 (ties -> lower index)"""
    dev = logits.buffer.device
    out = output_buffer if output_buffer is not None else dev.acquire_buffer(4 * (output_index + 1), "argmax_token")
    lc = logits.c()
    dev.check(dev.lib.dp_argmax(dev.h, _rec(recorder), C.byref(lc), vocab_size, pad_token_id, out.h, output_index))
    return out


def quantize_to_q4km_rowwise(data: Tensor, shape, *, output_buffer: Optional[Buffer] = None, recorder=None) -> WeightBuffer:
    """reference: quantizeToQ4KMRowWise(data, shape), src/converter/quantizer.js:253-288 (bit-exact, on the device)"""
    dev = data.buffer.device
    rows, cols = int(shape[0]), int(shape[1])
    d, out = data.c(), L.WeightS()
    dev.check(dev.lib.dp_quantize_q4k(dev.h, _rec(recorder), C.byref(d), rows, cols, 0,
                                      output_buffer.h if output_buffer is not None else None, C.byref(out)))
    nbytes = rows * ((cols + 255) // 256) * 144
    buf = output_buffer if output_buffer is not None else Buffer(dev, C.c_void_p(out.buf), nbytes, "q4k_quantized")
    return create_weight_buffer(buf, "q4k", "row", [rows, cols], "q4k_quantized")


def quantize_to_q4km(data: Tensor, num_elements: int, *, output_buffer: Optional[Buffer] = None, recorder=None) -> WeightBuffer:
    """reference: quantizeToQ4KM(data), src/converter/quantizer.js:223-251 (flat; a short tail is zero padded)"""
    dev = data.buffer.device
    d, out = data.c(), L.WeightS()
    dev.check(dev.lib.dp_quantize_q4k(dev.h, _rec(recorder), C.byref(d), 1, int(num_elements), 1,
                                      output_buffer.h if output_buffer is not None else None, C.byref(out)))
    nbytes = ((num_elements + 255) // 256) * 144
    buf = output_buffer if output_buffer is not None else Buffer(dev, C.c_void_p(out.buf), nbytes, "q4k_quantized")
    return create_weight_buffer(buf, "q4k", "row", [1, int(num_elements)], "q4k_quantized")


# ------------------------------------------------------------------------------
# fused decode ops (src/gpu/kernels/index.js:300-330)
# ------------------------------------------------------------------------------
def record_fused_ffn(recorder, input: Tensor, W_gate: WeightBuffer, W_up: WeightBuffer, hidden_size: int, intermediate_size: int, *,
                     batch_size: int = 1, activation: str = "silu", alpha: float = 1.0, output_buffer: Optional[Buffer] = None,
                     swiglu_limit: Optional[float] = None, **_ignored) -> Tensor:
    """reference: recordFusedFFN, src/gpu/kernels/fused_ffn.js:605"""
    dev = input.buffer.device
    if activation != "silu":
        raise DopplerError(L.ERR_UNSUPPORTED, f"Fused FFN: activation '{activation}' is outside this path (silu)")
    o = L.FfnOpts()
    dev.lib.dp_ffn_opts_default(C.byref(o))
    o.batch_size, o.alpha, o.swiglu_limit = batch_size, alpha, float(swiglu_limit or 0.0)
    o.out_buf = output_buffer.h if output_buffer is not None else None
    i, g, u, out = input.c(), W_gate.c(), W_up.c(), L.TensorS()
    dev.check(dev.lib.dp_fused_ffn(dev.h, _rec(recorder), C.byref(i), C.byref(g), C.byref(u), hidden_size, intermediate_size,
                                   C.byref(o), C.byref(out)))
    return _wrap(dev, out, output_buffer, "fused_ffn_output")


def run_fused_ffn(input, W_gate, W_up, hidden_size, intermediate_size, **options) -> Tensor:
    """reference: runFusedFFN, src/gpu/kernels/fused_ffn.js:501"""
    return record_fused_ffn(None, input, W_gate, W_up, hidden_size, intermediate_size, **options)


def record_matmul_residual_fused(recorder, input: Tensor, weight: WeightBuffer, residual: Tensor, *, N: int, K: int,
                                 alpha: float = 1.0, output_buffer: Optional[Buffer] = None, **_ignored) -> Tensor:
    """reference: recordMatmulResidualFused, src/gpu/kernels/fused_matmul_residual.js:105"""
    dev = input.buffer.device
    i, w, r, out = input.c(), weight.c(), residual.c(), L.TensorS()
    dev.check(dev.lib.dp_matmul_residual(dev.h, _rec(recorder), C.byref(i), C.byref(w), C.byref(r), N, K, alpha,
                                         output_buffer.h if output_buffer is not None else None, C.byref(out)))
    return _wrap(dev, out, output_buffer, "matmul_residual_output")


def run_matmul_residual_fused(input, weight, residual, **options) -> Tensor:
    """reference: runMatmulResidualFused, src/gpu/kernels/fused_matmul_residual.js:27"""
    return record_matmul_residual_fused(None, input, weight, residual, **options)


def record_matmul_rmsnorm_fused(recorder, input: Tensor, weight: WeightBuffer, norm_weight: Tensor, *, N: int, K: int,
                                eps: Optional[float] = None, residual: Optional[Tensor] = None,
                                output_buffer: Optional[Buffer] = None, rms_norm_weight_offset: bool = False, **_ignored) -> Tensor:
    """reference: recordMatmulRMSNormFused, src/gpu/kernels/fused_matmul_rmsnorm.js:171"""
    dev = input.buffer.device
    if eps is None:
        raise DopplerError(L.ERR_INVALID, "[MatmulRMSNormFused] eps is required.")
    i, w, nw, out = input.c(), weight.c(), norm_weight.c(), L.TensorS()
    r = residual.c() if residual is not None else None
    dev.check(dev.lib.dp_matmul_rmsnorm(dev.h, _rec(recorder), C.byref(i), C.byref(w), C.byref(nw), N, K, eps,
                                        C.byref(r) if r is not None else None, 1 if rms_norm_weight_offset else 0,
                                        output_buffer.h if output_buffer is not None else None, C.byref(out)))
    return _wrap(dev, out, output_buffer, "matmul_rmsnorm_output")


def run_matmul_rmsnorm_fused(input, weight, norm_weight, **options) -> Tensor:
    """reference: runMatmulRMSNormFused, src/gpu/kernels/fused_matmul_rmsnorm.js:52"""
    return record_matmul_rmsnorm_fused(None, input, weight, norm_weight, **options)


def record_lm_head_argmax(recorder, input: Tensor, lm_head: WeightBuffer, *, vocab_size: int, hidden_size: int,
                          pad_token_id: int = -1, output_buffer: Optional[Buffer] = None, output_index: int = 0,
                          **_ignored) -> Buffer:
    """reference: recordLmHeadArgmax, src/gpu/kernels/lm-head-argmax.js:292 (returns the token buffer)"""
    dev = input.buffer.device
    out = output_buffer if output_buffer is not None else dev.acquire_buffer(max(4, 4 * (output_index + 1)), "lm_head_argmax_output")
    i, w = input.c(), lm_head.c()
    try:
        dev.check(dev.lib.dp_lm_head_argmax(dev.h, _rec(recorder), C.byref(i), C.byref(w), vocab_size, hidden_size, pad_token_id,
                                            out.h, output_index))
    except DopplerError:
        if output_buffer is None:
            dev.release_buffer(out)
        raise
    return out


# ------------------------------------------------------------------------------
# KV cache
# ------------------------------------------------------------------------------
class KVCache:
    """reference: KVCache (contiguous, f16), src/inference/kv-cache/base.js:18"""

    def __init__(self, device: Device, num_layers: int, max_seq_len: int, num_kv_heads: int, head_dim: int,
                 batch: int = 1, _handle=None):
        self.device = device
        self.num_layers, self.max_seq_len, self.num_kv_heads, self.head_dim, self.batch = (
            num_layers, max_seq_len, num_kv_heads, head_dim, batch)
        if _handle is None:
            h = C.c_void_p()
            device.check(device.lib.dp_kv_cache_create(device.h, num_layers, max_seq_len, num_kv_heads, head_dim, batch,
                                                       C.byref(h)))
            _handle = h
        self.h = _handle

    def layer(self, i: int):
        k, v = C.c_void_p(), C.c_void_p()
        self.device.check(self.device.lib.dp_kv_layer(self.h, i, C.byref(k), C.byref(v)))
        n = self.batch * self.max_seq_len * self.num_kv_heads * self.head_dim * 2
        return Buffer(self.device, k, n, "kv_cache_keys"), Buffer(self.device, v, n, "kv_cache_values")

    @property
    def current_seq_len(self) -> int:
        return int(self.device.lib.dp_kv_seq_len(self.h))

    def set_seq_len(self, n: int):
        self.device.check(self.device.lib.dp_kv_set_seq_len(self.h, n))

    def truncate(self, n: int):
        self.device.check(self.device.lib.dp_kv_truncate(self.h, n))

    def clone(self) -> "KVCache":
        h = C.c_void_p()
        self.device.check(self.device.lib.dp_kv_clone(self.h, C.byref(h)))
        return KVCache(self.device, self.num_layers, self.max_seq_len, self.num_kv_heads, self.head_dim, self.batch, h)

    @property
    def nbytes(self) -> int:
        return int(self.device.lib.dp_kv_bytes(self.h))

    def destroy(self):
        if self.h:
            self.device.lib.dp_kv_cache_destroy(self.h)
            self.h = None
