"""The allocation-free decode-attention entry point (dp_attention_decode_static).

It exists for hosts that may not allocate device memory while they run (plugins called under a
foreign stream capture, workers that only receive buffers and a stream).  The test owns all the
buffers; the entry point gets raw device pointers and the stream, and must give the same numbers as
the regular dp_attention, on two calls in a row (the second with different inputs, so stale split
partials in the shared scratch would show)."""
import ctypes as C

import numpy as np
import pytest

from doppler_b200 import _lib as L
from doppler_b200 import ops, synthetic
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _free_device_bytes():
    import torch

    return torch.cuda.mem_get_info(0)[0]


def _case(dev, seed, B, H, Hkv, D, kv, measure_free=False):
    s = synthetic.key(seed, kv)
    qh, kh, vh = synthetic.normal_f32(s, B * H * D), synthetic.normal_f16(s + 1, B * kv * Hkv * D), synthetic.normal_f16(s + 2, B * kv * Hkv * D)
    q, k, v = dev.tensor_from(qh), dev.tensor_from(kh), dev.tensor_from(vh)
    ref = ops.run_attention(q, k, v, None, H, D, seq_len=1, kv_len=kv, num_kv_heads=Hkv, causal=False, batch=B,
                            kv_batch_stride=kv * Hkv * D)
    expected = dev.read_tensor(ref).ravel()
    out = dev.acquire_buffer(B * H * D * 4, "static_out")
    dev.lib.dp_buf_fill(dev.h, out.h, 0xFF, 0, B * H * D * 4)
    dev.sync()  # the shared scratch must not be in use by an earlier call
    free_before = _free_device_bytes() if measure_free else 0
    st = dev.lib.dp_attention_decode_static(C.c_void_p(dev.stream), q.buffer.device_ptr, k.buffer.device_ptr, v.buffer.device_ptr,
                                            out.device_ptr, B, H, Hkv, D, kv, kv * Hkv * D, 0.0)
    assert st == L.OK, dev.lib.dp_attention_decode_static_error()
    dev.sync()
    if measure_free:  # the call itself took no device memory (the first call on a device resolved the array's address)
        assert _free_device_bytes() == free_before
    got = dev.read_buffer(out, B * H * D * 4).view(np.float32)
    # independent of the pooled path: the oracle's restatement of attentionRef, sequence by sequence
    per = kv * Hkv * D
    ora = np.concatenate([O.attention_f16kv(qh[b * H * D:(b + 1) * H * D], kh[b * per:(b + 1) * per], vh[b * per:(b + 1) * per], 1, kv, H,
                                            Hkv, D, causal=False).ravel() for b in range(B)])
    rms = float(np.sqrt(np.mean(ora.astype(np.float64) ** 2)))
    assert np.all(np.abs(got - ora) <= 1e-3 * np.abs(ora) + 1e-3 * rms), "static-scratch attention differs from the oracle"
    for t in (q, k, v, ref):
        dev.release_buffer(t.buffer)
    dev.release_buffer(out)
    return got, expected


def test_static_scratch_attention_matches_pooled_path(dev):
    for i, (seed, shape) in enumerate(((901, (2, 32, 8, 128, 4096)), (902, (3, 16, 8, 128, 1777)))):
        got, expected = _case(dev, seed, *shape, measure_free=i > 0)
        assert np.all(np.isfinite(got))
        rms = float(np.sqrt(np.mean(expected.astype(np.float64) ** 2)))
        assert np.all(np.abs(got - expected) <= 1e-3 * np.abs(expected) + 1e-3 * rms)
        assert np.array_equal(got, expected), "same kernels, same split: the two paths should agree bit for bit"


def test_static_scratch_limit_is_enforced(dev):
    lib = dev.lib
    assert lib.dp_attention_decode_static_max_scratch() == 2 << 20
    dummy = dev.acquire_buffer(4096, "dummy")
    p = dummy.device_ptr
    # 591 heads of 512 dims, split in two: 591 * 2 * 514 floats of partials = 2.43 MB > the 2 MiB array
    # (rejected before anything is launched, so the dummy pointers are never touched)
    st = lib.dp_attention_decode_static(C.c_void_p(dev.stream), p, p, p, p, 1, 591, 591, 512, 4096, 0, 0.0)
    assert st == L.ERR_UNSUPPORTED and b"built-in array" in lib.dp_attention_decode_static_error()
    st = lib.dp_attention_decode_static(C.c_void_p(dev.stream), p, p, p, None, 1, 8, 8, 128, 16, 0, 0.0)
    assert st == L.ERR_INVALID
    st = lib.dp_attention_decode_static(C.c_void_p(dev.stream), p, p, p, p, 1, 8, 3, 128, 16, 0, 0.0)
    assert st == L.ERR_INVALID
    dev.release_buffer(dummy)
