"""Decode / prefill attention over the f16 KV cache, through the C ABI, against attentionRef."""
import numpy as np
import pytest

from doppler_b200 import ops, synthetic
from oracle import oracle as O
from parity import assert_close

pytestmark = pytest.mark.gpu


def _attn(dev, q, k16, v16, H, D, **opt):
    qt, kt, vt = dev.tensor_from(q.astype(np.float32)), dev.tensor_from(k16), dev.tensor_from(v16)
    out = ops.run_attention(qt, kt, vt, None, H, D, **opt)
    res = dev.read_tensor(out)
    for t in (out, qt, kt, vt):
        dev.release_buffer(t.buffer)
    return res


def test_reference_suite_case(dev):  # tests/kernels/browser/kernel-suite.js:717-733
    Q, K, V = O.lcg_test_data(32, 901), O.lcg_test_data(32, 902), O.lcg_test_data(32, 903)
    k16, v16 = K.astype(np.float16), V.astype(np.float16)
    got = _attn(dev, Q, k16, v16, 2, 8, seq_len=2, kv_len=4, num_kv_heads=1, causal=False)
    exp = O.attention(Q, k16.astype(np.float32), v16.astype(np.float32), 2, 4, 2, 1, 8)
    assert got.shape == (2, 2, 8)
    assert np.all(np.abs(got.ravel() - exp) <= 1e-5 + 1e-4 * np.abs(exp))  # KERNEL_TOLERANCES.attention
    # causal with startPos=2: first query sees keys 0..2, second 0..3
    got = _attn(dev, Q, k16, v16, 2, 8, seq_len=2, kv_len=4, num_kv_heads=1, causal=True, start_pos=2)
    exp = O.attention_f16kv(Q, k16, v16, 2, 4, 2, 1, 8, causal=True, start_pos=2)
    assert np.all(np.abs(got.ravel() - exp) <= 1e-5 + 1e-4 * np.abs(exp))


@pytest.mark.parametrize("H,Hkv,D,kv", [(32, 8, 128, 8192), (16, 8, 128, 700), (32, 8, 128, 1), (8, 8, 128, 257),
                                        (16, 2, 128, 4096), (8, 2, 64, 1000), (6, 3, 32, 333), (4, 4, 256, 129)])
def test_decode_shapes(dev, H, Hkv, D, kv):
    s = synthetic.key(51, H * 1000 + kv)
    q = synthetic.normal_f32(s, H * D)
    k16 = synthetic.normal_f16(s + 1, kv * Hkv * D)
    v16 = synthetic.normal_f16(s + 2, kv * Hkv * D)
    got = _attn(dev, q, k16, v16, H, D, seq_len=1, kv_len=kv, num_kv_heads=Hkv, start_pos=kv - 1)
    exp = O.attention_f16kv(q, k16, v16, 1, kv, H, Hkv, D, causal=True, start_pos=kv - 1)
    assert_close(got, exp, f"decode attention H{H}/Hkv{Hkv}/D{D}/kv{kv}")


def test_config2_batch(dev):
    """BASELINE config 2: batch 32, 32 heads, 8 KV heads, D 128, context 8192 (extension: batch dim)."""
    B, H, Hkv, D, kv = 32, 32, 8, 128, 8192
    s = synthetic.key(synthetic.DEFAULT_SEED, 20)
    q = synthetic.normal_f16(s, B * H * D).astype(np.float32)
    k16 = synthetic.normal_f16(s + 1, B * kv * Hkv * D)
    v16 = synthetic.normal_f16(s + 2, B * kv * Hkv * D)
    got = _attn(dev, q, k16, v16, H, D, seq_len=1, kv_len=kv, num_kv_heads=Hkv, causal=False, batch=B,
                kv_batch_stride=kv * Hkv * D)
    assert got.shape == (B, 1, H, D)
    got = got.reshape(B, H * D)
    n = kv * Hkv * D
    for b in (0, 13, 31):
        exp = O.attention_f16kv(q[b * H * D:(b + 1) * H * D], k16[b * n:(b + 1) * n], v16[b * n:(b + 1) * n], 1, kv, H, Hkv, D,
                                causal=False)
        assert_close(got[b], exp, f"config2 sequence {b}")
    # size-independent property: attention output is a convex combination of V rows
    vmax = np.abs(v16.astype(np.float32)).max()
    assert np.abs(got).max() <= vmax


def _np_attention(q, k16, v16, H, Hkv, D, lo, hi, scale, softcap=0.0):
    """Plain float64 restatement for options the C oracle does not take (softcap, key windows)."""
    q = q.reshape(H, D).astype(np.float64)
    k = k16.reshape(-1, Hkv, D)[lo:hi].astype(np.float64)
    v = v16.reshape(-1, Hkv, D)[lo:hi].astype(np.float64)
    out = np.zeros((H, D))
    for h in range(H):
        s = k[:, h // (H // Hkv), :] @ q[h] * scale
        if softcap > 0:
            s = np.tanh(s / softcap) * softcap
        pr = np.exp(s - s.max())
        out[h] = (pr / pr.sum()) @ v[:, h // (H // Hkv), :]
    return out.ravel()


# Shapes large enough (batch x KV heads x keys) to take the tensor-core decode kernel: GQA groups
# of 1, 3, 4, 8 and 16 heads, both head dims, ragged key counts, several sequences.
@pytest.mark.parametrize("B,H,Hkv,D,kv", [(4, 32, 4, 128, 2500), (8, 8, 8, 64, 777), (2, 64, 4, 128, 5001),
                                          (4, 12, 4, 64, 2400), (5, 16, 4, 128, 2047)])
def test_tensor_core_decode_shapes(dev, B, H, Hkv, D, kv):
    s = synthetic.key(55, B * 100000 + H * 1000 + kv)
    q = synthetic.normal_f32(s, B * H * D)
    n = kv * Hkv * D
    k16, v16 = synthetic.normal_f16(s + 1, B * n), synthetic.normal_f16(s + 2, B * n)
    got = _attn(dev, q, k16, v16, H, D, seq_len=1, kv_len=kv, num_kv_heads=Hkv, causal=False, batch=B,
                kv_batch_stride=n).reshape(B, H * D)
    for b in range(B):
        exp = O.attention_f16kv(q[b * H * D:(b + 1) * H * D], k16[b * n:(b + 1) * n], v16[b * n:(b + 1) * n], 1, kv, H, Hkv, D,
                                causal=False)
        assert_close(got[b], exp, f"tensor-core decode B{B}/H{H}/Hkv{Hkv}/D{D}/kv{kv} sequence {b}")


def test_tensor_core_decode_options(dev):
    """softcap, sliding window and per-sequence lengths on a shape the tensor-core kernel takes"""
    B, H, Hkv, D, kv = 3, 32, 8, 128, 3000
    s = synthetic.key(56, 0)
    q = synthetic.normal_f32(s, B * H * D) * 3.0
    n = kv * Hkv * D
    k16, v16 = synthetic.normal_f16(s + 1, B * n), synthetic.normal_f16(s + 2, B * n)
    scale = 1.0 / np.sqrt(D)
    got = _attn(dev, q, k16, v16, H, D, seq_len=1, kv_len=kv, num_kv_heads=Hkv, start_pos=kv - 1, sliding_window=1001,
                attn_softcap=5.0, batch=B, kv_batch_stride=n).reshape(B, H * D)
    for b in range(B):
        exp = _np_attention(q[b * H * D:(b + 1) * H * D], k16[b * n:(b + 1) * n], v16[b * n:(b + 1) * n], H, Hkv, D, kv - 1001, kv,
                            scale, softcap=5.0)
        assert_close(got[b], exp.astype(np.float32), f"softcap + sliding window, sequence {b}")
    lens_np = np.array([3000, 1, 1777], np.int32)
    lens = dev.tensor_from(lens_np)
    got = _attn(dev, q, k16, v16, H, D, seq_len=1, kv_len=kv, num_kv_heads=Hkv, causal=False, batch=B, kv_batch_stride=n,
                kv_len_buffer=lens.buffer).reshape(B, H * D)
    for b in range(B):
        exp = O.attention_f16kv(q[b * H * D:(b + 1) * H * D], k16[b * n:(b + 1) * n], v16[b * n:(b + 1) * n], 1, int(lens_np[b]), H,
                                Hkv, D, causal=False)
        assert_close(got[b], exp, f"per-sequence kv length {lens_np[b]}")
    dev.release_buffer(lens.buffer)


def test_kv_len_zero_and_kv_len_buffer(dev):
    H, Hkv, D, kv = 8, 2, 128, 512
    s = synthetic.key(52, 0)
    q, k16, v16 = synthetic.normal_f32(s, H * D), synthetic.normal_f16(s + 1, kv * Hkv * D), synthetic.normal_f16(s + 2, kv * Hkv * D)
    got = _attn(dev, q, k16, v16, H, D, seq_len=1, kv_len=0, num_kv_heads=Hkv, causal=False)
    assert np.all(got == 0)  # attention_decode_online_f16kv.wgsl:107-115
    lens = dev.tensor_from(np.array([300], np.int32))
    got = _attn(dev, q, k16, v16, H, D, seq_len=1, kv_len=kv, num_kv_heads=Hkv, causal=False, kv_len_buffer=lens.buffer)
    exp = O.attention_f16kv(q, k16, v16, 1, 300, H, Hkv, D, causal=False)
    assert_close(got, exp, "kvLenBuffer overrides kvLen")
    dev.release_buffer(lens.buffer)


def test_sliding_window_and_kv_start(dev):
    H, Hkv, D, kv, win = 8, 4, 128, 600, 128
    s = synthetic.key(53, 0)
    q, k16, v16 = synthetic.normal_f32(s, H * D), synthetic.normal_f16(s + 1, kv * Hkv * D), synthetic.normal_f16(s + 2, kv * Hkv * D)
    got = _attn(dev, q, k16, v16, H, D, seq_len=1, kv_len=kv, num_kv_heads=Hkv, start_pos=kv - 1, sliding_window=win)
    n = Hkv * D
    exp = O.attention_f16kv(q, k16[(kv - win) * n:], v16[(kv - win) * n:], 1, win, H, Hkv, D, causal=False)
    assert_close(got, exp, "sliding window keeps the last `win` keys")


def test_prefill_causal(dev):
    H, Hkv, D, T = 16, 8, 128, 96
    s = synthetic.key(54, 0)
    q = synthetic.normal_f32(s, T * H * D)
    k16, v16 = synthetic.normal_f16(s + 1, (T + 32) * Hkv * D), synthetic.normal_f16(s + 2, (T + 32) * Hkv * D)
    got = _attn(dev, q, k16, v16, H, D, seq_len=T, kv_len=T + 32, num_kv_heads=Hkv, causal=True, start_pos=32)
    exp = O.attention_f16kv(q, k16, v16, T, T + 32, H, Hkv, D, causal=True, start_pos=32)
    assert_close(got, exp, "prefill attention, causal with startPos")


@pytest.mark.parametrize("H,Hkv,D,T,start", [(32, 8, 128, 130, 0), (8, 8, 64, 33, 17), (16, 2, 128, 64, 500)])
def test_prefill_rows_on_tensor_cores(dev, H, Hkv, D, T, start):
    """seq_len > 1: every query row is its own causal problem (attention_streaming_f16kv.wgsl:96)"""
    s = synthetic.key(57, H * 1000 + T)
    kv = start + T
    q = synthetic.normal_f32(s, T * H * D)
    k16, v16 = synthetic.normal_f16(s + 1, kv * Hkv * D), synthetic.normal_f16(s + 2, kv * Hkv * D)
    got = _attn(dev, q, k16, v16, H, D, seq_len=T, kv_len=kv, num_kv_heads=Hkv, causal=True, start_pos=start)
    exp = O.attention_f16kv(q, k16, v16, T, kv, H, Hkv, D, causal=True, start_pos=start)
    assert_close(got, exp, f"prefill rows H{H}/Hkv{Hkv}/D{D}/T{T}/start{start}")


@pytest.mark.parametrize("H,Hkv,T,start", [(32, 8, 1024, 0), (8, 8, 257, 3), (16, 8, 100, 1000), (8, 1, 77, 0), (32, 8, 4096, 0)])
def test_prefill_query_tiled(dev, H, Hkv, T, start):
    """Causal prefill on the query-tiled kernel (head_dim 128, groups of 1 / 2 / 4 / 8 heads per KV head):
    tiles of query positions share each K / V tile; ragged last tiles, a start position inside the cache,
    and the BASELINE prompt lengths.  Semantics: tests/kernels/reference/attention.js:129-151.  At T = 4096
    the oracle checks a sample of the rows (every row of the first and the last tile, every 37th between)."""
    D = 128
    s = synthetic.key(58, H * 10000 + T)
    kv = start + T
    q = synthetic.normal_f32(s, T * H * D)
    k16, v16 = synthetic.normal_f16(s + 1, kv * Hkv * D), synthetic.normal_f16(s + 2, kv * Hkv * D)
    got = np.asarray(_attn(dev, q, k16, v16, H, D, seq_len=T, kv_len=kv, num_kv_heads=Hkv, causal=True, start_pos=start)).reshape(T, H * D)
    if T <= 1024:
        exp = np.asarray(O.attention_f16kv(q, k16, v16, T, kv, H, Hkv, D, causal=True, start_pos=start)).reshape(T, H * D)
        assert_close(got, exp, f"query-tiled prefill H{H}/Hkv{Hkv}/T{T}/start{start}")
    else:
        rows = sorted(set(list(range(0, 32)) + list(range(T - 32, T)) + list(range(0, T, 37))))
        qm = q.reshape(T, H * D)
        for r in rows:  # a single query row at position start + r sees keys 0 .. start + r
            exp = O.attention_f16kv(qm[r], k16, v16, 1, start + r + 1, H, Hkv, D, causal=True, start_pos=start + r)
            assert_close(got[r], np.asarray(exp).ravel(), f"query-tiled prefill row {r} of {T}")


def test_attention_argument_errors(dev):
    q = dev.tensor_from(np.zeros(8 * 128, np.float32))
    kv = dev.tensor_from(np.zeros(16 * 2 * 128, np.float16))
    with pytest.raises(ops.DopplerError):
        ops.run_attention(q, kv, kv, None, 8, 128, kv_len=17, num_kv_heads=2)  # cache too small
    with pytest.raises(ops.DopplerError):
        ops.run_attention(q, kv, kv, None, 8, 128, kv_len=16, num_kv_heads=3)  # heads not divisible
    with pytest.raises(ops.DopplerError):
        ops.run_attention(q, kv, kv, None, 8, 128, kv_len=16, num_kv_heads=2, kv_layout="paged")
    with pytest.raises(ops.DopplerError):
        ops.run_attention(kv, kv, kv, None, 8, 128, kv_len=16, num_kv_heads=2)  # Q must be f32
    dev.release_buffer(q.buffer)
    dev.release_buffer(kv.buffer)
