"""rmsnorm / rope / silu / residual / gather / kv-write / argmax, pool and recorder semantics."""
import numpy as np
import pytest

from doppler_b200 import ops, synthetic
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _close(a, b, rtol, atol):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    assert np.all(np.abs(a - b) <= atol + rtol * np.abs(b)), float(np.abs(a - b).max())


@pytest.mark.parametrize("rows,size", [(1, 1024), (4, 4096), (3, 100), (512, 1024)])
def test_rmsnorm(dev, rows, size):  # KERNEL_TOLERANCES.rmsnorm rtol 1e-5 atol 1e-6
    x = O.lcg_test_data(rows * size, 91)
    w = O.lcg_test_data(size, 92)
    xt, wt = dev.tensor_from(x.reshape(rows, size)), dev.tensor_from(w)
    y = ops.run_rmsnorm(xt, wt, 1e-6, batch_size=rows, hidden_size=size)
    _close(dev.read_tensor(y), O.rmsnorm(x, w, rows, size, 1e-6), 1e-5, 1e-6)
    # (1 + w), output scale, post-norm residual, pre-norm residual with the sum written out
    r = O.lcg_test_data(rows * size, 93)
    rt = dev.tensor_from(r.reshape(rows, size))
    y2 = ops.run_rmsnorm(xt, wt, 1e-6, batch_size=rows, hidden_size=size, rms_norm_weight_offset=True,
                         output_scale=0.5, residual=rt)
    exp = (O.rmsnorm(x, 1 + w, rows, size, 1e-6) + r) * 0.5
    _close(dev.read_tensor(y2), exp, 1e-5, 2e-6)
    sum_buf = dev.acquire_buffer(rows * size * 4, "sum")
    y3 = ops.run_rmsnorm(xt, wt, 1e-6, batch_size=rows, hidden_size=size, residual=rt, pre_residual=True,
                         residual_sum_output=sum_buf)
    _close(dev.read_tensor(y3), O.rmsnorm(x + r, w, rows, size, 1e-6), 1e-5, 1e-6)
    assert np.array_equal(dev.read_buffer(sum_buf, rows * size * 4).view(np.float32), x + r)
    w16 = dev.tensor_from(w.astype(np.float16))
    y4 = ops.run_rmsnorm(xt, w16, 1e-6, batch_size=rows, hidden_size=size)
    _close(dev.read_tensor(y4), O.rmsnorm(x, w.astype(np.float16).astype(np.float32), rows, size, 1e-6), 1e-5, 1e-6)
    for t in (y, y2, y3, y4, xt, wt, rt, w16):
        dev.release_buffer(t.buffer)
    dev.release_buffer(sum_buf)


def test_rmsnorm_qk_and_rope(dev):
    T, H, Hkv, D = 5, 16, 8, 128
    q, k = O.lcg_test_data(T * H * D, 314), O.lcg_test_data(T * Hkv * D, 315)
    qw, kw = 1 + 0.1 * O.lcg_test_data(D, 316), 1 + 0.1 * O.lcg_test_data(D, 317)
    qt, kt, qwt, kwt = dev.tensor_from(q), dev.tensor_from(k), dev.tensor_from(qw), dev.tensor_from(kw)
    ops.run_rmsnorm_qk(qt, qwt, kt, kwt, q_rows=T * H, k_rows=T * Hkv, head_dim=D, eps=1e-6)
    qn, kn = O.rmsnorm(q, qw, T * H, D, 1e-6), O.rmsnorm(k, kw, T * Hkv, D, 1e-6)
    _close(dev.read_tensor(qt), qn, 1e-5, 1e-6)
    _close(dev.read_tensor(kt), kn, 1e-5, 1e-6)
    cos, sin = ops.rope_tables(1e6, D, 64)
    ct, st = dev.tensor_from(cos), dev.tensor_from(sin)
    ops.run_rope(qt, ct, st, T, num_heads=H, head_dim=D, start_pos=7)
    _close(dev.read_tensor(qt), O.rope(dev.read_tensor(qt) * 0 + qn, cos, sin, T, H, D, 7), 1e-5, 2e-6)
    with pytest.raises(ops.DopplerError):
        ops.run_rope(qt, ct, st, T, num_heads=H, head_dim=D, start_pos=60)  # table too short
    # partial rotation (tests/kernels/rope-partial-rotation-reference.test.js): rotaryDim 64 inside D 128
    x = O.lcg_test_data(2 * 4 * D, 318)
    xt = dev.tensor_from(x)
    c2, s2 = ops.rope_tables(1e4, 64, 16)
    c2t, s2t = dev.tensor_from(c2), dev.tensor_from(s2)
    ops.run_rope(xt, c2t, s2t, 2, num_heads=4, head_dim=D, rotary_dim=64, start_pos=3)
    got = dev.read_tensor(xt).reshape(2, 4, D)
    xr = x.reshape(2, 4, D)
    for s in range(2):
        cc, ss = c2[s + 3].astype(np.float64), s2[s + 3].astype(np.float64)
        _close(got[s, :, :32], xr[s, :, :32] * cc - xr[s, :, 32:64] * ss, 1e-5, 2e-6)
        _close(got[s, :, 32:64], xr[s, :, :32] * ss + xr[s, :, 32:64] * cc, 1e-5, 2e-6)
        assert np.array_equal(got[s, :, 64:], xr[s, :, 64:])
    for t in (qt, kt, qwt, kwt, ct, st, xt, c2t, s2t):
        dev.release_buffer(t.buffer)


def test_silu_residual_gather_kvwrite_argmax(dev):
    g, u = O.lcg_test_data(1024, 124) * 40, O.lcg_test_data(1024, 125)
    gt, ut = dev.tensor_from(g), dev.tensor_from(u)
    y = ops.run_silu(ut, size=1024, gate=gt)
    _close(dev.read_tensor(y), O.silu_gated(g, u, clamped=True), 1e-5, 1e-6)
    a, b = O.lcg_test_data(512, 501), O.lcg_test_data(512, 502)
    at, bt = dev.tensor_from(a), dev.tensor_from(b)
    r = ops.run_residual_add(at, bt, 512)
    assert np.array_equal(dev.read_tensor(r), a + b)  # KERNEL_TOLERANCES.residual is ~exact
    emb = synthetic.normal_f16(synthetic.key(61, 0), 100 * 64).reshape(100, 64)
    ids = np.array([3, 99, 0, 42], np.int32)
    et, it = dev.tensor_from(emb), dev.tensor_from(ids)
    gth = ops.run_gather(it, et, 4, 64)
    assert np.array_equal(dev.read_tensor(gth), emb[ids].astype(np.float32))  # gather is exact
    cache = dev.acquire_buffer(4096 * 2, "cache")
    src = O.lcg_test_data(1024, 77) * 100
    srt = dev.tensor_from(src)
    ops.run_kv_cache_write_f32_to_f16(srt, cache, 512, 1024)
    got = dev.read_buffer(cache, 2048, 1024).view(np.float16)
    assert np.array_equal(got.view(np.uint16), src.astype(np.float16).view(np.uint16))
    with pytest.raises(ops.DopplerError):
        ops.run_kv_cache_write_f32_to_f16(srt, cache, 3584, 1024)  # runs past the cache
    logits = O.lcg_test_data(151936, 9)
    logits[[777, 90000]] = 5.0  # a tie: the lower index must win
    lt = dev.tensor_from(logits)
    tok = ops.run_argmax(lt, 151936)
    assert int(dev.read_buffer(tok, 4).view(np.int32)[0]) == 777 == O.argmax(logits)
    tok2 = ops.run_argmax(lt, 151936, pad_token_id=777)
    assert int(dev.read_buffer(tok2, 4).view(np.int32)[0]) == 90000
    for t in (y, gt, ut, r, at, bt, et, it, gth, srt, lt):
        dev.release_buffer(t.buffer)
    for bf in (cache, tok, tok2):
        dev.release_buffer(bf)


def test_pool_semantics(dev):  # src/memory/buffer-pool.js:249 acquire / release / reuse
    s0 = dev.pool_stats()
    a = dev.acquire_buffer(1000, "a")
    assert a.capacity == 1024
    dev.release_buffer(a)
    s1 = dev.pool_stats()
    b = dev.acquire_buffer(900, "b")  # same 1024-byte bucket: served from the pool, no new allocation
    s2 = dev.pool_stats()
    assert s2["reuses"] == s1["reuses"] + 1 and s2["allocations"] == s1["allocations"] and b.capacity == 1024
    assert s1["releases"] == s0["releases"] + 1
    dev.release_buffer(b)
    with pytest.raises(ops.DopplerError):
        dev.release_buffer(b)  # double release
    with pytest.raises(ops.DopplerError):
        dev.upload_data(b, np.zeros(4, np.float32))  # released buffer
    c = dev.acquire_buffer(16, "c")
    with pytest.raises(ops.DopplerError):
        dev.upload_data(c, np.zeros(1000, np.float32))  # overflow
    data = np.arange(4, dtype=np.int32)
    dev.upload_data(c, data)
    assert np.array_equal(dev.read_buffer(c, 16).view(np.int32), data)
    dev.release_buffer(c)


def test_recorder_and_graph(dev):  # src/gpu/command-recorder.js:14,419,560
    a, b = O.lcg_test_data(4096, 1), O.lcg_test_data(4096, 2)
    at, bt = dev.tensor_from(a), dev.tensor_from(b)
    out = dev.acquire_buffer(4096 * 4, "out")
    rec = ops.CommandRecorder(dev, "test")
    tmp = ops.run_residual_add(at, bt, 4096, recorder=rec)
    rec.track_temporary_buffer(tmp.buffer)
    ops.run_residual_add(tmp, bt, 4096, output_buffer=out, recorder=rec)
    assert rec.op_count == 2
    rec.submit_and_wait()
    assert np.array_equal(dev.read_buffer(out, 4096 * 4).view(np.float32), (a + b) + b)
    with pytest.raises(ops.DopplerError):
        dev.release_buffer(tmp.buffer)  # the recorder already returned it to the pool
    # graph capture + replay: out = out + b each launch
    ot = ops.create_tensor(out, "f32", [4096])
    rec = ops.CommandRecorder(dev, "graph", capture_graph=True)
    ops.run_residual_add(ot, bt, 4096, output_buffer=out, recorder=rec)
    graph = rec.finish_graph()
    before = dev.launch_count
    for _ in range(3):
        graph.launch()
    dev.sync()
    assert dev.launch_count == before + 3
    exp = (a + b) + b
    for _ in range(3):
        exp = exp + b
    assert np.array_equal(dev.read_buffer(out, 4096 * 4).view(np.float32), exp)
    graph.destroy()
    rec = ops.CommandRecorder(dev, "aborted")
    with pytest.raises(ops.DopplerError):
        ops.CommandRecorder(dev, "second")  # one open recorder per context
    rec.abort()
    for bf in (at.buffer, bt.buffer, out):
        dev.release_buffer(bf)


def test_kv_cache_allocator(dev):  # src/inference/kv-cache/base.js:99-153, :829, :962
    kv = ops.KVCache(dev, 2, 64, 2, 128)
    assert kv.nbytes == 2 * 2 * 64 * 2 * 128 * 2
    k0, v0 = kv.layer(0)
    src = O.lcg_test_data(2 * 128 * 3, 5)
    st = dev.tensor_from(src)
    ops.run_kv_cache_write_f32_to_f16(st, k0, 0, src.size)
    kv.set_seq_len(3)
    clone = kv.clone()
    assert clone.current_seq_len == 3
    ck0, _ = clone.layer(0)
    assert np.array_equal(dev.read_buffer(ck0, src.size * 2), dev.read_buffer(k0, src.size * 2))
    kv.truncate(1)
    assert kv.current_seq_len == 1 and clone.current_seq_len == 3
    kv.truncate(10)
    assert kv.current_seq_len == 1  # truncate never grows
    with pytest.raises(ops.DopplerError):
        kv.set_seq_len(65)
    with pytest.raises(ops.DopplerError):
        kv.layer(2)
    clone.destroy()
    kv.destroy()
    dev.release_buffer(st.buffer)
