"""Pins the CPU oracle to the reference.

Reference-produced numbers: the reference's retained 9B receipt
(reports/qwen-3-5-9b-metal/2026-07-12/layer0-ffn-gate-oracle.json) records the sha256 of the
decoded scales and minima its own dequantiser produced for the 196,608 block headers of a real
[12288, 4096] Q4_K tensor; the headers are committed under tests/golden/ and the oracle must
reproduce both digests (test_receipt_* below).  Beyond that the reference's JavaScript cannot
run here, so the oracle is also pinned three ways:
 1. the reference's own procedural unit tests are re-run against it (same inputs,
    same assertions): tests/converter/quantizer.test.js, tests/gpu/dequant-numeric.test.js,
    tests/tooling/q4k-projection-reference.test.js, tests/kernels/browser/kernel-suite.js;
 2. a second, independent transliteration of the JavaScript (pure Python floats are
    the same IEEE doubles as JS numbers) must agree bit for bit on those inputs;
 3. hand-derived known answers for the 144-byte layout.
"""
import math
import struct

import numpy as np

from oracle import oracle as O

QK_K, BLOCK = 256, 144


# ---- independent transliteration of src/converter/quantizer.js (pure Python) ------------
def _f32(x):
    return struct.unpack("<f", struct.pack("<f", x))[0]


def py_f32_to_f16(value):
    f = struct.unpack("<I", struct.pack("<f", value))[0]
    sign, exp, frac = (f >> 31) & 1, (f >> 23) & 0xFF, f & 0x7FFFFF
    if exp == 0xFF:
        return (sign << 15) | 0x7C00 | (0x200 if frac else 0)
    if exp == 0:
        return sign << 15
    exp = exp - 127 + 15
    if exp >= 31:
        return (sign << 15) | 0x7C00
    if exp <= 0:
        if exp < -10:
            return sign << 15
        frac = (frac | 0x800000) >> (1 - exp)
        return (sign << 15) | (frac >> 13)
    return (sign << 15) | (exp << 10) | (frac >> 13)


def py_f16_to_f32(h):
    sign, exp, frac = (h >> 15) & 1, (h >> 10) & 0x1F, h & 0x3FF
    if exp == 0:
        if frac == 0:
            return -0.0 if sign else 0.0
        return (-1 if sign else 1) * 2.0 ** -14 * (frac / 1024)
    if exp == 31:
        return math.nan if frac else (-math.inf if sign else math.inf)
    return (-1 if sign else 1) * 2.0 ** (exp - 15) * (1 + frac / 1024)


def py_quantize_block(data, valid=QK_K):
    block = bytearray(BLOCK)
    scales, mins, q = [0.0] * 8, [0.0] * 8, [0] * 256
    for sb in range(8):
        n = max(0, min(32, valid - sb * 32))
        if n == 0:
            continue
        seg = [float(v) for v in data[sb * 32: sb * 32 + n]]
        mn, mx = min(seg), max(seg)
        mins[sb] = _f32(-mn)
        rng = mx - mn
        scales[sb] = _f32(rng / 15) if rng > 0 else 0.0
        inv = 1 / scales[sb] if scales[sb] > 0 else 0
        for i, v in enumerate(seg):
            q[sb * 32 + i] = max(0, min(15, math.floor((v - mn) * inv + 0.5)))
    max_scale = max_min = 0.0
    for i in range(8):
        max_scale = max(max_scale, scales[i])
        max_min = max(max_min, mins[i])
        if mins[i] < 0:
            mins[i] = 0.0
    d, dmin = max_scale / 63, max_min / 63
    struct.pack_into("<HH", block, 0, py_f32_to_f16(d), py_f32_to_f16(dmin))
    inv_d = 1 / d if d > 0 else 0
    inv_dm = 1 / dmin if dmin > 0 else 0
    sc = [min(63, math.floor(scales[i] * inv_d + 0.5)) for i in range(8)]
    mb = [min(63, math.floor(max(0, mins[i]) * inv_dm + 0.5)) for i in range(8)]
    for i in range(4):
        block[4 + i] = (sc[i] & 0x3F) | (((sc[i + 4] >> 4) & 3) << 6)
        block[8 + i] = (mb[i] & 0x3F) | (((mb[i + 4] >> 4) & 3) << 6)
        block[12 + i] = (sc[i + 4] & 0xF) | ((mb[i + 4] & 0xF) << 4)
    for c in range(4):
        for i in range(32):
            block[16 + c * 32 + i] = (q[c * 64 + i] & 0xF) | ((q[c * 64 + 32 + i] & 0xF) << 4)
    return bytes(block)


def py_dequant_block(block):
    d = py_f16_to_f32(struct.unpack_from("<H", block, 0)[0])
    dmin = py_f16_to_f32(struct.unpack_from("<H", block, 2)[0])
    sc, mb = [0] * 8, [0] * 8
    for i in range(4):
        sc[i] = block[4 + i] & 0x3F
        sc[i + 4] = ((block[4 + i] >> 6) & 3) << 4
        mb[i] = block[8 + i] & 0x3F
        mb[i + 4] = ((block[8 + i] >> 6) & 3) << 4
    for i in range(4):
        sc[i + 4] |= block[12 + i] & 0xF
        mb[i + 4] |= (block[12 + i] >> 4) & 0xF
    scales = [_f32(d * s) for s in sc]
    mins = [_f32(dmin * m) for m in mb]
    out = [0.0] * 256
    for c in range(4):
        for i in range(32):
            b = block[16 + c * 32 + i]
            out[c * 64 + i] = _f32(scales[2 * c] * (b & 0xF) - mins[2 * c])
            out[c * 64 + 32 + i] = _f32(scales[2 * c + 1] * (b >> 4) - mins[2 * c + 1])
    return out


def quant_error(orig, rec):
    orig, rec = np.asarray(orig, np.float64), np.asarray(rec, np.float64)
    diff = orig - rec
    mse = float(np.mean(diff * diff))
    sp = float(np.mean(orig * orig))
    return {"mse": mse, "max": float(np.abs(diff).max()), "snr": 10 * math.log10(sp / mse) if sp > 0 and mse > 0 else math.inf}


def _f32arr(fn, n):
    return np.array([fn(i) for i in range(n)], dtype=np.float64).astype(np.float32)


# ---- 1. tests/converter/quantizer.test.js ---------------------------------------------------
def test_f16_round_trip_values():  # quantizer.test.js:22-40
    for v in [0, 1, -1, 0.5, -0.25, 12.25, -24.5]:
        rt = O.f16_to_f32(O.f32_to_f16_trunc(v))
        assert math.isfinite(rt) and abs(rt - v) < 0.05
        assert O.f32_to_f16_trunc(v) == py_f32_to_f16(v)
    assert O.f16_to_f32(O.f32_to_f16_trunc(math.inf)) == math.inf
    assert O.f16_to_f32(O.f32_to_f16_trunc(-math.inf)) == -math.inf
    assert math.isnan(O.f16_to_f32(O.f32_to_f16_trunc(math.nan)))


def test_f16_decode_all_codes_match_numpy():
    codes = np.arange(65536, dtype=np.uint16)
    ours = np.array([O.f16_to_f32(int(c)) for c in codes], np.float32)
    ref = codes.view(np.float16).astype(np.float32)
    ok = (ours == ref) | (np.isnan(ours) & np.isnan(ref))
    assert ok.all()


def test_f16_encoders():
    rng = np.random.default_rng(5)
    vals = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-7, 1e-4, 1.0, 300.0, 7e4)])
    for v in vals:
        v = float(v)
        assert O.f32_to_f16_rne(v) == int(np.float32(v).astype(np.float16).view(np.uint16)), v
        assert O.f32_to_f16_trunc(v) == py_f32_to_f16(v)
    # truncation never exceeds the magnitude; the kv-host encoder rounds half up (types.js:25-43)
    assert O.f32_to_f16_trunc(1.0 + 2**-11 + 2**-12) == 0x3C00
    assert O.f32_to_f16_kvhost(1.0 + 2**-11) == 0x3C01
    assert O.f32_to_f16_rne(1.0 + 2**-11) == 0x3C00  # tie -> even


def test_quantize_block_size_and_layout():  # quantizer.test.js:42-49, dequant-numeric.test.js:180-188
    blk = O.q4k_quantize_block(_f32arr(lambda i: math.sin(i / 16), 256))
    assert blk.size == 144
    blk = O.q4k_quantize_block(_f32arr(lambda i: math.sin(i / 16) * 5, 256))
    assert blk.size == 144 == BLOCK


def test_sizes_2x300():  # quantizer.test.js:51-80
    data = _f32arr(lambda i: ((i % 29) - 14) / 7, 600)
    flat = O.q4k_quantize_flat(data)
    row = O.q4k_quantize_rowwise(data, 2, 300)
    assert flat.size == math.ceil(600 / 256) * 144
    assert row.size == 2 * 2 * 144
    deq = O.q4k_dequant_flat(flat, 600)
    e = quant_error(data, deq)
    assert all(math.isfinite(e[k]) for k in ("mse", "max", "snr"))


def test_rowwise_tail_1x300():  # quantizer.test.js:82-101, dequant-numeric.test.js:112-134
    data = np.zeros(300, np.float32)
    data[:256] = _f32arr(lambda i: ((i % 17) - 8) / 4, 256)
    data[256:] = _f32arr(lambda i: -10 + i * 0.01, 44)
    row = O.q4k_quantize_rowwise(data, 1, 300)
    deq = O.q4k_dequant_rowwise(row, 1, 300).ravel()
    assert quant_error(data, deq)["max"] < 0.25
    assert deq[256:].max() < -9.5


def test_batched_rowwise_2x2x300():  # quantizer.test.js:103-121
    data = _f32arr(lambda i: ((i % 37) - 18) / 9, 1200)
    row = O.q4k_quantize_rowwise(data, 4, 300)
    assert row.size == 4 * 2 * 144 > math.ceil(1200 / 256) * 144
    deq = O.q4k_dequant_rowwise(row, 4, 300)
    assert deq.size == 1200 and math.isfinite(quant_error(data, deq.ravel())["mse"])


# ---- 2. tests/gpu/dequant-numeric.test.js ------------------------------------------------------
def test_flat_single_block():  # :15-33
    data = _f32arr(lambda i: math.sin(i * 0.05) * 2.0, 256)
    q = O.q4k_quantize_flat(data)
    assert q.size == 144
    e = quant_error(data, O.q4k_dequant_flat(q, 256))
    assert e["max"] < 0.5 and e["snr"] > 15


def test_flat_multi_block():  # :36-53
    data = _f32arr(lambda i: ((i % 37) - 18) / 9, 768)
    q = O.q4k_quantize_flat(data)
    assert q.size == 3 * 144
    assert quant_error(data, O.q4k_dequant_flat(q, 768))["max"] < 0.5


def test_rowwise_k300():  # :58-87
    data = _f32arr(lambda i: ((i % 23) - 11) / 5.5, 1200)
    q = O.q4k_quantize_rowwise(data, 4, 300)
    assert q.size == 4 * 2 * 144
    deq = O.q4k_dequant_rowwise(q, 4, 300)
    assert deq.shape == (4, 300)
    assert np.abs(deq.ravel() - data).max() < 0.5


def test_rowwise_k192_k256_k384():  # :90-109, :137-154, :191-213
    for rows, K, fn in ((2, 192, lambda i: math.cos(i * 0.1) * 3.0), (3, 256, lambda i: ((i % 41) - 20) / 10),
                        (5, 384, lambda i: ((i % 31) - 15) / 7.5)):
        data = _f32arr(fn, rows * K)
        q = O.q4k_quantize_rowwise(data, rows, K)
        assert q.size == rows * math.ceil(K / 256) * 144
        deq = O.q4k_dequant_rowwise(q, rows, K)
        assert deq.size == rows * K and quant_error(data, deq.ravel())["max"] < 0.5


def test_flat_equals_rowwise_when_aligned():  # :156-177 (exact equality)
    data = _f32arr(lambda i: ((i % 19) - 9) / 4.5, 1024)
    flat, row = O.q4k_quantize_flat(data), O.q4k_quantize_rowwise(data, 2, 512)
    assert np.array_equal(flat, row)
    a, b = O.q4k_dequant_flat(flat, 1024), O.q4k_dequant_rowwise(row, 2, 512).ravel()
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


# ---- 3. tests/tooling/q4k-projection-reference.test.js ---------------------------------------------
def test_projection_reference():
    rows, cols = 5, 512
    w = _f32arr(lambda i: math.sin(i * 0.017) * 0.25 + math.cos(i * 0.003) * 0.1, rows * cols)
    act = _f32arr(lambda i: math.sin(i * 0.011) * 0.5, cols)
    q = O.q4k_quantize_rowwise(w, rows, cols)
    deq = O.q4k_dequant_rowwise(q, rows, cols)
    first = O.q4k_dequant_block(q[:144])
    assert np.array_equal(first, deq.ravel()[:256])  # :31-32 deepEqual
    out = O.q4k_gemv(q, rows, cols, act)
    expected = np.array([np.float32(sum(float(act[c]) * float(deq[r, c]) for c in range(cols))) for r in range(rows)])
    assert np.array_equal(out.view(np.uint32), expected.view(np.uint32))  # :36-44 deepEqual
    # the GEMM restatement is the same sum for every row of A
    gm = O.q4k_gemm(q, rows, cols, np.stack([act, act * 0.5]), 2)
    assert np.array_equal(gm[0].view(np.uint32), out.view(np.uint32))


# ---- 4. harness generators + kernel-suite cases -----------------------------------------------------
def test_lcg_generator_matches_js_semantics():  # tests/kernels/harness/tolerance.js:110-141
    def js(seed, n, lo=-1.0, hi=1.0):
        state, out = seed, []
        for _ in range(n):
            p = float(state) * 1103515245.0 + 12345.0  # double arithmetic, like JS
            state = int(p) & 0x7FFFFFFF
            out.append(_f32(lo + (state / 0x7FFFFFFF) * (hi - lo)))
        return np.array(out, np.float32)
    for seed in (42, 901, 1001, 2101, 2102):
        assert np.array_equal(O.lcg_test_data(300, seed), js(seed, 300))
    assert np.array_equal(O.lcg_test_data(64, 2101, -0.5, 0.5), js(2101, 64, -0.5, 0.5))
    # hand-computed first draw for seed 42: (42*1103515245+12345) & 0x7fffffff = 1250496027
    assert abs(float(O.lcg_test_data(1, 42)[0]) - (-1 + 2 * 1250496027 / 0x7FFFFFFF)) < 1e-7


def test_prng1664525():
    v = O.prng1664525(3, 7)
    s = (7 * 1664525 + 1013904223) % 2**32
    assert v[0] == s / 2**32


def test_kernel_suite_dequant_case():  # kernel-suite.js:735-746 (2 blocks, seed 1001)
    vals = O.lcg_test_data(512, 1001)
    q = O.q4k_quantize_flat(vals)
    deq = O.q4k_dequant_flat(q, 512)
    assert np.abs(deq - vals).max() < 0.2  # quantisation error of a [-1,1] signal
    for b in range(2):  # second implementation agrees bit for bit
        assert bytes(q[b * 144:(b + 1) * 144]) == py_quantize_block(vals[b * 256:(b + 1) * 256])
        assert np.array_equal(np.array(py_dequant_block(bytes(q[b * 144:(b + 1) * 144])), np.float32), deq[b * 256:(b + 1) * 256])


def test_kernel_suite_matmul_q4k_case():  # kernel-suite.js:218-232 (M=2,N=4,K=256)
    A = O.lcg_test_data(512, 2101, -0.5, 0.5)
    B = O.lcg_test_data(1024, 2102, -0.5, 0.5)
    q = O.q4k_quantize_flat(B)
    deq = O.q4k_dequant_flat(q, 1024).reshape(4, 256)
    exp = (A.reshape(2, 256).astype(np.float64) @ deq.T.astype(np.float64))
    got = O.q4k_gemm(q, 4, 256, A, 2)
    assert np.allclose(got, exp, rtol=1e-6, atol=1e-6)


def test_kernel_suite_attention_case():  # kernel-suite.js:717-733
    Q, K, V = O.lcg_test_data(32, 901), O.lcg_test_data(32, 902), O.lcg_test_data(32, 903)
    out = O.attention(Q, K, V, 2, 4, 2, 1, 8)
    # numpy restatement of attentionRef
    q, k, v = Q.reshape(2, 2, 8).astype(np.float64), K.reshape(4, 8).astype(np.float64), V.reshape(4, 8).astype(np.float64)
    s = np.einsum("shd,kd->shk", q, k) / math.sqrt(8)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    ref = np.einsum("shk,kd->shd", p, v).ravel()
    assert np.allclose(out, ref, rtol=1e-5, atol=1e-6)
    # f16-KV + causal variant equals the masked f32 form when K,V are f16-exact
    k16, v16 = K.astype(np.float16), V.astype(np.float16)
    a = O.attention_f16kv(Q, k16, v16, 2, 4, 2, 1, 8, causal=True, start_pos=2)
    mask = np.array([[0, 0, 0, -np.inf], [0, 0, 0, 0]], np.float32)
    b = O.attention(Q, k16.astype(np.float32), v16.astype(np.float32), 2, 4, 2, 1, 8, mask=mask)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_second_implementation_agrees_on_all_reference_inputs():
    cases = [_f32arr(lambda i: math.sin(i * 0.05) * 2.0, 256), _f32arr(lambda i: ((i % 37) - 18) / 9, 256),
             _f32arr(lambda i: math.sin(i / 16) * 5, 256), O.lcg_test_data(256, 2102, -0.5, 0.5),
             np.zeros(256, np.float32), np.full(256, 3.25, np.float32)]
    for data in cases:
        for valid in (256, 44, 192):
            blk = O.q4k_quantize_block(data, valid)
            assert bytes(blk) == py_quantize_block(data, valid)
            assert np.array_equal(O.q4k_dequant_block(blk), np.array(py_dequant_block(bytes(blk)), np.float32))


# ---- 5. hand-derived known answers for the 144-byte layout -------------------------------------------
def test_known_answer_block():
    blk = bytearray(144)
    struct.pack_into("<HH", blk, 0, 0x3C00, 0x3800)  # d = 1.0, dmin = 0.5
    sc = [1, 2, 3, 4, 17, 34, 51, 63]
    mn = [0, 1, 2, 3, 16, 33, 50, 63]
    for i in range(4):
        blk[4 + i] = sc[i] | ((sc[i + 4] >> 4) << 6)
        blk[8 + i] = mn[i] | ((mn[i + 4] >> 4) << 6)
        blk[12 + i] = (sc[i + 4] & 15) | ((mn[i + 4] & 15) << 4)
    for c in range(4):
        for i in range(32):
            blk[16 + 32 * c + i] = (i % 16) | (((15 - i) % 16) << 4)
    scodes, mcodes, d, dm = O.q4k_decode_header(np.frombuffer(bytes(blk), np.uint8))
    assert list(scodes) == sc and list(mcodes) == mn and d == 1.0 and dm == 0.5
    out = O.q4k_dequant_block(np.frombuffer(bytes(blk), np.uint8))
    for e in range(256):
        s, i = e // 32, e % 32
        qv = (i % 16) if s % 2 == 0 else ((15 - i) % 16)
        assert out[e] == sc[s] * qv - 0.5 * mn[s], e


def test_small_ops_against_numpy():
    rng = np.random.default_rng(0)
    x, w = rng.standard_normal((3, 64)).astype(np.float32), rng.standard_normal(64).astype(np.float32)
    y = O.rmsnorm(x, w, 3, 64, 1e-6).reshape(3, 64)
    ref = x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6) * w
    assert np.allclose(y, ref, rtol=1e-6, atol=1e-7)
    c, s = O.rope_tables(1e6, 8, 5)
    f = np.float32(1.0) / np.float32(1e6) ** (np.arange(4) * 2 / 8)
    assert np.allclose(c, np.cos(np.arange(5)[:, None] * f[None].astype(np.float32).astype(np.float64)), atol=1e-7)
    xr = rng.standard_normal((2, 3, 8)).astype(np.float32)
    yr = O.rope(xr, c, s, 2, 3, 8, start_pos=1).reshape(2, 3, 8)
    for t in range(2):
        cc, ss = c[t + 1], s[t + 1]
        assert np.allclose(yr[t, :, :4], xr[t, :, :4] * cc - xr[t, :, 4:] * ss, atol=1e-6)
        assert np.allclose(yr[t, :, 4:], xr[t, :, :4] * ss + xr[t, :, 4:] * cc, atol=1e-6)
    g, u = rng.standard_normal(100).astype(np.float32) * 10, rng.standard_normal(100).astype(np.float32)
    assert np.allclose(O.silu_gated(g, u), g / (1 + np.exp(-g.astype(np.float64))) * u, rtol=1e-6)
    assert np.allclose(O.silu_gated(g, u, clamped=True), O.silu_gated(g, u), rtol=1e-5, atol=1e-5)
    assert O.argmax(np.array([1, 5, 5, 2], np.float32)) == 1  # lower index wins (sample.wgsl:45-53)
    assert O.argmax(np.array([1, 5, 7, 2], np.float32), pad_id=2) == 1
    emb = rng.standard_normal((10, 4)).astype(np.float16)
    assert np.array_equal(O.gather_f16(emb, [3, 7], 4), emb[[3, 7]].astype(np.float32))


# ---- reference-produced digests: the 9B gate_proj receipt ---------------------------------
def test_receipt_header_fields_decode_back():
    """The a1 packing rule round-trips through the oracle's header reader on real headers."""
    from parity import pack_q4k_headers, receipt_headers

    z = receipt_headers()
    nb = 4096
    blocks = pack_q4k_headers(z["d_f16"][:nb], z["dmin_f16"][:nb], z["scale_codes"][: 8 * nb], z["min_codes"][: 8 * nb], 0x5A)
    for b in range(0, nb, 257):
        sc, mn, d, dm = O.q4k_decode_header(blocks[b * BLOCK:(b + 1) * BLOCK])
        assert np.array_equal(sc, z["scale_codes"][8 * b: 8 * b + 8]) and np.array_equal(mn, z["min_codes"][8 * b: 8 * b + 8])
        assert d == float(z["d_f16"][b: b + 1].view(np.float16)[0]) and dm == float(z["dmin_f16"][b: b + 1].view(np.float16)[0])


def test_receipt_decoded_scales_and_minima_match_the_reference_digests():
    """quantizer.js:204-209 / q4k-projection-reference.js:26-37 on 1,572,864 real sub-blocks: the
    oracle's dequantiser, fed the receipt's headers, yields exactly the bytes whose sha256 the
    reference recorded (artifactFiles.decodedScales / decodedMinima)."""
    from parity import receipt_headers, receipt_probe_blocks, sha256_f32

    z = receipt_headers()
    n_blocks = z["d_f16"].size
    assert n_blocks == int(z["shape"][0]) * int(z["shape"][1]) // QK_K == 196608
    for_minima, for_scales = receipt_probe_blocks()
    w = O.q4k_dequant_flat(for_minima, n_blocks * QK_K).reshape(-1, 32)
    assert np.all(w == w[:, :1])  # one value per sub-block
    minima = np.float32(0.0) - w[:, 0]
    assert sha256_f32(minima) == str(z["decoded_minima_sha256"])
    w = O.q4k_dequant_flat(for_scales, n_blocks * QK_K).reshape(-1, 32)
    assert np.all(w == w[:, :1])
    assert sha256_f32(w[:, 0]) == str(z["decoded_scales_sha256"])
