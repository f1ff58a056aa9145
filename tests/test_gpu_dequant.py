"""Q4_K dequant: bit-exact against the oracle (memcmp), through the C ABI."""
import math

import numpy as np
import pytest

from doppler_b200 import ops, synthetic
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _run_flat(dev, packed, nblocks, dtype="f32"):
    buf = dev.acquire_buffer(packed.nbytes, "q4k")
    dev.upload_data(buf, packed)
    t = ops.dequantize(buf, nblocks, output_dtype=dtype)
    out = dev.read_tensor(t)
    dev.release_buffer(t.buffer)
    dev.release_buffer(buf)
    return out


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint32 if a.dtype == np.float32 else np.uint16)


@pytest.mark.parametrize("nblocks", [1, 2, 10, 12288])  # 12288 blocks = BASELINE config 0 weight
def test_flat_bit_exact(dev, nblocks):
    packed = synthetic.q4k_blocks(synthetic.key(11, nblocks), nblocks)
    got = _run_flat(dev, packed, nblocks)
    exp = O.q4k_dequant_flat(packed, nblocks * 256)
    assert np.array_equal(_bits(got), _bits(exp))


def test_reference_suite_vectors(dev):  # tests/kernels/browser/kernel-suite.js:735-746 and :750-915
    for nb, seed in ((2, 1001), (1, 1002), (10, 1003)):
        q = O.q4k_quantize_flat(O.lcg_test_data(nb * 256, seed))
        assert np.array_equal(_bits(_run_flat(dev, q, nb)), _bits(O.q4k_dequant_flat(q, nb * 256)))


def test_f16_output_is_rne_of_f32(dev):
    packed = synthetic.q4k_blocks(synthetic.key(12, 0), 64)
    got = _run_flat(dev, packed, 64, "f16")
    exp = O.q4k_dequant_flat(packed, 64 * 256).astype(np.float16)
    assert np.array_equal(_bits(got), _bits(exp))


@pytest.mark.parametrize("rows,K", [(4, 300), (2, 192), (5, 384), (3, 256), (7, 1024)])
def test_rowwise_strips_tail(dev, rows, K):  # tests/gpu/dequant-numeric.test.js K=300/192/384/256
    data = np.array([((i % 23) - 11) / 5.5 for i in range(rows * K)], np.float32)
    q = O.q4k_quantize_rowwise(data, rows, K)
    buf = dev.acquire_buffer(q.nbytes, "q4k_rows")
    dev.upload_data(buf, q)
    for dt in ("f32", "f16"):
        t = ops.dequantize_rowwise(buf, rows, K, output_dtype=dt)
        assert t.shape == [rows, K]
        got = dev.read_tensor(t)
        exp = O.q4k_dequant_rowwise(q, rows, K)
        exp = exp if dt == "f32" else exp.astype(np.float16)
        assert np.array_equal(_bits(got), _bits(exp))
        dev.release_buffer(t.buffer)
    dev.release_buffer(buf)


def test_output_buffer_and_offset(dev):
    packed = synthetic.q4k_blocks(synthetic.key(13, 0), 8)
    buf = dev.acquire_buffer(packed.nbytes, "q4k")
    dev.upload_data(buf, packed)
    out = dev.acquire_buffer(8 * 256 * 4 + 1024, "mine")
    t = ops.dequantize(buf, 8, output_buffer=out, output_offset=1024)
    assert t.buffer is out and t.offset == 1024
    got = dev.read_buffer(out, 8 * 256 * 4, 1024).view(np.float32)
    assert np.array_equal(_bits(got), _bits(O.q4k_dequant_flat(packed, 2048)))
    with pytest.raises(ops.DopplerError):
        ops.dequantize(buf, 8, output_buffer=out, output_offset=100)  # not 256-aligned
    with pytest.raises(ops.DopplerError):
        ops.dequantize(buf, 9)  # more blocks than the buffer holds
    with pytest.raises(ops.DopplerError):
        ops.dequantize(buf, 8, output_dtype="i32")
    dev.release_buffer(out)
    dev.release_buffer(buf)


def test_full_size_round_trip_property(dev):
    """Config-1-sized weight [12288,4096]: dequant of a re-quantised row equals itself
    (quantise -> dequantise -> quantise -> dequantise is idempotent on this grid)."""
    rows, K = 64, 4096
    w = O.lcg_test_data(rows * K, 31, -0.1, 0.1)
    q1 = O.q4k_quantize_rowwise(w, rows, K)
    buf = dev.acquire_buffer(q1.nbytes, "q")
    dev.upload_data(buf, q1)
    t = ops.dequantize_rowwise(buf, rows, K)
    d1 = dev.read_tensor(t)
    assert np.array_equal(_bits(d1), _bits(O.q4k_dequant_rowwise(q1, rows, K)))
    assert np.abs(d1.ravel() - w).max() < 0.2 / 15 + 1e-3
    dev.release_buffer(t.buffer)
    dev.release_buffer(buf)


def test_receipt_headers_decode_to_the_reference_digests(dev):
    """The CUDA dequant kernel on the 196,608 real block headers of the reference's 9B gate_proj
    receipt: decoded scales and minima hash to the digests the reference recorded for its own
    dequantiser (layer0-ffn-gate-oracle.json, artifactFiles.decodedScales / decodedMinima)."""
    from parity import receipt_headers, receipt_probe_blocks, sha256_f32

    z = receipt_headers()
    nb = z["d_f16"].size
    for_minima, for_scales = receipt_probe_blocks()
    w = _run_flat(dev, for_minima, nb).reshape(-1, 32)
    assert np.all(w == w[:, :1])
    assert sha256_f32(np.float32(0.0) - w[:, 0]) == str(z["decoded_minima_sha256"])
    w = _run_flat(dev, for_scales, nb).reshape(-1, 32)
    assert np.all(w == w[:, :1])
    assert sha256_f32(w[:, 0]) == str(z["decoded_scales_sha256"])
