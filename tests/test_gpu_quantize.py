"""Device Q4_K quantizer against the oracle's restatement of src/converter/quantizer.js: bit-exact."""
import numpy as np
import pytest

from doppler_b200 import ops, synthetic
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _rowwise(dev, w, rows, cols):
    t = dev.tensor_from(np.ascontiguousarray(w, np.float32).reshape(rows, cols))
    wb = ops.quantize_to_q4km_rowwise(t, [rows, cols])
    assert wb.dtype == "q4k" and wb.layout == "row" and wb.shape == [rows, cols]
    got = dev.read_buffer(wb.buffer, rows * ((cols + 255) // 256) * 144)
    dev.release_buffer(t.buffer)
    return got, wb


@pytest.mark.parametrize("rows,cols", [(64, 1024), (7, 300), (3, 256), (5, 33), (1, 1), (130, 4096)])
def test_rowwise_bit_exact(dev, rows, cols):
    w = synthetic.normal_f32(synthetic.key(71, rows * 10000 + cols), rows * cols, 0.05)
    got, wb = _rowwise(dev, w, rows, cols)
    exp = O.q4k_quantize_rowwise(w, rows, cols)
    assert np.array_equal(got, np.asarray(exp, np.uint8).ravel()), "device quantizer differs from the reference restatement"
    # and the packed matrix is usable as a weight: GEMV on it equals the oracle GEMV on the oracle's bytes
    x = synthetic.normal_f32(synthetic.key(71, 5), cols)
    xt = dev.tensor_from(x.reshape(1, cols))
    y = ops.run_matmul(xt, wb, 1, rows, cols, output_dtype="f32")
    from parity import assert_close
    assert_close(dev.read_tensor(y), O.q4k_gemv(exp, rows, cols, x), f"gemv on device-quantised [{rows},{cols}]")
    for b in (wb.buffer, xt.buffer, y.buffer):
        dev.release_buffer(b)


def test_special_values(dev):
    """constant sub-blocks (range 0), all-negative and all-positive data, halves that round up,
    values large enough to saturate the 6-bit codes"""
    rows, cols = 6, 512
    w = np.zeros((rows, cols), np.float32)
    w[0] = 0.75                                   # constant: scale 0, min offset -0.75 -> clamped to 0
    w[1] = -np.abs(synthetic.normal_f32(synthetic.key(72, 1), cols)) - 1.0
    w[2] = np.abs(synthetic.normal_f32(synthetic.key(72, 2), cols)) + 1.0
    w[3] = np.tile(np.arange(32, dtype=np.float32) * 0.5 - 4.0, cols // 32)   # exact .5 quotients
    w[4] = synthetic.normal_f32(synthetic.key(72, 3), cols) * 1e4
    w[4, :32] *= 1e-6                             # tiny sub-block next to large ones
    w[5] = synthetic.normal_f32(synthetic.key(72, 4), cols) * 1e-9   # f16 header underflows
    got, wb = _rowwise(dev, w, rows, cols)
    assert np.array_equal(got, np.asarray(O.q4k_quantize_rowwise(w.ravel(), rows, cols), np.uint8).ravel())
    dev.release_buffer(wb.buffer)


def test_reference_suite_vector_and_flat_driver(dev):
    """the reference's own test vector (tests/kernels/browser/kernel-suite.js:735-746 data) and the
    flat driver's zero padding (quantizer.js:223-251)"""
    vals = O.lcg_test_data(512, 1001)
    t = dev.tensor_from(vals)
    wb = ops.quantize_to_q4km(t, 512)
    assert np.array_equal(dev.read_buffer(wb.buffer, 2 * 144), np.asarray(O.q4k_quantize_flat(vals), np.uint8).ravel())
    dev.release_buffer(wb.buffer)
    dev.release_buffer(t.buffer)
    ragged = synthetic.normal_f32(synthetic.key(73, 1), 700) + 2.0   # positive data: the zero padding changes the last block's range
    t = dev.tensor_from(ragged)
    wb = ops.quantize_to_q4km(t, 700)
    flat = np.asarray(O.q4k_quantize_flat(ragged), np.uint8).ravel()
    assert np.array_equal(dev.read_buffer(wb.buffer, 3 * 144), flat)
    rowwise = np.asarray(O.q4k_quantize_rowwise(ragged, 1, 700), np.uint8).ravel()
    assert not np.array_equal(flat, rowwise)      # the two drivers really differ on a tail
    dev.release_buffer(wb.buffer)
    dev.release_buffer(t.buffer)
    with pytest.raises(ops.DopplerError):
        ops.quantize_to_q4km_rowwise(dev.tensor_from(np.zeros(4, np.float32)), [2, 256])   # source too small
