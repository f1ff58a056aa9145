"""Q4_K fused dequant+matmul (decode GEMV, prefill GEMM) and the f16-weight GEMV, through
the C ABI, against the double-accumulate oracle."""
import numpy as np
import pytest

from doppler_b200 import ops, synthetic
from oracle import oracle as O
from parity import assert_close

pytestmark = pytest.mark.gpu


def _matmul(dev, W, N, K, A, M, out_dtype="f32", a_dtype="f32", wdtype="q4k", **opt):
    wb = dev.weight_from(W, wdtype, [N, K])
    a = np.ascontiguousarray(A, np.float32 if a_dtype == "f32" else np.float16).reshape(M, K)
    at = dev.tensor_from(a)
    ct = ops.run_matmul(at, wb, M, N, K, output_dtype=out_dtype, **opt)
    assert ct.shape == [M, N] and ct.dtype == out_dtype
    out = dev.read_tensor(ct)
    for b in (ct.buffer, at.buffer, wb.buffer):
        dev.release_buffer(b)
    return out


def test_config0_gemv(dev):
    """BASELINE config 0: x f32[1,1024] ~N(0,1), W [3072,1024] synthetic blocks."""
    N, K = 3072, 1024
    W = synthetic.q4k_matrix(synthetic.key(synthetic.DEFAULT_SEED, 1), N, K)
    x = synthetic.normal_f32(synthetic.key(synthetic.DEFAULT_SEED, 2), K)
    got = _matmul(dev, W, N, K, x, 1)
    assert_close(got, O.q4k_gemv(W, N, K, x), "config0 gemv [1,1024]x[3072,1024]")
    again = _matmul(dev, W, N, K, x, 1)
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32)), "GEMV is not run-to-run deterministic"


@pytest.mark.parametrize("N,K", [(12288, 4096), (4096, 12288), (6144, 4096), (4096, 4096)])
def test_9b_shape_gemv(dev, N, K):
    W = synthetic.q4k_matrix(synthetic.key(21, N * 7 + K), N, K)
    x = synthetic.normal_f32(synthetic.key(22, K), K)
    got = _matmul(dev, W, N, K, x, 1)
    assert_close(got, O.q4k_gemv(W, N, K, x), f"gemv [{N},{K}]")


def test_gemv_linearity_and_alpha(dev):
    N, K = 12288, 4096
    W = synthetic.q4k_matrix(synthetic.key(23, 0), N, K)
    x1, x2 = synthetic.normal_f32(synthetic.key(23, 1), K), synthetic.normal_f32(synthetic.key(23, 2), K)
    y1, y2, y12 = _matmul(dev, W, N, K, x1, 1), _matmul(dev, W, N, K, x2, 1), _matmul(dev, W, N, K, x1 + x2, 1)
    assert_close(y12, y1.astype(np.float64) + y2, "gemv linearity")
    ya = _matmul(dev, W, N, K, x1, 1, alpha=0.25)
    assert_close(ya, 0.25 * y1.astype(np.float64), "gemv alpha")


@pytest.mark.parametrize("N,K", [(5, 300), (3, 192), (33, 384), (1, 256), (257, 512), (100, 2560)])
def test_gemv_ragged_shapes(dev, N, K):  # K tails padded inside the last block of each row
    w = O.lcg_test_data(N * K, 77 + N, -0.5, 0.5)
    W = O.q4k_quantize_rowwise(w, N, K)
    x = O.lcg_test_data(K, 78)
    assert_close(_matmul(dev, W, N, K, x, 1), O.q4k_gemv(W, N, K, x), f"gemv ragged [{N},{K}]")


def test_gemv_f16_output_and_f16_activation(dev):
    N, K = 512, 1024
    w = O.lcg_test_data(N * K, 5, -0.05, 0.05)
    W = O.q4k_quantize_rowwise(w, N, K)
    x = O.lcg_test_data(K, 6)
    exp = O.q4k_gemv(W, N, K, x)
    got16 = _matmul(dev, W, N, K, x, 1, out_dtype="f16")
    assert np.abs(got16.astype(np.float64) - exp).max() <= np.abs(exp).max() * 2**-10
    x16 = x.astype(np.float16)
    got = _matmul(dev, W, N, K, x16, 1, a_dtype="f16")
    assert_close(got, O.q4k_gemv(W, N, K, x16.astype(np.float32)), "gemv f16 activations")


def test_reference_suite_matmul_q4k(dev):  # tests/kernels/browser/kernel-suite.js:218-232
    M, N, K = 2, 4, 256
    A = O.lcg_test_data(M * K, 2101, -0.5, 0.5)
    B = O.lcg_test_data(N * K, 2102, -0.5, 0.5)
    W = O.q4k_quantize_flat(B)
    got = _matmul(dev, W, N, K, A, M, exact_weights=True)
    exp = O.q4k_gemm(W, N, K, A, M)
    assert np.all(np.abs(got - exp) <= 1e-2 + 1e-2 * np.abs(exp))  # the reference's own tolerance
    assert_close(got, exp, "kernel-suite matmul_q4k")


def test_reference_widetile_parity_case(dev):
    """tests/kernels/fused-matmul-q4-widetile-f16a-parity.test.js: M=4,K=1536,N=6144, LCG seed 7,
    f16 activations, f16 output, max_abs_diff < 1.0 and no NaN/Inf."""
    M, K, N = 4, 1536, 6144
    r = O.prng1664525(M * K + N * K, 7)
    a32 = ((r[:M * K] - 0.5) * 1.0).astype(np.float32)
    w32 = ((r[M * K:] - 0.5) * 0.1).astype(np.float32)
    a16 = np.array([O.f32_to_f16_kvhost(float(v)) for v in a32], np.uint16).view(np.float16)
    W = O.q4k_quantize_rowwise(w32, N, K)
    exp = O.q4k_gemm(W, N, K, a16.astype(np.float32), M)
    got = _matmul(dev, W, N, K, a16, M, out_dtype="f16", a_dtype="f16")
    assert np.all(np.isfinite(got)) and np.abs(got.astype(np.float64) - exp).max() < 1.0
    got32 = _matmul(dev, W, N, K, a16, M, out_dtype="f32", a_dtype="f16", exact_weights=True)
    assert_close(got32, exp, "widetile parity case, f32 out")


@pytest.mark.parametrize("M,N,K", [(2, 64, 256), (7, 130, 300), (64, 256, 1024), (65, 96, 512)])
def test_gemm_exact_weight_path(dev, M, N, K):
    w = O.lcg_test_data(N * K, 11 + M, -0.5, 0.5)
    W = O.q4k_quantize_rowwise(w, N, K)
    A = O.lcg_test_data(M * K, 12 + M)
    got = _matmul(dev, W, N, K, A, M, exact_weights=True)
    assert_close(got, O.q4k_gemm(W, N, K, A, M), f"gemm exact [{M},{K}]x[{N},{K}]")


def test_config1_gemm(dev):
    """BASELINE config 1: A f16[512,4096] ~N(0,1), W [12288,4096], f32 accumulate, f16 out.
    Default path = the rule-selected kernel's numerics (weights to f32 accuracy): the stated 1e-3 gate
    against the double-accumulate oracle, f32 and f16 output (the oracle's sum rounded to f16 differs
    from ours by at most the last f16 bit, 4.9e-4 relative, inside the gate)."""
    M, N, K = 512, 12288, 4096
    W = synthetic.q4k_matrix(synthetic.key(synthetic.DEFAULT_SEED, 10), N, K)
    A = synthetic.normal_f16(synthetic.key(synthetic.DEFAULT_SEED, 11), M * K)
    exp = O.q4k_gemm(W, N, K, A.astype(np.float32), M)
    got32 = _matmul(dev, W, N, K, A, M, out_dtype="f32", a_dtype="f16")
    assert_close(got32, exp, "config1 gemm f32 out")
    got16 = _matmul(dev, W, N, K, A, M, out_dtype="f16", a_dtype="f16")
    assert np.all(np.isfinite(got16.astype(np.float32)))
    assert_close(got16.astype(np.float32), exp, "config1 gemm f16 out")
    # two runs give the same bits (no atomics on the default path)
    assert np.array_equal(got16.view(np.uint16), _matmul(dev, W, N, K, A, M, out_dtype="f16", a_dtype="f16").view(np.uint16))


def test_config1_gemm_opt_in_f16_weights(dev):
    """opts.f16_weights: the numerics of the reference's opt-in tiled prefill kernel
    (fused_matmul_q4_prefill_tiled_f16.wgsl:201, weights rounded to f16 first), one tensor-core product.
    Gate 1e-3 against the oracle's restatement of THAT kernel; its distance from the exact product is printed."""
    M, N, K = 512, 12288, 4096
    W = synthetic.q4k_matrix(synthetic.key(synthetic.DEFAULT_SEED, 10), N, K)
    A = synthetic.normal_f16(synthetic.key(synthetic.DEFAULT_SEED, 11), M * K)
    exp = O.q4k_gemm_f16_weights(W, N, K, A.astype(np.float32), M)
    got32 = _matmul(dev, W, N, K, A, M, out_dtype="f32", a_dtype="f16", f16_weights=True)
    assert_close(got32, exp, "config1 gemm, f16-rounded weights, f32 out")
    got16 = _matmul(dev, W, N, K, A, M, out_dtype="f16", a_dtype="f16", f16_weights=True)
    assert_close(got16.astype(np.float32), exp, "config1 gemm, f16-rounded weights, f16 out")
    from parity import stats
    print("[parity] f16-rounded weights vs the exact product:", stats(got32, O.q4k_gemm(W, N, K, A.astype(np.float32), M)))


def test_f16_weight_gemv_lm_head_shape(dev):
    N, K = 8192, 1024
    W = synthetic.normal_f16(synthetic.key(31, 0), N * K, 0.02)
    x = synthetic.normal_f32(synthetic.key(31, 1), K)
    got = _matmul(dev, W, N, K, x, 1, wdtype="f16")
    assert_close(got, O.f16_gemv(W, N, K, x), "f16-weight gemv")
    A = synthetic.normal_f32(synthetic.key(31, 2), 5 * K).reshape(5, K)
    gotm = _matmul(dev, W, N, K, A, 5, wdtype="f16")
    for m in range(5):
        assert_close(gotm[m], O.f16_gemv(W, N, K, A[m]), f"f16-weight gemv row {m}")


@pytest.mark.parametrize("M,N,K", [(64, 8192, 1024), (20, 1000, 512), (9, 136, 256), (70, 256, 128)])
def test_f16_weight_rows_kernel(dev, M, N, K):
    """Batched LM head: the weights are streamed once for all rows; ragged row tiles, ragged batches, a batch over 64
    and activations of a wide range (the per-row scaling) all reach the f32 result."""
    W = synthetic.normal_f16(synthetic.key(32, N), N * K, 0.02)
    A = synthetic.normal_f32(synthetic.key(32, M), M * K).reshape(M, K)
    A[1] *= 3.0e6
    A[M - 1] *= 1.0e-6
    got = _matmul(dev, W, N, K, A, M, wdtype="f16")
    for m in range(M):
        assert_close(got[m], O.f16_gemv(W, N, K, A[m]), f"f16-weight rows M={M} row {m}")
    again = _matmul(dev, W, N, K, A, M, wdtype="f16")
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32))
    # f16 activations, f16 output
    Ah = synthetic.normal_f32(synthetic.key(33, M), M * K).reshape(M, K).astype(np.float16)
    goth = _matmul(dev, W, N, K, Ah, M, wdtype="f16", a_dtype="f16", out_dtype="f16")
    for m in (0, M - 1):
        ref = O.f16_gemv(W, N, K, Ah[m].astype(np.float32))
        assert_close(goth[m].astype(np.float32), ref, f"f16-weight rows f16 act row {m}", rtol=2e-3)


def test_matmul_argument_errors(dev):
    N, K = 8, 256
    W = synthetic.q4k_matrix(synthetic.key(41, 0), N, K)
    wb = dev.weight_from(W, "q4k", [N, K])
    at = dev.tensor_from(np.zeros((1, K), np.float32))
    with pytest.raises(ops.DopplerError, match="outputDtype"):
        ops.run_matmul(at, wb, 1, N, K)
    with pytest.raises(ops.DopplerError):
        ops.run_matmul(at, wb, 1, N + 1, K, output_dtype="f32")  # weight shape mismatch
    with pytest.raises(ops.DopplerError):
        ops.run_matmul(at, wb, 1, N, K, output_dtype="f32", a_offset=128)  # misaligned offset
    with pytest.raises(ops.DopplerError):
        ops.run_matmul(at, wb, 2, N, K, output_dtype="f32")  # A too small for M=2
    with pytest.raises(ops.DopplerError):
        ops.run_matmul(at, wb, 1, N, K, output_dtype="f32", transpose_b=False)
    small = dev.acquire_buffer(16, "small")
    with pytest.raises(ops.DopplerError):
        ops.run_matmul(at, wb, 1, N, K, output_dtype="f32", output_buffer=small)
    stats0 = dev.pool_stats()
    with pytest.raises(ops.DopplerError):
        ops.run_matmul(at, wb, 0, N, K, output_dtype="f32")
    assert dev.pool_stats()["bytes_in_use"] == stats0["bytes_in_use"]  # nothing leaked on the error path
    for b in (small, at.buffer, wb.buffer):
        dev.release_buffer(b)


def test_large_m_gemm_takes_the_two_sm_kernel(dev):
    """M = 2048 on N = 12288 is several waves of tiles: the dispatcher then picks the two-SM kernel
    (tcgen05.mma.cta_group::2, 512 x 256 pair tiles); a ragged M checks the rows beyond the last tile.
    Default numerics: the exact product (double-accumulate oracle, 1e-3 gate).  With f16_weights the
    expectation is the float64 product with f16-rounded weights, the opt-in tiled prefill kernel's
    numerics (fused_matmul_q4_prefill_tiled_f16.wgsl:118-201); against exact weights that output differs
    by up to 4e-3 of the rms at K = 512."""
    N, K = 12288, 512
    W = synthetic.q4k_matrix(synthetic.key(91, 0), N, K)
    w32 = O.q4k_dequant_flat(W, N * K).reshape(N, K)
    w16 = w32.astype(np.float16).astype(np.float64)
    for M in (2048, 1300):
        A = synthetic.normal_f16(synthetic.key(92, M), M * K)
        a64 = A.astype(np.float64).reshape(M, K)
        got = _matmul(dev, W, N, K, A, M, out_dtype="f32", a_dtype="f16")
        assert_close(got, a64 @ w32.astype(np.float64).T, f"two-SM gemm [{M},{K}]x[{N},{K}] vs the exact product")
        got = _matmul(dev, W, N, K, A, M, out_dtype="f32", a_dtype="f16", f16_weights=True)
        assert_close(got, a64 @ w16.T, f"two-SM gemm [{M},{K}]x[{N},{K}], f16_weights, vs the f16-weight product")


def test_f32_activation_gemm_runs_on_the_tensor_cores(dev):
    """f32 activations select the f32-exact product (matmul.rules.json:15-22).  From 32 rows on it is computed
    on the tensor cores: every row is scaled into f16 range by a power of two, and ONE kernel multiplies the
    f16 halves and the f16 rounding residues of activations and weights into one accumulator
    (A_hi.W_hi + A_hi.W_lo + A_lo.W_hi per K step).
    Rows here span ten decades (FFN intermediates of the synthetic models reach 1e7) and one row is zero, so
    the gate is per row: |a - b| <= 2e-5 * (|b| + rms(row of b)), fifty times tighter than the f16-rounded
    kernel could meet."""
    M, N, K = 200, 384, 1024
    W = synthetic.q4k_matrix(synthetic.key(93, 0), N, K)
    A = synthetic.normal_f32(synthetic.key(93, 1), M * K).reshape(M, K)
    decades = np.linspace(-3.0, 7.0, M).astype(np.float32)
    A = (A * (10.0 ** decades)[:, None]).astype(np.float32)
    A[17] = 0.0
    exp = np.asarray(O.q4k_gemm(W, N, K, A.ravel(), M), np.float64).reshape(M, N)
    l0 = dev.launch_count
    got = np.asarray(_matmul(dev, W, N, K, A, M), np.float64).reshape(M, N)
    assert dev.launch_count - l0 == 2, "expected the scaling cast and one tensor-core kernel"
    assert np.all(np.isfinite(got))
    rms = np.sqrt(np.mean(exp * exp, axis=1, keepdims=True))
    ratio = np.abs(got - exp) / (2e-5 * (np.abs(exp) + rms) + 1e-300)
    print(f"[parity] f32-activation tensor-core gemm: worst per-row gate ratio {ratio.max():.3f}")
    assert ratio.max() <= 1.0
    assert np.all(got[17] == 0.0)
    exact = np.asarray(_matmul(dev, W, N, K, A, M, exact_weights=True), np.float64).reshape(M, N)
    assert (np.abs(exact - exp) / (2e-5 * (np.abs(exp) + rms) + 1e-300)).max() <= 1.0


@pytest.mark.parametrize("M,N,K", [(64, 4096, 12288), (64, 6144, 4096), (40, 1536, 2048), (2, 256, 256), (17, 128, 512), (33, 384, 1024)])
def test_small_batch_gemm_weights_on_the_m_side(dev, M, N, K):
    """2..64 activation rows (batched decode steps): the kernel with the 128 weight rows of a tile on the MMA's M
    side, units of (tile, super-block column) dealt evenly to one CTA per SM, split tiles added in CTA order.
    f32 activations spanning ten decades against the exact product per row (gate 2e-5 up to K = 2048, growing
    with sqrt(K) beyond); two runs give the same
    bits; f16 activations with both weight numerics."""
    W = synthetic.q4k_matrix(synthetic.key(95, N + K), N, K)
    A = synthetic.normal_f32(synthetic.key(95, M), M * K).reshape(M, K)
    A = (A * (10.0 ** np.linspace(-3.0, 7.0, M).astype(np.float32))[:, None]).astype(np.float32)
    if M > 8:
        A[5] = 0.0
    exp = np.asarray(O.q4k_gemm(W, N, K, A.ravel(), M), np.float64).reshape(M, N)
    got32 = _matmul(dev, W, N, K, A, M)
    got = np.asarray(got32, np.float64).reshape(M, N)
    assert np.all(np.isfinite(got))
    rms = np.sqrt(np.mean(exp * exp, axis=1, keepdims=True))
    gate = 2e-5 * max(1.0, (K / 2048.0) ** 0.5)  # f32 accumulation error grows with the square root of K
    ratio = np.abs(got - exp) / (gate * (np.abs(exp) + rms) + 1e-300)
    print(f"[parity] small-batch gemm [{M},{K}]x[{N},{K}]: worst per-row gate ratio {ratio.max():.3f} at gate {gate:.1e}")
    assert ratio.max() <= 1.0
    assert np.array_equal(got32.view(np.uint32), _matmul(dev, W, N, K, A, M).view(np.uint32)), "not run-to-run deterministic"
    A16 = synthetic.normal_f16(synthetic.key(96, M), M * K)
    got16 = _matmul(dev, W, N, K, A16, M, out_dtype="f32", a_dtype="f16")
    assert_close(got16, O.q4k_gemm(W, N, K, A16.astype(np.float32), M), "small-batch gemm, f16 activations")
    gotw = _matmul(dev, W, N, K, A16, M, out_dtype="f32", a_dtype="f16", f16_weights=True)
    assert_close(gotw, O.q4k_gemm_f16_weights(W, N, K, A16.astype(np.float32), M), "small-batch gemm, f16 activations, f16-rounded weights")


def test_two_sm_gemm_split_over_k(dev):
    """More than 256 rows on few 512 x 256 pair tiles (here two): the two-SM kernel runs several clusters per tile
    along K, every part writes its own partial tile and the parts are added in a fixed order.  f32 activations
    (three products per K step) against the exact product per row, a ragged row count, and the same bits twice."""
    M, N, K = 300, 512, 4096
    W = synthetic.q4k_matrix(synthetic.key(97, 0), N, K)
    A = synthetic.normal_f32(synthetic.key(97, 1), M * K).reshape(M, K)
    A = (A * (10.0 ** np.linspace(-2.0, 5.0, M).astype(np.float32))[:, None]).astype(np.float32)
    exp = np.asarray(O.q4k_gemm(W, N, K, A.ravel(), M), np.float64).reshape(M, N)
    l0 = dev.launch_count
    got32 = _matmul(dev, W, N, K, A, M)
    assert dev.launch_count - l0 == 3, "expected the scaling cast, one tensor-core kernel and the reduction of the K parts"
    got = np.asarray(got32, np.float64).reshape(M, N)
    rms = np.sqrt(np.mean(exp * exp, axis=1, keepdims=True))
    gate = 2e-5 * (K / 2048.0) ** 0.5
    ratio = np.abs(got - exp) / (gate * (np.abs(exp) + rms) + 1e-300)
    print(f"[parity] two-SM gemm split over K [{M},{K}]x[{N},{K}]: worst per-row gate ratio {ratio.max():.3f}")
    assert ratio.max() <= 1.0
    assert np.array_equal(got32.view(np.uint32), _matmul(dev, W, N, K, A, M).view(np.uint32)), "not run-to-run deterministic"


def test_few_tiles_long_k_is_deterministic(dev):
    """A problem of few output tiles and a long K (here two tiles, K = 4096) is split over K: several CTAs per
    tile take whole super-blocks each, write their own partial tile, and a second kernel adds the parts in a
    fixed order (no atomics), so two runs give the same bits; f16 activations against the exact product,
    f32 activations (three products per K step in one f32 accumulator) against it per row."""
    M, N, K = 96, 256, 4096
    W = synthetic.q4k_matrix(synthetic.key(94, 0), N, K)
    A = synthetic.normal_f16(synthetic.key(94, 1), M * K)
    exp = O.q4k_gemm(W, N, K, A.astype(np.float32), M)
    got = _matmul(dev, W, N, K, A, M, out_dtype="f32", a_dtype="f16")
    assert_close(got, exp, f"few-tile gemm [{M},{K}]x[{N},{K}] vs the exact product")
    assert np.array_equal(got.view(np.uint32), _matmul(dev, W, N, K, A, M, out_dtype="f32", a_dtype="f16").view(np.uint32))
    A32 = synthetic.normal_f32(synthetic.key(94, 2), M * K)
    exp32 = np.asarray(O.q4k_gemm(W, N, K, A32, M), np.float64).reshape(M, N)
    got32 = _matmul(dev, W, N, K, A32, M)
    assert np.array_equal(got32.view(np.uint32), _matmul(dev, W, N, K, A32, M).view(np.uint32))
    got32 = np.asarray(got32, np.float64).reshape(M, N)
    rms = np.sqrt(np.mean(exp32 * exp32, axis=1, keepdims=True))
    assert (np.abs(got32 - exp32) / (2e-5 * (np.abs(exp32) + rms) + 1e-300)).max() <= 1.0
