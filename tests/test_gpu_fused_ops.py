"""The reference's fused decode ops (src/gpu/kernels/index.js:300-330) through the C ABI, against
compositions of the oracle's single ops."""
import numpy as np
import pytest

from doppler_b200 import ops, synthetic
from oracle import oracle as O
from parity import assert_close

pytestmark = pytest.mark.gpu


def _w(dev, seed, n, k):
    W = synthetic.q4k_matrix(synthetic.key(61, seed), n, k)
    return W, dev.weight_from(W, "q4k", [n, k])


@pytest.mark.parametrize("batch,hidden,inter", [(1, 1024, 3072), (1, 4096, 12288), (3, 512, 768), (1, 300, 520)])
def test_fused_ffn(dev, batch, hidden, inter):
    Wg, wg = _w(dev, 1, inter, hidden)
    Wu, wu = _w(dev, 2, inter, hidden)
    x = synthetic.normal_f32(synthetic.key(61, 3), batch * hidden)
    xt = dev.tensor_from(x.reshape(batch, hidden))
    out = ops.run_fused_ffn(xt, wg, wu, hidden, inter, batch_size=batch, alpha=0.5)
    assert out.shape == [batch, inter] and out.dtype == "f32"
    got = dev.read_tensor(out).reshape(batch, inter)
    for b in range(batch):
        g = O.q4k_gemv(Wg, inter, hidden, x[b * hidden:(b + 1) * hidden]).astype(np.float64)
        u = O.q4k_gemv(Wu, inter, hidden, x[b * hidden:(b + 1) * hidden]).astype(np.float64)
        exp = g / (1.0 + np.exp(-g)) * u * 0.5   # fused_ffn_q4k.wgsl:115-117,246
        assert_close(got[b], exp, f"fused ffn [{batch},{hidden}]->[{inter}] row {b}")
    # swigluLimit clamps the product
    lim = float(np.percentile(np.abs(got), 90))
    assert lim > 0
    out2 = ops.run_fused_ffn(xt, wg, wu, hidden, inter, batch_size=batch, alpha=0.5, swiglu_limit=lim)
    got2 = dev.read_tensor(out2).reshape(batch, inter)
    assert np.array_equal(got2, np.clip(got, -lim, lim))
    for t in (out, out2, xt):
        dev.release_buffer(t.buffer)
    # gate / up dtype mismatch is refused with the reference's message
    f16 = dev.weight_from(np.zeros((inter, hidden), np.float16), "f16", [inter, hidden])
    xt = dev.tensor_from(x.reshape(batch, hidden))
    with pytest.raises(ops.DopplerError, match="matching gate/up dtypes"):
        ops.run_fused_ffn(xt, wg, f16, hidden, inter, batch_size=batch)
    for b in (wg.buffer, wu.buffer, f16.buffer, xt.buffer):
        dev.release_buffer(b)


@pytest.mark.parametrize("N,K", [(4096, 4096), (1024, 3072), (130, 300)])
def test_matmul_residual_fused(dev, N, K):
    W, wb = _w(dev, 4, N, K)
    x = synthetic.normal_f32(synthetic.key(61, 5), K)
    r = synthetic.normal_f32(synthetic.key(61, 6), N, 50.0)
    xt, rt = dev.tensor_from(x.reshape(1, K)), dev.tensor_from(r.reshape(1, N))
    out = ops.run_matmul_residual_fused(xt, wb, rt, N=N, K=K, alpha=2.0)
    exp = 2.0 * O.q4k_gemv(W, N, K, x).astype(np.float64) + r
    assert_close(dev.read_tensor(out), exp, f"matmul+residual [{N},{K}]")
    # f16 weights take the same op
    w16 = synthetic.normal_f16(synthetic.key(61, 7), N * K, 0.05).reshape(N, K)
    wb16 = dev.weight_from(w16, "f16", [N, K])
    out16 = ops.run_matmul_residual_fused(xt, wb16, rt, N=N, K=K)
    assert_close(dev.read_tensor(out16), O.f16_gemv(w16, N, K, x).astype(np.float64) + r, "f16 matmul+residual")
    for b in (out.buffer, out16.buffer, xt.buffer, rt.buffer, wb.buffer, wb16.buffer):
        dev.release_buffer(b)


def test_matmul_rmsnorm_fused(dev):
    N, K = 1024, 3072
    W, wb = _w(dev, 8, N, K)
    x = synthetic.normal_f32(synthetic.key(61, 9), K)
    nw = synthetic.normal_f32(synthetic.key(61, 10), N, 0.1, 1.0)
    r = synthetic.normal_f32(synthetic.key(61, 11), N)
    xt, nwt, rt = dev.tensor_from(x.reshape(1, K)), dev.tensor_from(nw), dev.tensor_from(r.reshape(1, N))
    y = O.q4k_gemv(W, N, K, x)
    normed = O.rmsnorm(y, nw, 1, N, 1e-6).astype(np.float64)
    out = ops.run_matmul_rmsnorm_fused(xt, wb, nwt, N=N, K=K, eps=1e-6)
    assert_close(dev.read_tensor(out), normed, "matmul+rmsnorm")
    out_r = ops.run_matmul_rmsnorm_fused(xt, wb, nwt, N=N, K=K, eps=1e-6, residual=rt)   # residual after the norm
    assert_close(dev.read_tensor(out_r), normed + r, "matmul+rmsnorm+residual")
    with pytest.raises(ops.DopplerError, match="eps is required"):
        ops.run_matmul_rmsnorm_fused(xt, wb, nwt, N=N, K=K)
    for b in (out.buffer, out_r.buffer, xt.buffer, nwt.buffer, rt.buffer, wb.buffer):
        dev.release_buffer(b)


def test_lm_head_argmax(dev):
    vocab, hidden = 40000, 1024
    head = synthetic.normal_f16(synthetic.key(61, 12), vocab * hidden, 0.05).reshape(vocab, hidden)
    x = synthetic.normal_f32(synthetic.key(61, 13), hidden)
    logits = O.f16_gemv(head, vocab, hidden, x)
    best = int(np.argmax(logits))
    wb = dev.weight_from(head, "f16", [vocab, hidden])
    xt = dev.tensor_from(x.reshape(1, hidden))
    tok = ops.record_lm_head_argmax(None, xt, wb, vocab_size=vocab, hidden_size=hidden, output_index=2)
    got = np.frombuffer(dev.read_buffer(tok, 12), np.int32)
    assert got[2] == best == O.argmax(logits)
    # the pad token is never chosen
    tok2 = ops.record_lm_head_argmax(None, xt, wb, vocab_size=vocab, hidden_size=hidden, pad_token_id=best)
    second = int(np.frombuffer(dev.read_buffer(tok2, 4), np.int32)[0])
    assert second == O.argmax(logits, best) and second != best
    # a Q4_K LM head (lm_head_argmax_q4k.wgsl)
    Wq = synthetic.q4k_matrix(synthetic.key(61, 14), 4096, hidden)
    wq = dev.weight_from(Wq, "q4k", [4096, hidden])
    tok3 = ops.record_lm_head_argmax(None, xt, wq, vocab_size=4096, hidden_size=hidden)
    assert int(np.frombuffer(dev.read_buffer(tok3, 4), np.int32)[0]) == O.argmax(O.q4k_gemv(Wq, 4096, hidden, x))
    with pytest.raises(ops.DopplerError, match="must be f32"):
        ops.record_lm_head_argmax(None, dev.tensor_from(np.zeros(hidden, np.float16)), wb, vocab_size=vocab, hidden_size=hidden)
    for b in (tok, tok2, tok3, xt.buffer, wb.buffer, wq.buffer):
        dev.release_buffer(b)
