// C ABI of the op surface: argument validation (the checks the reference does
// in src/gpu/kernels/matmul-selection.js:197-257, attention.js:1047-1311, ...)
// and dispatch to the kernels.  No op here has a CPU path.
#include "common.h"

#include <cmath>
#include <cstdlib>
#include <cstring>

dp_status dpk_gemm_q4k_tc(dp_ctx *ctx, const uint8_t *W, const void *A, dp_dtype a_dtype, void *C, dp_dtype c_dtype,
                          int M, int N, int K, float alpha, bool f16_weights, bool *handled);
dp_status dpk_gemv_q4k_fast(dp_ctx *ctx, const uint8_t *W, const float *x, void *y, dp_dtype y_dtype, int N, int K,
                            float alpha, const float *residual, bool *handled);

extern "C" void dp_matmul_opts_default(dp_matmul_opts *o) {
  if (!o) return;
  memset(o, 0, sizeof *o);
  o->alpha = 1.0f;
  o->out_dtype = DP_F32;
  o->transpose_b = 1;
}

extern "C" void dp_attn_opts_default(dp_attn_opts *o) {
  if (!o) return;
  memset(o, 0, sizeof *o);
  o->seq_len = 1;
  o->causal = 1;
  o->batch = 1;
}

extern "C" void dp_rmsnorm_opts_default(dp_rmsnorm_opts *o) {
  if (!o) return;
  memset(o, 0, sizeof *o);
  o->batch_size = 1;
  o->output_scale = 1.0f;
}

static dp_status check_tensor(dp_ctx *ctx, const dp_tensor *t, const char *op, const char *name, size_t need_bytes) {
  if (!t || !t->buf) return dp_fail(ctx, DP_ERR_INVALID, "%s: %s is null", op, name);
  if (!t->buf->active) return dp_fail(ctx, DP_ERR_STATE, "%s: %s buffer '%s' was released", op, name, t->buf->label.c_str());
  if (t->buf->ctx != ctx) return dp_fail(ctx, DP_ERR_STATE, "%s: %s belongs to another context", op, name);
  if (t->offset % DP_BUFFER_ALIGN) return dp_fail(ctx, DP_ERR_INVALID, "%s: %s offset %zu is not 256-byte aligned", op, name, t->offset);
  if (dp_tavail(t) < need_bytes)
    return dp_fail(ctx, DP_ERR_INVALID, "%s: %s too small: need %zu bytes at offset %zu, buffer has %zu", op, name,
                   need_bytes, t->offset, t->buf->bytes);
  return DP_OK;
}

static void fill_tensor(dp_tensor *out, dp_buf buf, size_t off, dp_dtype dt, int ndim, int64_t a, int64_t b, int64_t c) {
  if (!out) return;
  memset(out, 0, sizeof *out);
  out->buf = buf; out->offset = off; out->dtype = dt; out->ndim = ndim;
  out->shape[0] = a; out->shape[1] = b; out->shape[2] = c;
}

// ---- matmul ------------------------------------------------------------------
extern "C" dp_status dp_matmul(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *A, const dp_weight *B, int M, int N,
                               int K, const dp_matmul_opts *opts_in, dp_tensor *out) {
  DP_TRY(dp_check_rec(ctx, rec));
  dp_matmul_opts o;
  if (opts_in) o = *opts_in; else dp_matmul_opts_default(&o);
  DP_CHECK(ctx, M > 0 && N > 0 && K > 0, "matmul: invalid dimensions M=%d N=%d K=%d", M, N, K);
  DP_CHECK(ctx, A && A->buf, "matmul: A is null");
  DP_CHECK(ctx, B && B->buf, "matmul: B is null");
  DP_CHECK(ctx, out != nullptr, "matmul: out is null");
  if (!o.transpose_b || B->layout != 0)
    return dp_fail(ctx, DP_ERR_UNSUPPORTED, "matmul: only row-layout [N,K] weights (transposeB=true) are on this path");
  DP_CHECK(ctx, B->shape[0] == N && B->shape[1] == K, "matmul: weight shape [%lld,%lld] does not match N=%d K=%d",
           (long long)B->shape[0], (long long)B->shape[1], N, K);
  DP_CHECK(ctx, o.out_dtype == DP_F32 || o.out_dtype == DP_F16, "matmul: outputDtype must be f16 or f32, got %s",
           dp_dtype_name(o.out_dtype));
  DP_CHECK(ctx, A->dtype == DP_F32 || A->dtype == DP_F16, "matmul: A dtype must be f16 or f32, got %s", dp_dtype_name(A->dtype));
  DP_CHECK(ctx, (o.a_off | o.b_off | o.c_off) % DP_BUFFER_ALIGN == 0,
           "matmul: aOffset/bOffset/cOffset must be 256-byte aligned (got %zu/%zu/%zu)", o.a_off, o.b_off, o.c_off);

  dp_tensor a = *A;
  a.offset += o.a_off;
  DP_TRY(check_tensor(ctx, &a, "matmul", "A", (size_t)M * K * dp_dtype_size(A->dtype)));
  const size_t bpr = dp_cdiv((size_t)K, DP_QK_K);
  size_t b_need;
  switch (B->dtype) {
    case DP_Q4K: b_need = (size_t)N * bpr * DP_Q4K_BLOCK_BYTES; break;  // matmul-selection.js:230-233
    case DP_F16: b_need = (size_t)N * K * 2; break;
    case DP_F32: b_need = (size_t)N * K * 4; break;
    default: return dp_fail(ctx, DP_ERR_INVALID, "matmul: unsupported weight dtype %s", dp_dtype_name(B->dtype));
  }
  dp_tensor bt;
  memset(&bt, 0, sizeof bt);
  bt.buf = B->buf; bt.offset = B->offset + o.b_off;
  DP_TRY(check_tensor(ctx, &bt, "matmul", "B", b_need));

  const size_t c_bytes = (size_t)M * N * dp_dtype_size(o.out_dtype);
  dp_buf cbuf = nullptr;
  DP_TRY(dp_out_buffer(ctx, o.out_buf, o.c_off, c_bytes, "matmul_output", &cbuf));
  void *cptr = (char *)cbuf->dptr + o.c_off;
  const char *aptr = dp_tptr(&a);
  const char *bptr = dp_tptr(&bt);
  dp_status st = DP_OK;
  if (B->dtype == DP_Q4K) {
    if (M == 1 && A->dtype == DP_F32) {
      bool handled = false;
      st = dpk_gemv_q4k_fast(ctx, (const uint8_t *)bptr, (const float *)aptr, cptr, o.out_dtype, N, K, o.alpha, nullptr, &handled);
      if (st == DP_OK && !handled)
        st = dpk_gemv_q4k(ctx, (const uint8_t *)bptr, (const float *)aptr, cptr, o.out_dtype, N, K, o.alpha, nullptr);
    } else {
      bool handled = false;
      // f16 activations on the tensor cores.  Default: the rule-selected kernel's numerics (matmul.rules.json:17,
      // fused_matmul_q4_batched_f16a.wgsl:107,151: f32 weights, f32 accumulate, one rounding of an f16 output).
      // f16_weights: the opt-in tiled kernel's numerics (matmul-selection.js:550-620,
      // fused_matmul_q4_prefill_tiled_f16.wgsl:201: weights rounded to f16 first), one tensor-core product.
      if (!o.exact_weights && M > 1 && A->dtype == DP_F16)
        st = dpk_gemm_q4k_tc(ctx, (const uint8_t *)bptr, aptr, A->dtype, cptr, o.out_dtype, M, N, K, o.alpha, o.f16_weights != 0, &handled);
      // f32 activations select the f32-exact product (matmul.rules.json:15-22): from 32 rows on the tensor
      // cores compute it in three passes (f16 halves and rounding residues of activations and weights)
      else if (!o.exact_weights && M >= 2 && A->dtype == DP_F32 && o.out_dtype == DP_F32)
        st = dpk_gemm_q4k_tc_rowscaled(ctx, (const uint8_t *)bptr, (const float *)aptr, (float *)cptr, M, N, K, o.alpha, 3, &handled);
      if (st == DP_OK && !handled)
        st = dpk_gemm_q4k_simt(ctx, (const uint8_t *)bptr, aptr, A->dtype, cptr, o.out_dtype, M, N, K, o.alpha);
    }
  } else if (B->dtype == DP_F16) {
    st = dpk_gemv_f16w(ctx, (const __half *)bptr, aptr, A->dtype, cptr, o.out_dtype, M, N, K, o.alpha);
  } else {
    if (A->dtype != DP_F32 || o.out_dtype != DP_F32)
      st = dp_fail(ctx, DP_ERR_UNSUPPORTED, "matmul: f32 weights need f32 A and f32 output");
    else
      st = dpk_gemv_f32w(ctx, (const float *)bptr, (const float *)aptr, (float *)cptr, M, N, K, o.alpha);
  }
  if (st != DP_OK) {
    if (!o.out_buf) dp_buf_release(ctx, cbuf);  // reference releases owned buffers before rethrow (matmul.js:644-655)
    return st;
  }
  dp_note_op(ctx, rec);
  fill_tensor(out, cbuf, o.c_off, o.out_dtype, 2, M, N, 0);
  return DP_OK;
}

// ---- dequant -------------------------------------------------------------------
static dp_status dequant_common(dp_ctx *ctx, dp_recorder *rec, dp_buf packed, size_t packed_off, size_t rows, size_t bpr,
                                size_t K, dp_dtype out_dtype, size_t out_off, dp_buf out_buf, dp_tensor *out, int ndim) {
  DP_TRY(dp_check_rec(ctx, rec));
  DP_CHECK(ctx, packed != nullptr, "dequantize: quantized buffer is null");
  DP_CHECK(ctx, out != nullptr, "dequantize: out is null");
  DP_CHECK(ctx, out_dtype == DP_F32 || out_dtype == DP_F16, "dequantize: outputDtype must be f16 or f32, got %s",
           dp_dtype_name(out_dtype));
  DP_CHECK(ctx, packed_off % 16 == 0, "dequantize: packed offset %zu is not 16-byte aligned", packed_off);
  dp_tensor pt;
  memset(&pt, 0, sizeof pt);
  pt.buf = packed;
  DP_TRY(check_tensor(ctx, &pt, "dequantize", "quantized", packed_off + rows * bpr * DP_Q4K_BLOCK_BYTES));
  const size_t out_bytes = rows * K * dp_dtype_size(out_dtype);
  dp_buf obuf = nullptr;
  DP_TRY(dp_out_buffer(ctx, out_buf, out_off, out_bytes ? out_bytes : 4, "dequant_output", &obuf));
  dp_status st = dpk_dequant_q4k(ctx, (const uint8_t *)packed->dptr + packed_off, rows, bpr, K, (char *)obuf->dptr + out_off, out_dtype);
  if (st != DP_OK) {
    if (!out_buf) dp_buf_release(ctx, obuf);
    return st;
  }
  dp_note_op(ctx, rec);
  if (ndim == 1) fill_tensor(out, obuf, out_off, out_dtype, 1, (int64_t)(rows * K), 0, 0);
  else fill_tensor(out, obuf, out_off, out_dtype, 2, (int64_t)rows, (int64_t)K, 0);
  return DP_OK;
}

extern "C" dp_status dp_dequant_q4k(dp_ctx *ctx, dp_recorder *rec, dp_buf packed, size_t packed_off, uint32_t num_blocks,
                                    dp_dtype out_dtype, size_t out_off, dp_buf out_buf, dp_tensor *out) {
  if (!ctx) return DP_ERR_INVALID;
  return dequant_common(ctx, rec, packed, packed_off, 1, num_blocks, (size_t)num_blocks * DP_QK_K, out_dtype, out_off,
                        out_buf, out, 1);
}

extern "C" dp_status dp_dequant_q4k_rowwise(dp_ctx *ctx, dp_recorder *rec, dp_buf packed, size_t packed_off, int rows,
                                            int K, dp_dtype out_dtype, dp_buf out_buf, dp_tensor *out) {
  if (!ctx) return DP_ERR_INVALID;
  DP_CHECK(ctx, rows > 0 && K > 0, "dequantizeRowwise: invalid shape [%d,%d]", rows, K);
  return dequant_common(ctx, rec, packed, packed_off, (size_t)rows, dp_cdiv((size_t)K, DP_QK_K), (size_t)K, out_dtype, 0,
                        out_buf, out, 2);
}

// ---- attention -------------------------------------------------------------------
extern "C" dp_status dp_attention(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *Q, const dp_tensor *K,
                                  const dp_tensor *V, int num_heads, int head_dim, const dp_attn_opts *opts_in,
                                  dp_tensor *out) {
  DP_TRY(dp_check_rec(ctx, rec));
  dp_attn_opts o;
  if (opts_in) o = *opts_in; else dp_attn_opts_default(&o);
  if (o.batch <= 0) o.batch = 1;
  if (o.seq_len <= 0) o.seq_len = 1;
  if (o.num_kv_heads <= 0) o.num_kv_heads = num_heads;
  DP_CHECK(ctx, out != nullptr, "attention: out is null");
  DP_CHECK(ctx, num_heads > 0 && head_dim > 0 && head_dim <= 512, "attention: invalid numHeads=%d headDim=%d", num_heads, head_dim);
  DP_CHECK(ctx, num_heads % o.num_kv_heads == 0, "attention: numHeads %d is not a multiple of numKVHeads %d", num_heads, o.num_kv_heads);
  DP_CHECK(ctx, o.kv_len >= 0, "attention: invalid kvLen %d", o.kv_len);
  DP_CHECK(ctx, Q && Q->dtype == DP_F32, "attention: Q must be f32");
  DP_CHECK(ctx, K && V && K->dtype == DP_F16 && V->dtype == DP_F16, "attention: this path reads an f16 KV cache (K/V dtype f16)");
  const size_t q_elems = (size_t)o.batch * o.seq_len * num_heads * head_dim;
  DP_TRY(check_tensor(ctx, Q, "attention", "Q", q_elems * 4));
  const size_t kv_row = (size_t)o.num_kv_heads * head_dim;
  if (o.batch > 1) DP_CHECK(ctx, o.kv_batch_stride >= (size_t)o.kv_len * kv_row && o.kv_batch_stride % 8 == 0,
                            "attention: kv_batch_stride %zu too small or not a multiple of 8", o.kv_batch_stride);
  const size_t kv_need = ((size_t)(o.batch - 1) * o.kv_batch_stride + (size_t)o.kv_len * kv_row) * 2;
  DP_TRY(check_tensor(ctx, K, "attention", "K", kv_need));
  DP_TRY(check_tensor(ctx, V, "attention", "V", kv_need));
  if (o.kv_lens) DP_CHECK(ctx, o.kv_lens->active && o.kv_lens->bytes >= (size_t)o.batch * 4, "attention: kvLenBuffer too small");
  dp_buf obuf = nullptr;
  DP_TRY(dp_out_buffer(ctx, o.out_buf, 0, q_elems * 4, "attention_output", &obuf));
  dpk_attn_params p{};
  p.q = (const float *)dp_tptr(Q);
  p.k = (const __half *)dp_tptr(K);
  p.v = (const __half *)dp_tptr(V);
  p.out = (float *)obuf->dptr;
  p.batch = o.batch; p.seq_len = o.seq_len; p.kv_len = o.kv_len;
  p.num_heads = num_heads; p.num_kv_heads = o.num_kv_heads; p.head_dim = head_dim;
  p.scale = o.scale > 0.0f ? o.scale : 1.0f / sqrtf((float)head_dim);
  p.softcap = o.attn_softcap;
  p.causal = o.causal; p.start_pos = o.start_pos; p.sliding_window = o.sliding_window; p.kv_start = o.kv_start;
  p.kv_batch_stride = o.kv_batch_stride;
  p.kv_lens = o.kv_lens ? (const int *)o.kv_lens->dptr : nullptr;
  dp_status st = dpk_attention(ctx, p);
  if (st != DP_OK) {
    if (!o.out_buf) dp_buf_release(ctx, obuf);
    return st;
  }
  dp_note_op(ctx, rec);
  if (out) {
    memset(out, 0, sizeof *out);
    out->buf = obuf; out->dtype = DP_F32;
    if (o.batch > 1) { out->ndim = 4; out->shape[0] = o.batch; out->shape[1] = o.seq_len; out->shape[2] = num_heads; out->shape[3] = head_dim; }
    else { out->ndim = 3; out->shape[0] = o.seq_len; out->shape[1] = num_heads; out->shape[2] = head_dim; }
  }
  return DP_OK;
}

// ---- small ops ---------------------------------------------------------------------
extern "C" dp_status dp_rmsnorm(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *input, const dp_tensor *weight, float eps,
                                const dp_rmsnorm_opts *opts_in, dp_tensor *out) {
  DP_TRY(dp_check_rec(ctx, rec));
  dp_rmsnorm_opts o;
  if (opts_in) o = *opts_in; else dp_rmsnorm_opts_default(&o);
  DP_CHECK(ctx, out != nullptr, "rmsnorm: out is null");
  DP_CHECK(ctx, o.batch_size > 0 && o.hidden_size > 0, "rmsnorm: invalid batchSize=%d hiddenSize=%d", o.batch_size, o.hidden_size);
  DP_CHECK(ctx, input && input->dtype == DP_F32, "rmsnorm: input must be f32");
  DP_CHECK(ctx, weight && (weight->dtype == DP_F32 || weight->dtype == DP_F16), "rmsnorm: weight must be f32 or f16");
  const size_t n = (size_t)o.batch_size * o.hidden_size;
  DP_TRY(check_tensor(ctx, input, "rmsnorm", "input", n * 4));
  DP_TRY(check_tensor(ctx, weight, "rmsnorm", "weight", (size_t)o.hidden_size * dp_dtype_size(weight->dtype)));
  if (o.residual) DP_TRY(check_tensor(ctx, o.residual, "rmsnorm", "residual", n * 4));
  DP_CHECK(ctx, !o.pre_residual || o.residual, "rmsnorm: preResidual needs a residual tensor");
  if (o.residual_sum_output) DP_CHECK(ctx, o.residual_sum_output->active && o.residual_sum_output->bytes >= n * 4,
                                       "rmsnorm: residualSumOutput too small");
  dp_buf obuf = nullptr;
  DP_TRY(dp_out_buffer(ctx, o.out_buf, 0, n * 4, "rmsnorm_output", &obuf));
  dp_status st = dpk_rmsnorm(ctx, (const float *)dp_tptr(input), dp_tptr(weight), weight->dtype == DP_F16,
                             o.residual ? (const float *)dp_tptr(o.residual) : nullptr, o.pre_residual != 0,
                             o.residual_sum_output ? (float *)o.residual_sum_output->dptr : nullptr, (float *)obuf->dptr,
                             o.batch_size, o.hidden_size, eps, o.weight_offset != 0,
                             o.output_scale == 0.0f ? 1.0f : o.output_scale);
  if (st != DP_OK) {
    if (!o.out_buf) dp_buf_release(ctx, obuf);
    return st;
  }
  dp_note_op(ctx, rec);
  fill_tensor(out, obuf, 0, DP_F32, 2, o.batch_size, o.hidden_size, 0);
  return DP_OK;
}

extern "C" dp_status dp_rmsnorm_qk(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *q, const dp_tensor *q_weight,
                                   const dp_tensor *k, const dp_tensor *k_weight, int q_rows, int k_rows, int head_dim,
                                   float eps, int weight_offset) {
  DP_TRY(dp_check_rec(ctx, rec));
  DP_CHECK(ctx, q_rows >= 0 && k_rows >= 0 && head_dim > 0, "rmsnorm_qk: invalid rows/headDim");
  DP_CHECK(ctx, q && k && q->dtype == DP_F32 && k->dtype == DP_F32, "rmsnorm_qk: q and k must be f32");
  DP_CHECK(ctx, q_weight && k_weight && q_weight->dtype == DP_F32 && k_weight->dtype == DP_F32, "rmsnorm_qk: weights must be f32");
  DP_TRY(check_tensor(ctx, q, "rmsnorm_qk", "q", (size_t)q_rows * head_dim * 4));
  DP_TRY(check_tensor(ctx, k, "rmsnorm_qk", "k", (size_t)k_rows * head_dim * 4));
  DP_TRY(check_tensor(ctx, q_weight, "rmsnorm_qk", "q_weight", (size_t)head_dim * 4));
  DP_TRY(check_tensor(ctx, k_weight, "rmsnorm_qk", "k_weight", (size_t)head_dim * 4));
  DP_TRY(dpk_rmsnorm_qk(ctx, (float *)dp_tptr(q), (const float *)dp_tptr(q_weight), (float *)dp_tptr(k),
                        (const float *)dp_tptr(k_weight), q_rows, k_rows, head_dim, eps, weight_offset != 0));
  dp_note_op(ctx, rec);
  return DP_OK;
}

extern "C" dp_status dp_rope(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *input, const dp_tensor *freqs_cos,
                             const dp_tensor *freqs_sin, int seq_len, const dp_rope_opts *o) {
  DP_TRY(dp_check_rec(ctx, rec));
  DP_CHECK(ctx, o != nullptr, "rope: options are required (numHeads, headDim)");
  DP_CHECK(ctx, o->num_heads > 0 && o->head_dim > 0 && seq_len > 0, "rope: invalid numHeads=%d headDim=%d seqLen=%d",
           o->num_heads, o->head_dim, seq_len);
  const int rotary = o->rotary_dim > 0 ? o->rotary_dim : o->head_dim;
  const int span = o->pair_span_dim > 0 ? o->pair_span_dim : rotary;
  DP_CHECK(ctx, rotary % 2 == 0 && rotary <= o->head_dim && span <= o->head_dim && span >= rotary,
           "rope: rotaryDim=%d pairSpanDim=%d do not fit headDim=%d", rotary, span, o->head_dim);
  DP_CHECK(ctx, input && input->dtype == DP_F32, "rope: input must be f32");
  DP_CHECK(ctx, o->start_pos >= 0, "rope: negative startPos");
  DP_TRY(check_tensor(ctx, input, "rope", "input", (size_t)seq_len * o->num_heads * o->head_dim * 4));
  const size_t tbl = (size_t)(o->start_pos + seq_len) * (rotary / 2) * 4;
  DP_TRY(check_tensor(ctx, freqs_cos, "rope", "freqsCos", tbl));
  DP_TRY(check_tensor(ctx, freqs_sin, "rope", "freqsSin", tbl));
  DP_TRY(dpk_rope(ctx, (float *)dp_tptr(input), (const float *)dp_tptr(freqs_cos), (const float *)dp_tptr(freqs_sin),
                  seq_len, o->num_heads, o->head_dim, rotary, span, o->interleaved != 0, o->start_pos));
  dp_note_op(ctx, rec);
  return DP_OK;
}

// host-side table build, src/inference/pipelines/text/init-rope.js:22-25,121-131 (ropeScale 1):
// the frequency is rounded to f32 before it multiplies the position.
extern "C" dp_status dp_rope_tables(double theta, int rotary_dim, int max_seq, float *cos_out, float *sin_out) {
  if (!cos_out || !sin_out || rotary_dim <= 0 || rotary_dim % 2 || max_seq <= 0 || !(theta > 0)) return DP_ERR_INVALID;
  const int half = rotary_dim / 2;
  for (int i = 0; i < half; i++) {
    const float freq = (float)(1.0 / pow(theta, (double)(2 * i) / (double)rotary_dim));
    for (int pos = 0; pos < max_seq; pos++) {
      const double angle = (double)pos * (double)freq;
      cos_out[(size_t)pos * half + i] = (float)cos(angle);
      sin_out[(size_t)pos * half + i] = (float)sin(angle);
    }
  }
  return DP_OK;
}

extern "C" dp_status dp_silu_mul(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *up, const dp_tensor *gate, size_t n,
                                 float clamp_max, dp_buf out_buf, dp_tensor *out) {
  DP_TRY(dp_check_rec(ctx, rec));
  DP_CHECK(ctx, out != nullptr, "silu: out is null");
  DP_CHECK(ctx, up && gate && up->dtype == DP_F32 && gate->dtype == DP_F32, "silu: up and gate must be f32");
  DP_TRY(check_tensor(ctx, up, "silu", "input", n * 4));
  DP_TRY(check_tensor(ctx, gate, "silu", "gate", n * 4));
  dp_buf obuf = nullptr;
  DP_TRY(dp_out_buffer(ctx, out_buf, 0, n ? n * 4 : 4, "silu_output", &obuf));
  dp_status st = dpk_silu_mul(ctx, (const float *)dp_tptr(up), (const float *)dp_tptr(gate), (float *)obuf->dptr, n, clamp_max);
  if (st != DP_OK) { if (!out_buf) dp_buf_release(ctx, obuf); return st; }
  dp_note_op(ctx, rec);
  fill_tensor(out, obuf, 0, DP_F32, 1, (int64_t)n, 0, 0);
  return DP_OK;
}

extern "C" dp_status dp_residual_add(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *a, const dp_tensor *b, size_t n,
                                     float scale, dp_buf out_buf, dp_tensor *out) {
  DP_TRY(dp_check_rec(ctx, rec));
  DP_CHECK(ctx, out != nullptr, "residual: out is null");
  DP_CHECK(ctx, a && b && a->dtype == DP_F32 && b->dtype == DP_F32, "residual: a and b must be f32");
  DP_TRY(check_tensor(ctx, a, "residual", "a", n * 4));
  DP_TRY(check_tensor(ctx, b, "residual", "b", n * 4));
  dp_buf obuf = nullptr;
  DP_TRY(dp_out_buffer(ctx, out_buf, 0, n ? n * 4 : 4, "residual_output", &obuf));
  dp_status st = dpk_residual_add(ctx, (const float *)dp_tptr(a), (const float *)dp_tptr(b), (float *)obuf->dptr, n,
                                  scale == 0.0f ? 1.0f : scale);
  if (st != DP_OK) { if (!out_buf) dp_buf_release(ctx, obuf); return st; }
  dp_note_op(ctx, rec);
  fill_tensor(out, obuf, 0, DP_F32, 1, (int64_t)n, 0, 0);
  return DP_OK;
}

extern "C" dp_status dp_gather_f16(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *ids, const dp_tensor *table, int n_ids,
                                   int hidden, dp_buf out_buf, dp_tensor *out) {
  DP_TRY(dp_check_rec(ctx, rec));
  DP_CHECK(ctx, out != nullptr, "gather: out is null");
  DP_CHECK(ctx, n_ids > 0 && hidden > 0, "gather: invalid numTokens=%d hiddenSize=%d", n_ids, hidden);
  DP_CHECK(ctx, ids && ids->dtype == DP_I32, "gather: indices must be i32");
  DP_CHECK(ctx, table && table->dtype == DP_F16, "gather: embedding table must be f16");
  DP_TRY(check_tensor(ctx, ids, "gather", "indices", (size_t)n_ids * 4));
  DP_TRY(check_tensor(ctx, table, "gather", "embeddings", (size_t)hidden * 2));
  dp_buf obuf = nullptr;
  DP_TRY(dp_out_buffer(ctx, out_buf, 0, (size_t)n_ids * hidden * 4, "gather_output", &obuf));
  dp_status st = dpk_gather_f16(ctx, (const int *)dp_tptr(ids), (const __half *)dp_tptr(table), (float *)obuf->dptr, n_ids, hidden);
  if (st != DP_OK) { if (!out_buf) dp_buf_release(ctx, obuf); return st; }
  dp_note_op(ctx, rec);
  fill_tensor(out, obuf, 0, DP_F32, 2, n_ids, hidden, 0);
  return DP_OK;
}

extern "C" dp_status dp_kv_write_f32_to_f16(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *src, dp_buf dst,
                                            size_t dst_offset_elems, size_t n) {
  DP_TRY(dp_check_rec(ctx, rec));
  DP_CHECK(ctx, src && src->dtype == DP_F32, "kv_cache_write: source must be f32");
  DP_CHECK(ctx, dst && dst->active, "kv_cache_write: destination buffer is null or released");
  DP_TRY(check_tensor(ctx, src, "kv_cache_write", "source", n * 4));
  DP_CHECK(ctx, (dst_offset_elems + n) * 2 <= dst->bytes, "kv_cache_write: %zu elements at offset %zu exceed the cache buffer (%zu bytes)",
           n, dst_offset_elems, dst->bytes);
  DP_TRY(dpk_kv_write(ctx, (const float *)dp_tptr(src), (__half *)dst->dptr + dst_offset_elems, n));
  dp_note_op(ctx, rec);
  return DP_OK;
}

extern "C" dp_status dp_argmax(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *logits, int n, int pad_id,
                               dp_buf out_tokens, int output_index) {
  DP_TRY(dp_check_rec(ctx, rec));
  DP_CHECK(ctx, n > 0, "argmax: invalid vocab size %d", n);
  DP_CHECK(ctx, logits && logits->dtype == DP_F32, "argmax: logits must be f32");
  DP_TRY(check_tensor(ctx, logits, "argmax", "logits", (size_t)n * 4));
  DP_CHECK(ctx, out_tokens && out_tokens->active && output_index >= 0 && (size_t)(output_index + 1) * 4 <= out_tokens->bytes,
           "argmax: output token buffer too small for index %d", output_index);
  DP_TRY(dp_scratch(ctx, &ctx->argmax_scratch, 256 * 8, "argmax_partials"));
  float *vals = (float *)ctx->argmax_scratch->dptr;
  int *idxs = (int *)(vals + 256);
  DP_TRY(dpk_argmax(ctx, (const float *)dp_tptr(logits), n, pad_id, (int *)out_tokens->dptr, output_index, vals, idxs, 0, nullptr));
  dp_note_op(ctx, rec);
  return DP_OK;
}

// ---- quantizer -----------------------------------------------------------------------------
dp_status dpk_quantize_q4k(dp_ctx *ctx, const float *data, uint8_t *out, size_t rows, size_t cols, bool full_pad);

extern "C" dp_status dp_quantize_q4k(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *src, int64_t rows, int64_t cols, int full_pad,
                                     dp_buf out_buf, dp_weight *out) {
  DP_TRY(dp_check_rec(ctx, rec));
  DP_CHECK(ctx, out != nullptr, "quantize: out is null");
  DP_CHECK(ctx, rows > 0 && cols > 0, "quantize: invalid shape [%lld,%lld]", (long long)rows, (long long)cols);
  DP_CHECK(ctx, src && src->dtype == DP_F32, "quantize: source must be f32");
  DP_TRY(check_tensor(ctx, src, "quantize", "source", (size_t)rows * cols * 4));
  const size_t bytes = (size_t)rows * dp_cdiv((size_t)cols, DP_QK_K) * DP_Q4K_BLOCK_BYTES;
  dp_buf obuf = nullptr;
  DP_TRY(dp_out_buffer(ctx, out_buf, 0, bytes, "q4k_quantized", &obuf));
  dp_status st = dpk_quantize_q4k(ctx, (const float *)dp_tptr(src), (uint8_t *)obuf->dptr, (size_t)rows, (size_t)cols, full_pad != 0);
  if (st != DP_OK) { if (!out_buf) dp_buf_release(ctx, obuf); return st; }
  dp_note_op(ctx, rec);
  memset(out, 0, sizeof *out);
  out->buf = obuf; out->offset = 0; out->dtype = DP_Q4K; out->layout = 0;
  out->shape[0] = rows; out->shape[1] = cols;
  return DP_OK;
}

// ---- fused decode ops ------------------------------------------------------------------
extern "C" void dp_ffn_opts_default(dp_ffn_opts *o) {
  if (!o) return;
  memset(o, 0, sizeof *o);
  o->batch_size = 1;
  o->alpha = 1.0f;
}

// fused_ffn_q4k.wgsl:115-117,241-246
__global__ void ffn_activate_kernel(const float *__restrict__ g, const float *__restrict__ u, float *__restrict__ out, size_t n,
                                    float alpha, float clamp_max) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float x = g[i];
    float v = (x / (1.0f + expf(-x))) * u[i] * alpha;
    if (clamp_max > 0.0f) v = fminf(fmaxf(v, -clamp_max), clamp_max);
    out[i] = v;
  }
}

// validated device pointer of a row-layout [N,K] weight (Q4_K or f16)
static dp_status fused_weight(dp_ctx *ctx, const dp_weight *B, const char *op, const char *name, int N, int K, const char **ptr) {
  if (!B || !B->buf) return dp_fail(ctx, DP_ERR_INVALID, "%s: %s is null", op, name);
  if (B->layout != 0) return dp_fail(ctx, DP_ERR_UNSUPPORTED, "%s: %s must use the row layout [N,K]", op, name);
  if (B->shape[0] != N || B->shape[1] != K)
    return dp_fail(ctx, DP_ERR_INVALID, "%s: %s shape [%lld,%lld] does not match [%d,%d]", op, name, (long long)B->shape[0],
                   (long long)B->shape[1], N, K);
  size_t need;
  if (B->dtype == DP_Q4K) need = (size_t)N * dp_cdiv((size_t)K, DP_QK_K) * DP_Q4K_BLOCK_BYTES;
  else if (B->dtype == DP_F16) need = (size_t)N * K * 2;
  else return dp_fail(ctx, DP_ERR_UNSUPPORTED, "%s: %s dtype %s is outside this path (q4k or f16)", op, name, dp_dtype_name(B->dtype));
  dp_tensor t;
  memset(&t, 0, sizeof t);
  t.buf = B->buf; t.offset = B->offset;
  DP_TRY(check_tensor(ctx, &t, op, name, need));
  *ptr = dp_tptr(&t);
  return DP_OK;
}

// y[M,N] (f32) = alpha * x[M,K] . W^T (+ residual, M == 1 only)
static dp_status fused_matvec(dp_ctx *ctx, dp_dtype wdtype, const char *w, const float *x, float *y, int M, int N, int K, float alpha,
                              const float *residual) {
  if (wdtype == DP_Q4K) {
    if (M == 1) {
      bool handled = false;
      DP_TRY(dpk_gemv_q4k_fast(ctx, (const uint8_t *)w, x, y, DP_F32, N, K, alpha, residual, &handled));
      if (!handled) DP_TRY(dpk_gemv_q4k(ctx, (const uint8_t *)w, x, y, DP_F32, N, K, alpha, residual));
      return DP_OK;
    }
    bool handled = false;
    if (M >= 2) DP_TRY(dpk_gemm_q4k_tc_rowscaled(ctx, (const uint8_t *)w, x, y, M, N, K, alpha, 3, &handled));
    if (handled) return DP_OK;
    return dpk_gemm_q4k_simt(ctx, (const uint8_t *)w, x, DP_F32, y, DP_F32, M, N, K, alpha);
  }
  DP_TRY(dpk_gemv_f16w(ctx, (const __half *)w, x, DP_F32, y, DP_F32, M, N, K, alpha));
  if (residual) DP_TRY(dpk_residual_add(ctx, y, residual, y, (size_t)N, 1.0f));
  return DP_OK;
}

extern "C" dp_status dp_fused_ffn(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *input, const dp_weight *w_gate,
                                  const dp_weight *w_up, int hidden, int inter, const dp_ffn_opts *opts_in, dp_tensor *out) {
  DP_TRY(dp_check_rec(ctx, rec));
  dp_ffn_opts o;
  if (opts_in) o = *opts_in; else dp_ffn_opts_default(&o);
  DP_CHECK(ctx, out != nullptr, "fused_ffn: out is null");
  DP_CHECK(ctx, hidden > 0 && inter > 0 && o.batch_size > 0, "fused_ffn: invalid hiddenSize=%d intermediateSize=%d batchSize=%d", hidden,
           inter, o.batch_size);
  DP_CHECK(ctx, w_gate && w_up, "fused_ffn: gate/up weights are null");
  DP_CHECK(ctx, w_gate->dtype == w_up->dtype, "Fused FFN requires matching gate/up dtypes (gate=%s, up=%s)", dp_dtype_name(w_gate->dtype),
           dp_dtype_name(w_up->dtype));
  DP_CHECK(ctx, input && input->dtype == DP_F32, "Fused FFN requires f32 activations");
  const int M = o.batch_size;
  DP_TRY(check_tensor(ctx, input, "fused_ffn", "input", (size_t)M * hidden * 4));
  const char *wg = nullptr, *wu = nullptr;
  DP_TRY(fused_weight(ctx, w_gate, "fused_ffn", "W_gate", inter, hidden, &wg));
  DP_TRY(fused_weight(ctx, w_up, "fused_ffn", "W_up", inter, hidden, &wu));
  const size_t n = (size_t)M * inter;
  dp_buf obuf = nullptr, tmp = nullptr;
  DP_TRY(dp_out_buffer(ctx, o.out_buf, 0, n * 4, "fused_ffn_output", &obuf));
  dp_status st = dp_buf_acquire(ctx, 2 * n * 4, "fused_ffn_gate_up", &tmp);
  if (st == DP_OK) {
    float *g = (float *)tmp->dptr, *u = g + n;
    const float *x = (const float *)dp_tptr(input);
    st = fused_matvec(ctx, w_gate->dtype, wg, x, g, M, inter, hidden, 1.0f, nullptr);
    if (st == DP_OK) st = fused_matvec(ctx, w_up->dtype, wu, x, u, M, inter, hidden, 1.0f, nullptr);
    if (st == DP_OK) {
      size_t grid = (n + 255) / 256;
      if (grid > (size_t)ctx->sm_count * 8) grid = (size_t)ctx->sm_count * 8;
      cudaError_t e = dp_launch_impl(ctx, ffn_activate_kernel, dim3((unsigned)grid), dim3(256), 0, (const float *)g, (const float *)u,
                                     (float *)obuf->dptr, n, o.alpha, o.swiglu_limit);
      ctx->launches++;
      if (e != cudaSuccess) st = dp_fail(ctx, DP_ERR_CUDA, "launch of ffn_activate_kernel failed: %s", cudaGetErrorString(e));
    }
    dp_buf_release(ctx, tmp);  // stream ordered: reused only by later work
  }
  if (st != DP_OK) { if (!o.out_buf) dp_buf_release(ctx, obuf); return st; }
  dp_note_op(ctx, rec);
  fill_tensor(out, obuf, 0, DP_F32, 2, M, inter, 0);
  return DP_OK;
}

extern "C" dp_status dp_matmul_residual(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *input, const dp_weight *weight,
                                        const dp_tensor *residual, int N, int K, float alpha, dp_buf out_buf, dp_tensor *out) {
  DP_TRY(dp_check_rec(ctx, rec));
  DP_CHECK(ctx, out != nullptr, "matmul_residual: out is null");
  DP_CHECK(ctx, N > 0 && K > 0, "matmul_residual: invalid N=%d K=%d", N, K);
  DP_CHECK(ctx, input && input->dtype == DP_F32, "matmul_residual: input must be f32");
  DP_CHECK(ctx, residual && residual->dtype == DP_F32, "matmul_residual: residual must be f32");
  DP_TRY(check_tensor(ctx, input, "matmul_residual", "input", (size_t)K * 4));
  DP_TRY(check_tensor(ctx, residual, "matmul_residual", "residual", (size_t)N * 4));
  const char *w = nullptr;
  DP_TRY(fused_weight(ctx, weight, "matmul_residual", "weight", N, K, &w));
  dp_buf obuf = nullptr;
  DP_TRY(dp_out_buffer(ctx, out_buf, 0, (size_t)N * 4, "matmul_residual_output", &obuf));
  dp_status st = fused_matvec(ctx, weight->dtype, w, (const float *)dp_tptr(input), (float *)obuf->dptr, 1, N, K,
                              alpha == 0.0f ? 1.0f : alpha, (const float *)dp_tptr(residual));
  if (st != DP_OK) { if (!out_buf) dp_buf_release(ctx, obuf); return st; }
  dp_note_op(ctx, rec);
  fill_tensor(out, obuf, 0, DP_F32, 2, 1, N, 0);
  return DP_OK;
}

extern "C" dp_status dp_matmul_rmsnorm(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *input, const dp_weight *weight,
                                       const dp_tensor *norm_weight, int N, int K, float eps, const dp_tensor *residual,
                                       int weight_offset, dp_buf out_buf, dp_tensor *out) {
  DP_TRY(dp_check_rec(ctx, rec));
  DP_CHECK(ctx, out != nullptr, "matmul_rmsnorm: out is null");
  DP_CHECK(ctx, N > 0 && K > 0, "matmul_rmsnorm: invalid N=%d K=%d", N, K);
  DP_CHECK(ctx, eps > 0.0f, "[MatmulRMSNormFused] eps is required.");
  DP_CHECK(ctx, input && input->dtype == DP_F32, "matmul_rmsnorm: input must be f32");
  DP_TRY(check_tensor(ctx, input, "matmul_rmsnorm", "input", (size_t)K * 4));
  DP_CHECK(ctx, norm_weight && (norm_weight->dtype == DP_F32 || norm_weight->dtype == DP_F16), "matmul_rmsnorm: norm weight must be f32 or f16");
  DP_TRY(check_tensor(ctx, norm_weight, "matmul_rmsnorm", "normWeight", (size_t)N * dp_dtype_size(norm_weight->dtype)));
  if (residual) {
    DP_CHECK(ctx, residual->dtype == DP_F32, "matmul_rmsnorm: residual must be f32");
    DP_TRY(check_tensor(ctx, residual, "matmul_rmsnorm", "residual", (size_t)N * 4));
  }
  const char *w = nullptr;
  DP_TRY(fused_weight(ctx, weight, "matmul_rmsnorm", "weight", N, K, &w));
  dp_buf obuf = nullptr, tmp = nullptr;
  DP_TRY(dp_out_buffer(ctx, out_buf, 0, (size_t)N * 4, "matmul_rmsnorm_output", &obuf));
  dp_status st = dp_buf_acquire(ctx, (size_t)N * 4, "matmul_rmsnorm_projection", &tmp);
  if (st == DP_OK) {
    st = fused_matvec(ctx, weight->dtype, w, (const float *)dp_tptr(input), (float *)tmp->dptr, 1, N, K, 1.0f, nullptr);
    if (st == DP_OK)
      st = dpk_rmsnorm(ctx, (const float *)tmp->dptr, dp_tptr(norm_weight), norm_weight->dtype == DP_F16,
                       residual ? (const float *)dp_tptr(residual) : nullptr, false, nullptr, (float *)obuf->dptr, 1, N, eps,
                       weight_offset != 0, 1.0f);
    dp_buf_release(ctx, tmp);
  }
  if (st != DP_OK) { if (!out_buf) dp_buf_release(ctx, obuf); return st; }
  dp_note_op(ctx, rec);
  fill_tensor(out, obuf, 0, DP_F32, 2, 1, N, 0);
  return DP_OK;
}

extern "C" dp_status dp_lm_head_argmax(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *input, const dp_weight *lm_head, int vocab,
                                       int hidden, int pad_id, dp_buf out_tokens, int output_index) {
  DP_TRY(dp_check_rec(ctx, rec));
  DP_CHECK(ctx, vocab > 0 && hidden > 0, "[LmHeadArgmax] invalid vocabSize=%d hiddenSize=%d", vocab, hidden);
  DP_CHECK(ctx, input && input->dtype == DP_F32, "[LmHeadArgmax] input tensor must be f32, got \"%s\".",
           input ? dp_dtype_name(input->dtype) : "unknown");
  DP_TRY(check_tensor(ctx, input, "lm_head_argmax", "input", (size_t)hidden * 4));
  DP_CHECK(ctx, out_tokens && out_tokens->active && output_index >= 0 && (size_t)(output_index + 1) * 4 <= out_tokens->bytes,
           "[LmHeadArgmax] output buffer too small for outputIndex %d", output_index);
  const char *w = nullptr;
  DP_TRY(fused_weight(ctx, lm_head, "lm_head_argmax", "lmHead", vocab, hidden, &w));
  DP_TRY(dp_scratch(ctx, &ctx->argmax_scratch, 256 * 8, "argmax_partials"));
  dp_buf logits = nullptr;
  DP_TRY(dp_buf_acquire(ctx, (size_t)vocab * 4, "lm_head_argmax_temp_logits", &logits));
  dp_status st = fused_matvec(ctx, lm_head->dtype, w, (const float *)dp_tptr(input), (float *)logits->dptr, 1, vocab, hidden, 1.0f, nullptr);
  if (st == DP_OK) {
    float *vals = (float *)ctx->argmax_scratch->dptr;
    st = dpk_argmax(ctx, (const float *)logits->dptr, vocab, pad_id, (int *)out_tokens->dptr, output_index, vals, (int *)(vals + 256), 0,
                    nullptr);
  }
  dp_buf_release(ctx, logits);
  if (st != DP_OK) return st;
  dp_note_op(ctx, rec);
  return DP_OK;
}

// ---- KV cache ------------------------------------------------------------------------
struct dp_kv_cache {
  dp_ctx *ctx;
  int layers, max_seq, n_kv_heads, head_dim, batch, seq_len;
  std::vector<dp_buf> keys, values;
};

extern "C" dp_status dp_kv_cache_create(dp_ctx *ctx, int layers, int max_seq, int n_kv_heads, int head_dim, int batch,
                                        dp_kv_cache **out) {
  if (!ctx || !out) return DP_ERR_INVALID;
  DP_CHECK(ctx, layers > 0 && max_seq > 0 && n_kv_heads > 0 && head_dim > 0 && batch > 0, "KVCache: invalid geometry");
  dp_kv_cache *kv = new dp_kv_cache();
  kv->ctx = ctx; kv->layers = layers; kv->max_seq = max_seq; kv->n_kv_heads = n_kv_heads; kv->head_dim = head_dim;
  kv->batch = batch; kv->seq_len = 0;
  const size_t bytes = (size_t)batch * max_seq * n_kv_heads * head_dim * 2;
  for (int l = 0; l < layers; l++) {
    dp_buf k = nullptr, v = nullptr;
    dp_status st = dp_buf_acquire(ctx, bytes, "kv_cache_keys", &k);
    if (st == DP_OK) st = dp_buf_acquire(ctx, bytes, "kv_cache_values", &v);
    if (st != DP_OK) {
      if (k) dp_buf_release(ctx, k);
      dp_kv_cache_destroy(kv);
      return st;
    }
    kv->keys.push_back(k); kv->values.push_back(v);
  }
  *out = kv;
  return DP_OK;
}

extern "C" void dp_kv_cache_destroy(dp_kv_cache *kv) {
  if (!kv) return;
  for (dp_buf b : kv->keys) dp_buf_release(kv->ctx, b);
  for (dp_buf b : kv->values) dp_buf_release(kv->ctx, b);
  delete kv;
}

extern "C" dp_status dp_kv_layer(dp_kv_cache *kv, int layer, dp_buf *keys, dp_buf *values) {
  if (!kv) return DP_ERR_INVALID;
  DP_CHECK(kv->ctx, layer >= 0 && layer < kv->layers, "KVCache: layer %d out of range [0,%d)", layer, kv->layers);
  if (keys) *keys = kv->keys[layer];
  if (values) *values = kv->values[layer];
  return DP_OK;
}

extern "C" int dp_kv_seq_len(dp_kv_cache *kv) { return kv ? kv->seq_len : -1; }

extern "C" dp_status dp_kv_set_seq_len(dp_kv_cache *kv, int len) {
  if (!kv) return DP_ERR_INVALID;
  DP_CHECK(kv->ctx, len >= 0 && len <= kv->max_seq, "KVCache: length %d exceeds maxSeqLen %d", len, kv->max_seq);
  kv->seq_len = len;
  return DP_OK;
}

// src/inference/kv-cache/base.js:962: truncation only ever shortens
extern "C" dp_status dp_kv_truncate(dp_kv_cache *kv, int len) {
  if (!kv) return DP_ERR_INVALID;
  DP_CHECK(kv->ctx, len >= 0, "KVCache.truncate: negative length %d", len);
  if (len < kv->seq_len) kv->seq_len = len;
  return DP_OK;
}

// src/inference/kv-cache/base.js:829: deep copy, device to device
extern "C" dp_status dp_kv_clone(dp_kv_cache *kv, dp_kv_cache **out) {
  if (!kv || !out) return DP_ERR_INVALID;
  dp_kv_cache *c = nullptr;
  DP_TRY(dp_kv_cache_create(kv->ctx, kv->layers, kv->max_seq, kv->n_kv_heads, kv->head_dim, kv->batch, &c));
  const size_t bytes = (size_t)kv->batch * kv->max_seq * kv->n_kv_heads * kv->head_dim * 2;
  for (int l = 0; l < kv->layers; l++) {
    cudaError_t e = cudaMemcpyAsync(c->keys[l]->dptr, kv->keys[l]->dptr, bytes, cudaMemcpyDeviceToDevice, kv->ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(c->values[l]->dptr, kv->values[l]->dptr, bytes, cudaMemcpyDeviceToDevice, kv->ctx->stream);
    if (e != cudaSuccess) {
      dp_kv_cache_destroy(c);
      return dp_fail(kv->ctx, DP_ERR_CUDA, "KVCache.clone: %s", cudaGetErrorString(e));
    }
  }
  c->seq_len = kv->seq_len;
  *out = c;
  return DP_OK;
}

extern "C" size_t dp_kv_bytes(dp_kv_cache *kv) {
  return kv ? (size_t)kv->layers * 2 * kv->batch * kv->max_seq * kv->n_kv_heads * kv->head_dim * 2 : 0;
}
