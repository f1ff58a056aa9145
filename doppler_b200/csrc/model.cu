// Decoder runner: packed-Q4_K weight upload, f16 KV allocation and the
// decode / prefill schedule for a dense Qwen3-shaped model.
//
// Replaces the slices of the reference that feed the kernels:
//   - src/loader/tensors/tensor-loader.js:540-558 (loadQ4KFused: 144-byte blocks stay packed),
//   - src/inference/kv-cache/base.js:99-153 (contiguous f16 cache),
//   - src/inference/pipelines/text/generator-steps.js:588 (decodeStep) and layer.js:682
//     (processLayerGPU): one recorded command buffer per token there, one CUDA
//     graph per decode step here; the sampled token and the position stay on the
//     device so consecutive steps need no host round trip.
// Op order and rounding points follow the reference pipeline: rmsnorm -> q/k/v ->
// per-head QK RMSNorm -> rotate-half RoPE -> K,V rounded to f16 into the cache ->
// attention over the cache (including the new token) -> o_proj + residual ->
// rmsnorm -> gate/up -> silu(gate)*up -> down + residual; final rmsnorm -> f16 LM
// head -> greedy argmax (lower index wins ties).
#include "common.h"
#include "pdl.cuh"
#include "q4k.cuh"
#include "actq.cuh"
#include "tp_exchange.h"
#include "gemv_exchange.h"
#include "handoff.cuh"

#include <cfloat>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

dp_status dpk_gemm_q4k_tc(dp_ctx *ctx, const uint8_t *W, const void *A, dp_dtype a_dtype, void *C, dp_dtype c_dtype,
                          int M, int N, int K, float alpha, bool f16_weights, bool *handled);
dp_status dpk_gemv_q4k_fast(dp_ctx *ctx, const uint8_t *W, const float *x, void *y, dp_dtype y_dtype, int N, int K,
                            float alpha, const float *residual, bool *handled);
dp_status dpk_q4k_prep_act(dp_ctx *ctx, const float *x, void *actq, int K);
dp_status dpk_gemv_q4k_actq(dp_ctx *ctx, const uint8_t *W, const void *actq, void *y, dp_dtype y_dtype, int N, int K,
                            float alpha, const float *residual);
dp_status dpk_gemv_q4k_actq_tma(dp_ctx *ctx, const uint8_t *W, const void *actq, void *y, dp_dtype y_dtype, int N, int K,
                                float alpha, const float *residual, bool *handled);
size_t dpk_q4k_actq_bytes(int K);
dp_status dpk_gemv_q4k_tma_fused(dp_ctx *ctx, const uint8_t *W, int mode, const float *x, const float *w, float eps, int D,
                                 int splits, float *y, int N, int K, const float *residual, bool *handled, const GemvExchange *gx = nullptr);
bool dpk_gemv_q4k_fast_ok(int N, int K);
dp_status dpk_attention_split_only(dp_ctx *ctx, const dpk_attn_params &p, float *scratch, int splits);
dp_status dp_tp_allreduce_ptr(dp_ctx *ctx, float *ptr, size_t count);
dp_status dp_tp_allgather_ptr(dp_ctx *ctx, const void *send, void *recv, size_t bytes_per_rank);
bool dp_tp_ready(dp_ctx *ctx);
dp_tp_exchange *dp_tp_exchange_desc(dp_ctx *ctx);
bool dp_tp_exchange_view(dp_ctx *ctx, int *rank, int *size, uint2 **areas);
dp_status dp_take_dev_status(dp_ctx *ctx);

struct LayerW {
  dp_buf qkv = nullptr, o = nullptr, gateup = nullptr, down = nullptr;
  float *in_norm = nullptr, *post_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
};

struct dp_model {
  dp_ctx *ctx;
  dp_model_cfg cfg;
  int nh, nkv, qdim, kvdim, inter, vocab_l, vocab0;  // this rank's share
  int T;                                              // rows of the activation buffers
  std::vector<LayerW> layers;
  dp_buf norms = nullptr, embed = nullptr, lm_head = nullptr;
  float *final_norm = nullptr;
  std::vector<dp_buf> kc, vc;
  dp_buf rope = nullptr;
  float *rope_cos = nullptr, *rope_sin = nullptr;
  dp_buf act = nullptr;  // one slab for all activations
  float *h, *n, *qkv, *q, *att, *gu, *actv, *partial, *logits;
  float *hbuf[3];       // tensor-parallel single-token decode: the residual stream rotates over three buffers (hbuf[0] == h);
                        // a kernel reads one and its CTAs write their shares of the next, so none overwrites what another still reads
  float *h_last;        // where the last forward pass left the hidden state
  unsigned *d_ticket = nullptr;   // device counter of decode steps ever run on this CONTEXT (its exchange area outlives a model):
                                  // hand-off tickets derive from it and never repeat
  dp_buf state = nullptr;  // device ints: pos[B], kvlen[B], tok[B], step, then argmax scratch
  int *d_pos, *d_kvlen, *d_tok, *d_step;
  float *am_vals; int *am_idx; float *am_best; int *am_pair_i; float *am_gather;
  dp_buf out_tokens = nullptr;
  int out_tokens_cap = 0;
  int *pin_state = nullptr;   // page-locked staging of the per-call state block (1024 words) + the status word read back
  int *pin_out = nullptr;     // page-locked staging of the decoded tokens (out_tokens_cap words)
  dp_buf attn_scratch = nullptr;
  dp_buf actq = nullptr;  // fixed-point activation digits of the decode GEMV (sized for the largest K)
  int attn_splits_decode = 1;
  bool recording_decode = false;  // set while a decode step is recorded into its CUDA graph
  bool fuse_qk = true;  // decode: QK norm + RoPE + KV append inside the attention kernel
  std::vector<int> seq_len;
  dp_graph *graph[2] = {nullptr, nullptr};
  int graph_batch[2] = {0, 0};
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  double last_ms = 0;
  size_t weight_bytes = 0;
  int allreduce_mode = 0;
  bool final_norm_done = false;  // set by run_layers when the exchange kernel already applied the final RMSNorm
};

// ---- model-specific kernels ---------------------------------------------------

// Per-head QK RMSNorm + rotate-half RoPE + KV append, one warp per (token, head).
// Reference ops fused here: rmsnorm_qk.wgsl:75-118, rope.wgsl:62-106,
// kv_cache_write_f32_to_f16.wgsl:19 (the reference ships the same fusion as
// split_qkv_rmsnorm_rope_qk_f16kv_cache.wgsl).  head_dim must be a multiple of 64.
__global__ void __launch_bounds__(256) qk_norm_rope_kv_kernel(
    const float *__restrict__ qkv, float *__restrict__ q_out, __half *__restrict__ kc, __half *__restrict__ vc,
    const float *__restrict__ q_norm, const float *__restrict__ k_norm, const float *__restrict__ cos_t,
    const float *__restrict__ sin_t, const int *__restrict__ pos_arr, int start_pos, int seq, int tokens, int nh,
    int nkv, int D, float eps, size_t kv_seq_stride) {
  pdl_launch();
  pdl_wait();
  const int heads = nh + 2 * nkv;
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (gw >= tokens * heads) return;
  const int t = gw / heads, hd = gw % heads;
  const int pos = pos_arr ? pos_arr[t] : start_pos + t;
  const int sq = pos_arr ? t : seq;
  const float *src = qkv + (size_t)t * heads * D + (size_t)hd * D;
  const int half = D / 2, per = half / 32;  // pairs per lane
  float x0[4], x1[4];
#pragma unroll
  for (int i = 0; i < 4; i++) if (i < per) { x0[i] = src[lane + 32 * i]; x1[i] = src[lane + 32 * i + half]; }
  if (hd < nh + nkv) {
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; i++) if (i < per) ss = fmaf(x0[i], x0[i], fmaf(x1[i], x1[i], ss));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.0f / sqrtf(ss / (float)D + eps);
    const float *w = hd < nh ? q_norm : k_norm;
#pragma unroll
    for (int i = 0; i < 4; i++) if (i < per) {
      const int d = lane + 32 * i;
      const float a = x0[i] * inv * w[d], b = x1[i] * inv * w[d + half];
      const float c = cos_t[(size_t)pos * half + d], s = sin_t[(size_t)pos * half + d];
      x0[i] = a * c - b * s;
      x1[i] = a * s + b * c;
    }
  }
  if (hd < nh) {
    float *dst = q_out + ((size_t)t * nh + hd) * D;
#pragma unroll
    for (int i = 0; i < 4; i++) if (i < per) { dst[lane + 32 * i] = x0[i]; dst[lane + 32 * i + half] = x1[i]; }
  } else {
    const int kh = hd < nh + nkv ? hd - nh : hd - nh - nkv;
    __half *dst = (hd < nh + nkv ? kc : vc) + (size_t)sq * kv_seq_stride + ((size_t)pos * nkv + kh) * D;
#pragma unroll
    for (int i = 0; i < 4; i++) if (i < per) {
      dst[lane + 32 * i] = __float2half_rn(x0[i]);
      dst[lane + 32 * i + half] = __float2half_rn(x1[i]);
    }
  }
}

// The gate and up projections share one matrix whose rows are interleaved in groups of eight (eight gate rows,
// then their eight up rows), so a 16-row tile of the decode GEMV holds matching pairs: gate c is output
// (c / 8) * 16 + c % 8, up c is eight further.
__device__ __forceinline__ size_t gu_gate_index(size_t c) { return (c >> 3) * 16 + (c & 7); }

// out[t, c] = silu(gate[t, c]) * up[t, c]   (silu.wgsl:30-37,98-104, sigmoid argument clamped to +-15)
__global__ void silu_gateup_kernel(const float *__restrict__ gu, float *__restrict__ out, int tokens, int inter) {
  pdl_launch();
  pdl_wait();
  const size_t total = (size_t)tokens * inter;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / inter, c = i % inter;
    const float g = gu[t * 2 * inter + gu_gate_index(c)], u = gu[t * 2 * inter + gu_gate_index(c) + 8];
    const float cl = fminf(fmaxf(g, -15.0f), 15.0f);
    out[i] = (g * (1.0f / (1.0f + expf(-cl)))) * u;
  }
}

// after a decode step: record the sampled tokens and move every sequence on by one
__global__ void advance_kernel(int *pos, int *kvlen, const int *tok, int *step, int *out_tokens, int batch, unsigned *ticket) {
  pdl_launch();
  pdl_wait();
  const int b = threadIdx.x;
  const int s = *step;
  if (b < batch) { out_tokens[s * batch + b] = tok[b]; pos[b] += 1; kvlen[b] += 1; }
  __syncthreads();
  if (b == 0) { *step = s + 1; *ticket += 1u; }
}


// combine the per-rank (best value, index) pairs of a vocabulary-sharded argmax;
// ties go to the lower global index (sample.wgsl:45-53)
__global__ void argmax_merge_kernel(const float *pairs, int ranks, int batch, int *tok) {
  pdl_launch();
  pdl_wait();
  const int b = threadIdx.x;
  if (b >= batch) return;
  float bv = -3.402823e+38f;
  int bi = 0x7fffffff;
  for (int r = 0; r < ranks; r++) {
    const float v = pairs[(r * batch + b) * 2];
    const int i = __float_as_int(pairs[(r * batch + b) * 2 + 1]);
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
  tok[b] = bi;
}

__global__ void pack_pair_kernel(const float *best, const int *tok, float *pairs, int batch) {
  pdl_launch();
  pdl_wait();
  const int b = threadIdx.x;
  if (b < batch) { pairs[2 * b] = best[b]; pairs[2 * b + 1] = __int_as_float(tok[b]); }
}


// ---- single-token producers that also emit the GEMV's fixed-point activation digits ----
// (reference ops: rmsnorm.wgsl:119-187, silu.wgsl:98-104, and the split-K merge of the decode
// attention; the digits feed gemv_q4k_fast.cu, so no separate quantisation launch is needed)

// RMSNorm of one row of `size` values (size % 256 == 0, size <= 8192); warp w owns blocks w, w+8, ...
__global__ void __launch_bounds__(256) rmsnorm_actq_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                           float *__restrict__ y, void *__restrict__ actq, int size, float eps) {
  pdl_launch();
  pdl_wait();
  __shared__ float sh[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, bpr = size / QK_K;
  float v[4][8];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int b = warp + 8 * i;
    if (b < bpr) {
      const float4 a = *reinterpret_cast<const float4 *>(x + b * QK_K + lane * 8);
      const float4 c = *reinterpret_cast<const float4 *>(x + b * QK_K + lane * 8 + 4);
      v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w; v[i][4] = c.x; v[i][5] = c.y; v[i][6] = c.z; v[i][7] = c.w;
#pragma unroll
      for (int j = 0; j < 8; j++) ss = fmaf(v[i][j], v[i][j], ss);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) sh[warp] = ss;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; i++) total += sh[i];
  const float inv_rms = 1.0f / sqrtf(total / (float)size + eps);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int b = warp + 8 * i;
    if (b < bpr) {
      const float4 wa = *reinterpret_cast<const float4 *>(w + b * QK_K + lane * 8);
      const float4 wc = *reinterpret_cast<const float4 *>(w + b * QK_K + lane * 8 + 4);
      const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wc.x, wc.y, wc.z, wc.w};
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; j++) o[j] = v[i][j] * inv_rms * wv[j];
      *reinterpret_cast<float4 *>(y + b * QK_K + lane * 8) = make_float4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<float4 *>(y + b * QK_K + lane * 8 + 4) = make_float4(o[4], o[5], o[6], o[7]);
      actq_emit_block(o, lane, b, bpr, actq);
    }
  }
}

// act = silu(gate) * up for one token, inter % 256 == 0; one warp per block
__global__ void __launch_bounds__(256) silu_actq_kernel(const float *__restrict__ gu, float *__restrict__ out,
                                                        void *__restrict__ actq, int inter) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, bpr = inter / QK_K;
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (b >= bpr) return;
  const float *gp = gu + 2 * (b * QK_K + lane * 8), *up = gp + 8;  // interleaved in groups of eight
  const float4 g0 = *reinterpret_cast<const float4 *>(gp), g1 = *reinterpret_cast<const float4 *>(gp + 4);
  const float4 u0 = *reinterpret_cast<const float4 *>(up), u1 = *reinterpret_cast<const float4 *>(up + 4);
  const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w}, u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
  float o[8];
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const float cl = fminf(fmaxf(g[j], -15.0f), 15.0f);
    o[j] = (g[j] * (1.0f / (1.0f + expf(-cl)))) * u[j];
  }
  *reinterpret_cast<float4 *>(out + b * QK_K + lane * 8) = make_float4(o[0], o[1], o[2], o[3]);
  *reinterpret_cast<float4 *>(out + b * QK_K + lane * 8 + 4) = make_float4(o[4], o[5], o[6], o[7]);
  actq_emit_block(o, lane, b, bpr, actq);
}

// merge of the split-K attention partials of one token (layout of attention.cu: per (head, split)
// D values, then running max and sum); (H*D) % 256 == 0 and D % 8 == 0; one warp per 256 outputs
__global__ void __launch_bounds__(256) attn_combine_actq_kernel(const float *__restrict__ part, float *__restrict__ out,
                                                                void *__restrict__ actq, int H, int D, int splits) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, bpr = H * D / QK_K;
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (b >= bpr) return;
  const int e0 = b * QK_K + lane * 8, h = e0 / D, d0 = e0 % D;
  const float *pp = part + (size_t)h * splits * (D + 2);
  float mm = -FLT_MAX;
  for (int s = 0; s < splits; s++) mm = fmaxf(mm, pp[s * (D + 2) + D]);
  float ll = 0.0f, acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 2
  for (int s = 0; s < splits; s++) {
    const float *ps = pp + s * (D + 2);
    const float ms = ps[D];
    const float c = (ms == -FLT_MAX) ? 0.0f : exp2f(ms - mm);
    ll = fmaf(ps[D + 1], c, ll);
    const float2 a0 = *reinterpret_cast<const float2 *>(ps + d0), a1 = *reinterpret_cast<const float2 *>(ps + d0 + 2);
    const float2 a2 = *reinterpret_cast<const float2 *>(ps + d0 + 4), a3 = *reinterpret_cast<const float2 *>(ps + d0 + 6);
    acc[0] = fmaf(a0.x, c, acc[0]); acc[1] = fmaf(a0.y, c, acc[1]); acc[2] = fmaf(a1.x, c, acc[2]); acc[3] = fmaf(a1.y, c, acc[3]);
    acc[4] = fmaf(a2.x, c, acc[4]); acc[5] = fmaf(a2.y, c, acc[5]); acc[6] = fmaf(a3.x, c, acc[6]); acc[7] = fmaf(a3.y, c, acc[7]);
  }
  float o[8];
#pragma unroll
  for (int j = 0; j < 8; j++) o[j] = ll > 0.0f ? acc[j] / ll : 0.0f;
  *reinterpret_cast<float4 *>(out + e0) = make_float4(o[0], o[1], o[2], o[3]);
  *reinterpret_cast<float4 *>(out + e0 + 4) = make_float4(o[4], o[5], o[6], o[7]);
  actq_emit_block(o, lane, b, bpr, actq);
}

// ---- vocabulary-sharded greedy pick over the peer-memory exchange area ----
// (no counterpart in the reference, which has no collective backend).  One CTA per rank pushes this
// rank's (best logit, global index) of every sequence, each as an 8-byte (value, ticket) word, into its
// slot of EVERY rank's area (plain stores over NVLink), then re-reads all ranks' slots in its OWN memory
// until they carry this exchange's ticket (bounded; on give-up a status word is raised and the kernel
// carries on so nothing hangs), and merges in rank order: the largest value wins, ties go to the lower
// global index (sample.wgsl:45-53), so every rank picks the same token.
struct ArgmaxExchange {
  int rank, nr;
  uint2 *area[DP_TP_MAX_RANKS];
};
__global__ void __launch_bounds__(256) tp_argmax_exchange_kernel(const ArgmaxExchange xg, dp_tp_exchange *__restrict__ xd, const float *__restrict__ best,
                                                                 int *__restrict__ tok, int batch, unsigned wait_limit, int *__restrict__ err) {
  pdl_launch();
  pdl_wait();
  __shared__ unsigned s_ticket;
  const int tid = threadIdx.x;
  if (tid == 0) s_ticket = ++xd->am_ticket;
  __syncthreads();
  const unsigned e = s_ticket;
  if (tid < batch) {
    const unsigned v = __float_as_uint(best[tid]), idx = (unsigned)tok[tid];
    for (int r = 0; r < xg.nr; r++) {
      uint2 *dst = xg.area[r] + dp_tp_am_slot_offset(e, xg.rank) + 2 * tid;
      asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(v), "r"(e) : "memory");
      asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst + 1), "r"(idx), "r"(e) : "memory");
    }
    float bv = -3.402823e+38f;
    int bi = 0x7fffffff;
    bool ok = true;
    for (int r = 0; r < xg.nr && ok; r++) {
      const uint2 *src = xg.area[xg.rank] + dp_tp_am_slot_offset(e, r) + 2 * tid;
      uint4 w = make_uint4(0u, 0u, 0u, 0u);
      ok = false;
      for (unsigned it = 0; it < wait_limit; it++) {
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "l"(src) : "memory");
        if (w.y == e && w.w == e) { ok = true; break; }
      }
      const float v2 = __uint_as_float(w.x);
      const int i2 = (int)w.z;
      if (ok && (v2 > bv || (v2 == bv && i2 < bi))) { bv = v2; bi = i2; }
    }
    if (!ok) atomicExch(err, 3);
    tok[tid] = bi;
  }
}

// Tensor parallel, end of the last layer: h' = h + the partial vectors all ranks pushed after down_proj
// (rank order), n = rmsnorm(h', w) for the LM head.  One CTA; size % 256 == 0, size <= 8192.
__global__ void __launch_bounds__(256) xchg_rmsnorm_kernel(const __grid_constant__ GemvExchange gx, const float *__restrict__ h_in, float *__restrict__ h_out,
                                                           const float *__restrict__ w, float *__restrict__ n_out, int size, float eps,
                                                           int *__restrict__ err) {
  pdl_launch();
  pdl_wait();
  __shared__ float sh[8];
  __shared__ int s_abort;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, bpr = size / QK_K;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  const unsigned ticket = *reinterpret_cast<const volatile unsigned *>(gx.ticket_step) * gx.ticket_stride + 1u + gx.ticket_in;
  const uint2 *mine = gx.mine;
  float v[4][8];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int b = warp + 8 * i;
    if (b < bpr) {
      const int off = b * QK_K + lane * 8;
      const float4 a = *reinterpret_cast<const float4 *>(h_in + off), c = *reinterpret_cast<const float4 *>(h_in + off + 4);
      v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w; v[i][4] = c.x; v[i][5] = c.y; v[i][6] = c.z; v[i][7] = c.w;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int r = 0; r < gx.nr; r++) {
        float s8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        handoff_take8(mine + dp_tp_slot_offset((unsigned)gx.parity_in, r) + off, ticket, s8, gx.wait_limit, &s_abort);
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] += s8[j];
      }
#pragma unroll
      for (int j = 0; j < 8; j++) { v[i][j] += acc[j]; ss = fmaf(v[i][j], v[i][j], ss); }
      *reinterpret_cast<float4 *>(h_out + off) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
      *reinterpret_cast<float4 *>(h_out + off + 4) = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
    }
  }
  __syncwarp();
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) sh[warp] = ss;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; i++) total += sh[i];
  const float inv_rms = 1.0f / sqrtf(total / (float)size + eps);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int b = warp + 8 * i;
    if (b < bpr) {
      const int off = b * QK_K + lane * 8;
      const float4 wa = *reinterpret_cast<const float4 *>(w + off), wc = *reinterpret_cast<const float4 *>(w + off + 4);
      *reinterpret_cast<float4 *>(n_out + off) = make_float4(v[i][0] * inv_rms * wa.x, v[i][1] * inv_rms * wa.y, v[i][2] * inv_rms * wa.z, v[i][3] * inv_rms * wa.w);
      *reinterpret_cast<float4 *>(n_out + off + 4) = make_float4(v[i][4] * inv_rms * wc.x, v[i][5] * inv_rms * wc.y, v[i][6] * inv_rms * wc.z, v[i][7] * inv_rms * wc.w);
    }
  }
  if (s_abort && threadIdx.x == 0) atomicExch(err, 3);
}

// ---- create / destroy -----------------------------------------------------------
static size_t q4k_bytes(size_t n, size_t k) { return n * dp_cdiv(k, DP_QK_K) * DP_Q4K_BLOCK_BYTES; }
static size_t align_up(size_t v, size_t a) { return dp_cdiv(v, a) * a; }

extern "C" dp_status dp_model_create(dp_ctx *ctx, const dp_model_cfg *cfg, dp_model **out) {
  if (!ctx || !cfg || !out) return DP_ERR_INVALID;
  const dp_model_cfg &c = *cfg;
  const int p = c.tp_size > 0 ? c.tp_size : 1;
  DP_CHECK(ctx, c.n_layers > 0 && c.hidden > 0 && c.n_heads > 0 && c.n_kv_heads > 0 && c.head_dim > 0 && c.inter > 0 &&
                    c.vocab > 0 && c.max_seq > 0, "model: invalid configuration");
  DP_CHECK(ctx, c.head_dim % 64 == 0 && c.head_dim <= 256, "model: head_dim %d must be 64, 128, 192 or 256", c.head_dim);
  DP_CHECK(ctx, c.n_heads % c.n_kv_heads == 0, "model: n_heads %d not a multiple of n_kv_heads %d", c.n_heads, c.n_kv_heads);
  DP_CHECK(ctx, c.tp_rank >= 0 && c.tp_rank < p, "model: tp_rank %d outside [0,%d)", c.tp_rank, p);
  DP_CHECK(ctx, p <= DP_TP_MAX_RANKS, "model: tp_size %d exceeds the %d ranks a group holds", p, DP_TP_MAX_RANKS);
  DP_CHECK(ctx, c.max_batch <= 256, "model: max_batch %d > 256", c.max_batch);
  DP_CHECK(ctx, c.n_kv_heads % p == 0 && c.n_heads % p == 0, "model: heads (%d/%d) do not divide over %d ranks", c.n_heads, c.n_kv_heads, p);
  DP_CHECK(ctx, c.inter % (p * DP_QK_K) == 0 && (c.n_heads * c.head_dim) % (p * DP_QK_K) == 0,
           "model: row-parallel matrices must split on 256-element super-blocks over %d ranks", p);
  DP_CHECK(ctx, c.hidden % DP_QK_K == 0, "model: hidden %d must be a multiple of 256", c.hidden);
  DP_CHECK(ctx, c.vocab % p == 0, "model: vocab %d does not divide over %d ranks", c.vocab, p);
  DP_CHECK(ctx, p == 1 || dp_tp_ready(ctx), "model: tp_size %d needs dp_tp_init on this context first", p);
  dp_model *m = new dp_model();
  m->ctx = ctx; m->cfg = c; m->cfg.tp_size = p;
  if (m->cfg.max_batch <= 0) m->cfg.max_batch = 1;
  m->nh = c.n_heads / p; m->nkv = c.n_kv_heads / p;
  m->qdim = m->nh * c.head_dim; m->kvdim = m->nkv * c.head_dim;
  m->inter = c.inter / p; m->vocab_l = c.vocab / p; m->vocab0 = m->vocab_l * c.tp_rank;
  const int B = m->cfg.max_batch;
  // Prefill chunk: up to 2048 rows per GEMM (the tile grid of a 4096-column projection fills the GPU from
  // about 1536 rows on), no more than the longest sequence needs
  {
    int t = c.max_seq < 2048 ? (c.max_seq + 255) / 256 * 256 : 2048;
    if (t < 512) t = 512;
    m->T = B > t ? B : t;
  }
  m->layers.resize(c.n_layers);
  m->seq_len.assign(B, 0);
  dp_status st = DP_OK;
  auto acquire = [&](size_t bytes, const char *label, dp_buf *b) { if (st == DP_OK) st = dp_buf_acquire(ctx, bytes, label, b); };
  const int H = c.hidden, D = c.head_dim;
  for (int l = 0; l < c.n_layers; l++) {
    LayerW &L = m->layers[l];
    acquire(q4k_bytes(m->qdim + 2 * m->kvdim, H), "w_qkv_q4k", &L.qkv);
    acquire(q4k_bytes(H, m->qdim), "w_o_q4k", &L.o);
    acquire(q4k_bytes(2 * m->inter, H), "w_gateup_q4k", &L.gateup);
    acquire(q4k_bytes(H, m->inter), "w_down_q4k", &L.down);
    if (st == DP_OK) m->weight_bytes += L.qkv->bytes + L.o->bytes + L.gateup->bytes + L.down->bytes;
  }
  const size_t per_layer_norm = (size_t)2 * H + 2 * D;
  acquire(((size_t)c.n_layers * per_layer_norm + H) * 4, "norm_weights", &m->norms);
  acquire((size_t)c.vocab * H * 2, "embedding_f16", &m->embed);
  acquire((size_t)m->vocab_l * H * 2, "lm_head_f16", &m->lm_head);
  const size_t kv_bytes = (size_t)B * c.max_seq * m->kvdim * 2;
  m->kc.assign(c.n_layers, nullptr); m->vc.assign(c.n_layers, nullptr);
  for (int l = 0; l < c.n_layers; l++) { acquire(kv_bytes, "kv_cache_keys", &m->kc[l]); acquire(kv_bytes, "kv_cache_values", &m->vc[l]); }
  acquire((size_t)c.max_seq * D * 4, "rope_tables", &m->rope);
  const size_t T = m->T;
  const size_t n_h = align_up(T * H, 64), n_qkv = align_up(T * (m->qdim + 2 * m->kvdim), 64), n_q = align_up(T * m->qdim, 64);
  const size_t n_gu = align_up(T * 2 * m->inter, 64), n_act = align_up(T * m->inter, 64), n_log = align_up((size_t)B * m->vocab_l, 64);
  acquire((3 * n_h + n_qkv + 2 * n_q + n_gu + n_act + n_log + 2 * align_up(H, 64)) * 4, "activations", &m->act);
  acquire(4096 + 1024 + 2048 + 16384 + (size_t)B * 256 * 8, "decode_state", &m->state);
  // split-K scratch sized for the longest context
  dpk_attn_params ap{};
  ap.batch = B; ap.seq_len = 1; ap.kv_len = c.max_seq; ap.num_heads = m->nh; ap.num_kv_heads = m->nkv; ap.head_dim = D;
  size_t sbytes = dpk_attention_scratch_bytes(ctx, ap, &m->attn_splits_decode);
  acquire(sbytes ? sbytes : 256, "attention_split_partials", &m->attn_scratch);
  {
    int kmax = H > m->qdim ? H : m->qdim;
    if (m->inter > kmax) kmax = m->inter;
    acquire(dpk_q4k_actq_bytes(kmax), "gemv_activation_digits", &m->actq);
  }
  if (st != DP_OK) { dp_model_destroy(m); return st; }
  m->weight_bytes += m->lm_head->bytes;

  float *nb = (float *)m->norms->dptr;
  for (int l = 0; l < c.n_layers; l++) {
    LayerW &L = m->layers[l];
    L.in_norm = nb; nb += H; L.post_norm = nb; nb += H; L.q_norm = nb; nb += D; L.k_norm = nb; nb += D;
  }
  m->final_norm = nb;
  float *a = (float *)m->act->dptr;
  m->h = a; a += n_h; m->n = a; a += n_h; m->partial = a; a += n_h; m->qkv = a; a += n_qkv; m->q = a; a += n_q;
  m->att = a; a += n_q; m->gu = a; a += n_gu; m->actv = a; a += n_act; m->logits = a; a += n_log;
  m->hbuf[0] = m->h; m->hbuf[1] = a; a += align_up(H, 64); m->hbuf[2] = a; a += align_up(H, 64);
  m->h_last = m->h;
  int *si = (int *)m->state->dptr;
  m->d_pos = si; m->d_kvlen = si + 256; m->d_tok = si + 512; m->d_step = si + 768;
  char *sp = (char *)m->state->dptr + 4096;
  m->am_best = (float *)sp; sp += 1024;             // best logit per sequence
  m->am_pair_i = (int *)sp; sp += 2048;             // (value, index) per sequence, this rank
  m->am_gather = (float *)sp; sp += 16384;          // the pairs of up to 8 ranks
  m->am_vals = (float *)sp; m->am_idx = (int *)(m->am_vals + (size_t)B * 256);
  m->d_ticket = (unsigned *)(ctx->dev_status + 16);  // zeroed with the context, then only ever incremented
  // rope tables (host build, init-rope.js semantics)
  {
    std::vector<float> cs((size_t)c.max_seq * D / 2), sn((size_t)c.max_seq * D / 2);
    dp_rope_tables((double)c.rope_theta, D, c.max_seq, cs.data(), sn.data());
    m->rope_cos = (float *)m->rope->dptr; m->rope_sin = m->rope_cos + (size_t)c.max_seq * D / 2;
    st = dp_buf_upload(ctx, m->rope, cs.data(), 0, cs.size() * 4);
    if (st == DP_OK) st = dp_buf_upload(ctx, m->rope, sn.data(), cs.size() * 4, sn.size() * 4);
  }
  if (st == DP_OK && (cudaEventCreate(&m->ev0) != cudaSuccess || cudaEventCreate(&m->ev1) != cudaSuccess))
    st = dp_fail(ctx, DP_ERR_CUDA, "model: cudaEventCreate failed");
  if (st == DP_OK) st = dp_buf_fill(ctx, m->state, 0, 0, m->state->bytes);
  if (st != DP_OK) { dp_model_destroy(m); return st; }
  *out = m;
  return DP_OK;
}

extern "C" void dp_model_destroy(dp_model *m) {
  if (!m) return;
  dp_ctx *ctx = m->ctx;
  cudaStreamSynchronize(ctx->stream);
  for (int i = 0; i < 2; i++) if (m->graph[i]) dp_graph_destroy(m->graph[i]);
  auto rel = [&](dp_buf b) { if (b) dp_buf_release(ctx, b); };
  for (LayerW &L : m->layers) { rel(L.qkv); rel(L.o); rel(L.gateup); rel(L.down); }
  rel(m->norms); rel(m->embed); rel(m->lm_head); rel(m->rope); rel(m->act); rel(m->state); rel(m->out_tokens); rel(m->attn_scratch); rel(m->actq);
  for (dp_buf b : m->kc) rel(b);
  for (dp_buf b : m->vc) rel(b);
  if (m->pin_state) cudaFreeHost(m->pin_state);
  if (m->pin_out) cudaFreeHost(m->pin_out);
  if (m->ev0) cudaEventDestroy(m->ev0);
  if (m->ev1) cudaEventDestroy(m->ev1);
  delete m;
}

// ---- weight upload ------------------------------------------------------------------
extern "C" dp_status dp_model_load_q4k(dp_model *m, int layer, dp_weight_id which, const void *host, int N, int K) {
  if (!m) return DP_ERR_INVALID;
  dp_ctx *ctx = m->ctx;
  const dp_model_cfg &c = m->cfg;
  DP_CHECK(ctx, layer >= 0 && layer < c.n_layers, "loadQ4K: layer %d out of range", layer);
  DP_CHECK(ctx, host != nullptr, "loadQ4K: null host pointer");
  const int p = c.tp_size, r = c.tp_rank, H = c.hidden;
  LayerW &L = m->layers[layer];
  const size_t bpr = dp_cdiv((size_t)K, DP_QK_K), row_bytes = bpr * DP_Q4K_BLOCK_BYTES;
  auto expect = [&](int n, int k, const char *name) -> dp_status {
    if (N != n || K != k) return dp_fail(ctx, DP_ERR_INVALID, "loadQ4K: %s expects shape [%d,%d], got [%d,%d]", name, n, k, N, K);
    return DP_OK;
  };
  const uint8_t *src = (const uint8_t *)host;
  switch (which) {
    case DP_W_Q: case DP_W_K: case DP_W_V: {  // column parallel: contiguous rows of this rank
      const int full = which == DP_W_Q ? c.n_heads * c.head_dim : c.n_kv_heads * c.head_dim;
      DP_TRY(expect(full, H, which == DP_W_Q ? "q_proj" : which == DP_W_K ? "k_proj" : "v_proj"));
      const int rows = full / p;
      const size_t dst_row = which == DP_W_Q ? 0 : which == DP_W_K ? (size_t)m->qdim : (size_t)m->qdim + m->kvdim;
      return dp_buf_upload(ctx, L.qkv, src + (size_t)r * rows * row_bytes, dst_row * row_bytes, (size_t)rows * row_bytes);
    }
    case DP_W_GATE: case DP_W_UP: {
      // one matrix for both, rows interleaved in groups of eight: gate rows 8j..8j+7, then up rows 8j..8j+7
      DP_TRY(expect(c.inter, H, which == DP_W_GATE ? "gate_proj" : "up_proj"));
      const int rows = c.inter / p;
      DP_CHECK(ctx, rows % 8 == 0, "loadQ4K: %d gate/up rows per rank are not a multiple of 8", rows);
      const uint8_t *mine = src + (size_t)r * rows * row_bytes;
      DP_CUDA(ctx, cudaMemcpy2DAsync((char *)L.gateup->dptr + (which == DP_W_GATE ? 0 : 8) * row_bytes, 16 * row_bytes, mine, 8 * row_bytes,
                                     8 * row_bytes, (size_t)rows / 8, cudaMemcpyHostToDevice, ctx->stream));
      DP_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      return DP_OK;
    }
    case DP_W_O: case DP_W_DOWN: {  // row parallel: this rank's super-block columns of every row
      const int kfull = which == DP_W_O ? c.n_heads * c.head_dim : c.inter;
      DP_TRY(expect(H, kfull, which == DP_W_O ? "o_proj" : "down_proj"));
      dp_buf dst = which == DP_W_O ? L.o : L.down;
      if (p == 1) return dp_buf_upload(ctx, dst, src, 0, (size_t)N * row_bytes);
      const size_t bl = bpr / p, seg = bl * DP_Q4K_BLOCK_BYTES;
      std::vector<uint8_t> stage((size_t)N * seg);
      for (int n = 0; n < N; n++) memcpy(stage.data() + (size_t)n * seg, src + (size_t)n * row_bytes + (size_t)r * seg, seg);
      return dp_buf_upload(ctx, dst, stage.data(), 0, stage.size());
    }
    default:
      return dp_fail(ctx, DP_ERR_INVALID, "loadQ4K: weight id %d is not a Q4_K matrix", (int)which);
  }
}

extern "C" dp_status dp_model_load_norm(dp_model *m, int layer, dp_weight_id which, const float *host, int n) {
  if (!m) return DP_ERR_INVALID;
  dp_ctx *ctx = m->ctx;
  DP_CHECK(ctx, layer >= 0 && layer < m->cfg.n_layers && host, "loadNorm: bad layer or null pointer");
  LayerW &L = m->layers[layer];
  float *dst; int want;
  switch (which) {
    case DP_W_IN_NORM: dst = L.in_norm; want = m->cfg.hidden; break;
    case DP_W_POST_NORM: dst = L.post_norm; want = m->cfg.hidden; break;
    case DP_W_Q_NORM: dst = L.q_norm; want = m->cfg.head_dim; break;
    case DP_W_K_NORM: dst = L.k_norm; want = m->cfg.head_dim; break;
    default: return dp_fail(ctx, DP_ERR_INVALID, "loadNorm: weight id %d is not a norm", (int)which);
  }
  DP_CHECK(ctx, n == want, "loadNorm: expected %d values, got %d", want, n);
  return dp_buf_upload(ctx, m->norms, host, (size_t)((char *)dst - (char *)m->norms->dptr), (size_t)n * 4);
}

extern "C" dp_status dp_model_load_final_norm(dp_model *m, const float *host, int n) {
  if (!m || !host) return DP_ERR_INVALID;
  DP_CHECK(m->ctx, n == m->cfg.hidden, "loadFinalNorm: expected %d values, got %d", m->cfg.hidden, n);
  return dp_buf_upload(m->ctx, m->norms, host, (size_t)((char *)m->final_norm - (char *)m->norms->dptr), (size_t)n * 4);
}

extern "C" dp_status dp_model_load_embed(dp_model *m, const void *host, int row0, int rows) {
  if (!m || !host) return DP_ERR_INVALID;
  DP_CHECK(m->ctx, row0 >= 0 && rows >= 0 && row0 + rows <= m->cfg.vocab, "loadEmbed: rows [%d,%d) outside the vocabulary", row0, row0 + rows);
  return dp_buf_upload(m->ctx, m->embed, host, (size_t)row0 * m->cfg.hidden * 2, (size_t)rows * m->cfg.hidden * 2);
}

// rows are GLOBAL vocabulary rows; only the part that falls in this rank's shard is kept
extern "C" dp_status dp_model_load_lm_head(dp_model *m, const void *host, int row0, int rows) {
  if (!m || !host) return DP_ERR_INVALID;
  DP_CHECK(m->ctx, row0 >= 0 && rows >= 0 && row0 + rows <= m->cfg.vocab, "loadLmHead: rows [%d,%d) outside the vocabulary", row0, row0 + rows);
  int lo = row0 > m->vocab0 ? row0 : m->vocab0;
  int hi = row0 + rows < m->vocab0 + m->vocab_l ? row0 + rows : m->vocab0 + m->vocab_l;
  if (hi <= lo) return DP_OK;
  const size_t rb = (size_t)m->cfg.hidden * 2;
  return dp_buf_upload(m->ctx, m->lm_head, (const char *)host + (size_t)(lo - row0) * rb, (size_t)(lo - m->vocab0) * rb, (size_t)(hi - lo) * rb);
}

extern "C" dp_status dp_model_reset(dp_model *m) {
  if (!m) return DP_ERR_INVALID;
  for (int &s : m->seq_len) s = 0;
  return DP_OK;
}

extern "C" size_t dp_model_weight_bytes(dp_model *m) { return m ? m->weight_bytes : 0; }
extern "C" int dp_model_seq_len(dp_model *m, int seq) { return (m && seq >= 0 && seq < (int)m->seq_len.size()) ? m->seq_len[seq] : -1; }
extern "C" double dp_model_last_decode_ms(dp_model *m) { return m ? m->last_ms : 0.0; }

extern "C" dp_status dp_model_set_allreduce_mode(dp_model *m, int mode) {
  if (!m) return DP_ERR_INVALID;
  if (mode != 0 && mode != 1) return dp_fail(m->ctx, DP_ERR_INVALID, "model: unknown allreduce mode %d", mode);
  if (mode == 1) {
    if (m->cfg.tp_size > 1 && !dp_tp_exchange_desc(m->ctx))
      return dp_fail(m->ctx, DP_ERR_STATE, "model: allreduce mode 1 needs the peer-memory exchange area (dp_tp_ipc_export / dp_tp_ipc_attach)");
    if (m->cfg.hidden % DP_QK_K || m->cfg.hidden > DP_TP_SLOT_FLOATS)
      return dp_fail(m->ctx, DP_ERR_UNSUPPORTED, "model: allreduce mode 1 carries hidden sizes that are multiples of 256 up to %d", DP_TP_SLOT_FLOATS);
  }
  for (int i = 0; i < 2; i++) if (m->graph[i]) { dp_graph_destroy(m->graph[i]); m->graph[i] = nullptr; }
  m->allreduce_mode = mode;
  return DP_OK;
}

// ---- the schedule ---------------------------------------------------------------------
// silu_dst / silu_done (rows of gate|up pairs, M >= 2): the tensor-core GEMM may store silu(gate) * up, [M, N / 2], to
// silu_dst instead of y; *silu_done says whether it did.
// norm_w / eps: x holds un-normalised rows and y = q4k_linear(rmsnorm(x, norm_w, eps)); the multi-row tensor-core path
// folds the norm into its conversion of the rows, every other path runs it as a kernel of its own into m->n.
static dp_status q4k_linear(dp_model *m, const uint8_t *W, const float *x, float *y, int M, int N, int K,
                            const float *residual, bool digits_ready = false, float *silu_dst = nullptr, bool *silu_done = nullptr,
                            const float *norm_w = nullptr, float eps = 0.0f) {
  dp_ctx *ctx = m->ctx;
  if (norm_w && M == 1) {
    DP_TRY(dpk_rmsnorm(ctx, x, norm_w, false, nullptr, false, nullptr, m->n, M, K, eps, false, 1.0f));
    x = m->n;
    norm_w = nullptr;
  }
  if (M == 1) {
    if (dpk_gemv_q4k_fast_ok(N, K)) {
      if (!digits_ready) DP_TRY(dpk_q4k_prep_act(ctx, x, m->actq->dptr, K));
      bool tma = false;
      DP_TRY(dpk_gemv_q4k_actq_tma(ctx, W, m->actq->dptr, y, DP_F32, N, K, 1.0f, residual, &tma));
      if (!tma) DP_TRY(dpk_gemv_q4k_actq(ctx, W, m->actq->dptr, y, DP_F32, N, K, 1.0f, residual));
    } else {
      DP_TRY(dpk_gemv_q4k(ctx, W, x, y, DP_F32, N, K, 1.0f, residual));
    }
    return DP_OK;
  }
  // the GEMM may not alias its output with the residual: go through the partial buffer
  float *dst = (residual && residual == y) ? m->partial : y;
  // Prefill chunks of 32 rows or more run on the tensor-core kernel: each activation row is scaled into f16
  // range by a power of two (FFN intermediates of a random-init model reach 1e7, far outside f16) and
  // scaled back in the epilogue.  Default: three passes, A_hi.W_hi + A_lo.W_hi + A_hi.W_lo with the f16
  // rounding residues of activations and weights, which reproduces the f32-exact product (the reference's
  // rule for f32 activations, matmul.rules.json:15-22) to f32 accuracy at about a tenth of the CUDA-core
  // kernel's time.  DP_PREFILL_TC=1: one pass, activations and weights rounded to f16 as in the reference's
  // tiled f16 prefill kernel (fused_matmul_q4_prefill_tiled_f16.wgsl), about 1e-3 of the output's rms away
  // from the exact product; DP_PREFILL_TC=0, small chunks and shapes the tensor-core kernel does not tile:
  // the f32-exact CUDA-core kernel.
  static int prefill_tc = -1;
  if (prefill_tc < 0) { const char *e = getenv("DP_PREFILL_TC"); prefill_tc = e ? atoi(e) : 3; }
  bool handled = false;
  // (batched decode steps recorded into a CUDA graph take the same path: the f16 scratch belongs to the
  // context and is never recycled while a graph is alive)
  dpk_tc_fuse f;
  f.silu_dst = silu_dst;
  if (residual) { f.residual = residual; f.residual_out = y; }  // a K-split launch adds it in its reduction, in place
  if (norm_w) {
    if (prefill_tc) {
      f.norm_w = norm_w; f.eps = eps;
      DP_TRY(dpk_gemm_q4k_tc_rowscaled(ctx, W, x, dst, M, N, K, 1.0f, prefill_tc == 1 ? 1 : 3, &handled, &f));
      f.norm_w = nullptr;
    }
    if (!handled) {  // (nothing was launched): the norm as a kernel of its own
      DP_TRY(dpk_rmsnorm(ctx, x, norm_w, false, nullptr, false, nullptr, m->n, M, K, eps, false, 1.0f));
      x = m->n;
    }
  }
  if (!handled && prefill_tc && M >= 2) DP_TRY(dpk_gemm_q4k_tc_rowscaled(ctx, W, x, dst, M, N, K, 1.0f, prefill_tc == 1 ? 1 : 3, &handled, &f));
  if (!handled) DP_TRY(dpk_gemm_q4k_simt(ctx, W, x, DP_F32, dst, DP_F32, M, N, K, 1.0f));
  if (silu_done) *silu_done = handled && f.silu_done;
  if (residual && !(handled && f.residual_done)) DP_TRY(dpk_residual_add(ctx, residual, dst, y, (size_t)M * N, 1.0f));
  return DP_OK;
}

enum { SRC_DIGITS = 0, SRC_RMSNORM = 1, SRC_SILU = 2, SRC_COMBINE = 3, SRC_XCHG_RMSNORM = 4, SRC_PLAIN = 5, SRC_FLAG_SILU_OUT = 0x100 };

// One pass over `tokens` rows already gathered in m->h.  decode: rows are
// sequences (positions from the device arrays); prefill: rows are consecutive
// positions of sequence `seq` starting at start_pos.
//
// Single-token decode takes the fused schedule: each Q4_K GEMV kernel rebuilds its own input
// (RMSNorm, SiLU*up or the split-K merge) while its weight ring fills, so a layer is six kernels:
//   GEMV qkv [rmsnorm]  ->  qk-norm + rope + KV append  ->  attention split
//   -> GEMV o [split merge] + residual  ->  GEMV gate|up [rmsnorm]  ->  GEMV down [silu*up] + residual
// ---- the exchange group of tensor-parallel single-token decode ----
struct DecodeGroup {
  int rank = 0, nr = 0;
  uint2 *area[DP_TP_MAX_RANKS] = {};
};

// the group's areas (one-shot mode), or none (nr == 0: one GPU, or NCCL mode)
static dp_status decode_group(dp_model *m, DecodeGroup *g) {
  *g = DecodeGroup();
  if (m->cfg.tp_size > 1 && m->allreduce_mode == 1 && !dp_tp_exchange_view(m->ctx, &g->rank, &g->nr, g->area)) g->nr = 0;
  return DP_OK;
}

// attention of one decode step and layer: QK norm + RoPE + KV append + split-K partials in one kernel
static dp_status decode_attention(dp_model *m, int l, int tokens) {
  const dp_model_cfg &c = m->cfg;
  LayerW &L = m->layers[l];
  dpk_attn_params ap{};
  ap.q = m->q; ap.out = m->att;
  ap.num_heads = m->nh; ap.num_kv_heads = m->nkv; ap.head_dim = c.head_dim;
  ap.scale = 1.0f / sqrtf((float)c.head_dim); ap.softcap = 0.0f; ap.sliding_window = 0; ap.kv_start = 0;
  ap.k = (const __half *)m->kc[l]->dptr; ap.v = (const __half *)m->vc[l]->dptr;
  ap.batch = tokens; ap.seq_len = 1; ap.kv_len = c.max_seq; ap.causal = 0; ap.start_pos = 0;
  ap.kv_batch_stride = (size_t)c.max_seq * m->kvdim; ap.kv_lens = m->d_kvlen;
  ap.fuse.qkv = m->qkv;
  ap.fuse.q_norm = L.q_norm; ap.fuse.k_norm = L.k_norm;
  ap.fuse.cos_t = m->rope_cos; ap.fuse.sin_t = m->rope_sin;
  ap.fuse.pos = m->d_pos;
  ap.fuse.kc = (__half *)m->kc[l]->dptr; ap.fuse.vc = (__half *)m->vc[l]->dptr;
  ap.fuse.eps = c.eps; ap.fuse.nh = m->nh; ap.fuse.nkv = m->nkv;
  return dpk_attention_split_only(m->ctx, ap, (float *)m->attn_scratch->dptr, m->attn_splits_decode);
}

// ---- tensor-parallel single-token decode, one launch per projection, exchange inside the GEMVs ----
// Five kernels per layer, as on one GPU; the sum over ranks costs no kernel and no collective call:
//   q|k|v   [prologue: h += partials of down_proj (all ranks), RMSNorm]      (layer 0: plain RMSNorm)
//   attention (QK norm + RoPE + KV append + split-K)
//   o_proj  [prologue: split merge]          epilogue: rows pushed into every rank's exchange area (parity 0)
//   gate|up [prologue: h += partials of o_proj (all ranks), RMSNorm]
//   down    [prologue: silu(gate) * up]      epilogue: rows pushed (parity 1)
// and after the last layer one small kernel: h += partials, final RMSNorm.  The residual stream rotates over
// three buffers: a kernel reads one and its CTAs write their shares of the next.
static dp_status run_layers_tp_exchange(dp_model *m, const DecodeGroup &g) {
  dp_ctx *ctx = m->ctx;
  const dp_model_cfg &c = m->cfg;
  const int H = c.hidden, D = c.head_dim, nqkv = m->qdim + 2 * m->kvdim;
  GemvExchange base;
  base.rank = g.rank; base.nr = g.nr;
  for (int r = 0; r < g.nr; r++) base.area[r] = g.area[r];
  base.mine = g.area[g.rank];
  base.ticket_step = m->d_ticket; base.ticket_stride = 3u * (unsigned)c.n_layers + 4u;
  base.wait_limit = ctx->wait_limit;
  int cur = 0;  // hbuf index holding the residual stream
  auto fail = [&](const char *what, int l) { return dp_fail(ctx, DP_ERR_UNSUPPORTED, "decode (one-shot exchange): no kernel plan for %s of layer %d", what, l); };
  for (int l = 0; l < c.n_layers; l++) {
    LayerW &L = m->layers[l];
    bool done = false;
    if (l == 0) {
      DP_TRY(dpk_gemv_q4k_tma_fused(ctx, (const uint8_t *)L.qkv->dptr, SRC_RMSNORM, m->hbuf[cur], L.in_norm, c.eps, 0, 0, m->qkv, nqkv, H, nullptr, &done));
    } else {
      GemvExchange gx = base;
      gx.ticket_in = 3u * (unsigned)(l - 1) + 2u; gx.parity_in = 1; gx.h_out = m->hbuf[(cur + 1) % 3];
      DP_TRY(dpk_gemv_q4k_tma_fused(ctx, (const uint8_t *)L.qkv->dptr, SRC_XCHG_RMSNORM, m->hbuf[cur], L.in_norm, c.eps, 0, 0, m->qkv, nqkv, H, nullptr, &done, &gx));
      cur = (cur + 1) % 3;
    }
    if (!done) return fail("q|k|v", l);
    DP_TRY(decode_attention(m, l, 1));
    {
      GemvExchange gx = base;
      gx.push = 1; gx.parity_out = 0; gx.ticket_out = 3u * (unsigned)l;
      done = false;
      DP_TRY(dpk_gemv_q4k_tma_fused(ctx, (const uint8_t *)L.o->dptr, SRC_COMBINE, (const float *)m->attn_scratch->dptr, nullptr, 0.0f, D,
                                    m->attn_splits_decode, m->partial, H, m->qdim, nullptr, &done, &gx));
      if (!done) return fail("o_proj", l);
    }
    {
      GemvExchange gx = base;
      gx.ticket_in = 3u * (unsigned)l; gx.parity_in = 0; gx.h_out = m->hbuf[(cur + 1) % 3];
      done = false;
      // (the reducing warps store silu(gate) * up: down_proj then reads a plain vector of half the size)
      DP_TRY(dpk_gemv_q4k_tma_fused(ctx, (const uint8_t *)L.gateup->dptr, SRC_XCHG_RMSNORM | SRC_FLAG_SILU_OUT, m->hbuf[cur], L.post_norm, c.eps, 0, 0, m->actv,
                                    2 * m->inter, H, nullptr, &done, &gx));
      if (!done) return fail("gate|up", l);
      cur = (cur + 1) % 3;
    }
    {
      GemvExchange gx = base;
      gx.push = 1; gx.parity_out = 1; gx.ticket_out = 3u * (unsigned)l + 2u;
      done = false;
      DP_TRY(dpk_gemv_q4k_tma_fused(ctx, (const uint8_t *)L.down->dptr, SRC_PLAIN, m->actv, nullptr, 0.0f, 0, 0, m->partial, H, m->inter, nullptr, &done, &gx));
      if (!done) return fail("down_proj", l);
    }
  }
  GemvExchange gx = base;
  gx.ticket_in = 3u * (unsigned)(c.n_layers - 1) + 2u; gx.parity_in = 1;
  float *h_out = m->hbuf[(cur + 1) % 3];
  DP_LAUNCH(ctx, xchg_rmsnorm_kernel, 1, 256, 0, gx, (const float *)m->hbuf[cur], h_out, (const float *)m->final_norm, m->n, H, c.eps, ctx->dev_status);
  m->h_last = h_out;
  m->final_norm_done = true;
  return DP_OK;
}

static bool tp_exchange_decode_ok(dp_model *m, const DecodeGroup &g) {
  const dp_model_cfg &c = m->cfg;
  if (g.nr < 2 || !m->ctx->dev_status || !m->fuse_qk) return false;
  if (m->attn_splits_decode < 2 || c.head_dim % 8 || m->qdim % QK_K || c.hidden % QK_K || m->inter % QK_K || c.hidden > 8192) return false;
  dpk_attn_params ap{};
  ap.batch = 1; ap.seq_len = 1; ap.kv_len = c.max_seq; ap.num_heads = m->nh; ap.num_kv_heads = m->nkv; ap.head_dim = c.head_dim;
  return dpk_attention_uses_tc(m->ctx, ap);
}

// 2..64 rows on one GPU: a projection on the small-batch tensor-core kernel with the operation that precedes it in
// the layer (RMSNorm, silu(gate)*up) folded into that kernel's pre-pass and the residual added by its epilogue.
// *handled stays false when the kernel does not take the shape or a fallback switch is set; the caller then runs
// the separate kernels.
static dp_status rows_linear_fused(dp_model *m, const uint8_t *W, const float *A, float *C, int M, int N, int K, const dpk_rows_fuse &fuse,
                                   bool *handled) {
  *handled = false;
  static int on = -1;
  if (on < 0) {
    const char *a = getenv("DP_GEMM_TC"), *b = getenv("DP_PREFILL_TC");
    on = ((a && atoi(a) == 0) || (b && atoi(b) != 3)) ? 0 : 1;
  }
  // (up to 32 rows: beyond, one block per row is too little parallelism for the folded operations and the separate
  // kernels overlap with the projections' tails; measured on the 9B shapes, batch 16: 7.37 -> 6.63 ms per step,
  // batch 64: 9.18 -> 9.36 ms with everything folded, 9.51 ms with the residual alone; a 1024-token prefill with the
  // folded pre-pass in front of the prefill GEMM: 39.4 -> 41.5 ms)
  if (!on || M < 2 || M > 32 || m->cfg.tp_size != 1) return DP_OK;
  return dpk_gemm_q4k_tc_rows(m->ctx, W, A, DP_F32, C, M, N, K, 1.0f, handled, &fuse);
}

static dp_status run_layers(dp_model *m, int tokens, bool decode, int seq, int start_pos) {
  dp_ctx *ctx = m->ctx;
  const dp_model_cfg &c = m->cfg;
  const int H = c.hidden, D = c.head_dim, p = c.tp_size;
  const size_t kv_seq_stride = (size_t)c.max_seq * m->kvdim;
  const int heads = m->nh + 2 * m->nkv;
  const bool single = decode && tokens == 1;
  if (single) {
    DecodeGroup xd;
    DP_TRY(decode_group(m, &xd));
    if (tp_exchange_decode_ok(m, xd)) return run_layers_tp_exchange(m, xd);
    if (p > 1 && m->allreduce_mode == 1)
      return dp_fail(ctx, DP_ERR_UNSUPPORTED, "decode: the one-shot exchange needs shapes its kernels plan (sizes that are multiples of 256, hidden <= 8192, a split KV range)");
  }
  for (int l = 0; l < c.n_layers; l++) {
    LayerW &L = m->layers[l];
    const int nqkv = m->qdim + 2 * m->kvdim;
    // ---- q, k, v ----
    bool done = false;
    if (single) {
      DP_TRY(dpk_gemv_q4k_tma_fused(ctx, (const uint8_t *)L.qkv->dptr, SRC_RMSNORM, m->h, L.in_norm, c.eps, 0, 0, m->qkv, nqkv, H, nullptr, &done));
    }
    if (!done && !single) {
      dpk_rows_fuse f;
      f.pre = DPK_ROWS_PRE_RMSNORM; f.norm_w = L.in_norm; f.eps = c.eps;
      DP_TRY(rows_linear_fused(m, (const uint8_t *)L.qkv->dptr, m->h, m->qkv, tokens, nqkv, H, f, &done));
    }
    if (!done) {
      const bool emit = single && H % QK_K == 0 && H <= 8192 && dpk_gemv_q4k_fast_ok(nqkv, H);
      if (emit) {
        DP_LAUNCH(ctx, rmsnorm_actq_kernel, 1, 256, 0, (const float *)m->h, (const float *)L.in_norm, m->n, m->actq->dptr, H, c.eps);
      } else if (single) {
        DP_TRY(dpk_rmsnorm(ctx, m->h, L.in_norm, false, nullptr, false, nullptr, m->n, tokens, H, c.eps, false, 1.0f));
      }
      if (single) DP_TRY(q4k_linear(m, (const uint8_t *)L.qkv->dptr, m->n, m->qkv, tokens, nqkv, H, nullptr, emit));
      else DP_TRY(q4k_linear(m, (const uint8_t *)L.qkv->dptr, m->h, m->qkv, tokens, nqkv, H, nullptr, false, nullptr, nullptr, L.in_norm, c.eps));
    }
    // ---- attention parameters ----
    dpk_attn_params ap{};
    ap.q = m->q; ap.out = m->att;
    ap.num_heads = m->nh; ap.num_kv_heads = m->nkv; ap.head_dim = D;
    ap.scale = 1.0f / sqrtf((float)D); ap.softcap = 0.0f; ap.sliding_window = 0; ap.kv_start = 0;
    int splits;
    if (decode) {
      ap.k = (const __half *)m->kc[l]->dptr; ap.v = (const __half *)m->vc[l]->dptr;
      ap.batch = tokens; ap.seq_len = 1; ap.kv_len = c.max_seq; ap.causal = 0; ap.start_pos = 0;
      ap.kv_batch_stride = kv_seq_stride; ap.kv_lens = m->d_kvlen;
      splits = m->attn_splits_decode;
    } else {
      ap.k = (const __half *)m->kc[l]->dptr + (size_t)seq * kv_seq_stride;
      ap.v = (const __half *)m->vc[l]->dptr + (size_t)seq * kv_seq_stride;
      ap.batch = 1; ap.seq_len = tokens; ap.kv_len = start_pos + tokens; ap.causal = 1; ap.start_pos = start_pos;
      ap.kv_batch_stride = 0; ap.kv_lens = nullptr;
      splits = 1;
    }
    // ---- per-head QK norm, RoPE, KV append ----
    // Decode on the tensor-core attention kernel: that kernel does it itself (one launch less per layer).
    if (decode && m->fuse_qk && dpk_attention_uses_tc(ctx, ap)) {
      ap.fuse.qkv = m->qkv;
      ap.fuse.q_norm = L.q_norm; ap.fuse.k_norm = L.k_norm;
      ap.fuse.cos_t = m->rope_cos; ap.fuse.sin_t = m->rope_sin;
      ap.fuse.pos = m->d_pos;
      ap.fuse.kc = (__half *)m->kc[l]->dptr; ap.fuse.vc = (__half *)m->vc[l]->dptr;
      ap.fuse.eps = c.eps; ap.fuse.nh = m->nh; ap.fuse.nkv = m->nkv;
    } else {
      const int warps = tokens * heads;
      DP_LAUNCH(ctx, qk_norm_rope_kv_kernel, (warps + 7) / 8, 256, 0, m->qkv, m->q, (__half *)m->kc[l]->dptr,
                (__half *)m->vc[l]->dptr, L.q_norm, L.k_norm, m->rope_cos, m->rope_sin, decode ? m->d_pos : nullptr,
                start_pos, seq, tokens, m->nh, m->nkv, D, c.eps, kv_seq_stride);
    }
    float *o_dst = p == 1 ? m->h : m->partial;
    const float *o_res = p == 1 ? m->h : nullptr;
    done = false;
    const bool split_merge_ok = single && splits > 1 && D % 8 == 0 && m->qdim % QK_K == 0;
    if (split_merge_ok) {
      DP_TRY(dpk_attention_split_only(ctx, ap, (float *)m->attn_scratch->dptr, splits));
      DP_TRY(dpk_gemv_q4k_tma_fused(ctx, (const uint8_t *)L.o->dptr, SRC_COMBINE, (const float *)m->attn_scratch->dptr, nullptr, 0.0f, D,
                                    splits, o_dst, H, m->qdim, o_res, &done));
      if (!done) {
        const bool emit = dpk_gemv_q4k_fast_ok(H, m->qdim);
        const int blocks = m->qdim / QK_K;
        if (emit) {
          DP_LAUNCH(ctx, attn_combine_actq_kernel, (blocks + 7) / 8, 256, 0, (const float *)m->attn_scratch->dptr, m->att,
                    m->actq->dptr, m->nh, D, splits);
          DP_TRY(q4k_linear(m, (const uint8_t *)L.o->dptr, m->att, o_dst, tokens, H, m->qdim, o_res, true));
          done = true;
        }
      }
      if (!done) return dp_fail(ctx, DP_ERR_STATE, "decode schedule: split attention without a merge path");
    } else {
      DP_TRY(dpk_attention_with_scratch(ctx, ap, (float *)m->attn_scratch->dptr, splits));
      bool fused_o = false;
      if (p == 1) {  // h += o_proj(att) in the projection's epilogue
        dpk_rows_fuse f;
        f.residual = m->h;
        DP_TRY(rows_linear_fused(m, (const uint8_t *)L.o->dptr, m->att, m->h, tokens, H, m->qdim, f, &fused_o));
      }
      if (!fused_o) DP_TRY(q4k_linear(m, (const uint8_t *)L.o->dptr, m->att, o_dst, tokens, H, m->qdim, o_res));
    }
    // ---- exchange after o_proj (tensor parallel) and the post-attention norm ----
    if (p > 1) {
      DP_TRY(dp_tp_allreduce_ptr(ctx, m->partial, (size_t)tokens * H));
      DP_TRY(dpk_residual_add(ctx, m->h, m->partial, m->h, (size_t)tokens * H, 1.0f));
    }
    // ---- gate | up ----
    done = false;
    bool act_ready = false;  // the gate|up kernel stored silu(gate) * up itself
    bool act_rows_ready = false;  // ... and so did the tensor-core GEMM of a multi-row pass
    if (single) {
      if (m->inter % QK_K == 0 && dpk_gemv_q4k_fast_ok(H, m->inter)) {
        DP_TRY(dpk_gemv_q4k_tma_fused(ctx, (const uint8_t *)L.gateup->dptr, SRC_RMSNORM | SRC_FLAG_SILU_OUT, m->h, L.post_norm, c.eps, 0, 0, m->actv,
                                      2 * m->inter, H, nullptr, &done));
        act_ready = done;
      }
      if (!done)
        DP_TRY(dpk_gemv_q4k_tma_fused(ctx, (const uint8_t *)L.gateup->dptr, SRC_RMSNORM, m->h, L.post_norm, c.eps, 0, 0, m->gu, 2 * m->inter, H,
                                      nullptr, &done));
    }
    if (!done && !single) {
      dpk_rows_fuse f;
      f.pre = DPK_ROWS_PRE_RMSNORM; f.norm_w = L.post_norm; f.eps = c.eps;
      DP_TRY(rows_linear_fused(m, (const uint8_t *)L.gateup->dptr, m->h, m->gu, tokens, 2 * m->inter, H, f, &done));
    }
    if (!done) {
      const bool emit = single && H % QK_K == 0 && H <= 8192 && dpk_gemv_q4k_fast_ok(2 * m->inter, H);
      if (emit) {
        DP_LAUNCH(ctx, rmsnorm_actq_kernel, 1, 256, 0, (const float *)m->h, (const float *)L.post_norm, m->n, m->actq->dptr, H, c.eps);
      } else if (single) {
        DP_TRY(dpk_rmsnorm(ctx, m->h, L.post_norm, false, nullptr, false, nullptr, m->n, tokens, H, c.eps, false, 1.0f));
      }
      // (rows on the tensor-core kernel: the norm is folded into the conversion of the rows, the epilogue stores
      // silu(gate) * up and the raw gate|up rows are never written)
      if (single) DP_TRY(q4k_linear(m, (const uint8_t *)L.gateup->dptr, m->n, m->gu, tokens, 2 * m->inter, H, nullptr, emit));
      else DP_TRY(q4k_linear(m, (const uint8_t *)L.gateup->dptr, m->h, m->gu, tokens, 2 * m->inter, H, nullptr, false,
                             p == 1 ? m->actv : nullptr, &act_rows_ready, L.post_norm, c.eps));
    }
    // ---- silu(gate) * up, down ----
    float *d_dst = p == 1 ? m->h : m->partial;
    const float *d_res = p == 1 ? m->h : nullptr;
    done = false;
    if (act_ready) {
      DP_TRY(dpk_gemv_q4k_tma_fused(ctx, (const uint8_t *)L.down->dptr, SRC_PLAIN, m->actv, nullptr, 0.0f, 0, 0, d_dst, H, m->inter, d_res, &done));
      if (!done) return dp_fail(ctx, DP_ERR_STATE, "decode schedule: down_proj cannot read the fused silu(gate) * up vector");
    } else if (single && m->inter % QK_K == 0)
      DP_TRY(dpk_gemv_q4k_tma_fused(ctx, (const uint8_t *)L.down->dptr, SRC_SILU, m->gu, nullptr, 0.0f, 0, 0, d_dst, H, m->inter, d_res, &done));
    if (!done && !single && p == 1 && !act_rows_ready) {  // silu(gate) * up in the pre-pass, h += down_proj(...) in the epilogue
      dpk_rows_fuse f;
      f.pre = DPK_ROWS_PRE_SILU; f.residual = m->h;
      DP_TRY(rows_linear_fused(m, (const uint8_t *)L.down->dptr, m->gu, m->h, tokens, H, m->inter, f, &done));
    }
    if (!done) {
      const bool emit = single && m->inter % QK_K == 0 && dpk_gemv_q4k_fast_ok(H, m->inter);
      if (emit) {
        const int blocks = m->inter / QK_K;
        DP_LAUNCH(ctx, silu_actq_kernel, (blocks + 7) / 8, 256, 0, (const float *)m->gu, m->actv, m->actq->dptr, m->inter);
      } else if (!act_rows_ready) {
        const size_t total = (size_t)tokens * m->inter;
        size_t grid = (total + 255) / 256;
        if (grid > (size_t)ctx->sm_count * 8) grid = (size_t)ctx->sm_count * 8;
        DP_LAUNCH(ctx, silu_gateup_kernel, (unsigned)grid, 256, 0, m->gu, m->actv, tokens, m->inter);
      }
      DP_TRY(q4k_linear(m, (const uint8_t *)L.down->dptr, m->actv, d_dst, tokens, H, m->inter, d_res, emit));
    }
    if (p > 1) {
      DP_TRY(dp_tp_allreduce_ptr(ctx, m->partial, (size_t)tokens * H));
      DP_TRY(dpk_residual_add(ctx, m->h, m->partial, m->h, (size_t)tokens * H, 1.0f));
    }
  }
  m->final_norm_done = false;
  m->h_last = m->h;
  return DP_OK;
}

// final norm + LM head + greedy argmax for `rows` rows of hidden state starting at hrow
static dp_status run_head(dp_model *m, const float *hrow, int rows) {
  dp_ctx *ctx = m->ctx;
  const dp_model_cfg &c = m->cfg;
  if (!(m->final_norm_done && rows == 1))
    DP_TRY(dpk_rmsnorm(ctx, hrow, m->final_norm, false, nullptr, false, nullptr, m->n, rows, c.hidden, c.eps, false, 1.0f));
  m->final_norm_done = false;
  DP_TRY(dpk_gemv_f16w(ctx, (const __half *)m->lm_head->dptr, m->n, DP_F32, m->logits, DP_F32, rows, m->vocab_l, c.hidden, 1.0f));
  if (rows == 1)
    DP_TRY(dpk_argmax(ctx, m->logits, m->vocab_l, -1, m->d_tok, 0, m->am_vals, m->am_idx, m->vocab0, m->am_best));
  else  // all rows in two launches
    DP_TRY(dpk_argmax_rows(ctx, m->logits, m->vocab_l, (size_t)m->vocab_l, rows, m->d_tok, m->am_vals, m->am_idx, m->vocab0, m->am_best));
  if (c.tp_size > 1) {
    dp_tp_exchange *xd = dp_tp_exchange_desc(ctx);
    ArgmaxExchange xg{};
    if (m->allreduce_mode == 1 && xd && rows <= DP_TP_MAX_BATCH && dp_tp_exchange_view(ctx, &xg.rank, &xg.nr, xg.area)) {
      // pairs pushed into every rank's exchange area
      DP_LAUNCH(ctx, tp_argmax_exchange_kernel, 1, 256, 0, xg, xd, (const float *)m->am_best, m->d_tok, rows, ctx->wait_limit, ctx->dev_status);
    } else {
      float *pairs = (float *)m->am_pair_i;
      DP_LAUNCH(ctx, pack_pair_kernel, 1, 256, 0, m->am_best, m->d_tok, pairs, rows);
      DP_TRY(dp_tp_allgather_ptr(ctx, pairs, m->am_gather, (size_t)rows * 8));
      DP_LAUNCH(ctx, argmax_merge_kernel, 1, 256, 0, m->am_gather, c.tp_size, rows, m->d_tok);
    }
  }
  return DP_OK;
}

extern "C" dp_status dp_model_prefill(dp_model *m, int seq, const int32_t *tokens, int n, int32_t *next_token) {
  if (!m) return DP_ERR_INVALID;
  dp_ctx *ctx = m->ctx;
  const dp_model_cfg &c = m->cfg;
  DP_CHECK(ctx, seq >= 0 && seq < c.max_batch, "prefill: sequence %d outside [0,%d)", seq, c.max_batch);
  DP_CHECK(ctx, tokens && n > 0, "prefill: empty prompt");
  DP_CHECK(ctx, m->seq_len[seq] + n <= c.max_seq, "prefill: %d + %d tokens exceed max_seq %d", m->seq_len[seq], n, c.max_seq);
  for (int i = 0; i < n; i++) DP_CHECK(ctx, tokens[i] >= 0 && tokens[i] < c.vocab, "prefill: token id %d outside the vocabulary", tokens[i]);
  dp_buf ids = nullptr;
  DP_TRY(dp_buf_acquire(ctx, (size_t)m->T * 4, "prefill_token_ids", &ids));
  dp_status st = DP_OK;
  for (int off = 0; off < n && st == DP_OK; off += m->T) {
    const int cnt = n - off < m->T ? n - off : m->T;
    st = dp_buf_upload(ctx, ids, tokens + off, 0, (size_t)cnt * 4);
    if (st == DP_OK) st = dpk_gather_f16(ctx, (const int *)ids->dptr, (const __half *)m->embed->dptr, m->h, cnt, c.hidden);
    if (st == DP_OK) st = run_layers(m, cnt, false, seq, m->seq_len[seq]);
    if (st == DP_OK) {
      m->seq_len[seq] += cnt;
      if (off + cnt >= n) st = run_head(m, m->h + (size_t)(cnt - 1) * c.hidden, 1);
    }
  }
  dp_buf_release(ctx, ids);
  DP_TRY(st);
  int tok = 0;
  DP_CUDA(ctx, cudaMemcpyAsync(&tok, m->d_tok, 4, cudaMemcpyDeviceToHost, ctx->stream));
  DP_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  DP_TRY(dp_take_dev_status(ctx));  // a bounded device-side wait that gave up invalidates the result
  if (next_token) *next_token = tok;
  return DP_OK;
}

static dp_status record_decode_step(dp_model *m, int batch) {
  dp_ctx *ctx = m->ctx;
  DP_TRY(dpk_gather_f16(ctx, m->d_tok, (const __half *)m->embed->dptr, m->h, batch, m->cfg.hidden));
  DP_TRY(run_layers(m, batch, true, 0, 0));
  DP_TRY(run_head(m, m->h, batch));
  DP_LAUNCH(ctx, advance_kernel, 1, 256, 0, m->d_pos, m->d_kvlen, m->d_tok, m->d_step, (int *)m->out_tokens->dptr, batch, m->d_ticket);
  return DP_OK;
}

extern "C" dp_status dp_model_decode(dp_model *m, int batch, const int32_t *first_tokens, int steps, int32_t *out_tokens) {
  if (!m) return DP_ERR_INVALID;
  dp_ctx *ctx = m->ctx;
  const dp_model_cfg &c = m->cfg;
  DP_CHECK(ctx, batch > 0 && batch <= c.max_batch, "decode: batch %d outside [1,%d]", batch, c.max_batch);
  DP_CHECK(ctx, first_tokens && out_tokens && steps > 0, "decode: null tokens or no steps");
  for (int b = 0; b < batch; b++) {
    DP_CHECK(ctx, first_tokens[b] >= 0 && first_tokens[b] < c.vocab, "decode: token id %d outside the vocabulary", first_tokens[b]);
    DP_CHECK(ctx, m->seq_len[b] + steps <= c.max_seq, "decode: sequence %d would exceed max_seq %d", b, c.max_seq);
  }
  if (m->out_tokens_cap < steps * batch) {
    if (m->out_tokens) { dp_buf_release(ctx, m->out_tokens); m->out_tokens = nullptr; }
    for (int i = 0; i < 2; i++) if (m->graph[i]) { dp_graph_destroy(m->graph[i]); m->graph[i] = nullptr; }
    if (m->pin_out) { cudaFreeHost(m->pin_out); m->pin_out = nullptr; }
    m->out_tokens_cap = 0;
    DP_TRY(dp_buf_acquire(ctx, (size_t)steps * batch * 4, "decode_out_tokens", &m->out_tokens));
    DP_CUDA(ctx, cudaMallocHost(&m->pin_out, (size_t)steps * batch * 4));
    m->out_tokens_cap = steps * batch;
  }
  if (!m->pin_state) DP_CUDA(ctx, cudaMallocHost(&m->pin_state, 4096 + 16));
  // The state block goes up from page-locked memory without a synchronisation of its own: the previous call
  // ended with a stream synchronisation, so the staging block is free, and the step's graph follows it in stream order.
  int *st = m->pin_state;
  memset(st, 0, 4096);
  for (int b = 0; b < batch; b++) { st[b] = m->seq_len[b]; st[256 + b] = m->seq_len[b] + 1; st[512 + b] = first_tokens[b]; }
  DP_CUDA(ctx, cudaMemcpyAsync(m->state->dptr, st, 4096, cudaMemcpyHostToDevice, ctx->stream));
  const int slot = 0;
  if (!m->graph[slot] || m->graph_batch[slot] != batch) {
    if (m->graph[slot]) { dp_graph_destroy(m->graph[slot]); m->graph[slot] = nullptr; }
    dp_recorder *rec = nullptr;
    DP_TRY(dp_recorder_begin(ctx, "decode_step", 1, &rec));
    ctx->pdl = getenv("DP_PDL") ? atoi(getenv("DP_PDL")) != 0 : true;  // kernels of the step overlap their launch with the predecessor's tail
    m->recording_decode = true;
    dp_status s = record_decode_step(m, batch);
    m->recording_decode = false;
    ctx->pdl = false;
    if (s != DP_OK) { std::string keep = ctx->err; dp_recorder_abort(rec); ctx->err = keep; return s; }
    DP_TRY(dp_recorder_finish_graph(rec, &m->graph[slot]));
    m->graph_batch[slot] = batch;
  }
  DP_CUDA(ctx, cudaEventRecord(m->ev0, ctx->stream));
  for (int s = 0; s < steps; s++) DP_TRY(dp_graph_launch(m->graph[slot]));
  DP_CUDA(ctx, cudaEventRecord(m->ev1, ctx->stream));
  // tokens and the device status word come back together, one synchronisation per call
  DP_CUDA(ctx, cudaMemcpyAsync(m->pin_out, m->out_tokens->dptr, (size_t)steps * batch * 4, cudaMemcpyDeviceToHost, ctx->stream));
  DP_CUDA(ctx, cudaMemcpyAsync(st + 1024, ctx->dev_status, 4, cudaMemcpyDeviceToHost, ctx->stream));
  DP_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  float ms = 0;
  DP_CUDA(ctx, cudaEventElapsedTime(&ms, m->ev0, m->ev1));
  m->last_ms = ms;
  if (st[1024]) DP_TRY(dp_take_dev_status(ctx));  // a bounded device-side wait that gave up invalidates the tokens (DP_ERR_TIMEOUT)
  memcpy(out_tokens, m->pin_out, (size_t)steps * batch * 4);
  for (int b = 0; b < batch; b++) m->seq_len[b] += steps;
  return DP_OK;
}

extern "C" dp_status dp_model_read_logits(dp_model *m, float *host, int n) {
  if (!m || !host) return DP_ERR_INVALID;
  DP_CHECK(m->ctx, n > 0 && n <= m->cfg.max_batch * m->vocab_l, "readLogits: %d values requested, %d available", n, m->cfg.max_batch * m->vocab_l);
  DP_CUDA(m->ctx, cudaMemcpyAsync(host, m->logits, (size_t)n * 4, cudaMemcpyDeviceToHost, m->ctx->stream));
  DP_CUDA(m->ctx, cudaStreamSynchronize(m->ctx->stream));
  return DP_OK;
}

extern "C" dp_status dp_model_read_hidden(dp_model *m, float *host, int n) {
  if (!m || !host) return DP_ERR_INVALID;
  DP_CHECK(m->ctx, n > 0 && (size_t)n <= (size_t)m->T * m->cfg.hidden, "readHidden: %d values requested", n);
  DP_CUDA(m->ctx, cudaMemcpyAsync(host, n <= m->cfg.hidden ? m->h_last : m->h, (size_t)n * 4, cudaMemcpyDeviceToHost, m->ctx->stream));
  DP_CUDA(m->ctx, cudaStreamSynchronize(m->ctx->stream));
  return DP_OK;
}

extern "C" dp_status dp_model_bench_gemv(dp_model *m, int reps, double *ms_total, uint64_t *launches, uint64_t *bytes) {
  if (!m || !ms_total || !launches || !bytes) return DP_ERR_INVALID;
  dp_ctx *ctx = m->ctx;
  const dp_model_cfg &c = m->cfg;
  DP_CHECK(ctx, reps > 0, "bench_gemv: reps must be positive");
  const int H = c.hidden;
  struct Shape { int N, K; };
  const Shape sh[4] = {{m->qdim + 2 * m->kvdim, H}, {H, m->qdim}, {2 * m->inter, H}, {H, m->inter}};
  uint64_t n_bytes = 0;
  for (int i = 0; i < 4; i++)
    n_bytes += (uint64_t)sh[i].N * dp_cdiv((size_t)sh[i].K, DP_QK_K) * DP_Q4K_BLOCK_BYTES + 4ull * sh[i].K + 4ull * sh[i].N;
  n_bytes *= (uint64_t)c.n_layers * (uint64_t)reps;
  // The timed loop launches, per layer, the four GEMV kernels of the single-token decode step with the prologues
  // that step uses (RMSNorm for q|k|v and gate|up, split merge for o_proj, silu(gate)*up for down_proj), each
  // reading what its predecessor wrote, back to back without the attention kernel.  Shapes the fused kernels do
  // not plan fall back to the kernel that takes ready-made digits.
  DP_TRY(dpk_q4k_prep_act(ctx, m->actv, m->actq->dptr, m->inter > H ? (m->inter / QK_K) * QK_K : H));
  const int splits = m->attn_splits_decode > 1 ? m->attn_splits_decode : 2;
  const bool fused_ok = c.tp_size == 1 && m->attn_scratch && c.head_dim % 8 == 0 && m->qdim % QK_K == 0 && m->inter % QK_K == 0;
  const uint64_t l0 = ctx->launches;
  ctx->pdl = true;
  DP_CUDA(ctx, cudaEventRecord(m->ev0, ctx->stream));
  dp_status st = DP_OK;
  for (int r = 0; r < reps && st == DP_OK; r++) {
    for (int l = 0; l < c.n_layers && st == DP_OK; l++) {
      LayerW &L = m->layers[l];
      bool done[4] = {false, false, false, false};
      if (fused_ok) {
        st = dpk_gemv_q4k_tma_fused(ctx, (const uint8_t *)L.qkv->dptr, SRC_RMSNORM, m->h, L.in_norm, c.eps, 0, 0, m->qkv, sh[0].N, H, nullptr, &done[0]);
        if (st == DP_OK && !done[0]) st = q4k_linear(m, (const uint8_t *)L.qkv->dptr, m->n, m->qkv, 1, sh[0].N, sh[0].K, nullptr, dpk_gemv_q4k_fast_ok(sh[0].N, sh[0].K));
        if (st == DP_OK)
          st = dpk_gemv_q4k_tma_fused(ctx, (const uint8_t *)L.o->dptr, SRC_COMBINE, (const float *)m->attn_scratch->dptr, nullptr, 0.0f, c.head_dim, splits,
                                      m->partial, H, m->qdim, m->h, &done[1]);
        if (st == DP_OK && !done[1]) st = q4k_linear(m, (const uint8_t *)L.o->dptr, m->att, m->partial, 1, sh[1].N, sh[1].K, nullptr, dpk_gemv_q4k_fast_ok(sh[1].N, sh[1].K));
        if (st == DP_OK)
          st = dpk_gemv_q4k_tma_fused(ctx, (const uint8_t *)L.gateup->dptr, SRC_RMSNORM | SRC_FLAG_SILU_OUT, m->h, L.post_norm, c.eps, 0, 0, m->actv, sh[2].N, H, nullptr, &done[2]);
        if (st == DP_OK && !done[2]) st = q4k_linear(m, (const uint8_t *)L.gateup->dptr, m->n, m->gu, 1, sh[2].N, sh[2].K, nullptr, dpk_gemv_q4k_fast_ok(sh[2].N, sh[2].K));
        if (st == DP_OK) st = dpk_gemv_q4k_tma_fused(ctx, (const uint8_t *)L.down->dptr, SRC_PLAIN, m->actv, nullptr, 0.0f, 0, 0, m->partial, H, m->inter, m->h, &done[3]);
        if (st == DP_OK && !done[3]) st = q4k_linear(m, (const uint8_t *)L.down->dptr, m->actv, m->partial, 1, sh[3].N, sh[3].K, nullptr, dpk_gemv_q4k_fast_ok(sh[3].N, sh[3].K));
      } else {
        const uint8_t *W[4] = {(const uint8_t *)L.qkv->dptr, (const uint8_t *)L.o->dptr, (const uint8_t *)L.gateup->dptr,
                               (const uint8_t *)L.down->dptr};
        const float *X[4] = {m->n, m->att, m->n, m->actv};
        float *Y[4] = {m->qkv, m->partial, m->gu, m->partial};
        for (int i = 0; i < 4 && st == DP_OK; i++)
          st = q4k_linear(m, W[i], X[i], Y[i], 1, sh[i].N, sh[i].K, nullptr, dpk_gemv_q4k_fast_ok(sh[i].N, sh[i].K));
      }
    }
  }
  ctx->pdl = false;
  m->final_norm_done = false;
  DP_TRY(st);
  DP_CUDA(ctx, cudaEventRecord(m->ev1, ctx->stream));
  DP_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  float ms = 0;
  DP_CUDA(ctx, cudaEventElapsedTime(&ms, m->ev0, m->ev1));
  *ms_total = ms; *launches = ctx->launches - l0; *bytes = n_bytes;
  return DP_OK;
}
