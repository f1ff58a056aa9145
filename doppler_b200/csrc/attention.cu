// Attention over the f16 KV cache: split-K flash-decode with GQA head sharing.
//
// Replaces src/gpu/kernels/attention_decode_online_f16kv.wgsl:85 (one workgroup
// per query head, no KV split, each KV head re-read once per query head of its
// group) and, for seq_len > 1, attention_streaming_f16kv.wgsl:96.
//
// Layouts are the reference's: Q f32 [seq, H, D]; K,V f16 [pos, Hkv, D]; out f32
// [seq, H, D].  The kernel grid is (kv splits, KV heads x head tiles, batch x
// query rows).  A CTA streams its slice of keys ONCE and applies it to every
// query head of the KV group (up to four per CTA), so HBM traffic is the KV
// bytes.  Eight lanes share a key (each lane owns D/8 dims, two 16-byte loads
// for D=128); each 8-lane group keeps its own running max / sum / output and the
// groups are merged at the end (warp shuffles, then shared memory).  Split
// partials (m, l, o) go to a scratch buffer and a second kernel merges them.
#include "common.h"
#include "pdl.cuh"

#include <cfloat>
#include <cstdlib>

#define ATT_THREADS 256
#define ATT_GROUPS (ATT_THREADS / 8)

struct AttnRange { int lo, hi; };

// keys visible to query row qi: [lo, hi) in cache positions
__device__ __forceinline__ AttnRange attn_range(int kv_len, int causal, int start_pos, int qi, int sliding_window,
                                                int kv_start) {
  AttnRange r;
  r.lo = 0;
  r.hi = kv_len;
  const int abs_q = start_pos + qi;
  if (causal) {
    int lim = abs_q - kv_start + 1;  // abs_key <= abs_q
    if (lim < r.hi) r.hi = lim;
  }
  if (sliding_window > 0 && abs_q >= sliding_window) {
    int first = abs_q - sliding_window + 1 - kv_start;  // abs_key >= abs_q - window + 1
    if (first > r.lo) r.lo = first;
  }
  if (r.hi < r.lo) r.hi = r.lo;
  return r;
}

// LPK lanes share a key (each owns DPL = D/LPK dims).  More lanes per key = fewer registers per
// thread (q and the output accumulators shrink), which is what lets two CTAs share an SM.
template <int DPL, int GT, int LPK>
__global__ void __launch_bounds__(ATT_THREADS, LPK == 16 ? 2 : 1) attn_split_kernel(dpk_attn_params p, float *__restrict__ part, int splits,
                                                                                    int head_tiles) {
  pdl_launch();
  pdl_wait();
  constexpr int D = DPL * LPK;
  constexpr int KEY_GROUPS = ATT_THREADS / LPK;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sub = lane & (LPK - 1);  // which D/LPK slice of the key this lane owns
  const int grp = tid / LPK;         // key group index within the CTA
  const int split = blockIdx.x;
  const int kvh = blockIdx.y / head_tiles, ht = blockIdx.y % head_tiles;
  const int z = blockIdx.z, b = z / p.seq_len, qi = z % p.seq_len;
  const int G = p.num_heads / p.num_kv_heads;
  const int h0 = kvh * G + ht * GT;  // first query head of this CTA

  int kv_len = p.kv_lens ? min(max(p.kv_lens[b], 0), p.kv_len) : p.kv_len;  // the host checked the cache for p.kv_len keys
  const AttnRange r = attn_range(kv_len, p.causal, p.start_pos, qi, p.sliding_window, p.kv_start);
  const int n_keys = r.hi - r.lo;
  const int per_split = (n_keys + splits - 1) / splits;
  const int k_begin = r.lo + split * per_split;
  int k_end = k_begin + per_split;
  if (k_end > r.hi) k_end = r.hi;

  const float LOG2E = 1.4426950408889634f;
  // q for this lane's dims, pre-multiplied by the softmax scale
  float q[GT][DPL];
#pragma unroll
  for (int g = 0; g < GT; g++) {
    const float *qp = p.q + ((size_t)z * p.num_heads + h0 + g) * D + sub * DPL;
#pragma unroll
    for (int i = 0; i < DPL; i += 4) {
      const float4 v = *reinterpret_cast<const float4 *>(qp + i);
      q[g][i] = v.x * p.scale; q[g][i + 1] = v.y * p.scale; q[g][i + 2] = v.z * p.scale; q[g][i + 3] = v.w * p.scale;
    }
  }
  float m[GT], l[GT], o[GT][DPL];
#pragma unroll
  for (int g = 0; g < GT; g++) {
    m[g] = -FLT_MAX; l[g] = 0.0f;
#pragma unroll
    for (int i = 0; i < DPL; i++) o[g][i] = 0.0f;
  }

  const size_t row_stride = (size_t)p.num_kv_heads * D;
  const __half *kbase = p.k + (size_t)b * p.kv_batch_stride + (size_t)kvh * D + sub * DPL;
  const __half *vbase = p.v + (size_t)b * p.kv_batch_stride + (size_t)kvh * D + sub * DPL;

  // The four 8-lane groups of a warp may run different trip counts, so the shuffles inside
  // the loop name only the lanes of their own group.
  const unsigned gmask = (LPK == 16 ? 0xFFFFu : 0xFFu) << (lane & ~(LPK - 1));
#pragma unroll 2
  for (int key = k_begin + grp; key < k_end; key += KEY_GROUPS) {
    uint4 kraw[DPL / 8], vraw[DPL / 8];
#pragma unroll
    for (int i = 0; i < DPL / 8; i++) {
      kraw[i] = __ldg(reinterpret_cast<const uint4 *>(kbase + (size_t)key * row_stride) + i);
      vraw[i] = __ldg(reinterpret_cast<const uint4 *>(vbase + (size_t)key * row_stride) + i);
    }
    float kf[DPL];
#pragma unroll
    for (int i = 0; i < DPL / 8; i++) {
      const __half2 *h = reinterpret_cast<const __half2 *>(&kraw[i]);
#pragma unroll
      for (int jx = 0; jx < 4; jx++) { const float2 f = __half22float2(h[jx]); kf[i * 8 + 2 * jx] = f.x; kf[i * 8 + 2 * jx + 1] = f.y; }
    }
    float s[GT];
#pragma unroll
    for (int g = 0; g < GT; g++) {
      float a = 0.0f;
#pragma unroll
      for (int i = 0; i < DPL; i++) a = fmaf(q[g][i], kf[i], a);
      a += __shfl_xor_sync(gmask, a, 1);
      a += __shfl_xor_sync(gmask, a, 2);
      a += __shfl_xor_sync(gmask, a, 4);
      if (LPK == 16) a += __shfl_xor_sync(gmask, a, 8);
      if (p.softcap > 0.0f) a = tanhf(a / p.softcap) * p.softcap;
      s[g] = a * LOG2E;
    }
    float vf[DPL];
#pragma unroll
    for (int i = 0; i < DPL / 8; i++) {
      const __half2 *h = reinterpret_cast<const __half2 *>(&vraw[i]);
#pragma unroll
      for (int jx = 0; jx < 4; jx++) { const float2 f = __half22float2(h[jx]); vf[i * 8 + 2 * jx] = f.x; vf[i * 8 + 2 * jx + 1] = f.y; }
    }
#pragma unroll
    for (int g = 0; g < GT; g++) {
      if (s[g] > m[g]) {  // rare after the first keys: rescale the running state
        const float c = exp2f(m[g] - s[g]);
        l[g] *= c;
#pragma unroll
        for (int i = 0; i < DPL; i++) o[g][i] *= c;
        m[g] = s[g];
      }
      const float pr = exp2f(s[g] - m[g]);
      l[g] += pr;
#pragma unroll
      for (int i = 0; i < DPL; i++) o[g][i] = fmaf(pr, vf[i], o[g][i]);
    }
  }

  // merge the key groups of each warp
#pragma unroll
  for (int g = 0; g < GT; g++) {
    float mm = m[g];
    if (LPK == 8) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 8));
    mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, 16));
    const float c = (m[g] == -FLT_MAX) ? 0.0f : exp2f(m[g] - mm);
    float ll = l[g] * c;
    if (LPK == 8) ll += __shfl_xor_sync(0xffffffffu, ll, 8);
    ll += __shfl_xor_sync(0xffffffffu, ll, 16);
#pragma unroll
    for (int i = 0; i < DPL; i++) {
      float v = o[g][i] * c;
      if (LPK == 8) v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      o[g][i] = v;
    }
    m[g] = mm; l[g] = ll;
  }
  // merge the warps through shared memory
  __shared__ float sm_o[ATT_THREADS / 32][GT][D];
  __shared__ float sm_m[ATT_THREADS / 32][GT], sm_l[ATT_THREADS / 32][GT];
  if (lane < LPK) {
#pragma unroll
    for (int g = 0; g < GT; g++) {
#pragma unroll
      for (int i = 0; i < DPL; i++) sm_o[warp][g][sub * DPL + i] = o[g][i];
      if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
    }
  }
  __syncthreads();
  constexpr int NW = ATT_THREADS / 32;
  for (int idx = tid; idx < GT * D; idx += ATT_THREADS) {
    const int g = idx / D, d = idx % D;
    float mm = -FLT_MAX;
#pragma unroll
    for (int w = 0; w < NW; w++) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.0f, acc = 0.0f;
#pragma unroll
    for (int w = 0; w < NW; w++) {
      const float c = (sm_m[w][g] == -FLT_MAX) ? 0.0f : exp2f(sm_m[w][g] - mm);
      ll = fmaf(sm_l[w][g], c, ll);
      acc = fmaf(sm_o[w][g][d], c, acc);
    }
    const int h = h0 + g;
    if (splits == 1) {
      p.out[((size_t)z * p.num_heads + h) * D + d] = ll > 0.0f ? acc / ll : 0.0f;
    } else {
      float *pp = part + (((size_t)z * p.num_heads + h) * splits + split) * (D + 2);
      pp[d] = acc;
      if (d == 0) { pp[D] = mm; pp[D + 1] = ll; }
    }
  }
}

// Any head_dim <= 512 and any GQA ratio: one CTA per (split, query head, row),
// lanes over dims.  Used for shapes outside the fast kernel.
__global__ void __launch_bounds__(128) attn_split_generic_kernel(dpk_attn_params p, float *__restrict__ part, int splits) {
  pdl_launch();
  pdl_wait();
  const int D = p.head_dim;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x, h = blockIdx.y, z = blockIdx.z;
  const int b = z / p.seq_len, qi = z % p.seq_len;
  const int kvh = h / (p.num_heads / p.num_kv_heads);
  int kv_len = p.kv_lens ? min(max(p.kv_lens[b], 0), p.kv_len) : p.kv_len;  // the host checked the cache for p.kv_len keys
  const AttnRange r = attn_range(kv_len, p.causal, p.start_pos, qi, p.sliding_window, p.kv_start);
  const int n_keys = r.hi - r.lo;
  const int per_split = (n_keys + splits - 1) / splits;
  const int k_begin = r.lo + split * per_split;
  int k_end = k_begin + per_split;
  if (k_end > r.hi) k_end = r.hi;
  const float LOG2E = 1.4426950408889634f;
  constexpr int MAXE = 16;  // dims per lane
  float q[MAXE], o[MAXE];
  const float *qp = p.q + ((size_t)z * p.num_heads + h) * D;
#pragma unroll
  for (int i = 0; i < MAXE; i++) { const int d = lane + 32 * i; q[i] = d < D ? qp[d] * p.scale : 0.0f; o[i] = 0.0f; }
  float m = -FLT_MAX, l = 0.0f;
  const size_t row_stride = (size_t)p.num_kv_heads * D;
  const __half *kb = p.k + (size_t)b * p.kv_batch_stride + (size_t)kvh * D;
  const __half *vb = p.v + (size_t)b * p.kv_batch_stride + (size_t)kvh * D;
  for (int key = k_begin + warp; key < k_end; key += 4) {
    float a = 0.0f;
#pragma unroll
    for (int i = 0; i < MAXE; i++) { const int d = lane + 32 * i; if (d < D) a = fmaf(q[i], __half2float(kb[(size_t)key * row_stride + d]), a); }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) a += __shfl_xor_sync(0xffffffffu, a, s);
    if (p.softcap > 0.0f) a = tanhf(a / p.softcap) * p.softcap;
    a *= LOG2E;
    if (a > m) {
      const float c = exp2f(m - a);
      l *= c;
#pragma unroll
      for (int i = 0; i < MAXE; i++) o[i] *= c;
      m = a;
    }
    const float pr = exp2f(a - m);
    l += pr;
#pragma unroll
    for (int i = 0; i < MAXE; i++) { const int d = lane + 32 * i; if (d < D) o[i] = fmaf(pr, __half2float(vb[(size_t)key * row_stride + d]), o[i]); }
  }
  __shared__ float sm_o[4][512];
  __shared__ float sm_m[4], sm_l[4];
#pragma unroll
  for (int i = 0; i < MAXE; i++) { const int d = lane + 32 * i; if (d < D) sm_o[warp][d] = o[i]; }
  if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
  __syncthreads();
  for (int d = tid; d < D; d += 128) {
    float mm = -FLT_MAX;
    for (int w = 0; w < 4; w++) mm = fmaxf(mm, sm_m[w]);
    float ll = 0.0f, acc = 0.0f;
    for (int w = 0; w < 4; w++) {
      const float c = (sm_m[w] == -FLT_MAX) ? 0.0f : exp2f(sm_m[w] - mm);
      ll = fmaf(sm_l[w], c, ll);
      acc = fmaf(sm_o[w][d], c, acc);
    }
    if (splits == 1) {
      p.out[((size_t)z * p.num_heads + h) * D + d] = ll > 0.0f ? acc / ll : 0.0f;
    } else {
      float *pp = part + (((size_t)z * p.num_heads + h) * splits + split) * (D + 2);
      pp[d] = acc;
      if (d == 0) { pp[D] = mm; pp[D + 1] = ll; }
    }
  }
}

// merge the split partials of one (row, head)
__global__ void attn_combine_kernel(const float *__restrict__ part, float *__restrict__ out, int D, int splits) {
  pdl_launch();
  pdl_wait();
  const size_t rh = blockIdx.x;
  const float *pp = part + rh * splits * (D + 2);
  float mm = -FLT_MAX;
  for (int s = 0; s < splits; s++) mm = fmaxf(mm, pp[s * (D + 2) + D]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float ll = 0.0f, acc = 0.0f;
#pragma unroll 4
    for (int s = 0; s < splits; s++) {
      const float ms = pp[s * (D + 2) + D];
      const float c = (ms == -FLT_MAX) ? 0.0f : exp2f(ms - mm);
      ll = fmaf(pp[s * (D + 2) + D + 1], c, ll);
      acc = fmaf(pp[s * (D + 2) + d], c, acc);
    }
    out[rh * D + d] = ll > 0.0f ? acc / ll : 0.0f;
  }
}

static bool fast_shape(const dpk_attn_params &p, int *gt) {
  if (p.head_dim != 128 && p.head_dim != 64) return false;
  const int G = p.num_heads / p.num_kv_heads;
  if (G == 1 || G == 2 || G == 4) { *gt = G; return true; }
  if (G % 4 == 0) { *gt = 4; return true; }
  return false;
}

// tensor-core decode kernel (attention_tc.cu)
bool dpk_attention_tc_eligible(const dpk_attn_params &p, int *gt_out);
dp_status dpk_attention_tc_split(dp_ctx *ctx, const dpk_attn_params &p, float *scratch, int splits);

// Every single-row shape the tensor-core kernel takes goes to it: it also wins on short contexts
// (9B-shaped decode step at context 1024: 2.08 ms with it, 2.21 ms with the CUDA-core kernel).
// DP_ATTN_TC=0 keeps the CUDA-core kernel.
static bool use_tc(dp_ctx *ctx, const dpk_attn_params &p, int *gt) {
  (void)ctx;
  static const int mode = [] { const char *e = getenv("DP_ATTN_TC"); return e ? atoi(e) : 1; }();
  return mode && dpk_attention_tc_eligible(p, gt);
}

// whether a call with these parameters runs on the tensor-core kernel (the decode schedule asks before it
// hands the kernel the QK-norm / RoPE / KV-append fusion)
bool dpk_attention_uses_tc(dp_ctx *ctx, const dpk_attn_params &p) {
  int gt = 0;
  return use_tc(ctx, p, &gt);
}

// splits for the tensor-core kernel: fewest whole waves of (two CTAs per SM) x keys per CTA
static int tc_splits(dp_ctx *ctx, const dpk_attn_params &p, int gt) {
  const int G = p.num_heads / p.num_kv_heads;
  const long base = (long)p.batch * p.seq_len * p.num_kv_heads * (G / gt);
  const long slots = (long)ctx->sm_count * 2;
  long best = 1, best_cost = -1;
  for (long s = 1; s <= 32; s++) {
    const long keys = (p.kv_len + s - 1) / s;
    // at least two rounds of the CTA's four warps per split: finer splits only lengthen the merge that
    // follows (9B-shaped decode at context 1024, cache of 1450 keys: 4 / 6 / 8 / 11 / 16 splits 1.962 / 1.944 / 1.966 /
    // 1.989 / 2.046 ms per step)
    if (s > 1 && keys < 192) break;
    const long waves = (base * s + slots - 1) / slots;
    const long cost = waves * (keys + 64);
    if (best_cost < 0 || cost < best_cost) { best = s; best_cost = cost; }
  }
  return (int)best;
}

size_t dpk_attention_scratch_bytes(dp_ctx *ctx, const dpk_attn_params &p, int *splits_out) {
  int gt = 1;
  if (use_tc(ctx, p, &gt)) {
    const int s = tc_splits(ctx, p, gt);
    *splits_out = s;
    return s == 1 ? 0 : (size_t)p.batch * p.seq_len * p.num_heads * s * (p.head_dim + 2) * sizeof(float);
  }
  const bool fast = fast_shape(p, &gt);
  const int G = p.num_heads / p.num_kv_heads;
  const long rows = (long)p.batch * p.seq_len;
  const long base_ctas = fast ? rows * p.num_kv_heads * (G / gt) : rows * p.num_heads;
  const long target = (long)ctx->sm_count * 4;
  long splits = (target + base_ctas - 1) / base_ctas;
  const int keys_per_cta_min = fast ? 128 : 32;
  long max_splits = (p.kv_len + keys_per_cta_min - 1) / keys_per_cta_min;
  if (max_splits < 1) max_splits = 1;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  if (splits > 32) splits = 32;
  *splits_out = (int)splits;
  if (splits == 1) return 0;
  return (size_t)rows * p.num_heads * splits * (p.head_dim + 2) * sizeof(float);
}

template <int DPL, int GT, int LPK>
static dp_status launch_fast(dp_ctx *ctx, const dpk_attn_params &p, float *scratch, int splits) {
  const int G = p.num_heads / p.num_kv_heads;
  const int head_tiles = G / GT;
  dim3 grid(splits, p.num_kv_heads * head_tiles, p.batch * p.seq_len);
  DP_LAUNCH(ctx, (attn_split_kernel<DPL, GT, LPK>), grid, ATT_THREADS, 0, p, scratch, splits, head_tiles);
  return DP_OK;
}

static dp_status attention_impl(dp_ctx *ctx, const dpk_attn_params &p, float *scratch, int splits, bool combine);

dp_status dpk_attention_with_scratch(dp_ctx *ctx, const dpk_attn_params &p, float *scratch, int splits) {
  return attention_impl(ctx, p, scratch, splits, true);
}

// the split kernel alone (splits > 1): the caller merges the partials itself
dp_status dpk_attention_split_only(dp_ctx *ctx, const dpk_attn_params &p, float *scratch, int splits) {
  return attention_impl(ctx, p, scratch, splits, false);
}

// query-tiled causal prefill kernel (attention_prefill.cu)
bool dpk_attention_prefill_eligible(const dpk_attn_params &p);
dp_status dpk_attention_prefill(dp_ctx *ctx, const dpk_attn_params &p);

static dp_status attention_impl(dp_ctx *ctx, const dpk_attn_params &p, float *scratch, int splits, bool combine) {
  int gt = 1;
  // several causal query rows: one CTA per tile of query positions shares each K / V tile (DP_ATTN_TC=0: off)
  static const int tc_mode = [] { const char *e = getenv("DP_ATTN_TC"); return e ? atoi(e) : 1; }();
  if (tc_mode && combine && dpk_attention_prefill_eligible(p)) return dpk_attention_prefill(ctx, p);
  if (use_tc(ctx, p, &gt)) {
    DP_TRY(dpk_attention_tc_split(ctx, p, scratch, splits));
  } else if (fast_shape(p, &gt)) {
    if (p.head_dim == 128) {
      if (gt == 1) DP_TRY((launch_fast<16, 1, 8>(ctx, p, scratch, splits)));
      else if (gt == 2) DP_TRY((launch_fast<16, 2, 8>(ctx, p, scratch, splits)));
      else DP_TRY((launch_fast<8, 4, 16>(ctx, p, scratch, splits)));  // 4 heads: 16 lanes per key keep it under 128 registers
    } else {
      if (gt == 1) DP_TRY((launch_fast<8, 1, 8>(ctx, p, scratch, splits)));
      else if (gt == 2) DP_TRY((launch_fast<8, 2, 8>(ctx, p, scratch, splits)));
      else DP_TRY((launch_fast<8, 4, 8>(ctx, p, scratch, splits)));
    }
  } else {
    dim3 grid(splits, p.num_heads, p.batch * p.seq_len);
    DP_LAUNCH(ctx, attn_split_generic_kernel, grid, 128, 0, p, scratch, splits);
  }
  if (splits > 1 && combine) {
    const unsigned rows = (unsigned)((long)p.batch * p.seq_len * p.num_heads);
    int threads = p.head_dim < 128 ? ((p.head_dim + 31) / 32) * 32 : 128;
    DP_LAUNCH(ctx, attn_combine_kernel, rows, threads, 0, scratch, p.out, p.head_dim, splits);
  }
  return DP_OK;
}

dp_status dpk_attention(dp_ctx *ctx, const dpk_attn_params &p) {
  int splits = 1;
  const size_t bytes = dpk_attention_scratch_bytes(ctx, p, &splits);
  float *scratch = nullptr;
  if (bytes) {
    DP_TRY(dp_scratch(ctx, &ctx->attn_scratch, bytes, "attention_split_partials"));
    scratch = (float *)ctx->attn_scratch->dptr;
  }
  return dpk_attention_with_scratch(ctx, p, scratch, splits);
}
