// Decode attention over the f16 KV cache on the tensor cores (one query row per sequence).
//
// Same contract as attn_split_kernel (attention.cu) and the reference kernel it replaces
// (src/gpu/kernels/attention_decode_online_f16kv.wgsl:85): Q f32 [batch, H, D], K,V f16
// [pos, Hkv, D], split-K partials (o, m, l) per (sequence, head, split).  What changes is who
// does the arithmetic.  The CUDA-core kernel spends ~40 instructions per key; here a warp
// handles 16 keys per iteration with 24 mma.sync.m16n8k16 instructions:
//
//   S   = Q  K^T   M = 16 rows (query heads of the KV group), N = 8 keys, K = head_dim
//   O^T = V^T P^T  M = 16 dims, N = 8 head columns, K = 16 keys
//
// The M = 16 rows of the first product are only half used by a GQA group of <= 8 heads, so rows
// 8..15 carry the low halves of a hi/lo f16 split of Q (S = S_hi + S_lo lands in the same
// thread), which keeps Q at ~22 bits.  With <= 4 heads the eight head columns of the second
// product do the same for P.  K and V stay f16 (exact), all accumulation is f32.
//
// Data movement: every warp owns a private ring of three 16-key stages in shared memory filled
// with cp.async (16 B per lane, rows XOR-swizzled so that ldmatrix is conflict free), so warps
// never wait for one another inside the key loop.  K fragments come from ldmatrix, V^T fragments
// from ldmatrix.trans.  Two CTAs of four warps per SM keep 128 KB of KV reads in flight per SM.
#include "common.h"
#include "pdl.cuh"

#include <cfloat>
#include <cmath>

#define ATC_WARPS 4
#define ATC_THREADS (ATC_WARPS * 32)
#define ATC_STAGES 3

__device__ __forceinline__ uint32_t atc_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void atc_cp_async16(uint32_t dst, const void *src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void atc_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void atc_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ void atc_ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void atc_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void atc_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t atc_pack(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

// D = head_dim (64 or 128).  PLO: the group has <= 4 heads, head columns 4..7 carry the low halves of P.
template <int D, bool PLO>
__global__ void __launch_bounds__(ATC_THREADS, 2) attn_tc_kernel(dpk_attn_params p, float *__restrict__ part, int splits,
                                                                 int head_tiles, int gt) {
  pdl_launch();
  pdl_wait();
  constexpr int CH = D / 8;        // 16-byte chunks per key row
  constexpr int ROWB = D * 2;      // bytes per key row
  constexpr int TILE = 16 * ROWB;  // one 16-key K (or V) tile
  constexpr int STAGE = 2 * TILE;  // K tile then V tile
  constexpr int KS = D / 16;       // k-steps of Q K^T = m-blocks of V^T P^T
  extern __shared__ __align__(128) unsigned char atc_smem[];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x;
  const int kvh = blockIdx.y / head_tiles, ht = blockIdx.y % head_tiles;
  const int z = blockIdx.z, b = z / p.seq_len, qi = z % p.seq_len;  // one query row per CTA (prefill rows are independent)
  const int G = p.num_heads / p.num_kv_heads;
  const int h0 = kvh * G + ht * gt;

  int kv_len = p.kv_lens ? min(max(p.kv_lens[b], 0), p.kv_len) : p.kv_len;  // the host checked the cache for p.kv_len keys
  int lo = 0, hi = kv_len;
  {
    const int abs_q = p.start_pos + qi;
    if (p.causal) { const int lim = abs_q - p.kv_start + 1; if (lim < hi) hi = lim; }
    if (p.sliding_window > 0 && abs_q >= p.sliding_window) { const int first = abs_q - p.sliding_window + 1 - p.kv_start; if (first > lo) lo = first; }
    if (hi < lo) hi = lo;
  }
  const int n_keys = hi - lo;
  const int per_split = (n_keys + splits - 1) / splits;
  const int k_begin = lo + split * per_split;
  int k_end = k_begin + per_split;
  if (k_end > hi) k_end = hi;

  const float LOG2E = 1.4426950408889634f;
  const bool capped = p.softcap > 0.0f;
  const float qmul = capped ? p.scale : p.scale * LOG2E;

  // A fragments of Q for every k-step: rows g (hi) and g+8 (lo).  This lane owns dims 16ks + 2t + {0,1,8,9}.
  const bool fused = p.fuse.qkv != nullptr;
  const int new_pos = fused ? p.fuse.pos[b] : -1;  // the key that is not in the cache yet
  uint32_t qa[KS][4];
  {
    float x[KS][4];
    if (g < gt) {
      const float *qrow = fused ? p.fuse.qkv + ((size_t)b * (p.fuse.nh + 2 * p.fuse.nkv) + h0 + g) * D
                                : p.q + ((size_t)z * p.num_heads + h0 + g) * D;
#pragma unroll
      for (int ks = 0; ks < KS; ks++) {
        const float2 x0 = *reinterpret_cast<const float2 *>(qrow + 16 * ks + 2 * t);
        const float2 x1 = *reinterpret_cast<const float2 *>(qrow + 16 * ks + 2 * t + 8);
        x[ks][0] = x0.x; x[ks][1] = x0.y; x[ks][2] = x1.x; x[ks][3] = x1.y;
      }
    } else {
#pragma unroll
      for (int ks = 0; ks < KS; ks++) x[ks][0] = x[ks][1] = x[ks][2] = x[ks][3] = 0.0f;
    }
    if (fused) {
      // per-head RMSNorm (rmsnorm_qk.wgsl:75-118) and rotate-half RoPE (rope.wgsl:62-106): the four lanes
      // of a head hold all its dims, and the partner of dim d (d + D/2) sits KS/2 k-steps further in the
      // same lane
      float ss = 0.0f;
#pragma unroll
      for (int ks = 0; ks < KS; ks++)
#pragma unroll
        for (int j = 0; j < 4; j++) ss = fmaf(x[ks][j], x[ks][j], ss);
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      const float inv = 1.0f / sqrtf(ss / (float)D + p.fuse.eps);
      constexpr int HALF = D / 2;
      if (g < gt) {
#pragma unroll
        for (int ks = 0; ks < KS / 2; ks++)
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const int d = 16 * ks + 2 * t + (j & 1) + (j >> 1) * 8;
            const float a = x[ks][j] * inv * p.fuse.q_norm[d], bb = x[ks + KS / 2][j] * inv * p.fuse.q_norm[d + HALF];
            const float c = p.fuse.cos_t[(size_t)new_pos * HALF + d], sn = p.fuse.sin_t[(size_t)new_pos * HALF + d];
            x[ks][j] = a * c - bb * sn;
            x[ks + KS / 2][j] = a * sn + bb * c;
          }
      }
    }
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
      const __half2 h0v = __floats2half2_rn(x[ks][0] * qmul, x[ks][1] * qmul);
      const __half2 h1v = __floats2half2_rn(x[ks][2] * qmul, x[ks][3] * qmul);
      const float2 f0 = __half22float2(h0v), f1 = __half22float2(h1v);
      qa[ks][0] = atc_pack(h0v);
      qa[ks][1] = atc_pack(__floats2half2_rn(x[ks][0] * qmul - f0.x, x[ks][1] * qmul - f0.y));
      qa[ks][2] = atc_pack(h1v);
      qa[ks][3] = atc_pack(__floats2half2_rn(x[ks][2] * qmul - f1.x, x[ks][3] * qmul - f1.y));
    }
  }

  float o[KS][4];
#pragma unroll
  for (int j = 0; j < KS; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
  float m_run = -INFINITY, l_run = 0.0f;  // head g; l is this lane's share (keys 2t, 2t+1 of every block)

  const size_t row_stride = (size_t)p.num_kv_heads * D;
  const __half *kbase = p.k + (size_t)b * p.kv_batch_stride + (size_t)kvh * D;
  const __half *vbase = p.v + (size_t)b * p.kv_batch_stride + (size_t)kvh * D;

  unsigned char *ring = atc_smem + (size_t)warp * ATC_STAGES * STAGE;
  const uint32_t ring_u32 = atc_smem_u32(ring);
  const int n_blocks = (k_end > k_begin) ? (k_end - k_begin + 15) / 16 : 0;
  const int my_n = n_blocks > warp ? (n_blocks - warp + ATC_WARPS - 1) / ATC_WARPS : 0;

  auto issue = [&](int i, int stage) {
    const int key0 = k_begin + (warp + i * ATC_WARPS) * 16;
    const uint32_t sK = ring_u32 + stage * STAGE;
#pragma unroll
    for (int c = 0; c < (16 * CH) / 32; c++) {
      const int piece = c * 32 + lane;
      const int key = piece / CH, ch = piece % CH;
      const int kk = key0 + key;
      const bool ok = kk < k_end && kk != new_pos;  // the new token's row is built in place below
      const size_t off = (size_t)(ok ? kk : k_begin) * row_stride + ch * 8;
      const uint32_t dst = sK + key * ROWB + ((ch ^ (key & 7)) << 4);
      atc_cp_async16(dst, kbase + off, ok ? 16 : 0);          // rows past the range are zero filled
      atc_cp_async16(dst + TILE, vbase + off, ok ? 16 : 0);
    }
  };

#pragma unroll
  for (int s = 0; s < ATC_STAGES - 1; s++) {
    if (s < my_n) issue(s, s);
    atc_commit();
  }

  for (int i = 0; i < my_n; i++) {
    __syncwarp();  // every lane has finished reading the stage that is refilled next
    {
      const int nx = i + ATC_STAGES - 1;
      if (nx < my_n) issue(nx, nx % ATC_STAGES);
      atc_commit();
    }
    atc_wait<ATC_STAGES - 1>();
    __syncwarp();
    const int stage = i % ATC_STAGES;
    const uint32_t sK = ring_u32 + stage * STAGE, sV = sK + TILE;
    const int key0 = k_begin + (warp + i * ATC_WARPS) * 16;
    if (fused && new_pos >= key0 && new_pos < key0 + 16 && new_pos < k_end) {
      // This warp's block holds the position of the new token: build its K row (per-head RMSNorm + RoPE,
      // rounded to f16 as the cache write does) and V row, put them into the stage and, once per KV head,
      // append them to the cache (kv_cache_write_f32_to_f16.wgsl:19).
      constexpr int HALF = D / 2, PER = HALF / 32;
      const int heads_all = p.fuse.nh + 2 * p.fuse.nkv;
      const float *ksrc = p.fuse.qkv + ((size_t)b * heads_all + p.fuse.nh + kvh) * D;
      const float *vsrc = ksrc + (size_t)p.fuse.nkv * D;
      float k0[PER], k1[PER], v0[PER], v1[PER];
      float ss = 0.0f;
#pragma unroll
      for (int e = 0; e < PER; e++) {
        k0[e] = ksrc[lane + 32 * e]; k1[e] = ksrc[lane + 32 * e + HALF];
        v0[e] = vsrc[lane + 32 * e]; v1[e] = vsrc[lane + 32 * e + HALF];
        ss = fmaf(k0[e], k0[e], fmaf(k1[e], k1[e], ss));
      }
#pragma unroll
      for (int o2 = 16; o2 > 0; o2 >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o2);
      const float inv = 1.0f / sqrtf(ss / (float)D + p.fuse.eps);
      unsigned char *rowK = ring + (size_t)stage * STAGE + (size_t)(new_pos - key0) * ROWB, *rowV = rowK + TILE;
      const int rsw = (new_pos - key0) & 7;
      __half *kdst = p.fuse.kc + (size_t)b * p.kv_batch_stride + ((size_t)new_pos * p.num_kv_heads + kvh) * D;
      __half *vdst = p.fuse.vc + (size_t)b * p.kv_batch_stride + ((size_t)new_pos * p.num_kv_heads + kvh) * D;
#pragma unroll
      for (int e = 0; e < PER; e++) {
        const int d = lane + 32 * e;
        const float a = k0[e] * inv * p.fuse.k_norm[d], bb = k1[e] * inv * p.fuse.k_norm[d + HALF];
        const float c = p.fuse.cos_t[(size_t)new_pos * HALF + d], sn = p.fuse.sin_t[(size_t)new_pos * HALF + d];
        const __half ka = __float2half_rn(a * c - bb * sn), kb = __float2half_rn(a * sn + bb * c);
        const __half va = __float2half_rn(v0[e]), vb = __float2half_rn(v1[e]);
        const int d2 = d + HALF;
        *reinterpret_cast<__half *>(rowK + ((((d >> 3) ^ rsw)) << 4) + (d & 7) * 2) = ka;
        *reinterpret_cast<__half *>(rowK + ((((d2 >> 3) ^ rsw)) << 4) + (d2 & 7) * 2) = kb;
        *reinterpret_cast<__half *>(rowV + ((((d >> 3) ^ rsw)) << 4) + (d & 7) * 2) = va;
        *reinterpret_cast<__half *>(rowV + ((((d2 >> 3) ^ rsw)) << 4) + (d2 & 7) * 2) = vb;
        if (ht == 0) { kdst[d] = ka; kdst[d2] = kb; vdst[d] = va; vdst[d2] = vb; }
      }
      __syncwarp();
    }

    // ---- scores of 16 keys for head g: s[2nb], s[2nb+1] = keys 8nb+2t, 8nb+2t+1 ----
    float s[4];
#pragma unroll
    for (int nb = 0; nb < 2; nb++) {
      float c0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, c1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      const int key = 8 * nb + (lane & 7);
#pragma unroll
      for (int j = 0; j < KS / 2; j++) {
        uint32_t r[4];
        const int ch = 4 * j + (lane >> 3);
        atc_ldmatrix_x4(r, sK + key * ROWB + ((ch ^ (key & 7)) << 4));
        atc_mma(c0, qa[2 * j], r[0], r[1]);
        atc_mma(c1, qa[2 * j + 1], r[2], r[3]);
      }
      s[2 * nb] = (c0[0] + c1[0]) + (c0[2] + c1[2]);
      s[2 * nb + 1] = (c0[1] + c1[1]) + (c0[3] + c1[3]);
    }
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const int kk = key0 + 8 * (e >> 1) + 2 * t + (e & 1);
      float v = s[e];
      if (capped) v = tanhf(v / p.softcap) * p.softcap * LOG2E;
      s[e] = kk < k_end ? v : -INFINITY;
    }
    // ---- online softmax (the four lanes of a head agree on the maximum) ----
    float mx = fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
    const bool grew = m_new > m_run;
    if (__any_sync(0xffffffffu, grew)) {
      const float alpha = exp2f(m_run - m_use);  // 1 where the maximum stayed, 0 on the first keys
      l_run *= alpha;
      const int hc0 = PLO ? ((2 * t) & 3) : 2 * t;  // head whose column is 2t (columns 4..7 repeat heads 0..3 under PLO)
      const float a0 = __shfl_sync(0xffffffffu, alpha, 4 * hc0);
      const float a1 = __shfl_sync(0xffffffffu, alpha, 4 * (hc0 + 1));
#pragma unroll
      for (int j = 0; j < KS; j++) { o[j][0] *= a0; o[j][1] *= a1; o[j][2] *= a0; o[j][3] *= a1; }
    }
    m_run = m_new;
    float pr[4];
#pragma unroll
    for (int e = 0; e < 4; e++) pr[e] = exp2f(s[e] - m_use);
    l_run += (pr[0] + pr[1]) + (pr[2] + pr[3]);
    // ---- B fragments of P^T: column = head g (hi), under PLO column g+4 = low half of head g ----
    const __half2 ph0 = __floats2half2_rn(pr[0], pr[1]), ph1 = __floats2half2_rn(pr[2], pr[3]);
    uint32_t b0 = atc_pack(ph0), b1 = atc_pack(ph1);
    if (PLO) {
      const float2 f0 = __half22float2(ph0), f1 = __half22float2(ph1);
      const uint32_t l0 = atc_pack(__floats2half2_rn(pr[0] - f0.x, pr[1] - f0.y));
      const uint32_t l1 = atc_pack(__floats2half2_rn(pr[2] - f1.x, pr[3] - f1.y));
      const uint32_t u0 = __shfl_up_sync(0xffffffffu, l0, 16), u1 = __shfl_up_sync(0xffffffffu, l1, 16);
      if (g >= 4) { b0 = u0; b1 = u1; }
    }
    // ---- O^T += V^T P^T ----
#pragma unroll
    for (int j = 0; j < KS; j++) {
      uint32_t a[4];
      const int key = (lane & 7) + 8 * ((lane >> 4) & 1);
      const int ch = 2 * j + ((lane >> 3) & 1);
      atc_ldmatrix_x4_trans(a, sV + key * ROWB + ((ch ^ (key & 7)) << 4));
      atc_mma(o[j], a, b0, b1);
    }
  }
  atc_wait<0>();

  // ---- merge the lanes of a head, then the warps ----
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if (PLO) {
#pragma unroll
    for (int j = 0; j < KS; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) o[j][e] += __shfl_xor_sync(0xffffffffu, o[j][e], 2);  // hi column + lo column
  }
  __syncthreads();  // all rings are idle: reuse them
  float *sm_o = reinterpret_cast<float *>(atc_smem);             // [warp][8][D]
  float *sm_m = sm_o + ATC_WARPS * 8 * D;                         // [warp][8]
  float *sm_l = sm_m + ATC_WARPS * 8;
  if (t == 0) { sm_m[warp * 8 + g] = (m_run == -INFINITY) ? -FLT_MAX : m_run; sm_l[warp * 8 + g] = l_run; }
  if (!PLO || t < 2) {
#pragma unroll
    for (int j = 0; j < KS; j++) {
      float *o0 = sm_o + ((size_t)warp * 8 + 2 * t) * D, *o1 = o0 + D;
      o0[16 * j + g] = o[j][0]; o1[16 * j + g] = o[j][1];
      o0[16 * j + 8 + g] = o[j][2]; o1[16 * j + 8 + g] = o[j][3];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < gt * D; idx += ATC_THREADS) {
    const int hh = idx / D, d = idx % D;
    float mm = -FLT_MAX;
#pragma unroll
    for (int w = 0; w < ATC_WARPS; w++) mm = fmaxf(mm, sm_m[w * 8 + hh]);
    float ll = 0.0f, acc = 0.0f;
#pragma unroll
    for (int w = 0; w < ATC_WARPS; w++) {
      const float ms = sm_m[w * 8 + hh];
      const float c = (ms == -FLT_MAX) ? 0.0f : exp2f(ms - mm);
      ll = fmaf(sm_l[w * 8 + hh], c, ll);
      acc = fmaf(sm_o[((size_t)w * 8 + hh) * D + d], c, acc);
    }
    const int h = h0 + hh;
    if (splits == 1) {
      p.out[((size_t)z * p.num_heads + h) * D + d] = ll > 0.0f ? acc / ll : 0.0f;
    } else {
      float *pp = part + (((size_t)z * p.num_heads + h) * splits + split) * (D + 2);
      pp[d] = acc;
      if (d == 0) { pp[D] = mm; pp[D + 1] = ll; }
    }
  }
}

// Shapes the tensor-core kernel takes: head_dim 64 or 128, GQA groups of up to 8 heads (or a multiple
// of 8), 16-byte aligned rows.  Every query row (decode: one per sequence; prefill: seq_len per
// sequence, each with its own causal limit) is one grid.z slice.
bool dpk_attention_tc_eligible(const dpk_attn_params &p, int *gt_out) {
  if (p.seq_len < 1) return false;
  if (p.head_dim != 128 && p.head_dim != 64) return false;
  if (p.num_kv_heads <= 0 || p.num_heads % p.num_kv_heads) return false;
  const int G = p.num_heads / p.num_kv_heads;
  int gt;
  if (G <= 8) gt = G;
  else if (G % 8 == 0) gt = 8;
  else return false;
  if (p.kv_batch_stride % 8) return false;
  if (((uintptr_t)p.k | (uintptr_t)p.v) & 15) return false;
  if ((uintptr_t)p.q & 7) return false;
  if (gt_out) *gt_out = gt;
  return true;
}

template <int D, bool PLO>
static dp_status launch_tc(dp_ctx *ctx, const dpk_attn_params &p, float *scratch, int splits, int gt) {
  const int G = p.num_heads / p.num_kv_heads;
  const int head_tiles = G / gt;
  const size_t smem = (size_t)ATC_WARPS * ATC_STAGES * 2 * 16 * D * 2;
  DP_CUDA(ctx, cudaFuncSetAttribute(attn_tc_kernel<D, PLO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(splits, p.num_kv_heads * head_tiles, p.batch * p.seq_len);
  DP_LAUNCH(ctx, (attn_tc_kernel<D, PLO>), grid, ATC_THREADS, smem, p, scratch, splits, head_tiles, gt);
  return DP_OK;
}

dp_status dpk_attention_tc_split(dp_ctx *ctx, const dpk_attn_params &p, float *scratch, int splits) {
  int gt = 0;
  if (!dpk_attention_tc_eligible(p, &gt)) return dp_fail(ctx, DP_ERR_UNSUPPORTED, "attention: shape outside the tensor-core decode kernel");
  if (p.head_dim == 128) return gt <= 4 ? launch_tc<128, true>(ctx, p, scratch, splits, gt) : launch_tc<128, false>(ctx, p, scratch, splits, gt);
  return gt <= 4 ? launch_tc<64, true>(ctx, p, scratch, splits, gt) : launch_tc<64, false>(ctx, p, scratch, splits, gt);
}
