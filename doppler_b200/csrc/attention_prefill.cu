// Causal prefill attention over the f16 KV cache, query-tiled (head_dim 128, GQA groups of 1, 2, 4 or 8).
//
// Replaces src/gpu/kernels/attention_streaming_f16kv.wgsl:96 (one thread per (query, head), two passes
// over K) and, in this library, running every query row as its own CTA of the decode kernel, which
// re-read a KV group's keys once per row.  Semantics as tests/kernels/reference/attention.js:129-151:
// key j is visible to the query at absolute position q iff j <= q; scale * q.k, softmax, P.V.
//
// One CTA = one KV head and a tile of QT = 128 / G query positions, G = query heads per KV head: its
// eight warps are (16-row block, head) pairs, so the K / V tiles in shared memory are read from global
// memory once per 128 (query, head) rows instead of once per row.  Keys go through in tiles of 32 in
// a two-stage cp.async ring (rows padded by 16 bytes: conflict-free fragment reads).  Tensor-core math
// with mma.sync m16n8k16 in the flash-attention arrangement: S = Q K^T with Q held in registers as an
// f16 hi half and an f16 lo half (two products, so the f32 query loses nothing that matters), online
// softmax in f32 per 16 x 32 score tile, O += P V with P likewise as f16 hi + lo halves and V fragments
// from ldmatrix.trans.  f32 accumulators; the output is written once, normalised.
#include "common.h"
#include "pdl.cuh"

#include <cfloat>

#define APF_WARPS 8
#define APF_THREADS (APF_WARPS * 32)
#define APF_D 128
#define APF_KT 32                       // keys per tile
#define APF_ROWB (APF_D * 2 + 16)       // bytes per key row in shared memory
#define APF_TILE (APF_KT * APF_ROWB)    // one K (or V) tile
#define APF_STAGE (2 * APF_TILE)        // K tile then V tile

__device__ __forceinline__ void apf_cp_async16(uint32_t dst, const void *src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void apf_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void apf_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
__device__ __forceinline__ void apf_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void apf_ldmatrix_x2_trans(uint32_t &r0, uint32_t &r1, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr) : "memory");
}
__device__ __forceinline__ uint32_t apf_pack(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}

// grid: (query tiles, KV heads, batch); G = num_heads / num_kv_heads in {1, 2, 4, 8}
__global__ void __launch_bounds__(APF_THREADS, 1) attn_prefill_tc_kernel(dpk_attn_params p, int G) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(128) unsigned char apf_smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int QT = 16 * APF_WARPS / G;              // query positions per CTA
  // Causal tiles cost in proportion to their position, and blocks start in index order: hand the tiles out
  // last (longest) first, all KV heads of a tile together, so the short ones fill the tail of the launch.
  const int lin = blockIdx.x + gridDim.x * blockIdx.y;
  const int kvh = lin % p.num_kv_heads, b = blockIdx.z;
  const int qtile = (int)gridDim.x - 1 - lin / p.num_kv_heads;
  const int hh = warp % G, rb = warp / G;         // this warp: head hh of the group, 16-row block rb of the tile
  const int h = kvh * G + hh;
  const int q0 = qtile * QT + rb * 16;       // first query row (within the call) of this warp
  const int rowA = q0 + g, rowB = q0 + g + 8;     // the two query rows this lane's accumulators belong to
  const int posA = p.start_pos + rowA, posB = p.start_pos + rowB;  // their absolute positions
  // keys this CTA needs: up to the position of its last query (and what the cache holds)
  int kv_len = p.kv_lens ? min(max(p.kv_lens[b], 0), p.kv_len) : p.kv_len;
  const int last_q = min(qtile * QT + QT, p.seq_len) - 1;
  const int cta_keys = min(kv_len, p.start_pos + last_q + 1);
  const int warp_keys = min(kv_len, p.start_pos + min(q0 + 15, p.seq_len - 1) + 1);  // beyond this every key is masked for the warp
  const int n_tiles = (cta_keys + APF_KT - 1) / APF_KT;

  const __half *kbase = p.k + (size_t)b * p.kv_batch_stride + (size_t)kvh * APF_D;
  const __half *vbase = p.v + (size_t)b * p.kv_batch_stride + (size_t)kvh * APF_D;
  const size_t key_stride = (size_t)p.num_kv_heads * APF_D;  // elements between consecutive keys
  const uint32_t smem0 = (uint32_t)__cvta_generic_to_shared(apf_smem);

  auto issue_tile = [&](int tile) {
    const int s = tile & 1;
    const int key0 = tile * APF_KT;
    // 32 keys x 16 chunks of 16 bytes, for K and for V: two chunks of each per thread
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const int c = tid + i * APF_THREADS;       // 0 .. 511
      const int key = c >> 4, ch = c & 15;
      const bool ok = key0 + key < cta_keys;
      const size_t off = (size_t)(ok ? key0 + key : 0) * key_stride + (size_t)ch * 8;
      const uint32_t dst = smem0 + (uint32_t)s * APF_STAGE + (uint32_t)key * APF_ROWB + (uint32_t)ch * 16;
      apf_cp_async16(dst, kbase + off, ok ? 16 : 0);            // rows past the range are zero filled
      apf_cp_async16(dst + APF_TILE, vbase + off, ok ? 16 : 0);
    }
    apf_commit();
  };

  // ---- Q fragments (A operand, 16 rows x 128 dims): f16 hi and lo halves of scale * q ----
  const float LOG2E = 1.4426950408889634f;
  const float qmul = p.scale * LOG2E;  // scores in log2 units: softmax with exp2
  uint32_t qh[8][4], ql[8][4];
  {
    const bool okA = rowA < p.seq_len, okB = rowB < p.seq_len;
    const float *qa = p.q + (((size_t)b * p.seq_len + (okA ? rowA : 0)) * p.num_heads + h) * APF_D;
    const float *qb = p.q + (((size_t)b * p.seq_len + (okB ? rowB : 0)) * p.num_heads + h) * APF_D;
#pragma unroll
    for (int ks = 0; ks < 8; ks++) {
      const float2 a0 = okA ? *reinterpret_cast<const float2 *>(qa + 16 * ks + 2 * t) : make_float2(0.f, 0.f);
      const float2 a1 = okB ? *reinterpret_cast<const float2 *>(qb + 16 * ks + 2 * t) : make_float2(0.f, 0.f);
      const float2 a2 = okA ? *reinterpret_cast<const float2 *>(qa + 16 * ks + 2 * t + 8) : make_float2(0.f, 0.f);
      const float2 a3 = okB ? *reinterpret_cast<const float2 *>(qb + 16 * ks + 2 * t + 8) : make_float2(0.f, 0.f);
      const float x[8] = {a0.x * qmul, a0.y * qmul, a1.x * qmul, a1.y * qmul, a2.x * qmul, a2.y * qmul, a3.x * qmul, a3.y * qmul};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const __half2 hi = __floats2half2_rn(x[2 * j], x[2 * j + 1]);
        const float2 hf = __half22float2(hi);
        qh[ks][j] = *reinterpret_cast<const uint32_t *>(&hi);
        ql[ks][j] = apf_pack(x[2 * j] - hf.x, x[2 * j + 1] - hf.y);
      }
    }
  }

  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; j++) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
  float mA = -INFINITY, mB = -INFINITY, lA = 0.0f, lB = 0.0f;  // running max (log2 units) and this lane's share of the running sum

  if (n_tiles > 0) issue_tile(0);
  for (int tile = 0; tile < n_tiles; tile++) {
    if (tile + 1 < n_tiles) { issue_tile(tile + 1); apf_wait<1>(); } else { apf_wait<0>(); }
    __syncthreads();
    const int key0 = tile * APF_KT;
    if (key0 < warp_keys) {  // (warp-uniform) later tiles are masked for all of this warp's rows
      const unsigned char *sK = apf_smem + (tile & 1) * APF_STAGE;
      const uint32_t sV = smem0 + (uint32_t)(tile & 1) * APF_STAGE + APF_TILE;
      // ---- S = (scale * Q) K^T for 16 rows x 32 keys ----
      float sc[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; nt++) { sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.0f; }
#pragma unroll
      for (int ks = 0; ks < 8; ks++) {
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
          const unsigned char *kr = sK + (nt * 8 + g) * APF_ROWB + (16 * ks + 2 * t) * 2;
          const uint32_t b0 = *reinterpret_cast<const uint32_t *>(kr), b1 = *reinterpret_cast<const uint32_t *>(kr + 16);
          apf_mma(sc[nt], qh[ks], b0, b1);
          apf_mma(sc[nt], ql[ks], b0, b1);
        }
      }
      // ---- causal mask, online softmax ----
      float tmA = -INFINITY, tmB = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 4; nt++) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const int key = key0 + nt * 8 + 2 * t + (e & 1);
          const int pos = e < 2 ? posA : posB;
          if (key > pos || key >= kv_len) sc[nt][e] = -INFINITY;
        }
        tmA = fmaxf(tmA, fmaxf(sc[nt][0], sc[nt][1]));
        tmB = fmaxf(tmB, fmaxf(sc[nt][2], sc[nt][3]));
      }
      tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 1)); tmA = fmaxf(tmA, __shfl_xor_sync(0xffffffffu, tmA, 2));
      tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 1)); tmB = fmaxf(tmB, __shfl_xor_sync(0xffffffffu, tmB, 2));
      const float nmA = fmaxf(mA, tmA), nmB = fmaxf(mB, tmB);
      const float uA = nmA == -INFINITY ? 0.0f : nmA, uB = nmB == -INFINITY ? 0.0f : nmB;  // a row with nothing visible yet
      const float cA = exp2f(mA - uA), cB = exp2f(mB - uB);  // exp2(-inf) = 0 on the first visible tile
      mA = nmA; mB = nmB;
      float sA = 0.0f, sB = 0.0f;
#pragma unroll
      for (int nt = 0; nt < 4; nt++) {
        sc[nt][0] = exp2f(sc[nt][0] - uA); sc[nt][1] = exp2f(sc[nt][1] - uA);
        sc[nt][2] = exp2f(sc[nt][2] - uB); sc[nt][3] = exp2f(sc[nt][3] - uB);
        sA += sc[nt][0] + sc[nt][1];
        sB += sc[nt][2] + sc[nt][3];
      }
      lA = lA * cA + sA;
      lB = lB * cB + sB;
#pragma unroll
      for (int j = 0; j < 16; j++) { o[j][0] *= cA; o[j][1] *= cA; o[j][2] *= cB; o[j][3] *= cB; }
      // ---- O += P V: P (16 x 32) as two A fragments, V fragments transposed out of shared memory ----
#pragma unroll
      for (int kk = 0; kk < 2; kk++) {
        uint32_t pa[4], pl[4];  // P as an f16 hi half and an f16 lo half: rounding P to f16 alone costs ~5e-4 of a row's largest term
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const float x0 = sc[2 * kk + (i >> 1)][2 * (i & 1)], x1 = sc[2 * kk + (i >> 1)][2 * (i & 1) + 1];
          const __half2 hi = __floats2half2_rn(x0, x1);
          const float2 hf = __half22float2(hi);
          pa[i] = *reinterpret_cast<const uint32_t *>(&hi);
          pl[i] = apf_pack(x0 - hf.x, x1 - hf.y);
        }
        const uint32_t vrow = sV + (uint32_t)(16 * kk + (lane & 15)) * APF_ROWB;
#pragma unroll
        for (int j = 0; j < 16; j++) {
          uint32_t b0, b1;
          apf_ldmatrix_x2_trans(b0, b1, vrow + (uint32_t)j * 16u);
          apf_mma(o[j], pa, b0, b1);
          apf_mma(o[j], pl, b0, b1);
        }
      }
    }
    __syncthreads();  // every warp is done with this stage before the tile after next overwrites it
  }
  // ---- normalise and store ----
  lA += __shfl_xor_sync(0xffffffffu, lA, 1); lA += __shfl_xor_sync(0xffffffffu, lA, 2);
  lB += __shfl_xor_sync(0xffffffffu, lB, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 2);
  const float iA = lA > 0.0f ? 1.0f / lA : 0.0f, iB = lB > 0.0f ? 1.0f / lB : 0.0f;
  if (rowA < p.seq_len) {
    float *dst = p.out + (((size_t)b * p.seq_len + rowA) * p.num_heads + h) * APF_D + 2 * t;
#pragma unroll
    for (int j = 0; j < 16; j++) *reinterpret_cast<float2 *>(dst + 8 * j) = make_float2(o[j][0] * iA, o[j][1] * iA);
  }
  if (rowB < p.seq_len) {
    float *dst = p.out + (((size_t)b * p.seq_len + rowB) * p.num_heads + h) * APF_D + 2 * t;
#pragma unroll
    for (int j = 0; j < 16; j++) *reinterpret_cast<float2 *>(dst + 8 * j) = make_float2(o[j][2] * iB, o[j][3] * iB);
  }
}

// Shapes this kernel takes: seq_len > 1, causal, head_dim 128, groups of 1 / 2 / 4 / 8 query heads per KV head,
// no sliding window / softcap / kv_start, 16-byte aligned K and V rows.
bool dpk_attention_prefill_eligible(const dpk_attn_params &p) {
  if (p.seq_len < 2 || !p.causal || p.head_dim != APF_D || p.fuse.qkv) return false;
  if (p.num_kv_heads <= 0 || p.num_heads % p.num_kv_heads) return false;
  const int G = p.num_heads / p.num_kv_heads;
  if (G != 1 && G != 2 && G != 4 && G != 8) return false;
  if (p.sliding_window > 0 || p.softcap > 0.0f || p.kv_start != 0) return false;
  if (p.kv_batch_stride % 8 || (((uintptr_t)p.k | (uintptr_t)p.v) & 15) || ((uintptr_t)p.q & 7) || ((uintptr_t)p.out & 7)) return false;
  return true;
}

dp_status dpk_attention_prefill(dp_ctx *ctx, const dpk_attn_params &p) {
  const int G = p.num_heads / p.num_kv_heads;
  const int QT = 16 * APF_WARPS / G;
  const size_t smem = 2 * APF_STAGE;
  static dp_per_device_once attr;
  if (attr.pending(ctx->device)) {
    DP_CUDA(ctx, cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr.done(ctx->device);
  }
  dim3 grid((p.seq_len + QT - 1) / QT, p.num_kv_heads, p.batch);
  DP_LAUNCH(ctx, attn_prefill_tc_kernel, grid, APF_THREADS, smem, p, G);
  return DP_OK;
}
