// Standalone Q4_K -> f32/f16 dequantisation.
//
// Replaces src/gpu/kernels/dequant_shared.wgsl:86-145 (one workgroup per
// super-block) and its rowwise wrapper (src/gpu/kernels/dequant.js:162).  Pure
// bandwidth: 0.5625 B in, 4 B (or 2 B) out per weight.  One warp handles one
// super-block: lane l reads word l of the 32 quant words and writes two 16-byte
// runs, so both the loads and the stores of a warp are contiguous.
//
// w = fma(d*sc, q, -(dmin*m)) rounds the exact value once, which is the same
// f32 as the reference CPU dequantizer produces (d*sc and dmin*m are exact in
// f32, and so is (d*sc)*q).
#include "common.h"
#include "pdl.cuh"
#include "q4k.cuh"

template <typename OutT>
__device__ __forceinline__ void store4(OutT *p, float a, float b, float c, float d, bool vec);

template <>
__device__ __forceinline__ void store4<float>(float *p, float a, float b, float c, float d, bool vec) {
  if (vec) *reinterpret_cast<float4 *>(p) = make_float4(a, b, c, d);
  else { p[0] = a; p[1] = b; p[2] = c; p[3] = d; }
}
template <>
__device__ __forceinline__ void store4<__half>(__half *p, float a, float b, float c, float d, bool vec) {
  __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
  if (vec) {
    uint2 v;
    v.x = *reinterpret_cast<uint32_t *>(&lo);
    v.y = *reinterpret_cast<uint32_t *>(&hi);
    *reinterpret_cast<uint2 *>(p) = v;
  } else {
    p[0] = __low2half(lo); p[1] = __high2half(lo); p[2] = __low2half(hi); p[3] = __high2half(hi);
  }
}

template <typename OutT>
__global__ void __launch_bounds__(256) dequant_q4k_kernel(const uint32_t *__restrict__ packed, OutT *__restrict__ out,
                                                          size_t total_blocks, uint32_t bpr, uint32_t K) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const size_t warp0 = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const size_t nwarps = (size_t)gridDim.x * (blockDim.x >> 5);
  const bool full = (K % QK_K) == 0;  // rows pack back to back: vector stores are aligned
  for (size_t blk = warp0; blk < total_blocks; blk += nwarps) {
    const uint32_t *b = packed + blk * Q4K_BLOCK_WORDS;
    // header words broadcast to the warp
    uint32_t h = (lane < 4) ? __ldg(b + lane) : 0u;
    uint32_t w0 = __shfl_sync(0xffffffffu, h, 0), u0 = __shfl_sync(0xffffffffu, h, 1);
    uint32_t u1 = __shfl_sync(0xffffffffu, h, 2), u2 = __shfl_sync(0xffffffffu, h, 3);
    uint32_t q = __ldg(b + 4 + lane);
    float2 dd = q4k_d_dmin(w0);
    Q4KScales s = q4k_unpack_scales(u0, u1, u2);
    const int chunk = lane >> 3, j = lane & 7;
    float sc_lo = __fmul_rn(dd.x, (float)q4k_sc(s, 2 * chunk));
    float sc_hi = __fmul_rn(dd.x, (float)q4k_sc(s, 2 * chunk + 1));
    float mn_lo = __fmul_rn(dd.y, (float)q4k_mn(s, 2 * chunk));
    float mn_hi = __fmul_rn(dd.y, (float)q4k_mn(s, 2 * chunk + 1));
    float lo[4], hi[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      uint32_t byte = (q >> (8 * i)) & 0xffu;
      lo[i] = __fmaf_rn(sc_lo, (float)(byte & 15u), -mn_lo);
      hi[i] = __fmaf_rn(sc_hi, (float)(byte >> 4), -mn_hi);
    }
    const size_t row = blk / bpr;
    const uint32_t bir = (uint32_t)(blk - row * bpr);
    const uint32_t e_lo = bir * QK_K + chunk * 64 + j * 4, e_hi = e_lo + 32;
    OutT *orow = out + row * (size_t)K;
    if (full) {
      store4<OutT>(orow + e_lo, lo[0], lo[1], lo[2], lo[3], true);
      store4<OutT>(orow + e_hi, hi[0], hi[1], hi[2], hi[3], true);
    } else {
#pragma unroll
      for (int i = 0; i < 4; i++) {
        if (e_lo + i < K) { float v = lo[i]; if constexpr (sizeof(OutT) == 4) orow[e_lo + i] = v; else orow[e_lo + i] = __float2half_rn(v); }
        if (e_hi + i < K) { float v = hi[i]; if constexpr (sizeof(OutT) == 4) orow[e_hi + i] = v; else orow[e_hi + i] = __float2half_rn(v); }
      }
    }
  }
}

dp_status dpk_dequant_q4k(dp_ctx *ctx, const uint8_t *packed, size_t rows, size_t bpr, size_t K,
                          void *out, dp_dtype out_dtype) {
  size_t total = rows * bpr;
  if (total == 0) return DP_OK;
  const int threads = 256, wpb = threads / 32;
  size_t want = dp_cdiv(total, wpb);
  size_t cap = (size_t)ctx->sm_count * 16;
  unsigned grid = (unsigned)(want < cap ? want : cap);
  if (out_dtype == DP_F32) {
    DP_LAUNCH(ctx, dequant_q4k_kernel<float>, grid, threads, 0, (const uint32_t *)packed, (float *)out, total,
              (uint32_t)bpr, (uint32_t)K);
  } else if (out_dtype == DP_F16) {
    DP_LAUNCH(ctx, dequant_q4k_kernel<__half>, grid, threads, 0, (const uint32_t *)packed, (__half *)out, total,
              (uint32_t)bpr, (uint32_t)K);
  } else {
    return dp_fail(ctx, DP_ERR_INVALID, "dequantize: outputDtype must be f32 or f16, got %s", dp_dtype_name(out_dtype));
  }
  return DP_OK;
}
