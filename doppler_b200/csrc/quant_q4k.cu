// f32 -> Q4_K quantisation on the device.
//
// Bit-exact restatement of the reference converter (src/converter/quantizer.js:78-166,
// quantizeQ4KBlockWithValidLength; row-wise driver :253-288, flat driver :223-251).  The
// reference computes in JavaScript doubles with Float32Array stores in between, so the kernel
// does the same: sub-block ranges and reciprocals in f64, scales / minima rounded to f32 where the
// reference stores them in a Float32Array, Math.round (halves toward +infinity), the truncating
// f32 -> f16 conversion of the converter (:15-46).  None of the f64 operations may be contracted
// into an FMA, hence the explicit __dmul_rn / __dsub_rn.
//
// One warp quantises one super-block: lane l owns elements 8l..8l+7, the four lanes l>>2 == s
// form sub-block s.  HBM traffic is 4 B in and 0.5625 B out per weight.
#include "common.h"
#include "pdl.cuh"
#include "q4k.cuh"

#include <cmath>

__device__ __forceinline__ double js_round(double x) {  // Math.round
  double r = floor(x);
  if (__dsub_rn(x, r) >= 0.5) r += 1.0;
  return r;
}

// src/converter/quantizer.js:15-46: truncates the mantissa, flushes f32 subnormals to zero
__device__ __forceinline__ uint32_t f32_to_f16_trunc(double value) {
  const uint32_t f = __float_as_uint((float)value);
  const uint32_t sign = (f >> 31) & 1u;
  int exp = (int)((f >> 23) & 0xffu);
  uint32_t frac = f & 0x7fffffu;
  if (exp == 0xff) return (sign << 15) | 0x7c00u | (frac ? 0x200u : 0u);
  if (exp == 0) return sign << 15;
  exp = exp - 127 + 15;
  if (exp >= 31) return (sign << 15) | 0x7c00u;
  if (exp <= 0) {
    if (exp < -10) return sign << 15;
    frac = (frac | 0x800000u) >> (1 - exp);
    return (sign << 15) | (frac >> 13);
  }
  return (sign << 15) | ((uint32_t)exp << 10) | (frac >> 13);
}

// full_pad = 1: a short tail is zero padded and quantised as a full block (flat driver);
// full_pad = 0: only the valid elements of the row's last block enter the ranges (row-wise driver).
__global__ void __launch_bounds__(256) quantize_q4k_kernel(const float *__restrict__ data, uint8_t *__restrict__ out, size_t rows,
                                                           size_t cols, size_t bpr, int full_pad) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const size_t warp0 = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const size_t nwarps = (size_t)gridDim.x * (blockDim.x >> 5);
  const size_t total = rows * bpr;
  for (size_t blk = warp0; blk < total; blk += nwarps) {
    const size_t r = blk / bpr, b = blk - r * bpr;
    const size_t col0 = b * QK_K;
    const int have = (int)((cols - col0) < (size_t)QK_K ? (cols - col0) : (size_t)QK_K);  // elements that exist
    const int valid = full_pad ? QK_K : have;                                              // elements that count
    const float *src = data + r * cols + col0;
    float v[8];
    float mn = INFINITY, mx = -INFINITY;
    int n_valid = 0;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int e = lane * 8 + j;
      v[j] = e < have ? src[e] : 0.0f;
      if (e < valid) { mn = fminf(mn, v[j]); mx = fmaxf(mx, v[j]); n_valid++; }
    }
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      n_valid += __shfl_xor_sync(0xffffffffu, n_valid, o);
    }
    float scale = 0.0f, min_off = 0.0f;
    double inv_scale = 0.0;
    if (n_valid > 0) {
      min_off = -mn;
      const double range = __dsub_rn((double)mx, (double)mn);
      scale = (float)(range > 0.0 ? range / 15.0 : 0.0);
      inv_scale = scale > 0.0f ? 1.0 / (double)scale : 0.0;
    }
    uint32_t q[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int e = lane * 8 + j;
      double qq = 0.0;
      if (e < valid) {
        qq = js_round(__dmul_rn(__dsub_rn((double)v[j], (double)mn), inv_scale));
        qq = qq < 0.0 ? 0.0 : (qq > 15.0 ? 15.0 : qq);
      }
      q[j] = (uint32_t)qq;
    }
    // block-wide maxima (initial value 0, as in the reference)
    float max_scale = scale, max_min = fmaxf(min_off, 0.0f);
#pragma unroll
    for (int o = 4; o <= 16; o <<= 1) {
      max_scale = fmaxf(max_scale, __shfl_xor_sync(0xffffffffu, max_scale, o));
      max_min = fmaxf(max_min, __shfl_xor_sync(0xffffffffu, max_min, o));
    }
    const double d = (double)max_scale / 63.0, dmin = (double)max_min / 63.0;
    const double inv_d = d > 0.0 ? 1.0 / d : 0.0, inv_dmin = dmin > 0.0 ? 1.0 / dmin : 0.0;
    const double s_code = js_round(__dmul_rn((double)scale, inv_d));
    const double mo = min_off > 0.0f ? (double)min_off : 0.0;
    const double m_code = js_round(__dmul_rn(mo, inv_dmin));
    const uint32_t sc = (uint32_t)(s_code < 63.0 ? s_code : 63.0), mb = (uint32_t)(m_code < 63.0 ? m_code : 63.0);
    uint32_t scs[8], mbs[8];
#pragma unroll
    for (int i = 0; i < 8; i++) { scs[i] = __shfl_sync(0xffffffffu, sc, 4 * i); mbs[i] = __shfl_sync(0xffffffffu, mb, 4 * i); }
    // quants: even sub-blocks are the low nibbles, the next sub-block (four lanes up) the high ones
    const uint32_t lo_x = q[0] | (q[1] << 8) | (q[2] << 16) | (q[3] << 24), lo_y = q[4] | (q[5] << 8) | (q[6] << 16) | (q[7] << 24);
    const uint32_t hi_x = __shfl_down_sync(0xffffffffu, lo_x, 4), hi_y = __shfl_down_sync(0xffffffffu, lo_y, 4);
    uint8_t *dst = out + blk * Q4K_BLOCK_BYTES;
    const int sb = lane >> 2;
    if ((sb & 1) == 0)
      *reinterpret_cast<uint2 *>(dst + 16 + 32 * (sb >> 1) + 8 * (lane & 3)) = make_uint2(lo_x | (hi_x << 4), lo_y | (hi_y << 4));
    if (lane == 0) {
      uint32_t w[4] = {f32_to_f16_trunc(d) | (f32_to_f16_trunc(dmin) << 16), 0u, 0u, 0u};
#pragma unroll
      for (int i = 0; i < 4; i++) {
        w[1] |= ((scs[i] & 0x3fu) | (((scs[i + 4] >> 4) & 3u) << 6)) << (8 * i);
        w[2] |= ((mbs[i] & 0x3fu) | (((mbs[i + 4] >> 4) & 3u) << 6)) << (8 * i);
        w[3] |= ((scs[i + 4] & 0x0fu) | ((mbs[i + 4] & 0x0fu) << 4)) << (8 * i);
      }
      *reinterpret_cast<uint4 *>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

dp_status dpk_quantize_q4k(dp_ctx *ctx, const float *data, uint8_t *out, size_t rows, size_t cols, bool full_pad) {
  const size_t bpr = dp_cdiv(cols, (size_t)QK_K);
  const size_t total = rows * bpr;
  if (total == 0) return DP_OK;
  size_t grid = dp_cdiv(total, (size_t)8);
  const size_t cap = (size_t)ctx->sm_count * 16;
  if (grid > cap) grid = cap;
  DP_LAUNCH(ctx, quantize_q4k_kernel, (unsigned)grid, 256, 0, data, out, rows, cols, bpr, full_pad ? 1 : 0);
  return DP_OK;
}
