// Q4_K decode GEMV, fast path (K % 256 == 0, N % 16 == 0, f32 activations).
//
// Replaces src/gpu/kernels/fused_matmul_q4.wgsl main_gemv (:279) / main_multicol (:122).
//
// The kernel is bound by HBM (0.5625 B per weight), so the goal is to spend as few
// issue slots per weight as possible.  Converting each 4-bit quant to f32 and doing one
// FMA per weight costs ~3 slots per weight, which at full bandwidth is more than the
// SMs have.  Instead the dot product of a 32-weight sub-block with the activations is
// taken EXACTLY in integers:
//   - a small pre-pass turns the f32 activation vector into 24-bit fixed point per
//     256-block (shared power-of-two exponent, error <= 2^-22 of the block's max) and
//     splits every value into three signed 8-bit digits ("limbs");
//   - the nibbles are unpacked four at a time into bytes (one AND per four weights) and
//     fed, with the three limb columns, to the int8 tensor-core MMA m16n8k32
//     (u8 x s8 -> s32): one MMA covers 16 weight rows x one sub-block;
//   - per sub-block the s32 result is multiplied by the 6-bit scale code (integer),
//     summed over the 8 sub-blocks, and only then converted to f32 and multiplied by
//     d * 2^e; the min term uses precomputed per-sub-block activation sums.
// Everything up to the final f32 scaling is exact, so the result differs from the
// double-accumulate oracle only by the activation fixed-point step and a few f32
// roundings per super-block (well inside the 1e-3 gate).
//
// Work split: one CTA = 16 weight rows; its 8 warps take every 8th super-block of K and
// are summed through shared memory.  Thread (g = lane/4, t = lane%4) feeds rows g, g+8:
// it reads 8 bytes of each 32-byte quant chunk, so four threads cover a chunk and a
// warp-wide load touches whole 32-byte sectors.
#include "common.h"
#include "q4k.cuh"

// ---- activation pre-pass -------------------------------------------------------
// layout of the quantised activation buffer for K = 256*bpr:
//   limbs  int8 [K/32][4][32]   column c = digit c (c = 3 is zero), bytes in element order
//   xscale f32  [bpr]           2^(e_b - 22)
//   ssum   f32  [K/32]          sum of the fixed-point integers of each sub-block
__global__ void __launch_bounds__(256) q4k_prep_act_kernel(const float *__restrict__ x, int8_t *__restrict__ limbs,
                                                           float *__restrict__ xscale, float *__restrict__ ssum, int bpr) {
  const int lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * (blockDim.x >> 5);
  for (int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < bpr; b += warps_total) {
    const float4 v0 = *reinterpret_cast<const float4 *>(x + b * QK_K + lane * 8);
    const float4 v1 = *reinterpret_cast<const float4 *>(x + b * QK_K + lane * 8 + 4);
    const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    int e = 0;
    if (amax > 0.0f) frexpf(amax, &e);  // amax < 2^e
    if (e < -100) e = -100;
    const float up = ldexpf(1.0f, 22 - e);
    int q[8], s = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) { q[i] = __float2int_rn(v[i] * up); s += q[i]; }
    uint32_t d[3][2] = {{0, 0}, {0, 0}, {0, 0}};
#pragma unroll
    for (int i = 0; i < 8; i++) {
      int r = q[i];
      const int l0 = ((r + 128) & 255) - 128;
      r = (r - l0) >> 8;
      const int l1 = ((r + 128) & 255) - 128;
      const int l2 = (r - l1) >> 8;
      d[0][i >> 2] |= (uint32_t)(l0 & 255) << (8 * (i & 3));
      d[1][i >> 2] |= (uint32_t)(l1 & 255) << (8 * (i & 3));
      d[2][i >> 2] |= (uint32_t)(l2 & 255) << (8 * (i & 3));
    }
    const int sb = b * 8 + (lane >> 2);
    uint2 *dst = reinterpret_cast<uint2 *>(limbs + (size_t)sb * 128) + (lane & 3);
    dst[0] = make_uint2(d[0][0], d[0][1]);
    dst[4] = make_uint2(d[1][0], d[1][1]);
    dst[8] = make_uint2(d[2][0], d[2][1]);
    dst[12] = make_uint2(0u, 0u);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if ((lane & 3) == 0) ssum[sb] = (float)s;
    float sc = ldexpf(1.0f, e - 22);
    if (!(amax <= 3.0e38f)) sc = __int_as_float(0x7fc00000);  // inf / nan activations poison the block
    if (lane == 0) xscale[b] = sc;
  }
}

__device__ __forceinline__ void mma_u8s8(int &c0, int &c1, int &c2, int &c3, uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
      : "=r"(c0), "=r"(c1), "=r"(c2), "=r"(c3)
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

#define GEMV_WARPS 8

template <typename OutT>
__global__ void __launch_bounds__(GEMV_WARPS * 32) gemv_q4k_mma_kernel(
    const uint8_t *__restrict__ W, const int8_t *__restrict__ limbs, const float *__restrict__ xscale,
    const float *__restrict__ ssum, OutT *__restrict__ y, int N, int bpr, float alpha,
    const float *__restrict__ residual) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * 16;
  const size_t row_bytes = (size_t)bpr * Q4K_BLOCK_BYTES;
  const uint8_t *rowA = W + (size_t)(row0 + g) * row_bytes;
  const uint8_t *rowB = rowA + 8 * row_bytes;
  // weight of this thread's two accumulator columns (column = 2t, 2t+1; digits 0,1,2 live in columns 0,1,2)
  const float w0 = t == 0 ? 1.0f : (t == 1 ? 65536.0f : 0.0f);
  const float w1 = t == 0 ? 256.0f : 0.0f;
  const uint32_t M4 = 0x0f0f0f0fu;
  float resA = 0.0f, resB = 0.0f;

  for (int b = warp; b < bpr; b += GEMV_WARPS) {
    const uint32_t *pa = reinterpret_cast<const uint32_t *>(rowA + (size_t)b * Q4K_BLOCK_BYTES);
    const uint32_t *pb = reinterpret_cast<const uint32_t *>(rowB + (size_t)b * Q4K_BLOCK_BYTES);
    const uint4 ha = __ldg(reinterpret_cast<const uint4 *>(pa));
    const uint4 hb = __ldg(reinterpret_cast<const uint4 *>(pb));
    uint2 qa[4], qb[4];
#pragma unroll
    for (int c = 0; c < 4; c++) {
      qa[c] = __ldg(reinterpret_cast<const uint2 *>(pa + 4 + 8 * c) + t);
      qb[c] = __ldg(reinterpret_cast<const uint2 *>(pb + 4 + 8 * c) + t);
    }
    const Q4KScales sa = q4k_unpack_scales(ha.y, ha.z, ha.w);
    const Q4KScales sb_ = q4k_unpack_scales(hb.y, hb.z, hb.w);
    const uint2 *lb = reinterpret_cast<const uint2 *>(limbs + (size_t)b * 8 * 128) + g * 4 + t;
    int accA0 = 0, accA1 = 0, accB0 = 0, accB1 = 0;
#pragma unroll
    for (int c = 0; c < 4; c++) {
#pragma unroll
      for (int hi = 0; hi < 2; hi++) {
        const int sb = 2 * c + hi;
        uint2 bf = make_uint2(0u, 0u);
        if (g < 3) bf = __ldg(lb + sb * 16);
        const uint32_t a0 = hi ? (qa[c].x >> 4) & M4 : qa[c].x & M4;
        const uint32_t a1 = hi ? (qb[c].x >> 4) & M4 : qb[c].x & M4;
        const uint32_t a2 = hi ? (qa[c].y >> 4) & M4 : qa[c].y & M4;
        const uint32_t a3 = hi ? (qb[c].y >> 4) & M4 : qb[c].y & M4;
        int c0, c1, c2, c3;
        mma_u8s8(c0, c1, c2, c3, a0, a1, a2, a3, bf.x, bf.y);
        const int scA = (int)q4k_byte(sb < 4 ? sa.sc03 : sa.sc47, sb & 3);
        const int scB = (int)q4k_byte(sb < 4 ? sb_.sc03 : sb_.sc47, sb & 3);
        accA0 += scA * c0; accA1 += scA * c1;
        accB0 += scB * c2; accB1 += scB * c3;
      }
    }
    const float xs = __ldg(xscale + b);
    const float2 dA = q4k_d_dmin(ha.x), dB = q4k_d_dmin(hb.x);
    const float fa = fmaf((float)accA1, w1, (float)accA0 * w0);
    const float fb = fmaf((float)accB1, w1, (float)accB0 * w0);
    // min term: thread t covers sub-blocks 2t and 2t+1 of both rows
    const float s0 = __ldg(ssum + b * 8 + 2 * t), s1 = __ldg(ssum + b * 8 + 2 * t + 1);
    const uint32_t mwA = t < 2 ? sa.mn03 : sa.mn47, mwB = t < 2 ? sb_.mn03 : sb_.mn47;
    const int sh = (t & 1) * 16;
    const float mA = fmaf((float)((mwA >> (sh + 8)) & 0xffu), s1, (float)((mwA >> sh) & 0xffu) * s0);
    const float mB = fmaf((float)((mwB >> (sh + 8)) & 0xffu), s1, (float)((mwB >> sh) & 0xffu) * s0);
    resA = fmaf(xs, fmaf(dA.x, fa, -dA.y * mA), resA);
    resB = fmaf(xs, fmaf(dB.x, fb, -dB.y * mB), resB);
  }
  resA += __shfl_xor_sync(0xffffffffu, resA, 1);
  resA += __shfl_xor_sync(0xffffffffu, resA, 2);
  resB += __shfl_xor_sync(0xffffffffu, resB, 1);
  resB += __shfl_xor_sync(0xffffffffu, resB, 2);
  __shared__ float red[GEMV_WARPS][16];
  if (t == 0) { red[warp][g] = resA; red[warp][g + 8] = resB; }
  __syncthreads();
  if (tid < 16) {
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < GEMV_WARPS; w++) v += red[w][tid];
    const int row = row0 + tid;
    v *= alpha;
    if (residual) v += residual[row];
    if constexpr (sizeof(OutT) == 4) y[row] = v; else y[row] = __float2half_rn(v);
  }
}

static size_t actq_bytes(int K) { return (size_t)K * 4 + (size_t)(K / 256) * 4 + (size_t)(K / 32) * 4; }

// quantise x (f32[K]) into `actq` (actq_bytes(K)); exposed to the runner so producers can be fused later
dp_status dpk_q4k_prep_act(dp_ctx *ctx, const float *x, void *actq, int K) {
  const int bpr = K / QK_K;
  int8_t *limbs = (int8_t *)actq;
  float *xscale = (float *)(limbs + (size_t)K * 4);
  float *ssum = xscale + bpr;
  const int grid = (bpr + 7) / 8;
  DP_LAUNCH(ctx, q4k_prep_act_kernel, grid, 256, 0, x, limbs, xscale, ssum, bpr);
  return DP_OK;
}

dp_status dpk_gemv_q4k_actq(dp_ctx *ctx, const uint8_t *W, const void *actq, void *y, dp_dtype y_dtype, int N, int K,
                            float alpha, const float *residual) {
  const int bpr = K / QK_K;
  const int8_t *limbs = (const int8_t *)actq;
  const float *xscale = (const float *)(limbs + (size_t)K * 4);
  const float *ssum = xscale + bpr;
  if (y_dtype == DP_F32) {
    DP_LAUNCH(ctx, gemv_q4k_mma_kernel<float>, N / 16, GEMV_WARPS * 32, 0, W, limbs, xscale, ssum, (float *)y, N, bpr, alpha, residual);
  } else {
    DP_LAUNCH(ctx, gemv_q4k_mma_kernel<__half>, N / 16, GEMV_WARPS * 32, 0, W, limbs, xscale, ssum, (__half *)y, N, bpr, alpha, residual);
  }
  return DP_OK;
}

size_t dpk_q4k_actq_bytes(int K) { return actq_bytes(K); }

bool dpk_gemv_q4k_fast_ok(int N, int K) { return N > 0 && K > 0 && (K % QK_K) == 0 && (N % 16) == 0; }

dp_status dpk_gemv_q4k_fast(dp_ctx *ctx, const uint8_t *W, const float *x, void *y, dp_dtype y_dtype, int N, int K,
                            float alpha, const float *residual, bool *handled) {
  *handled = false;
  if (!dpk_gemv_q4k_fast_ok(N, K) || (y_dtype != DP_F32 && y_dtype != DP_F16)) return DP_OK;
  DP_TRY(dp_scratch(ctx, &ctx->gemv_scratch, actq_bytes(K), "gemv_activation_digits"));
  DP_TRY(dpk_q4k_prep_act(ctx, x, ctx->gemv_scratch->dptr, K));
  DP_TRY(dpk_gemv_q4k_actq(ctx, W, ctx->gemv_scratch->dptr, y, y_dtype, N, K, alpha, residual));
  *handled = true;
  return DP_OK;
}
