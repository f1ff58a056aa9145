// CUDA-core matmul kernels: the general Q4_K decode GEMV, a tiled Q4_K GEMM
// that keeps f32-exact weights, and the f16/f32-weight GEMV used for the LM head.
//
// Replaces src/gpu/kernels/fused_matmul_q4.wgsl (main_gemv :279, main_multicol
// :122), fused_matmul_q4_batched*.wgsl (:122) and matmul_gemv_subgroup.wgsl.
#include "common.h"
#include "pdl.cuh"
#include "q4k.cuh"

// ---------------------------------------------------------------------------
// Q4_K GEMV, any N and K (K tails are zero-padded in shared memory).
//
// One warp per output row, eight lanes per super-block: lane j reads word j of
// each of the four 32-byte quant chunks, so a warp's loads cover whole 32-byte
// sectors and its shared-memory reads of x are conflict free.  Per sub-block
//   sum_k x_k (s q_k - m) = s * sum_k x_k q_k - m * sum_k x_k
// and the second sum is precomputed once per CTA (xsum), so the inner loop is
// one FMA per weight plus the nibble unpack.  Accumulation is f32.
// ---------------------------------------------------------------------------
template <typename AT>
__device__ __forceinline__ float load_act(const AT *p, size_t i);
template <>
__device__ __forceinline__ float load_act<float>(const float *p, size_t i) { return __ldg(p + i); }
template <>
__device__ __forceinline__ float load_act<__half>(const __half *p, size_t i) { return __half2float(__ldg(p + i)); }

__device__ __forceinline__ float dot4_nibbles(uint32_t qlo, const float4 &xv) {
  // qlo holds four nibbles in the low half of each byte
  float a = q4k_u8_to_float(qlo & 0xffu) * xv.x;
  a = fmaf(q4k_u8_to_float((qlo >> 8) & 0xffu), xv.y, a);
  a = fmaf(q4k_u8_to_float((qlo >> 16) & 0xffu), xv.z, a);
  a = fmaf(q4k_u8_to_float(qlo >> 24), xv.w, a);
  return a;
}

template <typename OutT>
__global__ void __launch_bounds__(256) gemv_q4k_kernel(const uint8_t *__restrict__ W, const float *__restrict__ x,
                                                       OutT *__restrict__ y, int N, int K, int bpr, float alpha,
                                                       const float *__restrict__ residual) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float smem[];
  float *xs = smem;                  // [bpr*256], zero beyond K
  float *xsum = smem + bpr * QK_K;   // [bpr*8] sum of x over each 32-element sub-block
  const int tid = threadIdx.x;
  for (int i = tid; i < bpr * QK_K; i += blockDim.x) xs[i] = i < K ? __ldg(x + i) : 0.0f;
  __syncthreads();
  for (int g = tid; g < bpr * 8; g += blockDim.x) {
    float s = 0;
#pragma unroll 8
    for (int i = 0; i < 32; i++) s += xs[g * 32 + ((i + tid) & 31)];
    xsum[g] = s;
  }
  __syncthreads();

  const int lane = tid & 31, j = lane & 7, sub = lane >> 3;
  const int warps = blockDim.x >> 5;
  for (int row = blockIdx.x * warps + (tid >> 5); row < N; row += gridDim.x * warps) {
    const uint32_t *wrow = reinterpret_cast<const uint32_t *>(W + (size_t)row * bpr * Q4K_BLOCK_BYTES);
    float acc = 0.0f;
#pragma unroll 2
    for (int b = sub; b < bpr; b += 4) {
      const uint32_t *blk = wrow + b * Q4K_BLOCK_WORDS;
      const uint4 hdr = __ldg(reinterpret_cast<const uint4 *>(blk));
      uint32_t q[4];
#pragma unroll
      for (int c = 0; c < 4; c++) q[c] = __ldg(blk + 4 + 8 * c + j);
      const float2 dd = q4k_d_dmin(hdr.x);
      const Q4KScales s = q4k_unpack_scales(hdr.y, hdr.z, hdr.w);
      const float *xb = xs + b * QK_K + 4 * j;
      float blk_sum = 0.0f;
#pragma unroll
      for (int c = 0; c < 4; c++) {
        const float4 xlo = *reinterpret_cast<const float4 *>(xb + 64 * c);
        const float4 xhi = *reinterpret_cast<const float4 *>(xb + 64 * c + 32);
        const float dlo = dot4_nibbles(q[c] & 0x0f0f0f0fu, xlo);
        const float dhi = dot4_nibbles((q[c] >> 4) & 0x0f0f0f0fu, xhi);
        blk_sum = fmaf(q4k_u8_to_float(q4k_byte(c < 2 ? s.sc03 : s.sc47, (2 * c) & 3)), dlo, blk_sum);
        blk_sum = fmaf(q4k_u8_to_float(q4k_byte(c < 2 ? s.sc03 : s.sc47, (2 * c + 1) & 3)), dhi, blk_sum);
      }
      // lane j also owns the min term of sub-block j
      const float mn = q4k_u8_to_float(q4k_byte(j < 4 ? s.mn03 : s.mn47, j & 3));
      acc = fmaf(dd.x, blk_sum, acc);
      acc = fmaf(-dd.y * mn, xsum[b * 8 + j], acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
      float v = acc * alpha;
      if (residual) v += residual[row];
      if constexpr (sizeof(OutT) == 4) y[row] = v; else y[row] = __float2half_rn(v);
    }
  }
}

dp_status dpk_gemv_q4k(dp_ctx *ctx, const uint8_t *W, const float *x, void *y, dp_dtype y_dtype, int N, int K,
                       float alpha, const float *residual) {
  const int bpr = (K + QK_K - 1) / QK_K;
  const size_t smem = (size_t)bpr * (QK_K + 8) * sizeof(float);
  if (smem > ctx->smem_optin)
    return dp_fail(ctx, DP_ERR_UNSUPPORTED, "matmul q4k gemv: K=%d needs %zu bytes of shared memory (max %zu)", K, smem,
                   ctx->smem_optin);
  const int threads = 256, warps = threads / 32;
  int ctas_per_sm = smem > 0 ? (int)((200 * 1024) / (smem + 1024)) : 8;
  if (ctas_per_sm < 1) ctas_per_sm = 1;
  if (ctas_per_sm > 8) ctas_per_sm = 8;
  int grid = (N + warps - 1) / warps;
  if (grid > ctx->sm_count * ctas_per_sm) grid = ctx->sm_count * ctas_per_sm;
  if (y_dtype == DP_F32) {
    if (smem > 48 * 1024) DP_CUDA(ctx, cudaFuncSetAttribute(gemv_q4k_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    DP_LAUNCH(ctx, gemv_q4k_kernel<float>, grid, threads, smem, W, x, (float *)y, N, K, bpr, alpha, residual);
  } else {
    if (smem > 48 * 1024) DP_CUDA(ctx, cudaFuncSetAttribute(gemv_q4k_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    DP_LAUNCH(ctx, gemv_q4k_kernel<__half>, grid, threads, smem, W, x, (__half *)y, N, K, bpr, alpha, residual);
  }
  return DP_OK;
}

// ---------------------------------------------------------------------------
// Q4_K GEMM with f32-exact weights on the CUDA cores (any M, N, K).  64x64
// output tile, one 32-wide sub-block of K per step, 4x4 outputs per thread.
// This is the exact-weight path; the tensor-core path lives in gemm_q4k_tc.cu.
// ---------------------------------------------------------------------------
template <typename AT, typename OutT>
__global__ void __launch_bounds__(256) gemm_q4k_simt_kernel(const uint8_t *__restrict__ W, const AT *__restrict__ A,
                                                            OutT *__restrict__ C, int M, int N, int K, int bpr,
                                                            float alpha) {
  pdl_launch();
  pdl_wait();
  __shared__ float As[32][64 + 4];  // [k][m]
  __shared__ float Ws[32][64 + 4];  // [k][n]
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * 64, m0 = blockIdx.y * 64;
  const int tn = tid & 15, tm = tid >> 4;  // outputs (m0+tm*4.., n0+tn*4..)
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int jx = 0; jx < 4; jx++) acc[i][jx] = 0.0f;

  const int wr = tid >> 2, part = tid & 3;  // dequant role: weight row n0+wr, 8 k's at part*8
  const int ar = tid >> 2, ak = (tid & 3) * 8;  // A role: row m0+ar, 8 k's at ak
  for (int kb = 0; kb < bpr * 8; kb++) {  // sub-block index along K
    const int b = kb >> 3, sbk = kb & 7;
    // A tile
    {
      const int m = m0 + ar;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const int k = kb * 32 + ak + i;
        float v = 0.0f;
        if (m < M && k < K) v = load_act<AT>(A, (size_t)m * K + k);
        As[ak + i][ar] = v;
      }
    }
    // W tile: dequantise 8 weights of sub-block sbk
    {
      const int n = n0 + wr;
      float wv[8];
      if (n < N) {
        const uint32_t *blk = reinterpret_cast<const uint32_t *>(W + ((size_t)n * bpr + b) * Q4K_BLOCK_BYTES);
        const uint4 hdr = __ldg(reinterpret_cast<const uint4 *>(blk));
        const float2 dd = q4k_d_dmin(hdr.x);
        const Q4KScales s = q4k_unpack_scales(hdr.y, hdr.z, hdr.w);
        const float sc = __fmul_rn(dd.x, (float)q4k_sc(s, sbk));
        const float mn = __fmul_rn(dd.y, (float)q4k_mn(s, sbk));
        const int chunk = sbk >> 1, hi = sbk & 1;
        const uint32_t q0 = __ldg(blk + 4 + chunk * 8 + part * 2), q1 = __ldg(blk + 4 + chunk * 8 + part * 2 + 1);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const uint32_t word = i < 4 ? q0 : q1;
          const uint32_t byte = (word >> (8 * (i & 3))) & 0xffu;
          const uint32_t nib = hi ? (byte >> 4) : (byte & 15u);
          wv[i] = __fmaf_rn(sc, (float)nib, -mn);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; i++) wv[i] = 0.0f;
      }
#pragma unroll
      for (int i = 0; i < 8; i++) Ws[part * 8 + i][wr] = wv[i];
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < 32; k++) {
      const float4 a4 = *reinterpret_cast<const float4 *>(&As[k][tm * 4]);
      const float4 w4 = *reinterpret_cast<const float4 *>(&Ws[k][tn * 4]);
      const float av[4] = {a4.x, a4.y, a4.z, a4.w}, wv4[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int jx = 0; jx < 4; jx++) acc[i][jx] = fmaf(av[i], wv4[jx], acc[i][jx]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + tm * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int jx = 0; jx < 4; jx++) {
      const int n = n0 + tn * 4 + jx;
      if (n >= N) continue;
      const float v = acc[i][jx] * alpha;
      if constexpr (sizeof(OutT) == 4) C[(size_t)m * N + n] = v; else C[(size_t)m * N + n] = __float2half_rn(v);
    }
  }
}

dp_status dpk_gemm_q4k_simt(dp_ctx *ctx, const uint8_t *W, const void *A, dp_dtype a_dtype, void *C, dp_dtype c_dtype,
                            int M, int N, int K, float alpha) {
  const int bpr = (K + QK_K - 1) / QK_K;
  dim3 grid((N + 63) / 64, (M + 63) / 64);
  if (a_dtype == DP_F32 && c_dtype == DP_F32) {
    DP_LAUNCH(ctx, (gemm_q4k_simt_kernel<float, float>), grid, 256, 0, W, (const float *)A, (float *)C, M, N, K, bpr, alpha);
  } else if (a_dtype == DP_F32 && c_dtype == DP_F16) {
    DP_LAUNCH(ctx, (gemm_q4k_simt_kernel<float, __half>), grid, 256, 0, W, (const float *)A, (__half *)C, M, N, K, bpr, alpha);
  } else if (a_dtype == DP_F16 && c_dtype == DP_F32) {
    DP_LAUNCH(ctx, (gemm_q4k_simt_kernel<__half, float>), grid, 256, 0, W, (const __half *)A, (float *)C, M, N, K, bpr, alpha);
  } else if (a_dtype == DP_F16 && c_dtype == DP_F16) {
    DP_LAUNCH(ctx, (gemm_q4k_simt_kernel<__half, __half>), grid, 256, 0, W, (const __half *)A, (__half *)C, M, N, K, bpr, alpha);
  } else {
    return dp_fail(ctx, DP_ERR_INVALID, "matmul q4k: unsupported dtypes A=%s C=%s", dp_dtype_name(a_dtype), dp_dtype_name(c_dtype));
  }
  return DP_OK;
}

// ---------------------------------------------------------------------------
// Dense-weight GEMV (f16 weights: LM head / embeddings on 'ehf16' models).
// One warp per weight row, up to MT activation rows per pass; the weight row is
// streamed with 16-byte loads and reused for all MT rows.
// ---------------------------------------------------------------------------
template <typename AT, typename OutT, int MT>
__global__ void __launch_bounds__(256) gemv_f16w_kernel(const __half *__restrict__ W, const AT *__restrict__ A,
                                                        OutT *__restrict__ C, int M, int m_base, int N, int K, float alpha) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const bool vec_ok = (K % 8) == 0;
  for (int row = blockIdx.x * warps + (threadIdx.x >> 5); row < N; row += gridDim.x * warps) {
    const __half *wr = W + (size_t)row * K;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = 0.0f;
    if (vec_ok) {
#pragma unroll 4
      for (int k = lane * 8; k < K; k += 256) {
        const uint4 wv = __ldg(reinterpret_cast<const uint4 *>(wr + k));
        const __half2 *h = reinterpret_cast<const __half2 *>(&wv);
        float wf[8];
#pragma unroll
        for (int i = 0; i < 4; i++) { float2 f = __half22float2(h[i]); wf[2 * i] = f.x; wf[2 * i + 1] = f.y; }
#pragma unroll
        for (int m = 0; m < MT; m++) {
          if (m_base + m < M) {
            const size_t ao = (size_t)(m_base + m) * K + k;
#pragma unroll
            for (int i = 0; i < 8; i++) acc[m] = fmaf(wf[i], load_act<AT>(A, ao + i), acc[m]);
          }
        }
      }
    } else {
      for (int k = lane; k < K; k += 32) {
        const float wv = __half2float(__ldg(wr + k));
#pragma unroll
        for (int m = 0; m < MT; m++)
          if (m_base + m < M) acc[m] = fmaf(wv, load_act<AT>(A, (size_t)(m_base + m) * K + k), acc[m]);
      }
    }
#pragma unroll
    for (int m = 0; m < MT; m++) {
      float v = acc[m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && m_base + m < M) {
        v *= alpha;
        if constexpr (sizeof(OutT) == 4) C[(size_t)(m_base + m) * N + row] = v;
        else C[(size_t)(m_base + m) * N + row] = __float2half_rn(v);
      }
    }
  }
}

// M == 1, f32 activations: x is staged once per CTA in shared memory; a warp streams FOUR weight rows at a time
// (four 16-byte loads in flight per lane and pass, two passes unrolled), so the shared-memory reads of x are
// shared by four rows and the shuffle reduction is paid once per 32 KB of weights instead of once per 8 KB.
template <typename OutT>
__global__ void __launch_bounds__(256) gemv_f16w_m1_kernel(const __half *__restrict__ W, const float *__restrict__ x,
                                                           OutT *__restrict__ y, int N, int K, float alpha) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float xs[];
  for (int i = threadIdx.x; i < K / 4; i += blockDim.x)
    reinterpret_cast<float4 *>(xs)[i] = __ldg(reinterpret_cast<const float4 *>(x) + i);
  __syncthreads();
  const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int n16 = K / 8;
  for (int row0 = (blockIdx.x * warps + (threadIdx.x >> 5)) * 4; row0 < N; row0 += gridDim.x * warps * 4) {
    const uint4 *wr[4];
#pragma unroll
    for (int r = 0; r < 4; r++) wr[r] = reinterpret_cast<const uint4 *>(W + (size_t)min(row0 + r, N - 1) * K);
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 2
    for (int c = lane; c < n16; c += 32) {
      uint4 wv[4];
#pragma unroll
      for (int r = 0; r < 4; r++) wv[r] = __ldg(wr[r] + c);
      const float4 x0 = *reinterpret_cast<const float4 *>(xs + 8 * c), x1 = *reinterpret_cast<const float4 *>(xs + 8 * c + 4);
#pragma unroll
      for (int r = 0; r < 4; r++) {
        const __half2 *h = reinterpret_cast<const __half2 *>(&wv[r]);
        const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]), f2 = __half22float2(h[2]), f3 = __half22float2(h[3]);
        float a = acc[r];
        a = fmaf(f0.x, x0.x, a); a = fmaf(f0.y, x0.y, a); a = fmaf(f1.x, x0.z, a); a = fmaf(f1.y, x0.w, a);
        a = fmaf(f2.x, x1.x, a); a = fmaf(f2.y, x1.y, a); a = fmaf(f3.x, x1.z, a); a = fmaf(f3.y, x1.w, a);
        acc[r] = a;
      }
    }
#pragma unroll
    for (int r = 0; r < 4; r++) {
      float a = acc[r];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      if (lane == 0 && row0 + r < N) {
        const float v = a * alpha;
        if constexpr (sizeof(OutT) == 4) y[row0 + r] = v; else y[row0 + r] = __float2half_rn(v);
      }
    }
  }
}

template <typename AT, typename OutT>
static dp_status launch_f16w(dp_ctx *ctx, const __half *W, const AT *A, OutT *C, int M, int N, int K, float alpha) {
  const int threads = 256, warps = 8;
  int grid = (N + warps - 1) / warps;
  const int cap = ctx->sm_count * 8;
  if (grid > cap) grid = cap;
  for (int m0 = 0; m0 < M; m0 += 4) {
    if (M - m0 == 1) {
      DP_LAUNCH(ctx, (gemv_f16w_kernel<AT, OutT, 1>), grid, threads, 0, W, A, C, M, m0, N, K, alpha);
    } else {
      DP_LAUNCH(ctx, (gemv_f16w_kernel<AT, OutT, 4>), grid, threads, 0, W, A, C, M, m0, N, K, alpha);
    }
  }
  return DP_OK;
}

dp_status dpk_gemv_f16w(dp_ctx *ctx, const __half *W, const void *A, dp_dtype a_dtype, void *C, dp_dtype c_dtype, int M,
                        int N, int K, float alpha) {
  if (M == 1 && a_dtype == DP_F32 && K % 8 == 0 && (size_t)K * 4 <= 48 * 1024) {
    int grid = (N + 31) / 32;  // eight warps of four rows
    if (grid > ctx->sm_count * 8) grid = ctx->sm_count * 8;
    if (c_dtype == DP_F32) {
      DP_LAUNCH(ctx, gemv_f16w_m1_kernel<float>, grid, 256, (size_t)K * 4, W, (const float *)A, (float *)C, N, K, alpha);
    } else {
      DP_LAUNCH(ctx, gemv_f16w_m1_kernel<__half>, grid, 256, (size_t)K * 4, W, (const float *)A, (__half *)C, N, K, alpha);
    }
    return DP_OK;
  }
  if (M >= 2) {
    bool handled = false;
    DP_TRY(dpk_gemm_f16w_rows(ctx, W, A, a_dtype, C, c_dtype, M, N, K, alpha, &handled));
    if (handled) return DP_OK;
  }
  if (a_dtype == DP_F32 && c_dtype == DP_F32) return launch_f16w<float, float>(ctx, W, (const float *)A, (float *)C, M, N, K, alpha);
  if (a_dtype == DP_F32 && c_dtype == DP_F16) return launch_f16w<float, __half>(ctx, W, (const float *)A, (__half *)C, M, N, K, alpha);
  if (a_dtype == DP_F16 && c_dtype == DP_F32) return launch_f16w<__half, float>(ctx, W, (const __half *)A, (float *)C, M, N, K, alpha);
  if (a_dtype == DP_F16 && c_dtype == DP_F16) return launch_f16w<__half, __half>(ctx, W, (const __half *)A, (__half *)C, M, N, K, alpha);
  return dp_fail(ctx, DP_ERR_INVALID, "matmul f16 weights: unsupported dtypes A=%s C=%s", dp_dtype_name(a_dtype), dp_dtype_name(c_dtype));
}

// f32 weights: plain warp-per-row kernel (kept for API completeness)
__global__ void __launch_bounds__(256) gemv_f32w_kernel(const float *__restrict__ W, const float *__restrict__ A,
                                                        float *__restrict__ C, int M, int N, int K, float alpha) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const long total = (long)M * N;
  for (long o = (long)blockIdx.x * warps + (threadIdx.x >> 5); o < total; o += (long)gridDim.x * warps) {
    const int m = (int)(o / N), n = (int)(o % N);
    float acc = 0.0f;
    for (int k = lane; k < K; k += 32) acc = fmaf(__ldg(W + (size_t)n * K + k), __ldg(A + (size_t)m * K + k), acc);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) C[(size_t)m * N + n] = acc * alpha;
  }
}

dp_status dpk_gemv_f32w(dp_ctx *ctx, const float *W, const float *A, float *C, int M, int N, int K, float alpha) {
  long total = (long)M * N;
  long want = (total + 7) / 8;
  int grid = (int)(want < (long)ctx->sm_count * 16 ? want : (long)ctx->sm_count * 16);
  DP_LAUNCH(ctx, gemv_f32w_kernel, grid, 256, 0, W, A, C, M, N, K, alpha);
  return DP_OK;
}
