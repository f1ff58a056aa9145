// Dense f16 weights times a small batch of activation rows (2..64 per launch): the LM head of a batched
// decode step (reference: the tied-embedding logits matmul, src/inference/pipelines/text/logits/gpu.js:245,
// which runs matmul_f16w_f32a.wgsl for 'ehf16' heads).
//
// HBM-bound: the weight matrix (1.24 GB for a 151936 x 4096 head) is streamed ONCE for all rows of the batch.
// A CTA of eight warps owns 128 weight rows; every warp keeps a 16 x (8 * NT) tile of the output in registers
// (mma.sync m16n8k16, the weights as the A operand straight from global memory with 16-byte loads, two 32-wide
// K chunks in flight per lane) and walks the whole of K.  The activation rows are the B operand: f32 rows are
// split beforehand into an f16 half and its rounding residue, both scaled per row by a power of two
// (scale_cast_rows in gemm_q4k_tc.cu), so that hi + lo carries about 22 bits and the product is the f32 one
// to f32 accuracy; 64-wide K slices of both are staged through shared memory with cp.async (two stages).
//
// K order inside an MMA: summation order is free, so the kernel permutes K to fit the loads.  A lane's 16-byte
// load of 8 consecutive halves at k = 32c + 8t feeds two MMAs: halves 0..3 as the lane's (k 2t, 2t+1, 2t+8,
// 2t+9) of the first, halves 4..7 of the second; the B fragments use the same assignment, which makes them one
// 16-byte shared-memory load per MMA pair.
#include <cuda_fp16.h>
#include <stdint.h>

#include "common.h"
#include "pdl.cuh"

namespace {

constexpr int ROWS_PER_CTA = 128;
constexpr int KS = 64;                 // K slice per stage
constexpr int B_STRIDE = KS * 2 + 64;  // bytes per staged activation row: 128 data + 64 pad (conflict-free 16-byte reads)

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid) {
  const int n = valid ? 16 : 0;  // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: 8-row groups of the batch this launch covers (1, 2, 4 or 8); LO: the residue halves are multiplied in as well.
template <typename OutT, int NT, bool LO>
__global__ void __launch_bounds__(256, 2) gemm_f16w_rows_kernel(const __half *__restrict__ W, const __half *__restrict__ a_hi,
                                                                const __half *__restrict__ a_lo, const float *__restrict__ row_scale,
                                                                OutT *__restrict__ C, int M, int m_base, int N, int K, float alpha) {
  extern __shared__ __align__(16) unsigned char smem[];
  constexpr int BROWS = NT * 8;
  constexpr int ARR_BYTES = BROWS * B_STRIDE;             // one array (hi or lo) of one stage
  constexpr int STAGE_BYTES = ARR_BYTES * (LO ? 2 : 1);
  pdl_launch();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * ROWS_PER_CTA + warp * 16;
  const int ra = min(row0 + g, N - 1), rb = min(row0 + g + 8, N - 1);
  const uint4 *wa = reinterpret_cast<const uint4 *>(W + (size_t)ra * K) + t;
  const uint4 *wb = reinterpret_cast<const uint4 *>(W + (size_t)rb * K) + t;
  const int nslice = K / KS;
  const uint32_t smem_u = (uint32_t)__cvta_generic_to_shared(smem);

  // weights of the first slice: nothing earlier in the stream writes them, so the loads go out before the wait
  uint4 curA[2], curB[2], nxtA[2], nxtB[2];
  curA[0] = __ldg(wa); curB[0] = __ldg(wb);
  curA[1] = __ldg(wa + 4); curB[1] = __ldg(wb + 4);
  pdl_wait();

  auto stage_load = [&](int s) {
    const uint32_t base = smem_u + (uint32_t)(s & 1) * STAGE_BYTES;
    constexpr int PIECES = BROWS * 8 * (LO ? 2 : 1);
#pragma unroll
    for (int p = tid; p < PIECES; p += 256) {
      const int arr = p / (BROWS * 8), rem = p % (BROWS * 8), r = rem >> 3, c = rem & 7;
      const int m = m_base + r;
      const bool ok = m < M;
      const __half *src = (arr ? a_lo : a_hi) + (size_t)(ok ? m : m_base) * K + (size_t)s * KS + c * 8;
      cp_async16(base + arr * ARR_BYTES + r * B_STRIDE + c * 16, src, ok);
    }
  };

  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f; }

  stage_load(0);
  cp_async_commit();
  for (int s = 0; s < nslice; s++) {
    if (s + 1 < nslice) {
      // (the stage written here was last read in iteration s - 1, which ended with a CTA barrier)
      stage_load(s + 1);
      cp_async_commit();
      const uint4 *na = wa + (size_t)(s + 1) * 8, *nb = wb + (size_t)(s + 1) * 8;
      nxtA[0] = __ldg(na); nxtB[0] = __ldg(nb);
      nxtA[1] = __ldg(na + 4); nxtB[1] = __ldg(nb + 4);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const unsigned char *st = smem + (s & 1) * STAGE_BYTES;
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const uint4 A = curA[h], B = curB[h];
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        const unsigned char *bp = st + (nt * 8 + g) * B_STRIDE + h * 64 + t * 16;
        const uint4 bh = *reinterpret_cast<const uint4 *>(bp);
        mma_f16(acc[nt], A.x, B.x, A.y, B.y, bh.x, bh.y);
        mma_f16(acc[nt], A.z, B.z, A.w, B.w, bh.z, bh.w);
        if constexpr (LO) {
          const uint4 bl = *reinterpret_cast<const uint4 *>(bp + ARR_BYTES);
          mma_f16(acc[nt], A.x, B.x, A.y, B.y, bl.x, bl.y);
          mma_f16(acc[nt], A.z, B.z, A.w, B.w, bl.z, bl.w);
        }
      }
    }
    __syncthreads();
    curA[0] = nxtA[0]; curA[1] = nxtA[1];
    curB[0] = nxtB[0]; curB[1] = nxtB[1];
  }

  // accumulator (weight row g / g + 8, batch row 2t / 2t + 1 of every group) -> C[batch row][weight row]
#pragma unroll
  for (int nt = 0; nt < NT; nt++) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int m = m_base + nt * 8 + 2 * t + (j & 1);
      const int row = row0 + g + (j >> 1) * 8;
      if (m < M && row < N) {
        const float v = acc[nt][j] * alpha * (row_scale ? __ldg(row_scale + m) : 1.0f);
        if constexpr (sizeof(OutT) == 4) C[(size_t)m * N + row] = v;
        else C[(size_t)m * N + row] = __float2half_rn(v);
      }
    }
  }
}

template <typename OutT, int NT, bool LO>
dp_status launch_rows(dp_ctx *ctx, const __half *W, const __half *hi, const __half *lo, const float *scales, OutT *C, int M, int m_base,
                      int N, int K, float alpha) {
  constexpr size_t smem = (size_t)2 * NT * 8 * B_STRIDE * (LO ? 2 : 1);
  auto kernel = gemm_f16w_rows_kernel<OutT, NT, LO>;
  if (smem > 48 * 1024) DP_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const unsigned grid = (unsigned)((N + ROWS_PER_CTA - 1) / ROWS_PER_CTA);
  DP_LAUNCH(ctx, kernel, grid, 256, smem, W, hi, lo, scales, C, M, m_base, N, K, alpha);
  return DP_OK;
}

template <typename OutT, bool LO>
dp_status dispatch_rows(dp_ctx *ctx, const __half *W, const __half *hi, const __half *lo, const float *scales, OutT *C, int M, int N, int K,
                        float alpha) {
  for (int m0 = 0; m0 < M; m0 += 64) {
    const int mb = M - m0 < 64 ? M - m0 : 64;
    dp_status st;
    if (mb <= 8) st = launch_rows<OutT, 1, LO>(ctx, W, hi, lo, scales, C, M, m0, N, K, alpha);
    else if (mb <= 16) st = launch_rows<OutT, 2, LO>(ctx, W, hi, lo, scales, C, M, m0, N, K, alpha);
    else if (mb <= 32) st = launch_rows<OutT, 4, LO>(ctx, W, hi, lo, scales, C, M, m0, N, K, alpha);
    else st = launch_rows<OutT, 8, LO>(ctx, W, hi, lo, scales, C, M, m0, N, K, alpha);
    if (st != DP_OK) return st;
  }
  return DP_OK;
}

}  // namespace

// C[M, N] = alpha * A[M, K] . W[N, K]^T for f16 weights and M >= 2.  f32 activations are multiplied in to f32
// accuracy (two f16 halves per element), f16 activations as they are.  *handled stays false for shapes the
// kernel does not take (K not a multiple of 64).
dp_status dpk_gemm_f16w_rows(dp_ctx *ctx, const __half *W, const void *A, dp_dtype a_dtype, void *C, dp_dtype c_dtype, int M, int N, int K,
                             float alpha, bool *handled) {
  *handled = false;
  if (M < 2 || K % KS || N < 1) return DP_OK;
  if ((c_dtype != DP_F32 && c_dtype != DP_F16) || (a_dtype != DP_F32 && a_dtype != DP_F16)) return DP_OK;
  dp_status st;
  if (a_dtype == DP_F32) {
    const size_t a_bytes = ((size_t)M * K * 2 + 255) / 256 * 256;
    DP_TRY(dp_scratch(ctx, &ctx->gemm_scratch, 2 * a_bytes + (size_t)M * 4, "matmul_a_f16"));
    char *base = (char *)ctx->gemm_scratch->dptr;
    __half *hi = (__half *)base, *lo = (__half *)(base + a_bytes);
    float *scales = (float *)(base + 2 * a_bytes);
    DP_TRY(dpk_scale_cast_rows(ctx, (const float *)A, hi, lo, scales, M, K));
    if (c_dtype == DP_F32) st = dispatch_rows<float, true>(ctx, W, hi, lo, scales, (float *)C, M, N, K, alpha);
    else st = dispatch_rows<__half, true>(ctx, W, hi, lo, scales, (__half *)C, M, N, K, alpha);
  } else {
    const __half *hi = (const __half *)A;
    if (c_dtype == DP_F32) st = dispatch_rows<float, false>(ctx, W, hi, hi, nullptr, (float *)C, M, N, K, alpha);
    else st = dispatch_rows<__half, false>(ctx, W, hi, hi, nullptr, (__half *)C, M, N, K, alpha);
  }
  if (st == DP_OK) *handled = true;
  return st;
}
