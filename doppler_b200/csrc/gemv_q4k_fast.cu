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
#include "pdl.cuh"
#include "q4k.cuh"
#include "actq.cuh"

// ---- activation pre-pass -------------------------------------------------------
// layout of the quantised activation buffer for K = 256*bpr:
//   limbs  int8 [K/32][4][32]   column c = digit c (c = 3 is zero), bytes in element order
//   xscale f32  [bpr]           2^(e_b - 22)
//   ssum   f32  [K/32]          sum of the fixed-point integers of each sub-block
__global__ void __launch_bounds__(256) q4k_prep_act_kernel(const float *__restrict__ x, void *__restrict__ actq, int bpr) {
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * (blockDim.x >> 5);
  for (int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < bpr; b += warps_total) {
    const float4 v0 = *reinterpret_cast<const float4 *>(x + b * QK_K + lane * 8);
    const float4 v1 = *reinterpret_cast<const float4 *>(x + b * QK_K + lane * 8 + 4);
    const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    actq_emit_block(v, lane, b, bpr, actq);
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
  pdl_launch();
  pdl_wait();
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
    const uint2 *lb = reinterpret_cast<const uint2 *>(limbs + (size_t)b * 1024) + t;  // digit layout: actq.cuh
    int accA0 = 0, accA1 = 0, accB0 = 0, accB1 = 0;
#pragma unroll
    for (int c = 0; c < 4; c++) {
#pragma unroll
      for (int hi = 0; hi < 2; hi++) {
        const int sb = 2 * c + hi;
        uint2 bf = make_uint2(0u, 0u);
        if (g < 3) bf = __ldg(lb + c * 32 + (2 * g + hi) * 4);
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

dp_status dpk_gemv_q4k_actq_tma(dp_ctx *ctx, const uint8_t *W, const void *actq, void *y, dp_dtype y_dtype, int N, int K,
                                float alpha, const float *residual, bool *handled);

static size_t actq_bytes(int K) { return (size_t)K * 4 + (size_t)(K / 256) * 4 + (size_t)(K / 32) * 4; }

// quantise x (f32[K]) into `actq` (actq_bytes(K)); exposed to the runner so producers can be fused later
dp_status dpk_q4k_prep_act(dp_ctx *ctx, const float *x, void *actq, int K) {
  const int bpr = K / QK_K;
  const int grid = (bpr + 7) / 8;
  DP_LAUNCH(ctx, q4k_prep_act_kernel, grid, 256, 0, x, actq, bpr);
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

struct GemvExchange;
dp_status dpk_gemv_q4k_tma_fused(dp_ctx *ctx, const uint8_t *W, int mode, const float *x, const float *w, float eps, int D,
                                 int splits, float *y, int N, int K, const float *residual, bool *handled, const GemvExchange *gxp);

dp_status dpk_gemv_q4k_fast(dp_ctx *ctx, const uint8_t *W, const float *x, void *y, dp_dtype y_dtype, int N, int K,
                            float alpha, const float *residual, bool *handled) {
  *handled = false;
  if (!dpk_gemv_q4k_fast_ok(N, K) || (y_dtype != DP_F32 && y_dtype != DP_F16)) return DP_OK;
  // One launch when the shape has a TMA plan: the kernel splits the f32 vector into digits in its own prologue
  // (the same digits the pre-pass below writes), which is what a launch-bound GEMV of a couple of MB is made of.
  if (y_dtype == DP_F32 && alpha == 1.0f && ((uintptr_t)x & 15u) == 0) {
    bool one = false;
    DP_TRY(dpk_gemv_q4k_tma_fused(ctx, W, 5 /* SRC_PLAIN */, x, nullptr, 0.0f, 0, 0, (float *)y, N, K, residual, &one, nullptr));
    if (one) { *handled = true; return DP_OK; }
  }
  DP_TRY(dp_scratch(ctx, &ctx->gemv_scratch, actq_bytes(K), "gemv_activation_digits"));
  DP_TRY(dpk_q4k_prep_act(ctx, x, ctx->gemv_scratch->dptr, K));
  bool tma = false;
  DP_TRY(dpk_gemv_q4k_actq_tma(ctx, W, ctx->gemv_scratch->dptr, y, y_dtype, N, K, alpha, residual, &tma));
  if (!tma) DP_TRY(dpk_gemv_q4k_actq(ctx, W, ctx->gemv_scratch->dptr, y, y_dtype, N, K, alpha, residual));
  *handled = true;
  return DP_OK;
}

// ---------------------------------------------------------------------------
// Persistent, TMA-fed variant (needs ceil(K/256) to be a multiple of the chunk size).
//
// One CTA per SM loops over 16-row tiles.  A producer warp streams the packed weight
// rows into a ring of shared-memory stages with untiled bulk copies (one contiguous
// copy per row and chunk of up to eight super-blocks, completion counted on an
// mbarrier), so many tens of KB per SM are in flight regardless of what the consumer
// warps are doing.  The eight consumer warps each take one super-block column of the
// chunk out of shared memory (rows are padded by 32 bytes so that the 8-byte reads of a
// half-warp fall in distinct banks), run the integer MMAs as above and hand the stage
// back through an "empty" mbarrier.  The activation digits live in shared memory for
// the whole kernel.  Every wait is bounded: on give-up the CTA raises an abort flag, all
// its threads leave their loops, and a status word tells the host (DP_ERR_TIMEOUT).
// ---------------------------------------------------------------------------
#include "mbar.cuh"
#include "handoff.cuh"
#include "tp_exchange.h"
#include "gemv_exchange.h"

#include <cstdlib>

#define TG_CONSUMERS 8  // warps per consumer group (one per super-block column of a chunk)
#define TG_MAX_BW 2     // super-block columns of a stage per consumer warp: a stage holds at most 16 blocks per row
#define TG_ROW_PAD 32
#define TG_RED_SLOTS 16

struct TgLayout {
  uint32_t digits, ssum, xscale, stages, bars, red, abort_flag, total;
  uint32_t row_stride, stage_bytes;
};

__host__ __device__ inline TgLayout tg_layout(int K, int cb, int stages) {
  TgLayout l;
  const uint32_t bpr = (uint32_t)K / QK_K;
  l.digits = 0;
  l.xscale = (uint32_t)K * 4;  // same order as the global buffer: digits, block scales, sub-block sums
  l.ssum = l.xscale + bpr * 4;
  uint32_t off = l.ssum + (uint32_t)(K / 32) * 4;
  off = (off + 127u) & ~127u;
  l.row_stride = (uint32_t)cb * Q4K_BLOCK_BYTES + TG_ROW_PAD;
  l.stage_bytes = 16u * l.row_stride;
  l.stages = off;
  off += (uint32_t)stages * l.stage_bytes;
  l.bars = off;  // full[stages], empty[stages], red[TG_RED_SLOTS]
  off += (2u * (uint32_t)stages + TG_RED_SLOTS) * 8u;
  l.red = off;
  off += TG_RED_SLOTS * TG_CONSUMERS * 16u * 4u;
  l.abort_flag = off;
  l.total = off + 16u;
  return l;
}

// Where the GEMV's input vector comes from.  SRC_DIGITS: ready-made digits in global memory.  The
// other modes let every CTA rebuild the digits itself from the previous op's f32 output while its
// producer warp is already filling the weight ring, so the normalisation / activation / split merge
// needs no kernel of its own (148 CTAs redo a few KB of work each; the latency hides under the
// pipeline fill):
//   SRC_RMSNORM  x = rmsnorm(h, w, eps)                 (rmsnorm.wgsl:119-187)
//   SRC_SILU     x = silu(gate) * up, gu[2K] = eight gate values, their eight up values, ...   (silu.wgsl:98-104)
//   SRC_COMBINE  x = merge of the split-K attention partials (layout of attention.cu)
//   SRC_XCHG_RMSNORM  tensor parallel: h' = h + the partial vectors every rank pushed into this rank's
//                exchange area (summed in rank order, so all ranks hold the same bits), x = rmsnorm(h', w, eps);
//                each CTA also writes its share of h'.  Allreduce + residual add + RMSNorm in the prologue.
// Output: y[row] (+ residual), or, with GemvExchange::push, the rows go as (value, ticket) words into this
// rank's slot of every rank's exchange area (plain stores over NVLink): the allreduce's send side in the epilogue.
enum { SRC_DIGITS = 0, SRC_RMSNORM = 1, SRC_SILU = 2, SRC_COMBINE = 3, SRC_XCHG_RMSNORM = 4, SRC_PLAIN = 5 };
// mode flag of dpk_gemv_q4k_tma_fused: the rows are gate|up pairs (eight gate rows, then their eight up rows per
// 16-row tile) and the kernel stores silu(gate) * up, N / 2 values, instead of the N raw rows
enum { SRC_FLAG_SILU_OUT = 0x100 };
struct GemvSource {
  const float *x;   // h (SRC_RMSNORM), gu (SRC_SILU), partials (SRC_COMBINE)
  const float *w;   // norm weights
  float eps;
  int D, splits;    // SRC_COMBINE: head_dim and number of splits
};

// GROUPS consumer groups of eight warps each; consecutive row tiles alternate between the groups, so
// while one group is in the latency-bound tail of a tile the other keeps the tensor pipe busy.
// PUSH: the epilogue pushes the rows into the exchange areas (GemvExchange); instantiated only for the
// tensor-parallel launches, so the other instantiations carry none of that code.
template <typename OutT, int GROUPS, int SRC, bool PUSH = false, bool SILU_OUT = false>
__global__ void __launch_bounds__((GROUPS * TG_CONSUMERS + 1) * 32, 1) gemv_q4k_tma_kernel(
    const uint8_t *__restrict__ W, const int8_t *__restrict__ limbs, const float *__restrict__ xscale,
    const float *__restrict__ ssum, OutT *__restrict__ y, int N, int K, int cb, int stages, float alpha,
    const float *__restrict__ residual, int *__restrict__ err, const __grid_constant__ GemvSource gs, const __grid_constant__ GemvExchange gx) {
  extern __shared__ __align__(128) uint8_t smem[];
  const TgLayout L = tg_layout(K, cb, stages);
  const int tid = threadIdx.x, lane = tid & 31, warp_all = tid >> 5;
  const int group = warp_all / TG_CONSUMERS, warp = warp_all % TG_CONSUMERS;  // producer: group == GROUPS
  const int bpr = K / QK_K, chunks = bpr / cb, tiles = N / 16;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L.abort_flag);
  const uint32_t bars = smem_u32(smem + L.bars);
  auto full_bar = [&](int s) { return bars + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return bars + 8u * (uint32_t)(stages + s); };
  auto red_bar = [&](int s) { return bars + 8u * (uint32_t)(2 * stages + s); };

  if (tid == 0) {
    for (int s = 0; s < stages; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), TG_CONSUMERS); }
    for (int s = 0; s < TG_RED_SLOTS; s++) mbar_init(red_bar(s), TG_CONSUMERS);
    *abort_flag = 0;
    mbar_fence_init();
  }
  pdl_launch();
  __syncthreads();
  (void)xscale; (void)ssum;
  const float *sm_ssum = reinterpret_cast<const float *>(smem + L.ssum);
  const float *sm_xscale = reinterpret_cast<const float *>(smem + L.xscale);
  // The producer starts streaming weights at once: they are written by no kernel of the step,
  // so under programmatic dependent launch the ring fills while the previous kernel drains.
  // The consumers first wait for the previous kernel (which produced the activation digits).
  if (group < GROUPS) {
    constexpr int CT = GROUPS * TG_CONSUMERS * 32;  // consumer threads
    constexpr int NW = CT / 32;
    const int cw = tid >> 5;
    // The norm weights are written by no kernel of the step either: their loads are issued before the wait
    // for the previous kernel, so that their latency is off the critical path of the prologue.
    float4 nw[2][2];
    if constexpr (SRC == SRC_RMSNORM || SRC == SRC_XCHG_RMSNORM) {
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int b = cw + NW * i;
        if (b < bpr) {
          nw[i][0] = __ldg(reinterpret_cast<const float4 *>(gs.w + b * QK_K + lane * 8));
          nw[i][1] = __ldg(reinterpret_cast<const float4 *>(gs.w + b * QK_K + lane * 8 + 4));
        }
      }
    }
    pdl_wait();
    if constexpr (SRC == SRC_DIGITS) {
      const uint4 *src = reinterpret_cast<const uint4 *>(limbs);
      uint4 *dst = reinterpret_cast<uint4 *>(smem);
      const int total = K * 4 + (K / 32) * 4 + bpr * 4;
      const int n16 = total / 16;
      for (int i = tid; i < n16; i += CT) dst[i] = __ldg(src + i);
      const int rem_words = (total - n16 * 16) / 4;
      if (tid < rem_words) reinterpret_cast<uint32_t *>(smem)[n16 * 4 + tid] = __ldg(reinterpret_cast<const uint32_t *>(limbs) + n16 * 4 + tid);
    } else if constexpr (SRC == SRC_RMSNORM || SRC == SRC_XCHG_RMSNORM) {
      float *scratch = reinterpret_cast<float *>(smem + L.red);  // free until the first tile is reduced
      float v[2][8];
      float ss = 0.0f;
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int b = cw + NW * i;
        if (b < bpr) {
          const int off = b * QK_K + lane * 8;
          const float4 a = *reinterpret_cast<const float4 *>(gs.x + off);
          const float4 c = *reinterpret_cast<const float4 *>(gs.x + off + 4);
          v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w; v[i][4] = c.x; v[i][5] = c.y; v[i][6] = c.z; v[i][7] = c.w;
          if constexpr (SRC == SRC_XCHG_RMSNORM) {
            const unsigned ticket = *reinterpret_cast<const volatile unsigned *>(gx.ticket_step) * gx.ticket_stride + 1u + gx.ticket_in;
            const uint2 *mine = gx.mine;
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            // rank order: every rank computes the same bits; two ranks' words are fetched together
            for (int r = 0; r + 1 < gx.nr; r += 2) {
              float s8[8] = {0, 0, 0, 0, 0, 0, 0, 0}, t8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
              handoff_take8x2(mine + dp_tp_slot_offset((unsigned)gx.parity_in, r) + off, mine + dp_tp_slot_offset((unsigned)gx.parity_in, r + 1) + off,
                              ticket, s8, t8, gx.wait_limit, abort_flag);
#pragma unroll
              for (int j = 0; j < 8; j++) acc[j] = (acc[j] + s8[j]) + t8[j];
            }
            if (gx.nr & 1) {
              float s8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
              handoff_take8(mine + dp_tp_slot_offset((unsigned)gx.parity_in, gx.nr - 1) + off, ticket, s8, gx.wait_limit, abort_flag);
#pragma unroll
              for (int j = 0; j < 8; j++) acc[j] += s8[j];
            }
#pragma unroll
            for (int j = 0; j < 8; j++) v[i][j] += acc[j];
            if (gx.h_out && (b % (int)gridDim.x) == (int)blockIdx.x) {
              *reinterpret_cast<float4 *>(gx.h_out + off) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
              *reinterpret_cast<float4 *>(gx.h_out + off + 4) = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
            }
          }
#pragma unroll
          for (int j = 0; j < 8; j++) ss = fmaf(v[i][j], v[i][j], ss);
        }
      }
      __syncwarp();
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) scratch[cw] = ss;
      asm volatile("bar.sync 1, %0;" ::"r"(CT) : "memory");
      float total = 0.0f;
#pragma unroll
      for (int i = 0; i < NW; i++) total += scratch[i];
      const float inv_rms = 1.0f / sqrtf(total / (float)K + gs.eps);
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int b = cw + NW * i;
        if (b < bpr) {
          const float4 wa = nw[i][0], wc = nw[i][1];
          const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wc.x, wc.y, wc.z, wc.w};
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; j++) o[j] = v[i][j] * inv_rms * wv[j];
          actq_emit_block(o, lane, b, bpr, smem);
        }
      }
    } else if constexpr (SRC == SRC_PLAIN) {
      // the input vector as it is (the previous kernel stored silu(gate) * up); two blocks per round
      for (int b = cw; b < bpr; b += 2 * NW) {
        const int b2 = b + NW;
        const bool two = b2 < bpr;
        const float *xp = gs.x + b * QK_K + lane * 8, *xq = gs.x + (two ? b2 : b) * QK_K + lane * 8;
        const float4 a0 = *reinterpret_cast<const float4 *>(xp), a1 = *reinterpret_cast<const float4 *>(xp + 4);
        const float4 c0 = *reinterpret_cast<const float4 *>(xq), c1 = *reinterpret_cast<const float4 *>(xq + 4);
        {
          const float o[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
          actq_emit_block(o, lane, b, bpr, smem);
        }
        if (two) {
          const float o[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
          actq_emit_block(o, lane, b2, bpr, smem);
        }
      }
    } else if constexpr (SRC == SRC_SILU) {
      // two blocks per round: the second block's loads are in flight while the first is converted
      for (int b = cw; b < bpr; b += 2 * NW) {
        const int b2 = b + NW;
        const bool two = b2 < bpr;
        const float *gp = gs.x + 2 * (b * QK_K + lane * 8), *up = gp + 8;  // gate|up interleaved in groups of eight
        const float *gq = gs.x + 2 * ((two ? b2 : b) * QK_K + lane * 8), *uq = gq + 8;
        const float4 g0 = *reinterpret_cast<const float4 *>(gp), g1 = *reinterpret_cast<const float4 *>(gp + 4);
        const float4 u0 = *reinterpret_cast<const float4 *>(up), u1 = *reinterpret_cast<const float4 *>(up + 4);
        const float4 h0 = *reinterpret_cast<const float4 *>(gq), h1 = *reinterpret_cast<const float4 *>(gq + 4);
        const float4 w0 = *reinterpret_cast<const float4 *>(uq), w1 = *reinterpret_cast<const float4 *>(uq + 4);
        {
          const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w}, u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const float cl = fminf(fmaxf(g[j], -15.0f), 15.0f);
            o[j] = (g[j] * (1.0f / (1.0f + expf(-cl)))) * u[j];
          }
          actq_emit_block(o, lane, b, bpr, smem);
        }
        if (two) {
          const float g[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w}, u[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const float cl = fminf(fmaxf(g[j], -15.0f), 15.0f);
            o[j] = (g[j] * (1.0f / (1.0f + expf(-cl)))) * u[j];
          }
          actq_emit_block(o, lane, b2, bpr, smem);
        }
      }
    } else {
      const int D = gs.D, splits = gs.splits;
      // Fast form (a half-warp's 128 outputs lie in one head, at most 16 splits): lane j of the half-warp fetches
      // the running max and sum of split j, so all of them arrive in one round trip, and the partial rows are
      // read four splits at a time.  Same arithmetic, in the same order, as the sequential form below.
      const bool fast = (D % 128) == 0 && splits <= 16;
      for (int b = cw; b < bpr; b += NW) {
        const int e0 = b * QK_K + lane * 8, h = e0 / D, d0 = e0 % D;
        const float *pp = gs.x + (size_t)h * splits * (D + 2);
        float mm = -3.402823466e+38f;
        float ll = 0.0f, acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (fast) {
          const int hl = lane & 15;
          float m_mine = -3.402823466e+38f, l_mine = 0.0f;
          if (hl < splits) { m_mine = pp[hl * (D + 2) + D]; l_mine = pp[hl * (D + 2) + D + 1]; }
          mm = m_mine;
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
          const float c_mine = (m_mine == -3.402823466e+38f) ? 0.0f : exp2f(m_mine - mm);
#pragma unroll 4
          for (int sp = 0; sp < splits; sp++) {
            const float *ps = pp + sp * (D + 2);
            const float2 a0 = *reinterpret_cast<const float2 *>(ps + d0), a1 = *reinterpret_cast<const float2 *>(ps + d0 + 2);
            const float2 a2 = *reinterpret_cast<const float2 *>(ps + d0 + 4), a3 = *reinterpret_cast<const float2 *>(ps + d0 + 6);
            const float c = __shfl_sync(0xffffffffu, c_mine, (lane & 16) + sp);
            ll = fmaf(__shfl_sync(0xffffffffu, l_mine, (lane & 16) + sp), c, ll);
            acc[0] = fmaf(a0.x, c, acc[0]); acc[1] = fmaf(a0.y, c, acc[1]); acc[2] = fmaf(a1.x, c, acc[2]); acc[3] = fmaf(a1.y, c, acc[3]);
            acc[4] = fmaf(a2.x, c, acc[4]); acc[5] = fmaf(a2.y, c, acc[5]); acc[6] = fmaf(a3.x, c, acc[6]); acc[7] = fmaf(a3.y, c, acc[7]);
          }
        } else {
          for (int sp = 0; sp < splits; sp++) mm = fmaxf(mm, pp[sp * (D + 2) + D]);
#pragma unroll 2
          for (int sp = 0; sp < splits; sp++) {
            const float *ps = pp + sp * (D + 2);
            const float ms = ps[D];
            const float c = (ms == -3.402823466e+38f) ? 0.0f : exp2f(ms - mm);
            ll = fmaf(ps[D + 1], c, ll);
            const float2 a0 = *reinterpret_cast<const float2 *>(ps + d0), a1 = *reinterpret_cast<const float2 *>(ps + d0 + 2);
            const float2 a2 = *reinterpret_cast<const float2 *>(ps + d0 + 4), a3 = *reinterpret_cast<const float2 *>(ps + d0 + 6);
            acc[0] = fmaf(a0.x, c, acc[0]); acc[1] = fmaf(a0.y, c, acc[1]); acc[2] = fmaf(a1.x, c, acc[2]); acc[3] = fmaf(a1.y, c, acc[3]);
            acc[4] = fmaf(a2.x, c, acc[4]); acc[5] = fmaf(a2.y, c, acc[5]); acc[6] = fmaf(a3.x, c, acc[6]); acc[7] = fmaf(a3.y, c, acc[7]);
          }
        }
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; j++) o[j] = ll > 0.0f ? acc[j] / ll : 0.0f;
        actq_emit_block(o, lane, b, bpr, smem);
      }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(CT) : "memory");
  }

  if (group == GROUPS) {
    // ---------------- producer ----------------
    uint32_t u = 0;
    bool ok = true;
    for (int rt = blockIdx.x; rt < tiles && ok; rt += gridDim.x) {
      for (int ch = 0; ch < chunks && ok; ch++, u++) {
        const int s = (int)(u % (uint32_t)stages);
        const uint32_t n = u / (uint32_t)stages;
        int good = 1;
        if (lane == 0) {
          if (n > 0) good = mbar_wait_bounded(empty_bar(s), (n - 1) & 1u, abort_flag) ? 1 : 0;
          if (good) mbar_expect_tx(full_bar(s), 16u * (uint32_t)cb * Q4K_BLOCK_BYTES);
        }
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) { ok = false; break; }
        if (lane < 16) {
          const uint8_t *src = W + ((size_t)(rt * 16 + lane) * bpr + (size_t)ch * cb) * Q4K_BLOCK_BYTES;
          bulk_g2s(smem_u32(smem + L.stages + (uint32_t)s * L.stage_bytes + (uint32_t)lane * L.row_stride), src,
                   (uint32_t)cb * Q4K_BLOCK_BYTES, full_bar(s));
        }
      }
    }
    if (!ok && lane == 0) {  // gave up: let the copies already issued land before the CTA exits
      const uint32_t first = u > (uint32_t)stages ? u - (uint32_t)stages : 0u;
      for (uint32_t v = first; v < u; v++) {
        const uint32_t bar = full_bar((int)(v % (uint32_t)stages)), par = (v / (uint32_t)stages) & 1u;
        for (uint32_t i = 0; i < (1u << 20) && !mbar_try_wait(bar, par); i++) {}
      }
    }
  } else {
    // ---------------- consumers ----------------
    const int g = lane >> 2, t = lane & 3;
    // B operand columns 2l and 2l+1 carry activation limb l (of the even / odd sub-block of a chunk), so
    // lane t reads limb t from its accumulator registers (columns 2t and 2t+1); t == 3 holds nothing.
    const float wt = t == 0 ? 1.0f : (t == 1 ? 256.0f : (t == 2 ? 65536.0f : 0.0f));
    const bool limb_lane = g < 6;  // B fragment columns 6 and 7 are zero
    const uint32_t M4 = 0x0f0f0f0fu, M4H = 0xf0f0f0f0u;
    uint32_t tile_no = (uint32_t)group;
    bool ok = true;
    float *red = reinterpret_cast<float *>(smem + L.red);
    for (int rt = blockIdx.x + group * gridDim.x; rt < tiles && ok; rt += GROUPS * gridDim.x, tile_no += GROUPS) {
      float resA = 0.0f, resB = 0.0f;
      uint32_t u = tile_no * (uint32_t)chunks;
      for (int ch = 0; ch < chunks; ch++, u++) {
        const int s = (int)(u % (uint32_t)stages);
        const uint32_t n = u / (uint32_t)stages;
        if (!mbar_wait_bounded(full_bar(s), n & 1u, abort_flag)) { ok = false; break; }
        // Phase 1: pull this warp's share of the stage (up to TG_MAX_BW super-block columns of the 16 rows)
        // into registers and hand the stage back to the producer at once.  The arithmetic below then runs
        // while the ring slot is already being refilled, so nearly the whole ring stays in flight.
        uint4 ha[TG_MAX_BW], hb[TG_MAX_BW];
        uint2 qa[TG_MAX_BW][4], qb[TG_MAX_BW][4];
#pragma unroll
        for (int i = 0; i < TG_MAX_BW; i++) {
          const int bw = warp + i * TG_CONSUMERS;
          if (bw < cb) {
            const uint8_t *pa = smem + L.stages + (uint32_t)s * L.stage_bytes + (uint32_t)g * L.row_stride + (uint32_t)bw * Q4K_BLOCK_BYTES;
            const uint8_t *pb = pa + 8u * L.row_stride;
            ha[i] = *reinterpret_cast<const uint4 *>(pa);
            hb[i] = *reinterpret_cast<const uint4 *>(pb);
#pragma unroll
            for (int c = 0; c < 4; c++) {
              qa[i][c] = *reinterpret_cast<const uint2 *>(pa + 16 + 32 * c + 8 * t);
              qb[i][c] = *reinterpret_cast<const uint2 *>(pb + 16 + 32 * c + 8 * t);
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(s));
        // Phase 2: arithmetic from registers
#pragma unroll
        for (int i = 0; i < TG_MAX_BW; i++) {
          const int bw = warp + i * TG_CONSUMERS;
          if (bw >= cb) break;
          const int b = ch * cb + bw;
          const Q4KScales sa = q4k_unpack_scales(ha[i].y, ha[i].z, ha[i].w);
          const Q4KScales sb_ = q4k_unpack_scales(hb[i].y, hb[i].z, hb[i].w);
          const uint2 *lb = reinterpret_cast<const uint2 *>(smem + (size_t)b * 1024) + g * 4 + t;  // column g of a chunk
          // One B fragment per chunk serves both of its MMAs: even columns carry the limbs of sub-block 2c
          // (low nibbles, read back from c0 / c2), odd columns those of sub-block 2c+1 (high nibbles, c1 / c3).
          // The high nibbles stay in place (16 * q as a u8); their sums are accumulated apart and divided
          // by 16 exactly at the end, which saves the four shifts per MMA.
          int accA = 0, accB = 0, accAh = 0, accBh = 0;
#pragma unroll
          for (int c = 0; c < 4; c++) {
            uint2 bf = make_uint2(0u, 0u);
            if (limb_lane) bf = lb[c * 32];
            int c0, c1, c2, c3;
            mma_u8s8(c0, c1, c2, c3, qa[i][c].x & M4, qb[i][c].x & M4, qa[i][c].y & M4, qb[i][c].y & M4, bf.x, bf.y);
            (void)c1; (void)c3;
            const uint32_t wsa = c < 2 ? sa.sc03 : sa.sc47, wsb = c < 2 ? sb_.sc03 : sb_.sc47;
            accA += (int)__byte_perm(wsa, 0u, 0x4440u + (uint32_t)((2 * c) & 3)) * c0;
            accB += (int)__byte_perm(wsb, 0u, 0x4440u + (uint32_t)((2 * c) & 3)) * c2;
            int h0, h1, h2, h3;
            mma_u8s8(h0, h1, h2, h3, qa[i][c].x & M4H, qb[i][c].x & M4H, qa[i][c].y & M4H, qb[i][c].y & M4H, bf.x, bf.y);
            (void)h0; (void)h2;
            accAh += (int)__byte_perm(wsa, 0u, 0x4440u + (uint32_t)((2 * c + 1) & 3)) * h1;
            accBh += (int)__byte_perm(wsb, 0u, 0x4440u + (uint32_t)((2 * c + 1) & 3)) * h3;
          }
          const float xs = sm_xscale[b];
          const float2 dA = q4k_d_dmin(ha[i].x), dB = q4k_d_dmin(hb[i].x);
          const float fa = (float)(accA + (accAh >> 4)) * wt;
          const float fb = (float)(accB + (accBh >> 4)) * wt;
          const float s0 = sm_ssum[b * 8 + 2 * t], s1 = sm_ssum[b * 8 + 2 * t + 1];
          const uint32_t mwA = t < 2 ? sa.mn03 : sa.mn47, mwB = t < 2 ? sb_.mn03 : sb_.mn47;
          const int sh = (t & 1) * 16;
          const float mA = fmaf((float)((mwA >> (sh + 8)) & 0xffu), s1, (float)((mwA >> sh) & 0xffu) * s0);
          const float mB = fmaf((float)((mwB >> (sh + 8)) & 0xffu), s1, (float)((mwB >> sh) & 0xffu) * s0);
          resA = fmaf(xs, fmaf(dA.x, fa, -dA.y * mA), resA);
          resB = fmaf(xs, fmaf(dB.x, fb, -dB.y * mB), resB);
        }
      }
      if (!ok) break;
      // sum the eight warps' partial rows through a ring of reduction slots
      resA += __shfl_xor_sync(0xffffffffu, resA, 1);
      resA += __shfl_xor_sync(0xffffffffu, resA, 2);
      resB += __shfl_xor_sync(0xffffffffu, resB, 1);
      resB += __shfl_xor_sync(0xffffffffu, resB, 2);
      const int slot = (int)(tile_no % TG_RED_SLOTS);
      float *rs = red + slot * TG_CONSUMERS * 16;
      if (t == 0) { rs[warp * 16 + g] = resA; rs[warp * 16 + g + 8] = resB; }
      __syncwarp();
      if (lane == 0) mbar_arrive(red_bar(slot));
      // The reducing warp of group g is warp g+1: with 17 warps on four schedulers the producer (warp 16)
      // shares scheduler 0 with consumer warps 0, 4, 8, 12; the extra work goes to other schedulers.
      if (warp == group + 1) {
        if (!mbar_wait_bounded(red_bar(slot), (tile_no / TG_RED_SLOTS) & 1u, abort_flag)) { ok = false; break; }
        if (lane < 16) {
          float v = 0.0f;
#pragma unroll
          for (int w = 0; w < TG_CONSUMERS; w++) v += rs[w * 16 + lane];
          const int row = rt * 16 + lane;
          v *= alpha;
          if constexpr (PUSH) {  // this rank's partial of the row, with the exchange's ticket, into its slot on every rank
            const unsigned ticket = *reinterpret_cast<const volatile unsigned *>(gx.ticket_step) * gx.ticket_stride + 1u + gx.ticket_out;
            const size_t off = dp_tp_slot_offset((unsigned)gx.parity_out, gx.rank) + (size_t)row;
#pragma unroll
            for (int r = 0; r < 8; r++)  // (static indices: a run-time index would copy the parameter block to local memory)
              if (r < gx.nr) handoff_put(gx.area[r] + off, v, ticket);
          } else if constexpr (SILU_OUT) {
            // lanes 0..7 hold gate rows 8 rt .. 8 rt + 7, lanes 8..15 their up rows (the rows are stored in that order)
            const float u = __shfl_down_sync(0x0000ffffu, v, 8);
            if (lane < 8) {
              const float cl = fminf(fmaxf(v, -15.0f), 15.0f);
              const float a = (v * (1.0f / (1.0f + expf(-cl)))) * u;
              if constexpr (sizeof(OutT) == 4) y[rt * 8 + lane] = a; else y[rt * 8 + lane] = __float2half_rn(a);
            }
          } else {
            if (residual) v += residual[row];
            if constexpr (sizeof(OutT) == 4) y[row] = v; else y[row] = __float2half_rn(v);
          }
        }
      }
    }
  }
  if (*abort_flag && lane == 0) atomicExch(err, 1);
}

static bool tma_plan(dp_ctx *ctx, int N, int K, int *cb_out, int *stages_out, uint32_t *smem_out) {
  if (!dpk_gemv_q4k_fast_ok(N, K)) return false;
  const int bpr = K / QK_K;
  // chunk = the largest divisor of the row's block count whose stage (16 padded row pieces) stays
  // under 56 KB: long per-row copies keep the number of bulk-copy requests per byte low
  const int limit = 56 * 1024;
  int cb = 0;
  for (int c = bpr; c >= 1; c--)
    if (bpr % c == 0 && c <= TG_MAX_BW * TG_CONSUMERS && 16 * (c * Q4K_BLOCK_BYTES + TG_ROW_PAD) <= limit) { cb = c; break; }
  if (cb == 0) return false;
  size_t budget = (size_t)227 * 1024;
  if (budget > ctx->smem_optin) budget = ctx->smem_optin;
  int stages = 8;
  while (stages >= 2 && tg_layout(K, cb, stages).total > budget) stages--;
  if (stages < 2) return false;
  *cb_out = cb; *stages_out = stages; *smem_out = tg_layout(K, cb, stages).total;
  return true;
}

template <typename OutT, int GROUPS, int SRC, bool PUSH = false, bool SILU_OUT = false>
static dp_status launch_tma(dp_ctx *ctx, const uint8_t *W, const int8_t *limbs, OutT *y, int N, int K, int cb, int stages,
                            uint32_t smem, float alpha, const float *residual, const GemvSource &gs, const GemvExchange &gx = GemvExchange()) {
  const float *xscale = limbs ? (const float *)(limbs + (size_t)K * 4) : nullptr;
  const float *ssum = limbs ? xscale + K / QK_K : nullptr;
  const int grid = N / 16 < ctx->sm_count ? N / 16 : ctx->sm_count;
  static dp_per_device_once attr;  // per instantiation
  if (attr.pending(ctx->device)) {
    DP_CUDA(ctx, cudaFuncSetAttribute(gemv_q4k_tma_kernel<OutT, GROUPS, SRC, PUSH, SILU_OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr.done(ctx->device);
  }
  DP_LAUNCH(ctx, (gemv_q4k_tma_kernel<OutT, GROUPS, SRC, PUSH, SILU_OUT>), grid, (GROUPS * TG_CONSUMERS + 1) * 32, smem, W, limbs, xscale, ssum, y,
            N, K, cb, stages, alpha, residual, ctx->dev_status, gs, gx);
  return DP_OK;
}

// DP_GEMV_VARIANT=0: the plain-load MMA kernel instead of the TMA-fed one (fallback switch)
static int gemv_variant() {
  static int v = -1;
  if (v < 0) {
    const char *e = getenv("DP_GEMV_VARIANT");
    v = (e && atoi(e) == 0) ? 0 : 2;
  }
  return v;
}

dp_status dpk_gemv_q4k_actq_tma(dp_ctx *ctx, const uint8_t *W, const void *actq, void *y, dp_dtype y_dtype, int N, int K,
                                float alpha, const float *residual, bool *handled) {
  *handled = false;
  int cb, stages;
  uint32_t smem;
  const int variant = gemv_variant();
  if (variant == 0 || !ctx->dev_status || !tma_plan(ctx, N, K, &cb, &stages, &smem)) return DP_OK;
  const int8_t *limbs = (const int8_t *)actq;
  GemvSource gs{};
  if (y_dtype == DP_F32) DP_TRY((launch_tma<float, 2, SRC_DIGITS>(ctx, W, limbs, (float *)y, N, K, cb, stages, smem, alpha, residual, gs)));
  else DP_TRY((launch_tma<__half, 2, SRC_DIGITS>(ctx, W, limbs, (__half *)y, N, K, cb, stages, smem, alpha, residual, gs)));
  *handled = true;
  return DP_OK;
}

// f32 GEMV whose input is produced inside the kernel (mode = SRC_RMSNORM / SRC_SILU / SRC_COMBINE).
// Returns handled = false when the shape has no TMA plan (the caller then runs the separate kernels).
dp_status dpk_gemv_q4k_tma_fused(dp_ctx *ctx, const uint8_t *W, int mode, const float *x, const float *w, float eps, int D,
                                 int splits, float *y, int N, int K, const float *residual, bool *handled, const GemvExchange *gxp) {
  *handled = false;
  const bool silu_out = (mode & SRC_FLAG_SILU_OUT) != 0;
  mode &= ~SRC_FLAG_SILU_OUT;
  if (silu_out && (residual || (mode != SRC_RMSNORM && mode != SRC_XCHG_RMSNORM))) return DP_OK;
  int cb, stages;
  uint32_t smem;
  if (gemv_variant() == 0 || !ctx->dev_status || !tma_plan(ctx, N, K, &cb, &stages, &smem)) return DP_OK;
  if (K > 16 * 2 * QK_K && (mode == SRC_RMSNORM || mode == SRC_XCHG_RMSNORM)) return DP_OK;  // the norm keeps two blocks per warp in registers
  GemvSource gs{};
  gs.x = x; gs.w = w; gs.eps = eps; gs.D = D; gs.splits = splits;
  if (gxp) {
    const GemvExchange &gx = *gxp;
    if ((mode == SRC_XCHG_RMSNORM && K > DP_TP_SLOT_FLOATS) || (gx.push && N > DP_TP_SLOT_FLOATS)) return DP_OK;
    if (mode == SRC_XCHG_RMSNORM && !gx.push && silu_out) DP_TRY((launch_tma<float, 2, SRC_XCHG_RMSNORM, false, true>(ctx, W, nullptr, y, N, K, cb, stages, smem, 1.0f, residual, gs, gx)));
    else if (mode == SRC_XCHG_RMSNORM && !gx.push) DP_TRY((launch_tma<float, 2, SRC_XCHG_RMSNORM>(ctx, W, nullptr, y, N, K, cb, stages, smem, 1.0f, residual, gs, gx)));
    else if (mode == SRC_PLAIN && gx.push) DP_TRY((launch_tma<float, 2, SRC_PLAIN, true>(ctx, W, nullptr, y, N, K, cb, stages, smem, 1.0f, residual, gs, gx)));
    else if (mode == SRC_SILU && gx.push) DP_TRY((launch_tma<float, 2, SRC_SILU, true>(ctx, W, nullptr, y, N, K, cb, stages, smem, 1.0f, residual, gs, gx)));
    else if (mode == SRC_COMBINE && gx.push) DP_TRY((launch_tma<float, 2, SRC_COMBINE, true>(ctx, W, nullptr, y, N, K, cb, stages, smem, 1.0f, residual, gs, gx)));
    else return DP_OK;  // (the schedule uses exactly these three)
    *handled = true;
    return DP_OK;
  }
  if (mode == SRC_XCHG_RMSNORM) return DP_OK;
  if (mode == SRC_RMSNORM && silu_out) DP_TRY((launch_tma<float, 2, SRC_RMSNORM, false, true>(ctx, W, nullptr, y, N, K, cb, stages, smem, 1.0f, residual, gs)));
  else if (mode == SRC_RMSNORM) DP_TRY((launch_tma<float, 2, SRC_RMSNORM>(ctx, W, nullptr, y, N, K, cb, stages, smem, 1.0f, residual, gs)));
  else if (mode == SRC_PLAIN) DP_TRY((launch_tma<float, 2, SRC_PLAIN>(ctx, W, nullptr, y, N, K, cb, stages, smem, 1.0f, residual, gs)));
  else if (mode == SRC_SILU) DP_TRY((launch_tma<float, 2, SRC_SILU>(ctx, W, nullptr, y, N, K, cb, stages, smem, 1.0f, residual, gs)));
  else if (mode == SRC_COMBINE) DP_TRY((launch_tma<float, 2, SRC_COMBINE>(ctx, W, nullptr, y, N, K, cb, stages, smem, 1.0f, residual, gs)));
  else return DP_OK;
  *handled = true;
  return DP_OK;
}
