// Q4_K prefill GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
// Replaces src/gpu/kernels/fused_matmul_q4_batched*.wgsl (:122, one workgroup per 4 rows x 1
// column, every workgroup re-dequantises its weight row) and follows the numerics of the
// reference's tiled prefill kernel fused_matmul_q4_prefill_tiled_f16.wgsl (:118-201): the
// dequantised weight is rounded to f16 in shared memory, the contraction accumulates in f32.
//
//   C[M,N] = alpha * A[M,K] . W[N,K]^T,  A f16 (f32 inputs are cast first), W packed Q4_K.
//
// One CTA owns a 256 (M) x BN (N) output tile, two 128 x BN f32 accumulators in tensor memory.
// Per 64-wide K step and pipeline stage:
//   - warp 0 (one lane) brings the two 128 x 64 f16 activation tiles in with TMA tensor copies
//     (128-byte swizzle, zero fill beyond M);
//   - warps 2..9 read the packed Q4_K bytes of the BN weight rows (32 quant bytes + the block
//     header per row and step), dequantise in registers, w = fma(d*sc, q, -dmin*m) rounded to
//     f16, and store the BN x 64 tile into shared memory in the same 128-byte-swizzled K-major
//     layout the tensor core expects (each weight is dequantised once per CTA);
//   - warp 1 (one lane) issues tcgen05.mma (kind::f16, M=128, N=BN, K=16) for both accumulators
//     and commits to an mbarrier that frees the stage.
// After the last step warps 2..9 read the accumulators back with tcgen05.ld (each warp its own
// 32-lane quarter of tensor memory) and write C as f32 or f16.
// Every mbarrier wait is bounded; on give-up the CTA raises a status word and still frees its
// tensor memory.
#include "common.h"
#include "mbar.cuh"
#include "pdl.cuh"
#include "q4k.cuh"
#include "umma.cuh"

#include <cuda.h>

#include <cstdlib>
#include <map>

namespace {

using namespace umma;

// The activation ring (filled by TMA) and the weight ring (filled by the dequant warps) have their own
// depths and barriers: weight stages are smaller, so more of them fit, and the dequant warps can run
// further ahead of the tensor core than the TMA needs to.
// warp 0: TMA, warp 1: MMA issue, warps 2 .. 2+DQ_WARPS-1: dequant + epilogue (DQ_WARPS % 4 == 0)


struct TcSmem {
  uint32_t a, b, bars, tmem_slot, abort_flag, total;
  uint32_t stage_a, stage_b;
};
// NPROD = products per K step that go into the one f32 accumulator:
//   1  A . f16(W)                                   (weights rounded to f16: the opt-in tiled kernel's numerics)
//   2  A . f16(W) + A . (W - f16(W))                (f16 activations, weights to f32 accuracy)
//   3  A_hi . f16(W) + A_hi . (W - f16(W)) + A_lo . f16(W)   (f32 activations as two f16 halves: the f32-exact product)
// A weight stage then holds the f16 tile and the residue tile, an activation stage the hi and the lo tiles.
__host__ __device__ constexpr inline TcSmem tc_layout(int BN, int SA, int SB, int MT = 2, int NPROD = 1) {
  TcSmem l{};
  l.stage_a = (uint32_t)MT * 128u * 128u * (NPROD == 3 ? 2u : 1u);  // MT 128-row tiles of 64 f16 (x2: hi and lo halves)
  l.stage_b = (uint32_t)BN * 128u * (NPROD >= 2 ? 2u : 1u);
  l.a = 0;
  l.b = (uint32_t)SA * l.stage_a;
  l.bars = l.b + (uint32_t)SB * l.stage_b;  // full_a[SA], full_b[SB], done[max(SA, SB)], accum
  l.tmem_slot = l.bars + (2 * SA + 2 * SB + 1) * 8;
  l.abort_flag = l.tmem_slot + 8;
  l.total = l.abort_flag + 8;
  return l;
}

// MT = number of 128-row accumulators per CTA (output tile 128*MT x BN).
template <int BN, int DQ_WARPS, typename OutT, int SA, int SB, int MT = 2, int NPROD = 1>
__global__ void __launch_bounds__((DQ_WARPS + 2) * 32, 1) gemm_q4k_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                                    const __grid_constant__ CUtensorMap tmap_a_lo,
                                                                    const uint8_t *__restrict__ W, OutT *__restrict__ C, int M,
                                                                    int N, int K, TcAlpha alpha, int *__restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const TcSmem L = tc_layout(BN, SA, SB, MT, NPROD);
  static_assert(MT * BN <= 512, "accumulators exceed tensor memory");
  constexpr uint32_t A_TILES = (uint32_t)MT * 128u * 128u;  // bytes of the hi (or only) activation tiles of a stage
  constexpr uint32_t B_TILE = (uint32_t)BN * 128u;          // bytes of the f16 weight tile of a stage
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * (128 * MT);
  // Split over K (grid.z parts, whole super-blocks each): a problem of few tiles (N = 4096 at M <= 256 is 32)
  // fills the GPU with several CTAs per tile.  Every part writes its own f32 tile; a second kernel adds the
  // parts in a fixed order, so the result does not depend on which CTA finishes first.
  const int k_splits = alpha.k_splits > 1 ? alpha.k_splits : 1;
  const int bpr_row = K / QK_K;                       // super-blocks per weight row
  const int bpr = bpr_row / k_splits, kb0 = (int)blockIdx.z * bpr;  // this CTA's share
  const int num_k = bpr * (QK_K / BK);
  if (k_splits > 1) C += (size_t)blockIdx.z * (size_t)M * (size_t)N;
  // Every CTA walks K in its own rotation (by whole super-blocks).  All CTAs of a grid row need the same
  // activation tiles; in lockstep they would all ask the same few L2 lines for them at the same time, and
  // the L2 slices holding those lines, not the tensor pipe, would set the pace of every K step.
  const int rot_b = (int)(blockIdx.x % (unsigned)bpr);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L.abort_flag);
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L.tmem_slot);
  const uint32_t bars = smem_u32(smem + L.bars);
  // One "K step done" barrier per step, in a ring of SD, frees both the activation stage and the weight
  // stage of that step: the MMA thread commits once per step.  (tcgen05.commit is served at about one per
  // 500-600 cycles; with one commit per ring and step, two per step, the commits and not the tensor pipe
  // set the pace of every K step.)  The producer of stage ring X (depth SX) waits, before it refills the
  // stage of step kt, for done(kt - SX); SD >= SX keeps that barrier from being committed again first.
  constexpr int SD = SA > SB ? SA : SB;
  auto full_a = [&](int s) { return bars + 8u * (uint32_t)s; };
  auto full_b = [&](int s) { return bars + 8u * (uint32_t)(SA + s); };
  auto done = [&](int s) { return bars + 8u * (uint32_t)(SA + SB + s); };
  const uint32_t accum_bar = bars + 8u * (uint32_t)(SA + SB + SD);
  constexpr uint32_t TMEM_COLS = 512;  // two accumulators of BN columns, rounded up to a power of two

  pdl_launch();
  pdl_wait();
  if (tid == 0) {
    for (int s = 0; s < SA; s++) mbar_init(full_a(s), 1);
    for (int s = 0; s < SB; s++) mbar_init(full_b(s), DQ_WARPS);
    for (int s = 0; s < SD; s++) mbar_init(done(s), 1);
    mbar_init(accum_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {  // tensor-memory allocation is a warp-wide operation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem + L.tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- activation tiles: TMA ----------------
    if (lane == 0) {
      for (int kt = 0; kt < num_k; kt++) {
        const int s = kt % SA;
        if (kt >= SA && !mbar_wait_bounded(done((kt - SA) % SD), (uint32_t)((kt - SA) / SD) & 1u, abort_flag)) break;
        mbar_expect_tx(full_a(s), L.stage_a);
        const uint32_t dst = smem_u32(smem + L.a + (uint32_t)s * L.stage_a);
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
          tma_load_2d(dst + (uint32_t)mt * 128u * 128u, &tmap_a, ((kb0 + ((kt >> 2) + rot_b) % bpr) * 4 + (kt & 3)) * BK, m0 + 128 * mt, full_a(s));
          if constexpr (NPROD == 3)
            tma_load_2d(dst + A_TILES + (uint32_t)mt * 128u * 128u, &tmap_a_lo, ((kb0 + ((kt >> 2) + rot_b) % bpr) * 4 + (kt & 3)) * BK, m0 + 128 * mt, full_a(s));
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issue ----------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(128, BN);
      bool ok = true;
      for (int kt = 0; kt < num_k && ok; kt++) {
        const int sa = kt % SA, sb = kt % SB;
        if (!mbar_wait_bounded(full_a(sa), (uint32_t)(kt / SA) & 1u, abort_flag)) { ok = false; break; }
        if (!mbar_wait_bounded(full_b(sb), (uint32_t)(kt / SB) & 1u, abort_flag)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_u32(smem + L.a + (uint32_t)sa * L.stage_a);
        const uint32_t b_addr = smem_u32(smem + L.b + (uint32_t)sb * L.stage_b);
#pragma unroll
        for (int k16 = 0; k16 < BK / 16; k16++) {
          const uint64_t bdesc = umma_desc_sw128(b_addr + (uint32_t)k16 * 32u);
          const uint32_t acc = (kt > 0 || k16 > 0) ? 1u : 0u;
#pragma unroll
          for (int mt = 0; mt < MT; mt++) {
            const uint64_t adesc = umma_desc_sw128(a_addr + (uint32_t)mt * 128u * 128u + (uint32_t)k16 * 32u);
            umma_f16(tmem_base + (uint32_t)(mt * BN), adesc, bdesc, idesc, acc);
            if constexpr (NPROD >= 2) umma_f16(tmem_base + (uint32_t)(mt * BN), adesc, umma_desc_sw128(b_addr + B_TILE + (uint32_t)k16 * 32u), idesc, 1u);
            if constexpr (NPROD == 3)
              umma_f16(tmem_base + (uint32_t)(mt * BN), umma_desc_sw128(a_addr + A_TILES + (uint32_t)mt * 128u * 128u + (uint32_t)k16 * 32u), bdesc, idesc, 1u);
          }
        }
        // both stages are free once these MMAs have read them
        umma_commit(done(kt % SD));
      }
      if (ok) umma_commit(accum_bar);
    }
  } else {
    // ---------------- weight tiles: dequantise into swizzled shared memory ----------------
    const int dw = warp - 2;            // 0..7
    const int r8 = lane & 7, oct = lane >> 3;  // row within the 8-row group, byte octet of the 32-byte chunk
    bool ok = true;
    constexpr int RG = BN / 8 / DQ_WARPS;  // 8-row groups per warp
    static_assert(RG >= 1 && RG * DQ_WARPS * 8 == BN, "dequant warps must tile the weight rows");
    constexpr int grp0 = 0;
    // software pipeline at super-block granularity: while the four K steps of block b are dequantised,
    // the header and the four quant pieces of block b+1 are already in flight
    uint4 hdr[RG];
    uint2 qn[RG][4];
    const uint32_t *rowp[RG];
#pragma unroll
    for (int j = 0; j < RG; j++) {
      rowp[j] = reinterpret_cast<const uint32_t *>(W + (size_t)(n0 + (grp0 + dw + j * DQ_WARPS) * 8 + r8) * bpr_row * Q4K_BLOCK_BYTES) + (size_t)kb0 * Q4K_BLOCK_WORDS;
      const uint32_t *blk0 = rowp[j] + (size_t)rot_b * Q4K_BLOCK_WORDS;
      hdr[j] = __ldg(reinterpret_cast<const uint4 *>(blk0));
#pragma unroll
      for (int c = 0; c < 4; c++) qn[j][c] = __ldg(reinterpret_cast<const uint2 *>(blk0 + 4 + 8 * c) + oct);
    }
    for (int kb = 0; kb < bpr && ok; kb++) {
      // rotate the prefetch buffers; decode the block header once for the four K steps.  The four
      // lanes that share a weight row (oct = 0..3) split the work: lane oct decodes sub-blocks 2*oct and
      // 2*oct+1, K step c then takes its two (scale, min) pairs from lane oct == c by shuffle.
      float my_sc0[RG], my_sc1[RG], my_mn0[RG], my_mn1[RG];
      uint2 qcur[RG][4];
#pragma unroll
      for (int j = 0; j < RG; j++) {
        const float2 dd = q4k_d_dmin(hdr[j].x);
        const Q4KScales sc = q4k_unpack_scales(hdr[j].y, hdr[j].z, hdr[j].w);
        const uint32_t sh = (uint32_t)(oct & 1) * 16u;
        const uint32_t scp = ((oct < 2 ? sc.sc03 : sc.sc47) >> sh) & 0xffffu;
        const uint32_t mnp = ((oct < 2 ? sc.mn03 : sc.mn47) >> sh) & 0xffffu;
        my_sc0[j] = __fmul_rn(dd.x, q4k_u8_to_float(scp & 0xffu));
        my_sc1[j] = __fmul_rn(dd.x, q4k_u8_to_float(scp >> 8));
        my_mn0[j] = __fmul_rn(dd.y, q4k_u8_to_float(mnp & 0xffu));
        my_mn1[j] = __fmul_rn(dd.y, q4k_u8_to_float(mnp >> 8));
#pragma unroll
        for (int c = 0; c < 4; c++) qcur[j][c] = qn[j][c];
      }
      if (kb + 1 < bpr) {
#pragma unroll
        for (int j = 0; j < RG; j++) {
          const uint32_t *blk = rowp[j] + (size_t)((kb + 1 + rot_b) % bpr) * Q4K_BLOCK_WORDS;
          hdr[j] = __ldg(reinterpret_cast<const uint4 *>(blk));
#pragma unroll
          for (int c = 0; c < 4; c++) qn[j][c] = __ldg(reinterpret_cast<const uint2 *>(blk + 4 + 8 * c) + oct);
        }
      }
      // A weight ring of eight stages is filled a whole super-block at a time: the four stage waits, the
      // proxy fence and the arrives are paid once per four K steps, and the four dequantisations are
      // independent instruction streams (shallower rings synchronise every K step).
      constexpr bool BLOCK_SYNC = SB >= 8 && SB % 4 == 0;
      if constexpr (BLOCK_SYNC) {
        bool stages_free = true;
#pragma unroll
        for (int chunk = 0; chunk < 4; chunk++) {
          const int kt = kb * 4 + chunk;
          if (kt >= SB) stages_free = stages_free && mbar_wait_bounded(done((kt - SB) % SD), (uint32_t)((kt - SB) / SD) & 1u, abort_flag);
        }
        if (!__all_sync(0xffffffffu, stages_free)) { ok = false; break; }
      }
#pragma unroll
      for (int chunk = 0; chunk < 4; chunk++) {
        const int kt = kb * 4 + chunk;
        const int s = kt % SB;
        if constexpr (!BLOCK_SYNC) {
          bool stage_free = true;
          if (kt >= SB) stage_free = mbar_wait_bounded(done((kt - SB) % SD), (uint32_t)((kt - SB) / SD) & 1u, abort_flag);
          if (!__all_sync(0xffffffffu, stage_free)) { ok = false; break; }  // leave together: the shuffles below name every lane
        }
        uint8_t *bt = smem + L.b + (uint32_t)s * L.stage_b;
        const int src_lane = (chunk << 3) | r8;
#pragma unroll
        for (int j = 0; j < RG; j++) {
          const uint2 q = qcur[j][chunk];
          const float s_lo = __shfl_sync(0xffffffffu, my_sc0[j], src_lane), s_hi = __shfl_sync(0xffffffffu, my_sc1[j], src_lane);
          const float m_lo = __shfl_sync(0xffffffffu, my_mn0[j], src_lane), m_hi = __shfl_sync(0xffffffffu, my_mn1[j], src_lane);
          // nibble -> f32 without the conversion pipe: PRMT builds the float 2^23 + q from a byte
          uint32_t lo[4], hi[4], rlo[4], rhi[4];
          (void)rlo; (void)rhi;
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const uint32_t word = i < 2 ? q.x : q.y;
            const uint32_t wl = word & 0x0f0f0f0fu, wh = (word >> 4) & 0x0f0f0f0fu;
            const uint32_t sel0 = (i & 1) ? 0x7442u : 0x7440u, sel1 = (i & 1) ? 0x7443u : 0x7441u;
            const float ql0 = __uint_as_float(__byte_perm(wl, 0x4B000000u, sel0)) - 8388608.0f;
            const float ql1 = __uint_as_float(__byte_perm(wl, 0x4B000000u, sel1)) - 8388608.0f;
            const float qh0 = __uint_as_float(__byte_perm(wh, 0x4B000000u, sel0)) - 8388608.0f;
            const float qh1 = __uint_as_float(__byte_perm(wh, 0x4B000000u, sel1)) - 8388608.0f;
            const float wl0 = __fmaf_rn(s_lo, ql0, -m_lo), wl1 = __fmaf_rn(s_lo, ql1, -m_lo);
            const float wh0 = __fmaf_rn(s_hi, qh0, -m_hi), wh1 = __fmaf_rn(s_hi, qh1, -m_hi);
            lo[i] = tc_pack_hi(wl0, wl1);
            hi[i] = tc_pack_hi(wh0, wh1);
            if constexpr (NPROD >= 2) { rlo[i] = tc_pack_lo(wl0, wl1, lo[i]); rhi[i] = tc_pack_lo(wh0, wh1, hi[i]); }
          }
          // row r of an 8-row group: 16-byte chunk c lives at chunk (c ^ r) of the 128-byte line
          uint8_t *line = bt + (uint32_t)(grp0 + dw + j * DQ_WARPS) * 1024u + (uint32_t)r8 * 128u;
          const uint32_t off_lo = ((uint32_t)oct ^ (uint32_t)r8) << 4, off_hi = ((uint32_t)(oct + 4) ^ (uint32_t)r8) << 4;
          *reinterpret_cast<uint4 *>(line + off_lo) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
          *reinterpret_cast<uint4 *>(line + off_hi) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
          if constexpr (NPROD >= 2) {  // the residue tile, same layout, behind the f16 tile
            *reinterpret_cast<uint4 *>(line + B_TILE + off_lo) = make_uint4(rlo[0], rlo[1], rlo[2], rlo[3]);
            *reinterpret_cast<uint4 *>(line + B_TILE + off_hi) = make_uint4(rhi[0], rhi[1], rhi[2], rhi[3]);
          }
        }
        if constexpr (!BLOCK_SYNC) {
          // generic-proxy stores -> visible to the tensor core
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(full_b(s));
        }
      }
      if constexpr (BLOCK_SYNC) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
#pragma unroll
          for (int chunk = 0; chunk < 4; chunk++) mbar_arrive(full_b((kb * 4 + chunk) % SB));
        }
      }
    }
    // ---------------- epilogue: tensor memory -> registers -> shared memory -> C ----------------
    // Staged through the idle operand rings and copied out along the rows, like the two-SM kernel's.
    const bool accum_ready = ok && mbar_wait_bounded(accum_bar, 0u, abort_flag);
    const bool go = __all_sync(0xffffffffu, accum_ready);  // tcgen05.ld is warp-wide: enter together or not at all
    if (go) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    {
      constexpr int ET = DQ_WARPS * 32;  // epilogue threads
      static_assert(128 * (BN * (int)sizeof(OutT) + 16) <= MT * 128 * 128 * SA * (NPROD == 3 ? 2 : 1) + BN * 128 * SB * (NPROD >= 2 ? 2 : 1),
                    "the output tile of a pass must fit the idle operand rings");
      const int quad = warp & 3;         // the 32 TMEM lanes this warp may read
      const int half = dw >> 2;          // DQ_WARPS/4 warps share a quarter and split the column groups
      constexpr int GROUPS = BN / 32;
      constexpr uint32_t row_bytes = (uint32_t)BN * (uint32_t)sizeof(OutT), row_pitch = row_bytes + 16u;
      uint8_t *stage = smem + L.a;
      const int et = tid - 64;
#pragma unroll 1
      for (int mt = 0; mt < MT; mt++) {
        const int row0 = m0 + mt * 128;
        if (go) {
          const int lrow = quad * 32 + lane;
          const int row = row0 + lrow;
          const float arow = (alpha.row_scale && row < M) ? alpha.value * __ldg(alpha.row_scale + row) : alpha.value;
#pragma unroll 1
          for (int cg = half; cg < GROUPS; cg += DQ_WARPS / 4) {
            uint32_t r[32];
            tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(mt * BN + cg * 32), r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            uint8_t *dst = stage + (uint32_t)lrow * row_pitch + (uint32_t)cg * 32u * (uint32_t)sizeof(OutT);
            if (sizeof(OutT) == 4 && alpha.silu_out) {
              float o[16];
              tc_silu_group(r, arow, o);
              tc_silu_group(r + 16, arow, o + 8);
              float4 *d4 = reinterpret_cast<float4 *>(stage + (uint32_t)lrow * row_pitch + (uint32_t)cg * 64u);
#pragma unroll
              for (int i = 0; i < 4; i++) d4[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
            } else if constexpr (sizeof(OutT) == 4) {
#pragma unroll
              for (int i = 0; i < 32; i += 4)
                *reinterpret_cast<float4 *>(dst + 4 * i) = make_float4(__uint_as_float(r[i]) * arow, __uint_as_float(r[i + 1]) * arow,
                                                                       __uint_as_float(r[i + 2]) * arow, __uint_as_float(r[i + 3]) * arow);
            } else {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint32_t p[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                  const __half2 h = __floats2half2_rn(__uint_as_float(r[i + 2 * j]) * arow, __uint_as_float(r[i + 2 * j + 1]) * arow);
                  p[j] = *reinterpret_cast<const uint32_t *>(&h);
                }
                *reinterpret_cast<uint4 *>(dst + 2 * i) = make_uint4(p[0], p[1], p[2], p[3]);
              }
            }
          }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(ET) : "memory");  // the tile of these 128 rows is staged
        if (go) {
          const int fold = (sizeof(OutT) == 4 && alpha.silu_out) ? 2 : 1;  // silu(gate) * up: half the columns
          const int cpr = (int)(row_bytes >> 4) / fold;  // 16-byte chunks per row
          const int total = 128 * cpr;
          const size_t n_out = (size_t)(N / fold);
          char *cbase = reinterpret_cast<char *>(C + (size_t)row0 * n_out + (size_t)(n0 / fold));
#pragma unroll 2
          for (int c = et; c < total; c += ET) {
            const int lrow = c / cpr, ch = c - lrow * cpr;
            if (row0 + lrow >= M) break;  // rows grow with c
            uint4 v = *reinterpret_cast<const uint4 *>(stage + (uint32_t)lrow * row_pitch + ((uint32_t)ch << 4));
            char *g = cbase + (size_t)lrow * n_out * sizeof(OutT) + ((size_t)ch << 4);
            *reinterpret_cast<uint4 *>(g) = v;
          }
        }
        if (mt + 1 < MT) asm volatile("bar.sync 1, %0;" ::"r"(ET) : "memory");  // the stage is free for the next 128 rows
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
  if (*abort_flag && tid == 0) atomicExch(err, 2);
}

// =================================================================================================
// Two-SM variant: tcgen05.mma.cta_group::2
// =================================================================================================
// A cluster of two CTAs owns a 512 x BN output tile.  Each MMA is 256 x BN x 16 across the pair: CTA r
// holds rows r*128 .. r*128+127 of the 256 in its own tensor memory, supplies those rows of A from its
// own shared memory and HALF of the B tile (BN/2 weight rows) from its own shared memory; the tensor
// cores fetch the other half from the peer.  So every CTA dequantises only BN/2 weight rows per K step
// (a quarter of the 1-SM kernel's work per output), writes half as much B into shared memory, and B is
// read from shared memory once per pair.  Two passes (rows 0..255 and 256..511 of the tile) share each
// B stage.  CTA 0 issues all MMAs; all "stage full" barriers live in CTA 0 (CTA 1's TMA and dequant
// warps signal them across the cluster), "stage free" and "accumulators ready" are multicast to both.
__device__ __forceinline__ void umma_f16_2sm(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit_2sm(uint32_t bar) {  // arrives on this barrier offset in both CTAs
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"((uint16_t)3)
               : "memory");
}
// tensor copy into this CTA's shared memory whose completion bytes are counted on a barrier of CTA 0
__device__ __forceinline__ void tma_load_2d_2sm(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr)
               : "memory");
}

// The tile width is a run-time value (a multiple of 16 up to BNMAX): the first `wide_tiles` clusters of a
// grid row take `bn_wide` columns, the others `bn_narrow`.  With 28 tiles of 176 and 46 of 160 columns the
// 74 clusters of a B200 cover N = 12288 in one even wave, where uniform 256-wide tiles fill only 48.
// PS = passes: 256-row MMAs per pair tile (output tile 256*PS x bn).  One pass halves the activation bytes
// per stage, which buys twice as many stages for the same shared memory.
template <int BNMAX, typename OutT, int SA, int SB, int CH, int PS, int NPROD = 1>
__global__ void __launch_bounds__((BNMAX / 16 + 2) * 32, 1) gemm_q4k_tc2_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                                  const __grid_constant__ CUtensorMap tmap_a_lo, const uint8_t *__restrict__ W,
                                                                  OutT *__restrict__ C, int M, int N, int K, TcAlpha alpha,
                                                                  int *__restrict__ err, int wide_tiles, int bn_wide, int bn_narrow) {
  constexpr int HBMAX = BNMAX / 2, DQ_WARPS = HBMAX / 8;  // warps 2 .. 2+DQ_WARPS-1: one 8-row group of weights each, then the epilogue
  static_assert(DQ_WARPS % 4 == 0, "the epilogue needs whole sets of four warps (one per 32 tensor-memory lanes)");
  static_assert(PS * BNMAX <= 512, "the accumulators must fit tensor memory");
  static_assert((CH == 1 || CH == 2 || CH == 4) && SB >= 2 * CH, "the weight ring must hold two groups of CH stages");
  const int cluster_x = blockIdx.x >> 1;
  const int bn = cluster_x < wide_tiles ? bn_wide : bn_narrow;  // columns of this pair tile
  const int hb = bn / 2, dq = hb / 8;                            // this CTA's weight rows, its active dequant warps
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const TcSmem L = tc_layout(HBMAX, SA, SB, PS, NPROD);
  constexpr uint32_t A_TILES = (uint32_t)PS * 128u * 128u;  // bytes of the hi (or only) activation tiles of a stage
  constexpr uint32_t B_TILE = (uint32_t)HBMAX * 128u;       // bytes of this CTA's half of the f16 weight tile of a stage
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t rank = cluster_ctarank();
  const int n0 = cluster_x < wide_tiles ? cluster_x * bn_wide : wide_tiles * bn_wide + (cluster_x - wide_tiles) * bn_narrow;
  const int m0 = blockIdx.y * (256 * PS);
  // Split over K (grid.z parts of whole super-blocks, f32 output only): a problem of few pair tiles (N = 4096 at
  // M = 1024 is 32) fills the GPU with several clusters per tile; part z writes its sums to C + z * M * N and
  // splitk_reduce_kernel adds the parts in a fixed order.
  const int k_splits = alpha.k_splits > 1 ? alpha.k_splits : 1;
  const int bpr_row = K / QK_K;
  const int bpr = bpr_row / k_splits, kb0 = (int)blockIdx.z * bpr;
  const int num_k = bpr * (QK_K / BK);
  const int rot_b = cluster_x % bpr;  // K rotation of this pair (see the one-SM kernel)
  if (k_splits > 1) C += (size_t)blockIdx.z * (size_t)M * (size_t)N;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L.abort_flag);
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L.tmem_slot);
  const uint32_t bars = smem_u32(smem + L.bars);
  constexpr int SD = SA > SB ? SA : SB;  // ring of "K step done" barriers, one commit per step (see the one-SM kernel)
  auto full_a = [&](int s) { return bars + 8u * (uint32_t)s; };
  auto full_b = [&](int s) { return bars + 8u * (uint32_t)(SA + s); };
  auto done = [&](int s) { return bars + 8u * (uint32_t)(SA + SB + s); };
  const uint32_t accum_bar = bars + 8u * (uint32_t)(SA + SB + SD);
  constexpr uint32_t TMEM_COLS = 512;

  pdl_launch();
  pdl_wait();
  if (tid == 0) {
    for (int s = 0; s < SA; s++) mbar_init(full_a(s), 1);
    for (int s = 0; s < SD; s++) mbar_init(done(s), 1);
    // "weights full": CTA 0 waits for its own twelve dequant warps plus one arrival relayed from CTA 1,
    // whose twelve warps arrive on CTA 1's own barrier first (one cross-SM arrive per stage, not twelve)
    for (int s = 0; s < SB; s++) mbar_init(full_b(s), rank == 0 ? dq + 1 : dq);
    mbar_init(accum_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {  // the same warp of both CTAs allocates the pair's tensor memory
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem + L.tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist and both allocations are done before anyone signals across
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- activation tiles: this CTA's rows of both passes ----------------
    if (lane == 0) {
      for (int kt = 0; kt < num_k; kt++) {
        const int s = kt % SA;
        if (kt >= SA && !mbar_wait_bounded(done((kt - SA) % SD), (uint32_t)((kt - SA) / SD) & 1u, abort_flag)) break;
        if (rank == 0) mbar_expect_tx(full_a(s), 2u * L.stage_a);  // both CTAs' bytes (PS tiles each) are counted on CTA 0's barrier
        const uint32_t dst = smem_u32(smem + L.a + (uint32_t)s * L.stage_a);
        const uint32_t bar0 = mapa_shared(full_a(s), 0u);
#pragma unroll
        for (int ps = 0; ps < PS; ps++) {
          tma_load_2d_2sm(dst + (uint32_t)ps * 128u * 128u, &tmap_a, ((kb0 + ((kt >> 2) + rot_b) % bpr) * 4 + (kt & 3)) * BK, m0 + ps * 256 + (int)rank * 128, bar0);
          if constexpr (NPROD == 3)
            tma_load_2d_2sm(dst + A_TILES + (uint32_t)ps * 128u * 128u, &tmap_a_lo, ((kb0 + ((kt >> 2) + rot_b) % bpr) * 4 + (kt & 3)) * BK, m0 + ps * 256 + (int)rank * 128, bar0);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issue: CTA 0 only ----------------
    if (lane == 0 && rank == 1) {
      // CTA 1: relay "this CTA's half of the weight stage is written" to CTA 0
      const uint32_t full_b0 = mapa_shared(full_b(0), 0u);
      for (int kt = 0; kt < num_k; kt++) {
        const int sb = kt % SB;
        if (!mbar_wait_bounded(full_b(sb), (uint32_t)(kt / SB) & 1u, abort_flag)) break;
        mbar_arrive_remote(full_b0 + 8u * (uint32_t)sb);
      }
    }
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc_f16(256, bn);
      bool ok = true;
      for (int kt = 0; kt < num_k && ok; kt++) {
        const int sa = kt % SA, sb = kt % SB;
        if (!mbar_wait_bounded_cluster(full_a(sa), (uint32_t)(kt / SA) & 1u, abort_flag) ||
            !mbar_wait_bounded_cluster(full_b(sb), (uint32_t)(kt / SB) & 1u, abort_flag)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_u32(smem + L.a + (uint32_t)sa * L.stage_a);
        const uint32_t b_addr = smem_u32(smem + L.b + (uint32_t)sb * L.stage_b);
#pragma unroll
        for (int k16 = 0; k16 < BK / 16; k16++) {
          const uint64_t bdesc = umma_desc_sw128(b_addr + (uint32_t)k16 * 32u);
          const uint32_t acc = (kt > 0 || k16 > 0) ? 1u : 0u;
#pragma unroll
          for (int ps = 0; ps < PS; ps++) {
            const uint64_t adesc = umma_desc_sw128(a_addr + (uint32_t)ps * 128u * 128u + (uint32_t)k16 * 32u);
            umma_f16_2sm(tmem_base + (uint32_t)(ps * BNMAX), adesc, bdesc, idesc, acc);
            if constexpr (NPROD >= 2) umma_f16_2sm(tmem_base + (uint32_t)(ps * BNMAX), adesc, umma_desc_sw128(b_addr + B_TILE + (uint32_t)k16 * 32u), idesc, 1u);
            if constexpr (NPROD == 3)
              umma_f16_2sm(tmem_base + (uint32_t)(ps * BNMAX), umma_desc_sw128(a_addr + A_TILES + (uint32_t)ps * 128u * 128u + (uint32_t)k16 * 32u), bdesc, idesc, 1u);
          }
        }
        umma_commit_2sm(done(kt % SD));  // arrives on both CTAs' barrier: their stages of this step are free
      }
      if (ok) umma_commit_2sm(accum_bar);
    }
  } else {
    // ---------------- this CTA's half of the weight tile ----------------
    const int dw = warp - 2;
    const int r8 = lane & 7, oct = lane >> 3;
    bool ok = true;
    const bool active = dw < dq;  // narrower tiles leave the last dequant warps without rows (they still do the epilogue)
    const uint32_t *rowp = reinterpret_cast<const uint32_t *>(W + (size_t)(n0 + (int)rank * hb + (active ? dw : 0) * 8 + r8) * bpr_row * Q4K_BLOCK_BYTES) + (size_t)kb0 * Q4K_BLOCK_WORDS;
    const uint32_t *blk0 = rowp + (size_t)rot_b * Q4K_BLOCK_WORDS;
    uint4 hdr = __ldg(reinterpret_cast<const uint4 *>(blk0));
    uint2 qn[4];
#pragma unroll
    for (int c = 0; c < 4; c++) qn[c] = __ldg(reinterpret_cast<const uint2 *>(blk0 + 4 + 8 * c) + oct);
    for (int kb = 0; kb < bpr && ok && active; kb++) {
      const float2 dd = q4k_d_dmin(hdr.x);
      const Q4KScales sc = q4k_unpack_scales(hdr.y, hdr.z, hdr.w);
      const uint32_t sh = (uint32_t)(oct & 1) * 16u;
      const uint32_t scp = ((oct < 2 ? sc.sc03 : sc.sc47) >> sh) & 0xffffu;
      const uint32_t mnp = ((oct < 2 ? sc.mn03 : sc.mn47) >> sh) & 0xffffu;
      const float my_sc0 = __fmul_rn(dd.x, q4k_u8_to_float(scp & 0xffu)), my_sc1 = __fmul_rn(dd.x, q4k_u8_to_float(scp >> 8));
      const float my_mn0 = __fmul_rn(dd.y, q4k_u8_to_float(mnp & 0xffu)), my_mn1 = __fmul_rn(dd.y, q4k_u8_to_float(mnp >> 8));
      uint2 qcur[4];
#pragma unroll
      for (int c = 0; c < 4; c++) qcur[c] = qn[c];
      if (kb + 1 < bpr) {
        const uint32_t *blk = rowp + (size_t)((kb + 1 + rot_b) % bpr) * Q4K_BLOCK_WORDS;
        hdr = __ldg(reinterpret_cast<const uint4 *>(blk));
#pragma unroll
        for (int c = 0; c < 4; c++) qn[c] = __ldg(reinterpret_cast<const uint2 *>(blk + 4 + 8 * c) + oct);
      }
      // CH K steps per synchronisation: the CH dequantisations are independent instruction streams, so one
      // warp overlaps their latencies, and the stage waits, the proxy fence and the arrives are paid once
      // per CH steps.  (One step at a time, every warp needs about a microsecond per K step whatever the
      // tile width, and that, not the tensor pipe, set the pace.)
#pragma unroll
      for (int c0 = 0; c0 < 4; c0 += CH) {
        bool stage_free = true;
#pragma unroll
        for (int u = 0; u < CH; u++) {
          const int kt = kb * 4 + c0 + u;
          if (kt >= SB) stage_free = stage_free && mbar_wait_bounded(done((kt - SB) % SD), (uint32_t)((kt - SB) / SD) & 1u, abort_flag);
        }
        if (!__all_sync(0xffffffffu, stage_free)) { ok = false; break; }
#pragma unroll
        for (int u = 0; u < CH; u++) {
          const int chunk = c0 + u;
          const int s = (kb * 4 + chunk) % SB;
          const int src_lane = (chunk << 3) | r8;
          const float s_lo = __shfl_sync(0xffffffffu, my_sc0, src_lane), s_hi = __shfl_sync(0xffffffffu, my_sc1, src_lane);
          const float m_lo = __shfl_sync(0xffffffffu, my_mn0, src_lane), m_hi = __shfl_sync(0xffffffffu, my_mn1, src_lane);
          const uint2 q = qcur[chunk];
          uint32_t lo[4], hi[4], rlo[4], rhi[4];
          (void)rlo; (void)rhi;
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const uint32_t word = i < 2 ? q.x : q.y;
            const uint32_t wl = word & 0x0f0f0f0fu, wh = (word >> 4) & 0x0f0f0f0fu;
            const uint32_t sel0 = (i & 1) ? 0x7442u : 0x7440u, sel1 = (i & 1) ? 0x7443u : 0x7441u;
            const float ql0 = __uint_as_float(__byte_perm(wl, 0x4B000000u, sel0)) - 8388608.0f;
            const float ql1 = __uint_as_float(__byte_perm(wl, 0x4B000000u, sel1)) - 8388608.0f;
            const float qh0 = __uint_as_float(__byte_perm(wh, 0x4B000000u, sel0)) - 8388608.0f;
            const float qh1 = __uint_as_float(__byte_perm(wh, 0x4B000000u, sel1)) - 8388608.0f;
            const float wl0 = __fmaf_rn(s_lo, ql0, -m_lo), wl1 = __fmaf_rn(s_lo, ql1, -m_lo);
            const float wh0 = __fmaf_rn(s_hi, qh0, -m_hi), wh1 = __fmaf_rn(s_hi, qh1, -m_hi);
            lo[i] = tc_pack_hi(wl0, wl1);
            hi[i] = tc_pack_hi(wh0, wh1);
            if constexpr (NPROD >= 2) { rlo[i] = tc_pack_lo(wl0, wl1, lo[i]); rhi[i] = tc_pack_lo(wh0, wh1, hi[i]); }
          }
          uint8_t *line = smem + L.b + (uint32_t)s * L.stage_b + (uint32_t)dw * 1024u + (uint32_t)r8 * 128u;
          *reinterpret_cast<uint4 *>(line + (((uint32_t)oct ^ (uint32_t)r8) << 4)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
          *reinterpret_cast<uint4 *>(line + (((uint32_t)(oct + 4) ^ (uint32_t)r8) << 4)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
          if constexpr (NPROD >= 2) {  // the residue tile, same layout, behind this CTA's half of the f16 tile
            *reinterpret_cast<uint4 *>(line + B_TILE + (((uint32_t)oct ^ (uint32_t)r8) << 4)) = make_uint4(rlo[0], rlo[1], rlo[2], rlo[3]);
            *reinterpret_cast<uint4 *>(line + B_TILE + (((uint32_t)(oct + 4) ^ (uint32_t)r8) << 4)) = make_uint4(rhi[0], rhi[1], rhi[2], rhi[3]);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // this CTA's stores -> visible to the tensor cores
        __syncwarp();
        if (lane == 0) {
#pragma unroll
          for (int u = 0; u < CH; u++) mbar_arrive(full_b((kb * 4 + c0 + u) % SB));
        }
      }
    }
    // ---------------- epilogue: this CTA's 128 rows of both passes ----------------
    // Tensor memory hands a thread one output row, so storing from registers puts a warp's 32 lanes on 32
    // different rows (16 bytes each, and as many scattered loads when C is accumulated).  The tile of a
    // pass goes through shared memory instead (the operand rings are idle by now): rows padded by 16 bytes
    // keep the 16-byte shared stores conflict free, and the copy to C runs along the rows, a warp on 512
    // contiguous bytes.  Every warp takes part in the barriers, also one whose bounded wait gave up.
    const bool accum_ready = ok && mbar_wait_bounded(accum_bar, 0u, abort_flag);
    const bool go = __all_sync(0xffffffffu, accum_ready);
    if (go) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    {
      constexpr int ET = DQ_WARPS * 32;  // epilogue threads
      static_assert(128 * (BNMAX * (int)sizeof(OutT) + 16) <= PS * 128 * 128 * SA * (NPROD == 3 ? 2 : 1) + HBMAX * 128 * SB * (NPROD >= 2 ? 2 : 1),
                    "the output tile of a pass must fit the idle operand rings");
      const int quad = warp & 3, set = dw >> 2;  // DQ_WARPS / 4 sets of four warps share the 16-column groups
      const int groups = bn / 16;
      const uint32_t row_bytes = (uint32_t)bn * (uint32_t)sizeof(OutT), row_pitch = row_bytes + 16u;
      uint8_t *stage = smem + L.a;
      const int et = tid - 64;  // 0 .. ET-1
#pragma unroll 1
      for (int ps = 0; ps < PS; ps++) {
        const int row0 = m0 + ps * 256 + (int)rank * 128;  // first row of this CTA's part of the pass
        if (go) {
          const int lrow = quad * 32 + lane;
          const int row = row0 + lrow;
          const float arow = (alpha.row_scale && row < M) ? alpha.value * __ldg(alpha.row_scale + row) : alpha.value;
#pragma unroll 1
          for (int cg = set; cg < groups; cg += DQ_WARPS / 4) {
            uint32_t r[16];
            tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(ps * BNMAX + cg * 16), r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            uint8_t *dst = stage + (uint32_t)lrow * row_pitch + (uint32_t)cg * 16u * (uint32_t)sizeof(OutT);
            if (sizeof(OutT) == 4 && alpha.silu_out) {
              float o[8];
              tc_silu_group(r, arow, o);
              float4 *d4 = reinterpret_cast<float4 *>(stage + (uint32_t)lrow * row_pitch + (uint32_t)cg * 32u);
              d4[0] = make_float4(o[0], o[1], o[2], o[3]);
              d4[1] = make_float4(o[4], o[5], o[6], o[7]);
            } else if constexpr (sizeof(OutT) == 4) {
#pragma unroll
              for (int i = 0; i < 16; i += 4)
                *reinterpret_cast<float4 *>(dst + 4 * i) = make_float4(__uint_as_float(r[i]) * arow, __uint_as_float(r[i + 1]) * arow,
                                                                       __uint_as_float(r[i + 2]) * arow, __uint_as_float(r[i + 3]) * arow);
            } else {
#pragma unroll
              for (int i = 0; i < 16; i += 8) {
                uint32_t pk[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                  const __half2 h = __floats2half2_rn(__uint_as_float(r[i + 2 * j]) * arow, __uint_as_float(r[i + 2 * j + 1]) * arow);
                  pk[j] = *reinterpret_cast<const uint32_t *>(&h);
                }
                *reinterpret_cast<uint4 *>(dst + 2 * i) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              }
            }
          }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(ET) : "memory");  // the pass's tile is staged
        if (go) {
          const int fold = (sizeof(OutT) == 4 && alpha.silu_out) ? 2 : 1;  // silu(gate) * up: half the columns
          const int cpr = (int)(row_bytes >> 4) / fold;  // 16-byte chunks per row
          const int total = 128 * cpr;
          const size_t n_out = (size_t)(N / fold);
          char *cbase = reinterpret_cast<char *>(C + (size_t)row0 * n_out + (size_t)(n0 / fold));
#pragma unroll 2
          for (int c = et; c < total; c += ET) {
            const int lrow = c / cpr, ch = c - lrow * cpr;
            if (row0 + lrow >= M) break;  // rows grow with c
            uint4 v = *reinterpret_cast<const uint4 *>(stage + (uint32_t)lrow * row_pitch + ((uint32_t)ch << 4));
            char *g = cbase + (size_t)lrow * n_out * sizeof(OutT) + ((size_t)ch << 4);
            *reinterpret_cast<uint4 *>(g) = v;
          }
        }
        if (ps + 1 < PS) asm volatile("bar.sync 1, %0;" ::"r"(ET) : "memory");  // the stage is free for the next pass
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();  // neither CTA frees tensor memory or leaves while the peer still uses the pair's resources
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  if (*abort_flag && tid == 0) atomicExch(err, 2);
}

// f32 -> f16 (round to nearest even), the cast the reference inserts in front of an f16 kernel
// (src/gpu/kernels/matmul.js:431-450)
__global__ void cast_f32_f16_kernel(const float *__restrict__ in, __half *__restrict__ out, size_t n) {
  pdl_launch();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = __float2half_rn(in[i]);
}

// f32 row -> f16 row times a power of two, chosen per row so that the largest magnitude lands in [2^13, 2^14):
// activations of any range (FFN intermediates reach 1e7) fit f16 with its full 11-bit significand, and the
// scaling itself is exact.  row_scale[r] receives the inverse factor for the GEMM's epilogue.
// With out_lo, the f16 rounding residue of every scaled element goes there (x * 2^-e = hi + lo to about 22 bits).
__global__ void __launch_bounds__(256) scale_cast_rows_kernel(const float *__restrict__ in, __half *__restrict__ out, __half *__restrict__ out_lo,
                                                              float *__restrict__ row_scale, int K) {
  pdl_launch();
  pdl_wait();
  const float *x = in + (size_t)blockIdx.x * K;
  __half *y = out + (size_t)blockIdx.x * K;
  float mx = 0.0f;
  for (int i = threadIdx.x; i < K; i += 256) mx = fmaxf(mx, fabsf(__ldg(x + i)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  __shared__ float wmax[8];
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = wmax[0];
#pragma unroll
  for (int w = 1; w < 8; w++) mx = fmaxf(mx, wmax[w]);
  // exponent of the row maximum (0 for an all-zero or non-finite row: no scaling)
  int e = 0;
  if (mx > 0.0f && mx < __int_as_float(0x7f800000)) e = (int)((__float_as_uint(mx) >> 23) & 0xffu) - 127 - 13;
  e = max(-100, min(100, e));
  const float down = __int_as_float((uint32_t)(127 - e) << 23), up = __int_as_float((uint32_t)(127 + e) << 23);
  for (int i = threadIdx.x; i < K; i += 256) {
    const float v = __ldg(x + i) * down;
    const __half h = __float2half_rn(v);
    y[i] = h;
    if (out_lo) out_lo[(size_t)blockIdx.x * K + i] = __float2half_rn(v - __half2float(h));
  }
  if (threadIdx.x == 0) row_scale[blockIdx.x] = up;
}

// The same conversion with the row kept in registers (K % 4 == 0, K <= 1024 * NV): one pass over the input, 16-byte
// loads, 8-byte stores.  With norm_w the row is RMS-normalised first (rmsnorm.wgsl:119-187), element for element and
// reduction step for reduction step as rmsnorm_vec_kernel (small_ops.cu) does it for rows of 1024..4096 values, so
// the halves are the ones the two separate kernels produce.
__device__ __forceinline__ float sc_block_sum(float v, float *sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float t = (lane < 8) ? sh[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  __syncthreads();
  return t;
}

template <int NV>
__global__ void __launch_bounds__(256) scale_cast_rows_vec_kernel(const float *__restrict__ in, __half *__restrict__ out, __half *__restrict__ out_lo,
                                                                  float *__restrict__ row_scale, int K, const float *__restrict__ norm_w, float eps) {
  pdl_launch();
  pdl_wait();
  __shared__ float sh[32];
  const size_t base = (size_t)blockIdx.x * K;
  const int n4 = K >> 2;
  float4 v[NV];
#pragma unroll
  for (int i = 0; i < NV; i++) {
    const int idx = threadIdx.x + i * 256;
    v[i] = idx < n4 ? *reinterpret_cast<const float4 *>(in + base + 4 * idx) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  }
  if (norm_w) {
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; i++) ss = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, ss))));
    const float total = sc_block_sum(ss, sh);
    const float inv_rms = 1.0f / sqrtf(total / (float)K + eps);
#pragma unroll
    for (int i = 0; i < NV; i++) {
      const int idx = threadIdx.x + i * 256;
      if (idx < n4) {
        const float4 w = *reinterpret_cast<const float4 *>(norm_w + 4 * idx);
        v[i].x = v[i].x * inv_rms * w.x; v[i].y = v[i].y * inv_rms * w.y; v[i].z = v[i].z * inv_rms * w.z; v[i].w = v[i].w * inv_rms * w.w;
      }
    }
  }
  float mx = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; i++) mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v[i].x), fabsf(v[i].y))), fmaxf(fabsf(v[i].z), fabsf(v[i].w)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = sh[0];
#pragma unroll
  for (int w = 1; w < 8; w++) mx = fmaxf(mx, sh[w]);
  int e = 0;  // exponent of the row maximum (0 for an all-zero or non-finite row: no scaling), as in scale_cast_rows_kernel
  if (mx > 0.0f && mx < __int_as_float(0x7f800000)) e = (int)((__float_as_uint(mx) >> 23) & 0xffu) - 127 - 13;
  e = max(-100, min(100, e));
  const float down = __int_as_float((uint32_t)(127 - e) << 23), up = __int_as_float((uint32_t)(127 + e) << 23);
#pragma unroll
  for (int i = 0; i < NV; i++) {
    const int idx = threadIdx.x + i * 256;
    if (idx >= n4) continue;
    const float s0 = v[i].x * down, s1 = v[i].y * down, s2 = v[i].z * down, s3 = v[i].w * down;
    const __half2 h01 = __halves2half2(__float2half_rn(s0), __float2half_rn(s1)), h23 = __halves2half2(__float2half_rn(s2), __float2half_rn(s3));
    *reinterpret_cast<uint2 *>(out + base + 4 * idx) = make_uint2(*reinterpret_cast<const uint32_t *>(&h01), *reinterpret_cast<const uint32_t *>(&h23));
    if (out_lo) {
      const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
      const __half2 l01 = __halves2half2(__float2half_rn(s0 - f01.x), __float2half_rn(s1 - f01.y));
      const __half2 l23 = __halves2half2(__float2half_rn(s2 - f23.x), __float2half_rn(s3 - f23.y));
      *reinterpret_cast<uint2 *>(out_lo + base + 4 * idx) = make_uint2(*reinterpret_cast<const uint32_t *>(&l01), *reinterpret_cast<const uint32_t *>(&l23));
    }
  }
  if (threadIdx.x == 0) row_scale[blockIdx.x] = up;
}

static dp_status launch_scale_cast(dp_ctx *ctx, const float *A, __half *hi, __half *lo, float *row_scale, int M, int K, const float *norm_w, float eps) {
  if (K % 4 == 0 && K <= 16384 && (((uintptr_t)A | (uintptr_t)hi | (uintptr_t)lo) & 15) == 0 && (!norm_w || (((uintptr_t)norm_w & 15) == 0 && K <= 4096))) {
    if (K <= 4096) DP_LAUNCH(ctx, scale_cast_rows_vec_kernel<4>, (unsigned)M, 256, 0, A, hi, lo, row_scale, K, norm_w, eps);
    else if (K <= 8192) DP_LAUNCH(ctx, scale_cast_rows_vec_kernel<8>, (unsigned)M, 256, 0, A, hi, lo, row_scale, K, norm_w, eps);
    else if (K <= 12288) DP_LAUNCH(ctx, scale_cast_rows_vec_kernel<12>, (unsigned)M, 256, 0, A, hi, lo, row_scale, K, norm_w, eps);
    else DP_LAUNCH(ctx, scale_cast_rows_vec_kernel<16>, (unsigned)M, 256, 0, A, hi, lo, row_scale, K, norm_w, eps);
    return DP_OK;
  }
  if (norm_w) return dp_fail(ctx, DP_ERR_STATE, "matmul: the fused RMSNorm needs rows of 1024..4096 values");
  DP_LAUNCH(ctx, scale_cast_rows_kernel, (unsigned)M, 256, 0, A, hi, lo, row_scale, K);
  return DP_OK;
}

template <int BN, int DQ_WARPS, typename OutT, int SA, int SB, int MT, int NPROD>
dp_status launch_tc(dp_ctx *ctx, const CUtensorMap &tm, const CUtensorMap &tm_lo, const uint8_t *W, OutT *C, int M, int N, int K, TcAlpha alpha) {
  constexpr size_t smem = tc_layout(BN, SA, SB, MT, NPROD).total + 1024;
  static_assert(smem <= 227 * 1024, "rings exceed shared memory");
  auto kernel = gemm_q4k_tc_kernel<BN, DQ_WARPS, OutT, SA, SB, MT, NPROD>;
  DP_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(N / BN, (M + 128 * MT - 1) / (128 * MT), alpha.k_splits > 1 ? alpha.k_splits : 1);
  DP_LAUNCH(ctx, kernel, grid, (DQ_WARPS + 2) * 32, smem, tm, tm_lo, W, C, M, N, K, alpha, ctx->dev_status);
  return DP_OK;
}

// parts of K per output tile for a one-SM launch of `tiles` CTAs: as many as fill the GPU, whole super-blocks, four or more each
static int tc_k_splits(dp_ctx *ctx, int tiles, int K) {
  const int bpr = K / QK_K;
  int best = 1;
  for (int sp = 2; sp <= 8; sp++)
    if (tiles * sp <= ctx->sm_count && bpr % sp == 0 && bpr / sp >= 4) best = sp;
  return best;
}

// two-SM MMA variant: clusters of two CTAs along x, pair tiles of 256 * PS rows
template <typename OutT, int BNMAX, int SA, int SB, int CH, int PS, int NPROD>
dp_status launch_tc_2sm(dp_ctx *ctx, const CUtensorMap &tm, const CUtensorMap &tm_lo, const uint8_t *W, OutT *C, int M, int N, int K, TcAlpha alpha,
                        int tiles, int wide_tiles, int bn_wide, int bn_narrow) {
  constexpr size_t smem = tc_layout(BNMAX / 2, SA, SB, PS, NPROD).total + 1024;
  static_assert(smem <= 227 * 1024, "rings exceed shared memory");
  auto kernel = gemm_q4k_tc2_kernel<BNMAX, OutT, SA, SB, CH, PS, NPROD>;
  DP_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * tiles, (M + 256 * PS - 1) / (256 * PS), alpha.k_splits > 1 ? alpha.k_splits : 1);
  cfg.blockDim = dim3((BNMAX / 16 + 2) * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tm, tm_lo, W, C, M, N, K, alpha, ctx->dev_status, wide_tiles, bn_wide, bn_narrow);
  ctx->launches++;
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return dp_fail(ctx, DP_ERR_CUDA, "launch of gemm_q4k_tc2_kernel failed: %s", cudaGetErrorString(e));
  return DP_OK;
}

// Ring depths per number of products (a stage grows with the products, shared memory does not):
//   two-SM, tiles up to 192 wide:  1: 4 + 8 (four K steps per synchronisation)   2: 3 + 4   3: 2 + 4
//   two-SM, tiles up to 256 wide:  1: 3 + 4   2: 3 + 4   3: 2 + 3 (one K step per synchronisation)
//   one-SM, 192 / 128 wide:        1: 3 + 3   2: 3 + 2 / 3 + 3   3: 2 + 2 / 2 + 3
template <typename OutT, int NPROD>
dp_status dispatch_tc(dp_ctx *ctx, int bn, const CUtensorMap &tm, const CUtensorMap &tm_lo, const uint8_t *W, OutT *C, int M, int N, int K, TcAlpha alpha) {
  // Two-SM kernel (tcgen05.mma.cta_group::2) for M > 256.  On 512 x 256 pair tiles its 256-wide MMAs fetch
  // 8 KB of operands per SM and 128 cycles instead of 10 KB per 96, and the tensor pipe runs about 1.3x
  // faster per SM.  It needs whole waves of 74 clusters to win (at M = 512, 48 uniform tiles of 256 columns
  // occupy 96 SMs), so the tiles are sized to the waves: with R = ceil(M / 512) rows of pair tiles, take the
  // fewest waves of 74 clusters that 256-wide tiles need, then as many column tiles per row as those waves
  // hold, in two widths 16 apart.  N = 12288: M = 512 runs one wave of 28 x 176 + 46 x 160 columns; M = 2048
  // three waves of 55 tiles (53 x 224 + 2 x 208).  Tiles narrower than 128 columns are left to the one-SM
  // kernel (every SM re-reads its activation rows once per tile column, so narrow tiles are bound by L2).
  // Measurements of the alternatives that were tried and dropped: profiles/gemm_q4k_tc__config1.md.
  if (M > 256 && alpha.k_splits > 1 && N % 256 == 0) {  // few pair tiles: uniform 256-wide tiles, several clusters per tile along K
    const int cols = N / 256;
    if constexpr (NPROD == 1) return launch_tc_2sm<OutT, 256, 3, 4, 2, 2, 1>(ctx, tm, tm_lo, W, C, M, N, K, alpha, cols, 0, 256, 256);
    else if constexpr (NPROD == 2) return launch_tc_2sm<OutT, 256, 3, 4, 2, 2, 2>(ctx, tm, tm_lo, W, C, M, N, K, alpha, cols, 0, 256, 256);
    else return launch_tc_2sm<OutT, 256, 2, 3, 1, 2, 3>(ctx, tm, tm_lo, W, C, M, N, K, alpha, cols, 0, 256, 256);
  }
  if (M > 256 && N % 16 == 0) {
    const int clusters = ctx->sm_count / 2, rows = (M + 511) / 512;
    const int waves = (rows * ((N + 255) / 256) + clusters - 1) / clusters;
    int cols = waves * clusters / rows;
    if (cols > N / 96) cols = N / 96;
    if (cols > 0) {
      const int narrow = (N / 16 / cols) * 16;
      const int n_wide = (N - cols * narrow) / 16;  // cols * narrow + 16 * n_wide == N, n_wide < cols
      const int wide = narrow + 16, widest = n_wide ? wide : narrow;
      if (narrow >= 128 && widest <= 192) {
        if constexpr (NPROD == 1) return launch_tc_2sm<OutT, 192, 4, 8, 4, 2, 1>(ctx, tm, tm_lo, W, C, M, N, K, alpha, cols, n_wide, wide, narrow);
        else if constexpr (NPROD == 2) return launch_tc_2sm<OutT, 192, 3, 4, 2, 2, 2>(ctx, tm, tm_lo, W, C, M, N, K, alpha, cols, n_wide, wide, narrow);
        else return launch_tc_2sm<OutT, 192, 2, 4, 2, 2, 3>(ctx, tm, tm_lo, W, C, M, N, K, alpha, cols, n_wide, wide, narrow);
      }
      if (narrow >= 128 && widest <= 256) {
        if constexpr (NPROD == 1) return launch_tc_2sm<OutT, 256, 3, 4, 2, 2, 1>(ctx, tm, tm_lo, W, C, M, N, K, alpha, cols, n_wide, wide, narrow);
        else if constexpr (NPROD == 2) return launch_tc_2sm<OutT, 256, 3, 4, 2, 2, 2>(ctx, tm, tm_lo, W, C, M, N, K, alpha, cols, n_wide, wide, narrow);
        else return launch_tc_2sm<OutT, 256, 2, 3, 1, 2, 3>(ctx, tm, tm_lo, W, C, M, N, K, alpha, cols, n_wide, wide, narrow);
      }
    }
  }
  // one-SM kernel; up to 128 rows (batched decode steps) one 128-row accumulator per CTA, else two
  if (M <= 128) {
    if constexpr (NPROD == 1) {
      if (bn == 192) return launch_tc<192, 12, OutT, 4, 4, 1, 1>(ctx, tm, tm_lo, W, C, M, N, K, alpha);
      return launch_tc<128, 8, OutT, 4, 4, 1, 1>(ctx, tm, tm_lo, W, C, M, N, K, alpha);
    } else if constexpr (NPROD == 2) {
      if (bn == 192) return launch_tc<192, 12, OutT, 4, 3, 1, 2>(ctx, tm, tm_lo, W, C, M, N, K, alpha);
      return launch_tc<128, 8, OutT, 4, 4, 1, 2>(ctx, tm, tm_lo, W, C, M, N, K, alpha);
    } else {
      if (bn == 192) return launch_tc<192, 12, OutT, 3, 2, 1, 3>(ctx, tm, tm_lo, W, C, M, N, K, alpha);
      return launch_tc<128, 8, OutT, 3, 3, 1, 3>(ctx, tm, tm_lo, W, C, M, N, K, alpha);
    }
  }
  if constexpr (NPROD == 1) {
    if (bn == 192) return launch_tc<192, 12, OutT, 3, 3, 2, 1>(ctx, tm, tm_lo, W, C, M, N, K, alpha);
    return launch_tc<128, 8, OutT, 3, 3, 2, 1>(ctx, tm, tm_lo, W, C, M, N, K, alpha);
  } else if constexpr (NPROD == 2) {
    if (bn == 192) return launch_tc<192, 12, OutT, 3, 2, 2, 2>(ctx, tm, tm_lo, W, C, M, N, K, alpha);
    return launch_tc<128, 8, OutT, 3, 3, 2, 2>(ctx, tm, tm_lo, W, C, M, N, K, alpha);
  } else {
    if (bn == 192) return launch_tc<192, 12, OutT, 2, 2, 2, 3>(ctx, tm, tm_lo, W, C, M, N, K, alpha);
    return launch_tc<128, 8, OutT, 2, 3, 2, 3>(ctx, tm, tm_lo, W, C, M, N, K, alpha);
  }
}

}  // namespace

// C = sum of the `splits` partial tiles of a K-split launch, added in a fixed order
// (+ residual, which may be C itself: every element is read and written by the same thread)
__global__ void splitk_reduce_kernel(const float *__restrict__ parts, float *C, size_t n, int splits, const float *residual) {
  pdl_launch();
  pdl_wait();
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (size_t)gridDim.x * blockDim.x * 4) {
    float4 acc = *reinterpret_cast<const float4 *>(parts + i);
    for (int z = 1; z < splits; z++) {
      const float4 v = *reinterpret_cast<const float4 *>(parts + (size_t)z * n + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (residual) {
      const float4 v = *reinterpret_cast<const float4 *>(residual + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4 *>(C + i) = acc;
  }
}

static dp_status gemm_q4k_tc_impl(dp_ctx *ctx, const uint8_t *W, const void *A, dp_dtype a_dtype, void *C, dp_dtype c_dtype, int M,
                                  int N, int K, float alpha, int mode, bool *handled, dpk_tc_fuse *fuse = nullptr) {
  // mode 0: A as given (f32 is cast to f16), weights rounded to f16: one product per K step.
  //      1: f32 rows scaled into f16 range, weights rounded to f16: one product.
  //      2: as 1, three products per K step into the one accumulator, A_hi.W_hi + A_hi.W_lo + A_lo.W_hi with the f16
  //         rounding residues of A and W: the f32-exact product to about 2^-21 of each term (f32 output only).
  //      3: f16 A, two products A.W_hi + A.W_lo: the product with weights kept to f32 accuracy (what the
  //         reference's rule-selected kernel for f16 activations computes, fused_matmul_q4_batched_f16a.wgsl:107);
  //         an f16 output is rounded once, from the f32 accumulator.
  const bool row_scaled = mode == 1 || mode == 2;
  *handled = false;
  static int enabled = -1;
  if (enabled < 0) { const char *e = getenv("DP_GEMM_TC"); enabled = e ? atoi(e) : 1; }
  if (!enabled || !ctx->dev_status) return DP_OK;
  if (K % QK_K || M < 1) return DP_OK;
  int bn = 0;
  if (N % 192 == 0) bn = 192;
  else if (N % 128 == 0) bn = 128;
  if (!bn) return DP_OK;
  EncodeTiledFn encode = get_encode();
  if (!encode) return DP_OK;
  if (mode == 3 && a_dtype != DP_F16) return DP_OK;
  // an RMSNorm folded into the activation conversion: row-scaled f32 rows of 1024..4096 values on the kernels below only
  if (fuse && fuse->norm_w && !(row_scaled && a_dtype == DP_F32 && c_dtype == DP_F32 && M > 64 && K % 4 == 0 && K >= 1024 && K <= 4096 &&
                                 ((uintptr_t)fuse->norm_w & 15) == 0 && ((uintptr_t)A & 15) == 0))
    return DP_OK;
  // up to 64 rows, f32 out, exact weights (modes 2 and 3): the integer-tile kernel (gemm_q4k_tc_rows.cu)
  if (M <= 64 && c_dtype == DP_F32 && ((mode == 2 && a_dtype == DP_F32) || mode == 3)) {
    DP_TRY(dpk_gemm_q4k_tc_rows(ctx, W, A, a_dtype, (float *)C, M, N, K, alpha, handled));
    if (*handled) return DP_OK;
  }

  if (M < 32 && a_dtype == DP_F32) return DP_OK;  // few f32 rows on a shape that kernel does not tile: the CUDA-core kernel
  const __half *a16 = (const __half *)A;
  // The f16 copies of f32 activations live in one scratch allocation of the context, reused in stream order.
  const __half *a_lo = nullptr;
  const float *scales = nullptr;
  if (a_dtype == DP_F32) {
    if (mode == 2 && c_dtype != DP_F32) return DP_OK;
    const size_t a_bytes = ((size_t)M * K * 2 + 255) / 256 * 256;
    DP_TRY(dp_scratch(ctx, &ctx->gemm_scratch, 2 * a_bytes + (size_t)M * 4, "matmul_a_f16"));
    char *base = (char *)ctx->gemm_scratch->dptr;
    a16 = (const __half *)base;
    if (row_scaled) {
      if (mode == 2) a_lo = (const __half *)(base + a_bytes);
      scales = (const float *)(base + 2 * a_bytes);
      DP_TRY(launch_scale_cast(ctx, (const float *)A, (__half *)base, mode == 2 ? (__half *)(base + a_bytes) : (__half *)nullptr,
                               (float *)(base + 2 * a_bytes), M, K, fuse ? fuse->norm_w : nullptr, fuse ? fuse->eps : 0.0f));
    } else {
      size_t n = (size_t)M * K, grid = (n + 255) / 256;
      if (grid > (size_t)ctx->sm_count * 16) grid = (size_t)ctx->sm_count * 16;
      DP_LAUNCH(ctx, cast_f32_f16_kernel, (unsigned)grid, 256, 0, (const float *)A, (__half *)base, n);
    }
  } else if (a_dtype != DP_F16) {
    return DP_OK;
  }
  CUtensorMap tm, tm_lo;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {BK, 128};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = encode(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)a16, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS)  // (without a lo half the second map is a copy of the first; the kernel then never uses it)
    r = encode(&tm_lo, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)(a_lo ? a_lo : a16), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  dp_status st = DP_OK;
  TcAlpha ta = {alpha, scales, 1, 0};
  // few output tiles (one-SM kernel, f32 output): split K over several CTAs per tile, partial tiles in a scratch
  // of the context, summed in a fixed order afterwards
  float *cdst = (float *)C;
  if (r == CUDA_SUCCESS && c_dtype == DP_F32 && M <= 256 && ((size_t)M * N) % 4 == 0) {
    const int tiles = (N / bn) * ((M + (M <= 128 ? 127 : 255)) / (M <= 128 ? 128 : 256));
    const int sp = tc_k_splits(ctx, tiles, K);
    if (sp > 1) {
      DP_TRY(dp_scratch(ctx, &ctx->gemm_split_scratch, (size_t)sp * M * N * 4, "matmul_k_split_parts"));
      ta.k_splits = sp;
      cdst = (float *)ctx->gemm_split_scratch->dptr;
    }
  } else if (r == CUDA_SUCCESS && c_dtype == DP_F32 && M > 256 && N % 256 == 0 && ((size_t)M * N) % 4 == 0) {
    // two-SM kernel on few pair tiles (512 x 256): as many parts of K as keep the clusters within one wave
    const int pair_tiles = ((M + 511) / 512) * (N / 256), clusters = ctx->sm_count / 2, bpr = K / QK_K;
    int sp = 1;
    for (int s2 = 2; s2 <= 8; s2++)
      if (pair_tiles * s2 <= clusters && bpr % s2 == 0 && bpr / s2 >= 4) sp = s2;
    if (sp > 1 && pair_tiles * 2 <= clusters) {
      DP_TRY(dp_scratch(ctx, &ctx->gemm_split_scratch, (size_t)sp * M * N * 4, "matmul_k_split_parts"));
      ta.k_splits = sp;
      cdst = (float *)ctx->gemm_split_scratch->dptr;
    }
  }
  // Optional fusions (f32 output): silu(gate) * up in the epilogue of an unsplit launch, written to fuse->silu_dst
  // [M, N / 2] instead of C; a residual added by the reduction that follows a K-split launch, written to
  // fuse->residual_out (which may be the residual itself).  What was not fused is left to the caller.
  float *c_final = (float *)C;
  const float *red_residual = nullptr;
  if (fuse && r == CUDA_SUCCESS && c_dtype == DP_F32) {
    if (fuse->silu_dst && ta.k_splits == 1 && N % 32 == 0) {
      ta.silu_out = 1;
      cdst = fuse->silu_dst;
      fuse->silu_done = true;
    }
    if (fuse->residual && fuse->residual_out && ta.k_splits > 1) {
      red_residual = fuse->residual;
      c_final = fuse->residual_out;
      fuse->residual_done = true;
    }
  }
  if (r != CUDA_SUCCESS) {
    st = dp_fail(ctx, DP_ERR_CUDA, "matmul: cuTensorMapEncodeTiled failed (%d) for A[%d,%d]", (int)r, M, K);
  } else if (c_dtype == DP_F32) {
    if (mode == 2) st = dispatch_tc<float, 3>(ctx, bn, tm, tm_lo, W, cdst, M, N, K, ta);
    else if (mode == 3) st = dispatch_tc<float, 2>(ctx, bn, tm, tm_lo, W, cdst, M, N, K, ta);
    else st = dispatch_tc<float, 1>(ctx, bn, tm, tm_lo, W, cdst, M, N, K, ta);
    if (st == DP_OK && ta.k_splits > 1) {
      const size_t n = (size_t)M * N;
      size_t grid = (n / 4 + 255) / 256;
      if (grid > (size_t)ctx->sm_count * 8) grid = (size_t)ctx->sm_count * 8;
      DP_LAUNCH(ctx, splitk_reduce_kernel, (unsigned)grid, 256, 0, (const float *)cdst, c_final, n, ta.k_splits, red_residual);
    }
  } else if (c_dtype == DP_F16) {
    if (mode == 3) st = dispatch_tc<__half, 2>(ctx, bn, tm, tm_lo, W, (__half *)C, M, N, K, ta);
    else st = dispatch_tc<__half, 1>(ctx, bn, tm, tm_lo, W, (__half *)C, M, N, K, ta);
  } else {
    st = dp_fail(ctx, DP_ERR_INVALID, "matmul: unsupported output dtype");
  }
  if (st == DP_OK) *handled = true;
  return st;
}

// f32 rows -> f16 halves, rounding residues and per-row inverse scales (see scale_cast_rows_kernel); lo may be null.
dp_status dpk_scale_cast_rows(dp_ctx *ctx, const float *A, __half *hi, __half *lo, float *row_scale, int M, int K) {
  return launch_scale_cast(ctx, A, hi, lo, row_scale, M, K, nullptr, 0.0f);
}

// f16 (or f32, cast to f16) activations.  f16_weights: one product with the dequantised weights rounded to f16,
// the numerics of the reference's opt-in tiled kernel (fused_matmul_q4_prefill_tiled_f16.wgsl:201).  Otherwise,
// for f16 activations, two products that keep the weights to f32 accuracy (the rule-selected kernel's numerics).
dp_status dpk_gemm_q4k_tc(dp_ctx *ctx, const uint8_t *W, const void *A, dp_dtype a_dtype, void *C, dp_dtype c_dtype, int M,
                          int N, int K, float alpha, bool f16_weights, bool *handled) {
  return gemm_q4k_tc_impl(ctx, W, A, a_dtype, C, c_dtype, M, N, K, alpha, (!f16_weights && a_dtype == DP_F16) ? 3 : 0, handled);
}

// f32 activations of any range on the tensor-core kernel: every row is scaled into f16 range by a power
// of two and scaled back in the epilogue.  passes == 1: activations and weights rounded to f16 (11-bit
// significands, what the reference's tiled f16 prefill kernel computes).  passes == 3: the rounding
// residues of both are multiplied in as well (three products per K step in one kernel), which gives the
// f32-exact product to f32 accuracy.
dp_status dpk_gemm_q4k_tc_rowscaled(dp_ctx *ctx, const uint8_t *W, const float *A, float *C, int M, int N, int K, float alpha, int passes,
                                    bool *handled, dpk_tc_fuse *fuse) {
  if (fuse) fuse->silu_done = fuse->residual_done = false;
  return gemm_q4k_tc_impl(ctx, W, A, DP_F32, C, DP_F32, M, N, K, alpha, passes == 3 ? 2 : 1, handled, fuse);
}
