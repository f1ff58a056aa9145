// Q4_K GEMM for a SMALL number of activation rows (batched decode steps, 2..64 rows) on the tcgen05 tensor
// cores, WITHOUT dequantising to floating point on the CUDA cores.
//
// Replaces src/gpu/kernels/fused_matmul_q4_batched*.wgsl for the batched decode step.
//
//   C[M, N] = alpha * A[M, K] . W[N, K]^T,   M <= 64, N % 128 == 0, K % 256 == 0, f32 out.
//
// A Q4_K weight is  w = d * (sc * q) - dmin * m  with q a 4-bit and sc, m 6-bit integers per 32-weight sub-block
// and d, dmin f16 per 256-weight super-block.  sc * q <= 945 is an integer that f16 holds EXACTLY, so for every
// super-block the tensor core multiplies an integer tile and the f16 scales are applied once per super-block:
//
//   y[n, m] = sum over super-blocks B of  d[n,B] * P[n,m,B] - dmin[n,B] * Pm[n,m,B]
//   P  = sum over the 256 k of B   (sc*q)[n,k] * x[m,k]            four K steps of 64, f32 accumulate in tensor memory
//   Pm = sum over the 8 sub-blocks (64*m)[n,s] * (xsum[m,s] / 64)   one K step of 16: the sums' f16 halves in columns
//        0..7 and their rounding residues in columns 8..15, the codes in both (xsum = sub-block sums of x, from a
//        pre-pass; divided by 64 so that they fit f16)
//
// The CUDA cores only widen nibbles to f16 integers (one byte permute and one half2 FMA per two weights) and,
// once per super-block, read P and Pm back from tensor memory (M / 128 values per weight) to apply d and dmin.
// (Taking the min term on the CUDA cores instead, 8 FMAs per output and super-block, made the drain warps the
// pace of the whole kernel: 4700 cycles per super-block against 2400 of MMAs.)  The weights enter exactly; f32 activations enter as two f16
// halves (x * 2^-e = hi + lo, two MMAs per K step), f16 activations as they are.  The weights are the MMA's M
// side (128 rows per tile), the activation rows its N side (32 or 64 columns), so no tensor-core work is spent
// on padding the batch to 128 rows.
//
// A tcgen05.commit costs about as much tensor-pipe time as eight of these small MMAs (measured: with one
// commit per 64-wide K step the kernel ran at 1300 cycles per step for 520 cycles of MMAs), so a pipeline
// stage is TWO K steps (128 of K) and the only commits are the two "stage consumed" ones per super-block; the
// second doubles as "P is complete".
//
// Work split ("stream K"): one CTA per SM.  The work is cut into units of one weight tile x one super-block
// column; the tiles x K/256 units are dealt out in order, the same number (+-1) to every CTA.  A CTA's units are
// contiguous: the tail of one tile, whole tiles, the head of another.  A run of units inside one tile is a
// segment: a segment that covers the whole of K writes C, any other writes its partial sums to its own slot of
// a scratch buffer, and a second kernel adds the slots of every split tile in CTA order (fixed order: the
// result does not depend on timing).
//
// Roles: warp 0 brings the activation tiles in with TMA, warp 1 issues the MMAs, eight warps build the integer
// weight tiles and eight others drain tensor memory (two accumulator buffers, so the drain of super-block B
// runs while B + 1 is multiplied, and the builders never wait for a drain).  Every mbarrier wait is bounded; on give-up the CTA raises the status word and
// still frees its tensor memory.
#include "common.h"
#include "mbar.cuh"
#include "pdl.cuh"
#include "q4k.cuh"
#include "umma.cuh"

namespace {

using namespace umma;

constexpr int TILE_N = 128;  // weight rows per tile (the MMA's M)
constexpr int BUILDERS = 8;  // tile-building warps: two 8-row groups each
constexpr int DRAINERS = 8;  // tensor-memory drain warps: two per lane quarter
constexpr int DQW = BUILDERS + DRAINERS;
constexpr int STAGES = 3;    // operand ring depth; a stage holds two K steps, a super-block takes two stages

__host__ __device__ inline long rows_unit_begin(long c, long units, long ctas) { return c * units / ctas; }
// the CTA that owns unit u: the largest c with unit_begin(c) <= u
__host__ __device__ inline int rows_unit_owner(long u, long units, long ctas) { return (int)(((u + 1) * ctas + units - 1) / units - 1); }

struct RowsPlan {
  int tiles, bpr, ctas, max_segs;  // max_segs: most tiles a CTA's run of units can touch
  long units;
};

// bounded wait that backs off between polls: for the drain warps, whose spinning would otherwise take issue slots
// from the tile-building warps of the same schedulers
__device__ __forceinline__ bool mbar_wait_bounded_backoff(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  for (uint32_t i = 0; i < (1u << 20); i++) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(100);
    if ((i & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

template <int BM, bool LO>
struct RowsSmem {
  static constexpr uint32_t w_tile = TILE_N * 128u;                  // one 128 x 64 f16 tile (one K step)
  static constexpr uint32_t stage_w = 2u * w_tile;
  static constexpr uint32_t x_tile = BM * 128u;
  static constexpr uint32_t x_step = x_tile * (LO ? 2u : 1u);        // hi halves, lo halves of one K step
  static constexpr uint32_t stage_x = 2u * x_step;
  // min-term operands: one 64-wide tile each whose four 16-wide K slices serve four consecutive super-blocks
  static constexpr uint32_t wm_tile = TILE_N * 128u, xm_tile = BM * 128u;
  static constexpr uint32_t w = 0, x = STAGES * stage_w, wm = x + STAGES * stage_x, xm = wm + wm_tile, bars = xm + xm_tile;
  // full_w[S], full_x[S], done[S], tmem_empty[2]
  static constexpr uint32_t tmem_slot = bars + (3 * STAGES + 2) * 8, abort_flag = tmem_slot + 8, total = abort_flag + 8;
};

// One block per activation row.  f32 rows: the row is scaled by a power of two so that its largest magnitude
// lands in [2^13, 2^14) and split into an f16 half and an f16 rounding residue (x * 2^-e = hi + lo to about 22
// bits; row_scale receives 2^e for the epilogue).  Both kinds: the f32 sums of the (scaled) row over every
// 32-wide sub-block, divided by 64, as f16 half and rounding residue: 16 halves per super-block.
template <typename AT>
__global__ void __launch_bounds__(1024) rows_prepass_kernel(const AT *__restrict__ in, __half *__restrict__ hi, __half *__restrict__ lo,
                                                           float *__restrict__ row_scale, __half *__restrict__ xs16, int K) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const AT *x = in + (size_t)row * K;
  float down = 1.0f;
  if constexpr (sizeof(AT) == 4) {
    float mx = 0.0f;
    for (int i = tid; i < K; i += 1024) mx = fmaxf(mx, fabsf(__ldg(x + i)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    __shared__ float wmax[32];
    if (lane == 0) wmax[warp] = mx;
    __syncthreads();
    mx = wmax[0];
#pragma unroll
    for (int w = 1; w < 32; w++) mx = fmaxf(mx, wmax[w]);
    int e = 0;  // exponent of the row maximum (0 for an all-zero or non-finite row: no scaling)
    if (mx > 0.0f && mx < __int_as_float(0x7f800000)) e = (int)((__float_as_uint(mx) >> 23) & 0xffu) - 127 - 13;
    e = max(-100, min(100, e));
    down = __int_as_float((uint32_t)(127 - e) << 23);
    if (tid == 0) row_scale[row] = __int_as_float((uint32_t)(127 + e) << 23);
  }
  const int nsub = K / 32;
  for (int s = warp; s < nsub; s += 32) {
    float v;
    if constexpr (sizeof(AT) == 4) {
      v = __ldg(x + s * 32 + lane) * down;
      const __half h = __float2half_rn(v);
      hi[(size_t)row * K + s * 32 + lane] = h;
      lo[(size_t)row * K + s * 32 + lane] = __float2half_rn(v - __half2float(h));
    } else {
      v = __half2float(x[s * 32 + lane]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) {  // [row][super-block][8 halves | 8 residues]
      const float q = v * 0.015625f;
      const __half h = __float2half_rn(q);
      __half *at = xs16 + ((size_t)row * (nsub >> 3) + (s >> 3)) * 16 + (s & 7);
      at[0] = h;
      at[8] = __float2half_rn(q - __half2float(h));
    }
  }
}

// The same pre-pass with the operation that precedes the projection in the layer folded in (f32 rows, up to 32 of them).
// One block per activation row.  f32 rows: the row is scaled by a power of two so that its largest magnitude
// lands in [2^13, 2^14) and split into an f16 half and an f16 rounding residue (x * 2^-e = hi + lo to about 22
// bits; row_scale receives 2^e for the epilogue).  Both kinds: the f32 sums of the (scaled) row over every
// 32-wide sub-block, divided by 64, as f16 half and rounding residue: 16 halves per super-block.
// PRE (f32 rows) applies the operation that precedes the projection in the layer, so that it costs no kernel
// and no pass over global memory of its own:
//   1  x = rmsnorm(in) * w      (rmsnorm.wgsl:119-187: x * 1/sqrt(mean(x^2) + eps) * w)
//   2  x = silu(gate) * up      (silu.wgsl:98-104, sigmoid argument clamped to +-15); `in` rows hold 2K values,
//                               eight gate values, then their eight up values, and so on
// A thread keeps its share of the row (elements tid, tid + 1024, ...; up to PREPASS_MAXV of them, K <= 16384) in
// registers, so the row is read from memory once whatever PRE is; a warp then holds 32 consecutive elements of
// every round, i.e. one sub-block, and sums it with shuffles.
constexpr int PREPASS_MAXV = 16;
template <typename AT, int PRE>
__global__ void __launch_bounds__(1024) rows_prepass_fused_kernel(const AT *__restrict__ in, __half *__restrict__ hi, __half *__restrict__ lo,
                                                                  float *__restrict__ row_scale, __half *__restrict__ xs16, int K,
                                                                  const float *__restrict__ norm_w, float eps) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const AT *x = in + (size_t)row * (PRE == 2 ? 2 * K : K);
  __shared__ float wred[32];
  const int rounds = K / 1024 + ((K % 1024) ? 1 : 0);
  float v[PREPASS_MAXV];
#pragma unroll
  for (int j = 0; j < PREPASS_MAXV; j++) {
    const int i = tid + j * 1024;
    v[j] = 0.0f;
    if (j < rounds && i < K) {
      if constexpr (PRE == 2) {
        const int gi = (i >> 3) * 16 + (i & 7);
        const float g = (float)x[gi], u = (float)x[gi + 8];
        const float cl = fminf(fmaxf(g, -15.0f), 15.0f);
        v[j] = (g * (1.0f / (1.0f + expf(-cl)))) * u;
      } else {
        v[j] = (float)x[i];
      }
    }
  }
  if constexpr (PRE == 1) {
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < PREPASS_MAXV; j++) ss = fmaf(v[j], v[j], ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) wred[warp] = ss;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < 32; w++) total += wred[w];
    const float inv_rms = 1.0f / sqrtf(total / (float)K + eps);
    __syncthreads();
#pragma unroll
    for (int j = 0; j < PREPASS_MAXV; j++) {
      const int i = tid + j * 1024;
      if (j < rounds && i < K) v[j] = v[j] * inv_rms * __ldg(norm_w + i);
    }
  }
  float down = 1.0f;
  if constexpr (sizeof(AT) == 4) {
    float mx = 0.0f;
#pragma unroll
    for (int j = 0; j < PREPASS_MAXV; j++) mx = fmaxf(mx, fabsf(v[j]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) wred[warp] = mx;
    __syncthreads();
    mx = wred[0];
#pragma unroll
    for (int w = 1; w < 32; w++) mx = fmaxf(mx, wred[w]);
    int e = 0;  // exponent of the row maximum (0 for an all-zero or non-finite row: no scaling)
    if (mx > 0.0f && mx < __int_as_float(0x7f800000)) e = (int)((__float_as_uint(mx) >> 23) & 0xffu) - 127 - 13;
    e = max(-100, min(100, e));
    down = __int_as_float((uint32_t)(127 - e) << 23);
    if (tid == 0) row_scale[row] = __int_as_float((uint32_t)(127 + e) << 23);
  }
  const int nsub = K / 32;
#pragma unroll
  for (int j = 0; j < PREPASS_MAXV; j++) {
    const int s = j * 32 + warp;  // the sub-block this warp holds in round j
    if (j >= rounds || s >= nsub) continue;  // (warp-uniform)
    float t = v[j];
    if constexpr (sizeof(AT) == 4) {
      t *= down;
      const __half h = __float2half_rn(t);
      hi[(size_t)row * K + s * 32 + lane] = h;
      lo[(size_t)row * K + s * 32 + lane] = __float2half_rn(t - __half2float(h));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) {  // [row][super-block][8 halves | 8 residues]
      const float q = t * 0.015625f;
      const __half h = __float2half_rn(q);
      __half *at = xs16 + ((size_t)row * (nsub >> 3) + (s >> 3)) * 16 + (s & 7);
      at[0] = h;
      at[8] = __float2half_rn(q - __half2float(h));
    }
  }
}

template <int BM, bool LO, bool RESID>
__global__ void __launch_bounds__((DQW + 2) * 32, 1) gemm_q4k_tc_rows_kernel(const __grid_constant__ CUtensorMap tmap_x,
                                                                              const __grid_constant__ CUtensorMap tmap_x_lo,
                                                                              const uint8_t *__restrict__ W, const __half *__restrict__ xs16,
                                                                              float *__restrict__ C, float *__restrict__ parts, int M, int N,
                                                                              TcAlpha alpha, RowsPlan plan, const float *__restrict__ residual,
                                                                              int *__restrict__ err) {
  using L = RowsSmem<BM, LO>;
  static_assert(BM == 32 || BM == 64, "activation rows per MMA: 32 or 64");
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bpr = plan.bpr;
  const int u0 = (int)rows_unit_begin(blockIdx.x, plan.units, plan.ctas), u1 = (int)rows_unit_begin((long)blockIdx.x + 1, plan.units, plan.ctas);
  const int num_units = u1 - u0, num_g = num_units * 2;  // stages: two per super-block
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::abort_flag);
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L::tmem_slot);
  const uint32_t bars = smem_u32(smem + L::bars);
  auto full_w = [&](int s) { return bars + 8u * (uint32_t)s; };
  auto full_x = [&](int s) { return bars + 8u * (uint32_t)(STAGES + s); };
  auto done = [&](int s) { return bars + 8u * (uint32_t)(2 * STAGES + s); };
  auto tmem_empty = [&](int b) { return bars + 8u * (uint32_t)(3 * STAGES + b); };
  // per buffer: P (BM columns; with f32 activations 2 * BM: the products with the hi and the lo halves side by side)
  // and Pm (BM columns)
  constexpr uint32_t PCOLS = LO ? 2 * BM : BM, BUFCOLS = PCOLS + BM;
  constexpr uint32_t TMEM_COLS = 2 * BUFCOLS <= 128 ? 128 : (2 * BUFCOLS <= 256 ? 256 : 512);

  pdl_launch();
  if (tid == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(full_w(s), BUILDERS); mbar_init(full_x(s), 1); mbar_init(done(s), 1); }
    for (int b = 0; b < 2; b++) mbar_init(tmem_empty(b), DRAINERS);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {  // tensor-memory allocation is a warp-wide operation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem + L::tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- activation tiles: TMA ----------------
    if (lane == 0) {
      pdl_wait();  // the activations are the previous kernel's output
      for (int g = 0; g < num_g; g++) {
        const int s = g % STAGES;
        if (g >= STAGES && !mbar_wait_bounded(done(s), (uint32_t)(g / STAGES - 1) & 1u, abort_flag)) break;
        const int sb = (u0 + (g >> 1)) % bpr;
        mbar_expect_tx(full_x(s), L::stage_x);
        const uint32_t dst = smem_u32(smem + L::x + (uint32_t)s * L::stage_x);
#pragma unroll
        for (int j = 0; j < 2; j++) {
          const int kx = (sb * 4 + (g & 1) * 2 + j) * BK;
          tma_load_2d(dst + (uint32_t)j * L::x_step, &tmap_x, kx, 0, full_x(s));
          if constexpr (LO) tma_load_2d(dst + (uint32_t)j * L::x_step + L::x_tile, &tmap_x_lo, kx, 0, full_x(s));
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issue: P[128 weight rows, BM] = I_tile . X_tile^T per super-block ----------------
    if (lane == 0) {
      // f32 activations: the hi and the lo tile of a K step lie back to back in shared memory, so ONE MMA of
      // N = 2 * BM multiplies the weight slice with both (the weight slice is fetched once instead of twice;
      // these small MMAs are bound by that fetch: about 80 cycles each whatever N)
      const uint32_t idesc = umma_idesc_f16(TILE_N, (int)PCOLS), idesc_m = umma_idesc_f16(TILE_N, BM);
      bool ok = true;
      for (int ui = 0; ui < num_units && ok; ui++) {
        const int buf = ui & 1;
        if (ui >= 2) {  // the buffer's previous super-block has been read back
          if (!mbar_wait_bounded(tmem_empty(buf), (uint32_t)((ui >> 1) - 1) & 1u, abort_flag)) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t tp = tmem_base + (uint32_t)buf * BUFCOLS, tpm = tp + PCOLS;
#pragma unroll 1
        for (int h = 0; h < 2; h++) {
          const int g = ui * 2 + h, s = g % STAGES;
          const uint32_t ph = (uint32_t)(g / STAGES) & 1u;
          if (!mbar_wait_bounded(full_x(s), ph, abort_flag) || !mbar_wait_bounded(full_w(s), ph, abort_flag)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t w_addr = smem_u32(smem + L::w + (uint32_t)s * L::stage_w);
          const uint32_t x_addr = smem_u32(smem + L::x + (uint32_t)s * L::stage_x);
#pragma unroll
          for (int j = 0; j < 2; j++) {
#pragma unroll
            for (int k16 = 0; k16 < BK / 16; k16++) {
              const uint64_t wdesc = umma_desc_sw128(w_addr + (uint32_t)j * L::w_tile + (uint32_t)k16 * 32u);
              umma_f16(tp, wdesc, umma_desc_sw128(x_addr + (uint32_t)j * L::x_step + (uint32_t)k16 * 32u), idesc, (h == 0 && j == 0 && k16 == 0) ? 0u : 1u);
            }
          }
          if (h == 1)  // the min term: one K step of 16 from this super-block's slice of the min tiles
            umma_f16(tpm, umma_desc_sw128(smem_u32(smem + L::wm) + (uint32_t)(ui & 3) * 32u), umma_desc_sw128(smem_u32(smem + L::xm) + (uint32_t)(ui & 3) * 32u), idesc_m, 0u);
          umma_commit(done(s));  // the stage is free once these MMAs have read it; after the second stage P and Pm are complete
        }
      }
    }
  } else if (warp < 2 + BUILDERS) {
    // ---------------- integer weight tiles into swizzled shared memory ----------------
    // Builder warp b builds the 8-row groups b and b + 8 of the tile.  The builders never wait for a drain, so
    // they run as far ahead of the tensor core as the ring allows.
    const int bw = warp - 2;
    const int r8 = lane & 7, oct = lane >> 3;  // row within the group, byte octet of a 32-byte quant chunk
    constexpr uint32_t Y64 = 0x64646464u, K1024 = 0x64006400u, KM1024 = 0xE400E400u, K64 = 0x54005400u;
    bool ok = true;
    uint4 hdr[2];
    uint2 qn[2][4];
    uint4 xsn[2];  // builder warps 0 (and 1): sub-block sums of activation row bw * 32 + lane, 8 halves | 8 residues
    const bool xs_warp = bw < BM / 32;
    const int xs_m = bw * 32 + lane;
    auto fetch_xs = [&](int u) {
      xsn[0] = xsn[1] = make_uint4(0u, 0u, 0u, 0u);
      if (xs_warp && xs_m < M) {
        const uint4 *src = reinterpret_cast<const uint4 *>(xs16 + ((size_t)xs_m * bpr + u % bpr) * 16);
        xsn[0] = __ldg(src);
        xsn[1] = __ldg(src + 1);
      }
    };
    auto fetch = [&](int u) {
      const int tile = u / bpr, sb = u - tile * bpr;
#pragma unroll
      for (int rg = 0; rg < 2; rg++) {
        const uint32_t *blk = reinterpret_cast<const uint32_t *>(W + ((size_t)(tile * TILE_N + (bw + rg * BUILDERS) * 8 + r8) * bpr + sb) * Q4K_BLOCK_BYTES);
        hdr[rg] = __ldg(reinterpret_cast<const uint4 *>(blk));
#pragma unroll
        for (int c = 0; c < 4; c++) qn[rg][c] = __ldg(reinterpret_cast<const uint2 *>(blk + 4 + 8 * c) + oct);
      }
    };
    fetch(u0);   // packed weights: nothing earlier in the stream writes them
    pdl_wait();  // the sub-block sums are the pre-pass's output
    fetch_xs(u0);
    for (int ui = 0; ui < num_units && ok; ui++) {
      Q4KScales sc[2];
      uint2 qcur[2][4];
#pragma unroll
      for (int rg = 0; rg < 2; rg++) {
        sc[rg] = q4k_unpack_scales(hdr[rg].y, hdr[rg].z, hdr[rg].w);
#pragma unroll
        for (int c = 0; c < 4; c++) qcur[rg][c] = qn[rg][c];
      }
      const uint4 xs0 = xsn[0], xs1 = xsn[1];
      if (ui + 1 < num_units) { fetch(u0 + ui + 1); fetch_xs(u0 + ui + 1); }
#pragma unroll
      for (int h = 0; h < 2; h++) {
        const int g = ui * 2 + h, s = g % STAGES;
        bool stage_free = true;
        if (g >= STAGES) stage_free = mbar_wait_bounded(done(s), (uint32_t)(g / STAGES - 1) & 1u, abort_flag);
        if (!__all_sync(0xffffffffu, stage_free)) { ok = false; break; }
#pragma unroll
        for (int j = 0; j < 2; j++) {
          const int c = 2 * h + j;  // K step of the super-block: sub-blocks 2c (low nibbles) and 2c+1 (high nibbles)
#pragma unroll
          for (int rg = 0; rg < 2; rg++) {
            // row r of an 8-row group: 16-byte chunk i lives at chunk (i ^ r) of the 128-byte line
            uint8_t *line = smem + L::w + (uint32_t)s * L::stage_w + (uint32_t)j * L::w_tile + (uint32_t)(bw + rg * BUILDERS) * 1024u + (uint32_t)r8 * 128u;
            const uint32_t cw = c < 2 ? sc[rg].sc03 : sc[rg].sc47;
            const uint32_t b = (uint32_t)((2 * c) & 3);
            // the two 6-bit scale codes as f16 pairs, and -1024 * code
            const uint32_t sca = hsub2_u32(__byte_perm(cw, Y64, 0x4040u | b | (b << 8)), K1024);
            const uint32_t scb = hsub2_u32(__byte_perm(cw, Y64, 0x4040u | (b + 1u) | ((b + 1u) << 8)), K1024);
            const uint32_t nega = hmul2_u32(sca, KM1024), negb = hmul2_u32(scb, KM1024);
            uint32_t lo[4], hi[4];
#pragma unroll
            for (int i = 0; i < 2; i++) {
              // byte -> f16 1024 + q with one permute; (1024 + q) * sc - 1024 * sc = sc * q exactly
              const uint32_t word = i ? qcur[rg][c].y : qcur[rg][c].x;
              const uint32_t tl = word & 0x0f0f0f0fu, th = (word >> 4) & 0x0f0f0f0fu;
              lo[2 * i] = hfma2_u32(__byte_perm(tl, Y64, 0x4140u), sca, nega);
              lo[2 * i + 1] = hfma2_u32(__byte_perm(tl, Y64, 0x4342u), sca, nega);
              hi[2 * i] = hfma2_u32(__byte_perm(th, Y64, 0x4140u), scb, negb);
              hi[2 * i + 1] = hfma2_u32(__byte_perm(th, Y64, 0x4342u), scb, negb);
            }
            const uint32_t off_lo = ((uint32_t)oct ^ (uint32_t)r8) << 4, off_hi = ((uint32_t)(oct + 4) ^ (uint32_t)r8) << 4;
            *reinterpret_cast<uint4 *>(line + off_lo) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            *reinterpret_cast<uint4 *>(line + off_hi) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
          }
        }
        if (h == 1) {
          // the min term's operands: K slice (ui & 3) of the two min tiles.  (Its previous user, super-block
          // ui - 4, has been multiplied: this stage was only free after super-block ui - 1 had started.)
          const uint32_t k0 = 2u * (uint32_t)(ui & 3);
          if (oct < 2) {  // 64 * the eight min codes of the row, in columns 0..7 and again in 8..15
#pragma unroll
            for (int rg = 0; rg < 2; rg++) {
              uint32_t mm[4];
#pragma unroll
              for (int i = 0; i < 4; i++)
                mm[i] = hmul2_u32(hsub2_u32(__byte_perm(i < 2 ? sc[rg].mn03 : sc[rg].mn47, Y64, (i & 1) ? 0x4342u : 0x4140u), K1024), K64);
              uint8_t *line = smem + L::wm + (uint32_t)(bw + rg * BUILDERS) * 1024u + (uint32_t)r8 * 128u;
              *reinterpret_cast<uint4 *>(line + (((k0 + (uint32_t)oct) ^ (uint32_t)r8) << 4)) = make_uint4(mm[0], mm[1], mm[2], mm[3]);
            }
          }
          if (xs_warp) {  // activation row xs_m: the sums' halves in columns 0..7, their residues in 8..15
            uint8_t *line = smem + L::xm + (uint32_t)(xs_m >> 3) * 1024u + (uint32_t)(xs_m & 7) * 128u;
            *reinterpret_cast<uint4 *>(line + ((k0 ^ (uint32_t)(xs_m & 7)) << 4)) = xs0;
            *reinterpret_cast<uint4 *>(line + (((k0 + 1u) ^ (uint32_t)(xs_m & 7)) << 4)) = xs1;
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(full_w(s));
      }
    }
  } else {
    // ---------------- drains: tensor memory -> d * P - dmin * (min term) -> running sums -> C / partial slot ----------------
    // Two warps per tensor-memory lane quarter, each with half of the columns (activation rows).
    const int dwi = warp - 2 - BUILDERS;
    const int quad = warp & 3, half = dwi >> 2;
    constexpr int CW = BM / 2;  // columns per drain warp
    auto fetch_hd = [&](int ui) -> uint32_t {  // (d, dmin) of the row this thread drains
      if (ui >= num_units) return 0u;
      const int u = u0 + ui, tile = u / bpr;
      return __ldg(reinterpret_cast<const uint32_t *>(W + ((size_t)(tile * TILE_N + quad * 32 + lane) * bpr + (u - tile * bpr)) * Q4K_BLOCK_BYTES));
    };
    float acc[CW];
#pragma unroll
    for (int i = 0; i < CW; i++) acc[i] = 0.0f;
    int seg = 0, seg_sb0 = u0 % bpr;
    uint32_t hd_next = fetch_hd(0);
    pdl_wait();  // C and the partial slots may still be read by earlier kernels
    for (int uj = 0; uj < num_units; uj++) {
      const uint32_t hd = hd_next;
      hd_next = fetch_hd(uj + 1);
      const int buf = uj & 1, g = uj * 2 + 1;
      const bool ready = mbar_wait_bounded_backoff(done(g % STAGES), (uint32_t)(g / STAGES) & 1u, abort_flag);
      if (!__all_sync(0xffffffffu, ready)) break;  // tcgen05.ld is warp-wide: enter together or not at all
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int u = u0 + uj, tile = u / bpr, sb = u - tile * bpr;
      const float2 dd = q4k_d_dmin(hd);
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)buf * BUFCOLS + (uint32_t)(half * CW);
#pragma unroll
      for (int ch = 0; ch < CW / 16; ch++) {  // sixteen columns at a time (register budget)
        uint32_t p[16], pl[16], pm[16];
        tmem_ld16(taddr + (uint32_t)(ch * 16), p);
        if constexpr (LO) tmem_ld16(taddr + (uint32_t)(BM + ch * 16), pl);
        tmem_ld16(taddr + PCOLS + (uint32_t)(ch * 16), pm);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (ch == CW / 16 - 1) {  // everything of this buffer is in registers: hand it back to the MMA warp
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(tmem_empty(buf));
        }
#pragma unroll
        for (int i = 0; i < 16; i++) {
          float v = __uint_as_float(p[i]);
          if constexpr (LO) v += __uint_as_float(pl[i]);
          acc[ch * 16 + i] += fmaf(dd.x, v, -dd.y * __uint_as_float(pm[i]));
        }
      }
      if (sb == bpr - 1 || uj == num_units - 1) {
        const bool whole = seg_sb0 == 0 && sb == bpr - 1;
        float *dst = whole ? C + (size_t)tile * TILE_N : parts + ((size_t)blockIdx.x * plan.max_segs + seg) * (size_t)M * TILE_N;
        const size_t pitch = whole ? (size_t)N : (size_t)TILE_N;
#pragma unroll
        for (int i = 0; i < CW; i++) {
          const int m = half * CW + i;
          if (m < M) {
            float v = acc[i] * (alpha.row_scale ? alpha.value * __ldg(alpha.row_scale + m) : alpha.value);
            if constexpr (RESID) if (whole) v += residual[(size_t)m * N + (size_t)tile * TILE_N + quad * 32 + lane];  // (may be C itself: same element, same thread)
            dst[(size_t)m * pitch + quad * 32 + lane] = v;
          }
          acc[i] = 0.0f;
        }
        seg++;
        seg_sb0 = 0;
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  if (*abort_flag && tid == 0) atomicExch(err, 2);
}

// C[m, tile columns] = sum over the CTAs that share the tile, in CTA order, of their partial slots.  Tiles one CTA
// computed alone were written to C by that CTA and are skipped.
__global__ void __launch_bounds__(256) rows_reduce_kernel(const float *__restrict__ parts, float *__restrict__ C, int M, int N, RowsPlan plan,
                                                          const float *__restrict__ residual) {
  pdl_launch();
  pdl_wait();
  // one thread per four columns of a tile row; blockIdx.y = tile, so the owners are computed once per block
  const int tile = blockIdx.y;
  const int units = (int)plan.units, ctas = plan.ctas, bpr = plan.bpr;
  const int cf = rows_unit_owner((long)tile * bpr, units, ctas), cl = rows_unit_owner((long)tile * bpr + bpr - 1, units, ctas);
  if (cf == cl) return;  // one CTA computed the whole tile and wrote C itself
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < M * (TILE_N / 4); i += gridDim.x * blockDim.x) {
    const int m = i / (TILE_N / 4), n = (i - m * (TILE_N / 4)) * 4;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int c = cf; c <= cl; c++) {
      const int seg = tile - (int)(rows_unit_begin(c, units, ctas) / bpr);
      const float4 v = *reinterpret_cast<const float4 *>(parts + ((size_t)c * plan.max_segs + seg) * (size_t)M * TILE_N + (size_t)m * TILE_N + n);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (residual) {
      const float4 rv = *reinterpret_cast<const float4 *>(residual + (size_t)m * N + (size_t)tile * TILE_N + n);
      acc.x += rv.x; acc.y += rv.y; acc.z += rv.z; acc.w += rv.w;
    }
    *reinterpret_cast<float4 *>(C + (size_t)m * N + (size_t)tile * TILE_N + n) = acc;
  }
}

template <int BM, bool LO, bool RESID>
dp_status launch_rows(dp_ctx *ctx, const CUtensorMap *tm, const uint8_t *W, const __half *xs16, float *C, float *parts, int M, int N,
                      TcAlpha alpha, const RowsPlan &plan, const float *residual) {
  constexpr size_t smem = RowsSmem<BM, LO>::total + 1024;
  static_assert(smem <= 227 * 1024, "rings exceed shared memory");
  auto kernel = gemm_q4k_tc_rows_kernel<BM, LO, RESID>;
  DP_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  DP_LAUNCH(ctx, kernel, (unsigned)plan.ctas, (DQW + 2) * 32, smem, tm[0], tm[1], W, xs16, C, parts, M, N, alpha, plan, residual, ctx->dev_status);
  return DP_OK;
}

}  // namespace

// A: f32 (multiplied in as two f16 halves: the f32-exact product) or f16 activations [M, K].  The dequantised
// weights enter exactly in both cases.  *handled stays false for shapes this kernel does not take.
// fuse (optional): an operation on the f32 input rows folded into the pre-pass (DPK_ROWS_PRE_RMSNORM: A is the
// un-normalised row, norm_w / eps the norm; DPK_ROWS_PRE_SILU: A rows hold 2K interleaved gate|up values) and a
// residual added to the output (may be C itself).
dp_status dpk_gemm_q4k_tc_rows(dp_ctx *ctx, const uint8_t *W, const void *A, dp_dtype a_dtype, float *C, int M, int N, int K, float alpha,
                               bool *handled, const dpk_rows_fuse *fuse) {
  *handled = false;
  const int pre = fuse ? fuse->pre : 0;
  const float *residual = fuse ? fuse->residual : nullptr;
  if (pre && a_dtype != DP_F32) return DP_OK;
  if (M < 2 || M > 64 || N % TILE_N || K % QK_K || !ctx->dev_status) return DP_OK;
  if (pre && K > 1024 * PREPASS_MAXV) return DP_OK;
  if (a_dtype != DP_F32 && a_dtype != DP_F16) return DP_OK;
  EncodeTiledFn encode = get_encode();
  if (!encode) return DP_OK;
  const int bm = M <= 32 ? 32 : 64;
  const bool f32a = a_dtype == DP_F32;
  if (residual && !(f32a && bm == 32)) return DP_OK;  // the residual is folded in for up to 32 f32 rows only (nothing launched yet)
  RowsPlan plan;
  plan.tiles = N / TILE_N;
  plan.bpr = K / QK_K;
  plan.units = (long)plan.tiles * plan.bpr;
  plan.ctas = (int)(plan.units < ctx->sm_count ? plan.units : ctx->sm_count);
  const long per_cta = (plan.units + plan.ctas - 1) / plan.ctas;
  plan.max_segs = (int)((per_cta + plan.bpr - 1) / plan.bpr) + 1;
  DP_TRY(dp_scratch(ctx, &ctx->gemm_split_scratch, (size_t)plan.ctas * plan.max_segs * M * TILE_N * 4, "matmul_k_split_parts"));
  float *parts = (float *)ctx->gemm_split_scratch->dptr;

  // f16 halves and residues of f32 rows, sub-block sums, row scales: one scratch of the context
  const size_t a_bytes = f32a ? ((size_t)M * K * 2 + 255) / 256 * 256 : 0;
  const size_t s_bytes = ((size_t)M * plan.bpr * 16 * 2 + 255) / 256 * 256;
  DP_TRY(dp_scratch(ctx, &ctx->gemm_scratch, 2 * a_bytes + s_bytes + (size_t)M * 4, "matmul_a_f16"));
  char *base = (char *)ctx->gemm_scratch->dptr;
  __half *hi = (__half *)base, *lo = (__half *)(base + a_bytes);
  __half *xs16 = (__half *)(base + 2 * a_bytes);
  float *scales = (float *)(base + 2 * a_bytes + s_bytes);
  if (f32a) {
    const float *nw = fuse ? fuse->norm_w : nullptr;
    const float eps = fuse ? fuse->eps : 0.0f;
    if (pre == DPK_ROWS_PRE_RMSNORM) DP_LAUNCH(ctx, (rows_prepass_fused_kernel<float, 1>), (unsigned)M, 1024, 0, (const float *)A, hi, lo, scales, xs16, K, nw, eps);
    else if (pre == DPK_ROWS_PRE_SILU) DP_LAUNCH(ctx, (rows_prepass_fused_kernel<float, 2>), (unsigned)M, 1024, 0, (const float *)A, hi, lo, scales, xs16, K, nw, eps);
    else DP_LAUNCH(ctx, rows_prepass_kernel<float>, (unsigned)M, 1024, 0, (const float *)A, hi, lo, scales, xs16, K);
  } else {
    DP_LAUNCH(ctx, rows_prepass_kernel<__half>, (unsigned)M, 1024, 0, (const __half *)A, (__half *)nullptr, (__half *)nullptr, (float *)nullptr, xs16, K);
    hi = (__half *)A;
    lo = hi;
  }

  CUtensorMap tm[2];
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)bm};
  const cuuint32_t estr[2] = {1, 1};
  void *ptrs[2] = {(void *)hi, (void *)lo};
  for (int i = 0; i < 2; i++) {
    CUresult r = encode(&tm[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, ptrs[i], dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return dp_fail(ctx, DP_ERR_CUDA, "matmul: cuTensorMapEncodeTiled failed (%d) for A[%d,%d]", (int)r, M, K);
  }
  const TcAlpha ta = {alpha, f32a ? scales : nullptr, 1};
  dp_status st;
  if (residual) st = launch_rows<32, true, true>(ctx, tm, W, xs16, C, parts, M, N, ta, plan, residual);
  else if (bm == 32) st = f32a ? launch_rows<32, true, false>(ctx, tm, W, xs16, C, parts, M, N, ta, plan, nullptr) : launch_rows<32, false, false>(ctx, tm, W, xs16, C, parts, M, N, ta, plan, nullptr);
  else st = f32a ? launch_rows<64, true, false>(ctx, tm, W, xs16, C, parts, M, N, ta, plan, nullptr) : launch_rows<64, false, false>(ctx, tm, W, xs16, C, parts, M, N, ta, plan, nullptr);
  if (st != DP_OK) return st;
  if (plan.units % plan.ctas != 0 || (plan.units / plan.ctas) % plan.bpr != 0) {  // some tile is shared between CTAs
    const int per_tile = M * (TILE_N / 4);
    DP_LAUNCH(ctx, rows_reduce_kernel, dim3((unsigned)((per_tile + 255) / 256), (unsigned)plan.tiles), 256, 0, (const float *)parts, C, M, N, plan, residual);
  }
  *handled = true;
  return DP_OK;
}
