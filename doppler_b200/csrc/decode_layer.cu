// Single-token decode: the Q4_K GEMVs of a layer as ONE persistent kernel.
//
// Replaces, for the decode step, one launch per projection (the reference records ~15 dispatches per
// layer, src/inference/pipelines/text/layer.js:682, matmuls via fused_matmul_q4.wgsl:279).  A decode
// GEMV reads 0.5625 B per weight and nothing else of note, so the only thing worth optimising is that
// HBM never idles; per-matrix launches idle it at every boundary (a 27 MB matrix takes 4.2 us of HBM
// time, and about as long again to drain one launch, start the next and fill its pipeline).  Here one
// CTA per SM walks a list of up to four projections ("phases"),
//      o_proj -> gate|up -> down_proj -> q|k|v of the next layer
// (the attention kernel sits between two such launches), and its producer warp streams the packed
// weight rows of ALL phases through one shared-memory ring with bulk copies: weights depend on nothing,
// so the stream runs straight through the phase boundaries.  The sixteen consumer warps are the
// arithmetic of gemv_q4k_fast.cu (fixed-point activation digits, int8 tensor-core MMAs).
//
// Between phases every CTA needs the WHOLE output vector of the previous phase.  There is no grid
// barrier: a measured barrier (fence, counter, flag, acquire) cost 8-10 us here, more than a phase's
// weight stream.  Instead every output element is handed over as one aligned 8-byte word
// (value, ticket), stored by the warp that reduced the row and re-read by each consumer until the ticket
// is the one of this hand-off (tp_exchange.h); tickets grow from hand-off to hand-off and never repeat.
// An 8-byte store is one transaction, so no fence is needed on either side.
//   - o_proj and down_proj (row-parallel under tensor parallelism) push their rows into this rank's slot
//     of EVERY rank's exchange area (plain stores over NVLink).  The next phase's prologue gathers the
//     slots of all ranks from its OWN memory, sums them in rank order (every rank gets the same bits),
//     adds them to the residual stream, which each CTA keeps in shared memory, and normalises
//     (rmsnorm.wgsl:119-187).  Allreduce, residual add and RMSNorm thus cost no kernel and no collective
//     call; a single GPU runs the very same code with one rank.  No load ever targets peer memory.
//   - gate|up rows are stored interleaved (eight gate rows, then their eight up rows), so the warp that
//     reduces a 16-row tile holds matching pairs: it applies silu(gate) * up itself (silu.wgsl:98-104)
//     and hands eight activations to down_proj's prologue the same way.
//
// Every wait is bounded (mbarriers: ~1M polls; hand-offs: `wait_limit` polls).  On give-up the CTA
// raises an abort flag, its threads skip the remaining work but still meet at every CTA barrier, the
// producer lets its copies in flight land, and a status word tells the host (DP_ERR_TIMEOUT).
#include "common.h"
#include "pdl.cuh"
#include "q4k.cuh"
#include "actq.cuh"
#include "mbar.cuh"
#include "tp_exchange.h"
#include "decode_layer.h"

#define DL_CONSUMERS 8   // warps per consumer group (one per super-block column of a chunk)
#define DL_GROUPS 2      // consecutive row tiles alternate between the groups
#define DL_MAX_BW 2      // super-block columns of a stage per consumer warp: a stage holds at most 16 blocks per row
#define DL_ROW_PAD 32
#define DL_RED_SLOTS 16
#define DL_CT (DL_GROUPS * DL_CONSUMERS * 32)  // consumer threads
#define DL_NW (DL_GROUPS * DL_CONSUMERS)       // consumer warps

struct DlLayout {
  uint32_t digits, h, stages, bars, red, abort_flag, total;
};

__host__ __device__ static inline uint32_t dl_digit_bytes(int K) { return (uint32_t)K * 4u + (uint32_t)(K / QK_K) * 4u + (uint32_t)(K / 32) * 4u; }

__host__ __device__ static inline DlLayout dl_layout(uint32_t digit_bytes, uint32_t h_bytes, uint32_t slot_bytes, int stages) {
  DlLayout l;
  l.digits = 0;
  uint32_t off = (digit_bytes + 127u) & ~127u;
  l.h = off;  // the residual stream, one copy per CTA
  off += (h_bytes + 127u) & ~127u;
  l.stages = off;
  off += (uint32_t)stages * slot_bytes;
  l.bars = off;  // full[stages], empty[stages], red[DL_RED_SLOTS]
  off += (2u * (uint32_t)stages + DL_RED_SLOTS) * 8u;
  l.red = off;
  off += DL_RED_SLOTS * DL_CONSUMERS * 16u * 4u;
  l.abort_flag = off;
  l.total = off + 16u;
  return l;
}

__device__ __forceinline__ void dl_mma_u8s8(int &c0, int &c1, int &c2, int &c3, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                            uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
      : "=r"(c0), "=r"(c1), "=r"(c2), "=r"(c3)
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

// one (value, ticket) word: a single 8-byte store
__device__ __forceinline__ void dl_put(uint2 *p, float v, unsigned ticket) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(ticket) : "memory");
}
__device__ __forceinline__ uint4 dl_peek2(const uint2 *p) {  // two words, straight from L2
  uint4 r;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
  return r;
}
// Eight consecutive (value, ticket) words: re-read until all carry `ticket` (bounded).  false: gave up.
__device__ __forceinline__ bool dl_take8(const uint2 *p, unsigned ticket, float (&v)[8], unsigned limit, volatile int *abort_flag) {
  for (unsigned it = 0; it < limit; it++) {
    const uint4 a = dl_peek2(p), b = dl_peek2(p + 2), c = dl_peek2(p + 4), d = dl_peek2(p + 6);
    if (a.y == ticket && a.w == ticket && b.y == ticket && b.w == ticket && c.y == ticket && c.w == ticket && d.y == ticket && d.w == ticket) {
      v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.z); v[2] = __uint_as_float(b.x); v[3] = __uint_as_float(b.z);
      v[4] = __uint_as_float(c.x); v[5] = __uint_as_float(c.z); v[6] = __uint_as_float(d.x); v[7] = __uint_as_float(d.z);
      return true;
    }
    if ((it & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
// eight consecutive floats written earlier in this kernel by other SMs (or by peers): from L2, never a stale L1 line
__device__ __forceinline__ void dl_load8(const float *p, float (&v)[8]) {
  const float4 a = __ldcg(reinterpret_cast<const float4 *>(p)), c = __ldcg(reinterpret_cast<const float4 *>(p + 4));
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
}
__device__ __forceinline__ void dl_store8(float *p, const float (&v)[8]) {
  *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4 *>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

// The prologue of a phase: the activation digits of its input vector, rebuilt by every CTA (all consumer
// threads call it together).
// (The helpers below name the dynamic shared memory themselves: through a pointer argument every access
// would be a generic load instead of a shared-memory one.)
extern __shared__ __align__(128) uint8_t dl_smem[];

// x = rmsnorm(h) * w; with an exchange in front, first h += the partial vectors of all ranks
__device__ __forceinline__ void dl_prologue_norm(const DlParams &P, const DlPhase ph, uint32_t red_off, uint32_t h_off, unsigned ticket_base, uint32_t abort_off, bool live) {
  uint8_t *smem = dl_smem;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(dl_smem + abort_off);
  const int tid = threadIdx.x, lane = tid & 31, cw = tid >> 5;
  const int K = ph.K, bpr = K / QK_K;
  float *h_s = reinterpret_cast<float *>(smem + h_off);
  float *scratch = reinterpret_cast<float *>(smem + red_off);  // free between phases
  {
    // x = rmsnorm(h) * w; XCHG: first h += the partial vectors of all ranks, summed in rank order.
    // The norm weights depend on nothing: their loads are in flight while the hand-off is awaited.
    const unsigned ticket = ticket_base + ph.ticket_in;
    const int nr = P.nr;
    const uint2 *my_area = P.area[P.rank];
    float4 nw[2][2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const int b = cw + DL_NW * i;
      if (b < bpr && live) {
        nw[i][0] = __ldg(reinterpret_cast<const float4 *>(ph.norm_w + b * QK_K + lane * 8));
        nw[i][1] = __ldg(reinterpret_cast<const float4 *>(ph.norm_w + b * QK_K + lane * 8 + 4));
      }
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const int b = cw + DL_NW * i;
      if (b < bpr && live) {
        const int off = b * QK_K + lane * 8;
        float v[8];
        const float4 ha = *reinterpret_cast<const float4 *>(h_s + off), hc = *reinterpret_cast<const float4 *>(h_s + off + 4);
        v[0] = ha.x; v[1] = ha.y; v[2] = ha.z; v[3] = ha.w; v[4] = hc.x; v[5] = hc.y; v[6] = hc.z; v[7] = hc.w;
        if (ph.src == DL_SRC_XCHG_RMSNORM) {
          float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int r = 0; r < nr; r++) {
            float s8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            dl_take8(my_area + dp_tp_slot_offset((unsigned)ph.parity, r) + off, ticket, s8, P.wait_limit, abort_flag);
#pragma unroll
            for (int j = 0; j < 8; j++) acc[j] += s8[j];
          }
#pragma unroll
          for (int j = 0; j < 8; j++) v[j] += acc[j];
          dl_store8(h_s + off, v);  // the stream stays in shared memory; it is read back below
          if (ph.h_out && (b % (int)gridDim.x) == (int)blockIdx.x) dl_store8(ph.h_out + off, v);
        }
#pragma unroll
        for (int j = 0; j < 8; j++) ss = fmaf(v[j], v[j], ss);
      }
    }
    __syncwarp();
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) scratch[cw] = ss;
    asm volatile("bar.sync 1, %0;" ::"r"(DL_CT) : "memory");
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < DL_NW; i++) total += scratch[i];
    const float inv_rms = 1.0f / sqrtf(total / (float)K + P.eps);
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const int b = cw + DL_NW * i;
      if (b < bpr && live) {
        const int off = b * QK_K + lane * 8;
        const float4 ha = *reinterpret_cast<const float4 *>(h_s + off), hc = *reinterpret_cast<const float4 *>(h_s + off + 4);
        const float4 wa = nw[i][0], wc = nw[i][1];
        float o[8];
        o[0] = ha.x * inv_rms * wa.x; o[1] = ha.y * inv_rms * wa.y; o[2] = ha.z * inv_rms * wa.z; o[3] = ha.w * inv_rms * wa.w;
        o[4] = hc.x * inv_rms * wc.x; o[5] = hc.y * inv_rms * wc.y; o[6] = hc.z * inv_rms * wc.z; o[7] = hc.w * inv_rms * wc.w;
        if (ph.n_out && blockIdx.x == 0) dl_store8(ph.n_out + off, o);
        if (ph.N > 0) actq_emit_block(o, lane, b, bpr, smem);
      }
    }
  }
}

// x = silu(gate) * up, handed over element by element by the previous phase's reducing warps
__device__ __forceinline__ void dl_prologue_act(const DlParams &P, const DlPhase ph, unsigned ticket_base, uint32_t abort_off, bool live) {
  uint8_t *smem = dl_smem;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(dl_smem + abort_off);
  const int tid = threadIdx.x, lane = tid & 31, cw = tid >> 5;
  const int K = ph.K, bpr = K / QK_K;
  {
    const unsigned ticket = ticket_base + ph.ticket_in;
    for (int b = cw; b < bpr && live; b += DL_NW) {
      float o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      dl_take8(P.act + b * QK_K + lane * 8, ticket, o, P.wait_limit, abort_flag);
      __syncwarp();
      actq_emit_block(o, lane, b, bpr, smem);
    }
  }
}

// x = an f32 vector left by the previous kernel, or the merge of the split-K attention partials
__device__ __forceinline__ void dl_prologue_vector(const DlParams &P, const DlPhase ph, bool live) {
  uint8_t *smem = dl_smem;
  const int tid = threadIdx.x, lane = tid & 31, cw = tid >> 5;
  const int K = ph.K, bpr = K / QK_K;
  if (ph.src == DL_SRC_VECTOR) {
    for (int b = cw; b < bpr && live; b += DL_NW) {
      float o[8];
      dl_load8(ph.x + b * QK_K + lane * 8, o);
      actq_emit_block(o, lane, b, bpr, smem);
    }
  } else {
    const int D = P.D, splits = P.splits;
    for (int b = cw; b < bpr && live; b += DL_NW) {
      const int e0 = b * QK_K + lane * 8, h = e0 / D, d0 = e0 % D;
      const float *pp = ph.x + (size_t)h * splits * (D + 2);
      float mm = -3.402823466e+38f, ll = 0.0f, acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int sp = 0; sp < splits; sp++) mm = fmaxf(mm, __ldcg(pp + sp * (D + 2) + D));
#pragma unroll 2
      for (int sp = 0; sp < splits; sp++) {
        const float *ps = pp + sp * (D + 2);
        const float ms = __ldcg(ps + D);
        const float c = (ms == -3.402823466e+38f) ? 0.0f : exp2f(ms - mm);
        ll = fmaf(__ldcg(ps + D + 1), c, ll);
        const float2 a0 = __ldcg(reinterpret_cast<const float2 *>(ps + d0)), a1 = __ldcg(reinterpret_cast<const float2 *>(ps + d0 + 2));
        const float2 a2 = __ldcg(reinterpret_cast<const float2 *>(ps + d0 + 4)), a3 = __ldcg(reinterpret_cast<const float2 *>(ps + d0 + 6));
        acc[0] = fmaf(a0.x, c, acc[0]); acc[1] = fmaf(a0.y, c, acc[1]); acc[2] = fmaf(a1.x, c, acc[2]); acc[3] = fmaf(a1.y, c, acc[3]);
        acc[4] = fmaf(a2.x, c, acc[4]); acc[5] = fmaf(a2.y, c, acc[5]); acc[6] = fmaf(a3.x, c, acc[6]); acc[7] = fmaf(a3.y, c, acc[7]);
      }
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; j++) o[j] = ll > 0.0f ? acc[j] / ll : 0.0f;
      actq_emit_block(o, lane, b, bpr, smem);
    }
  }
}

__device__ __forceinline__ void dl_prologue(const DlParams &P, int p, uint32_t red_off, uint32_t h_off, unsigned ticket_base, uint32_t abort_off, bool live) {
  const int src = P.ph[p].src;
  if (src == DL_SRC_RMSNORM || src == DL_SRC_XCHG_RMSNORM) dl_prologue_norm(P, P.ph[p], red_off, h_off, ticket_base, abort_off, live);
  else if (src == DL_SRC_ACT) dl_prologue_act(P, P.ph[p], ticket_base, abort_off, live);
  else dl_prologue_vector(P, P.ph[p], live);
}

// The row tiles of one phase for this CTA (consumer warps).  Returns the number of row tiles this CTA has in the phase.
struct DlTileCtx {
  uint32_t stages_off, bars, red_off, slot_bytes, abort_off;
  int stages;
  unsigned ticket_base;
};
__device__ __forceinline__ uint32_t dl_phase_tiles(const DlParams &P, int p, const DlTileCtx X, uint32_t tile_no, uint32_t u_base) {
  uint8_t *smem = dl_smem;
  const DlPhase ph = P.ph[p];  // a private copy: the fields are read many times
  const int tid = threadIdx.x, lane = tid & 31, warp_all = tid >> 5;
  const int group = warp_all / DL_CONSUMERS, warp = warp_all % DL_CONSUMERS;
  const int g = lane >> 2, t = lane & 3;
  const int stages = X.stages;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(dl_smem + X.abort_off);
  const uint32_t bars = X.bars;
  auto full_bar = [&](int s) { return bars + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return bars + 8u * (uint32_t)(stages + s); };
  auto red_bar = [&](int s) { return bars + 8u * (uint32_t)(2 * stages + s); };
  // B operand columns 2l and 2l+1 carry activation limb l (of the even / odd sub-block of a chunk), so
  // lane t reads limb t from its accumulator registers (columns 2t and 2t+1); t == 3 holds nothing.
  const float wt = t == 0 ? 1.0f : (t == 1 ? 256.0f : (t == 2 ? 65536.0f : 0.0f));
  const bool limb_lane = g < 6;  // B fragment columns 6 and 7 are zero
  const uint32_t M4 = 0x0f0f0f0fu, M4H = 0xf0f0f0f0u;
  float *red = reinterpret_cast<float *>(smem + X.red_off);
  const int K = ph.K, bpr = K / QK_K;
  const int rank = P.rank, nr = P.nr;
  const unsigned ticket_base = X.ticket_base;
  struct { uint32_t stages; } L = {X.stages_off};
      // ---- this CTA's row tiles of the phase ----
      const int tiles = ph.N / 16, cb = ph.cb, chunks = cb ? bpr / cb : 0;
      const uint32_t row_stride = (uint32_t)cb * Q4K_BLOCK_BYTES + DL_ROW_PAD;
      const float *sm_xscale = reinterpret_cast<const float *>(smem + (size_t)K * 4);
      const float *sm_ssum = sm_xscale + bpr;
      const unsigned ticket_out = ticket_base + ph.ticket_out;
      uint32_t local = 0;
      for (int rt = blockIdx.x; rt < tiles; rt += gridDim.x, local++, tile_no++) {
        if ((tile_no % DL_GROUPS) != (uint32_t)group) continue;
        if (__shfl_sync(0xffffffffu, *abort_flag, 0)) continue;  // warp-uniform: the MMAs need the whole warp
        float resA = 0.0f, resB = 0.0f;
        uint32_t u = u_base + local * (uint32_t)chunks;
        bool ok = true;
        for (int ch = 0; ch < chunks; ch++, u++) {
          const int s = (int)(u % (uint32_t)stages);
          const uint32_t n = u / (uint32_t)stages;
          if (!__all_sync(0xffffffffu, mbar_wait_bounded(full_bar(s), n & 1u, abort_flag))) { ok = false; break; }
          // Phase 1: pull this warp's share of the stage (up to DL_MAX_BW super-block columns of the 16 rows)
          // into registers and hand the stage back to the producer at once.  The arithmetic below then runs
          // while the ring slot is already being refilled, so nearly the whole ring stays in flight.
          uint4 ha[DL_MAX_BW], hb[DL_MAX_BW];
          uint2 qa[DL_MAX_BW][4], qb[DL_MAX_BW][4];
#pragma unroll
          for (int i = 0; i < DL_MAX_BW; i++) {
            const int bw = warp + i * DL_CONSUMERS;
            if (bw < cb) {
              const uint8_t *pa = smem + L.stages + (uint32_t)s * X.slot_bytes + (uint32_t)g * row_stride + (uint32_t)bw * Q4K_BLOCK_BYTES;
              const uint8_t *pb = pa + 8u * row_stride;
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
          for (int i = 0; i < DL_MAX_BW; i++) {
            const int bw = warp + i * DL_CONSUMERS;
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
              dl_mma_u8s8(c0, c1, c2, c3, qa[i][c].x & M4, qb[i][c].x & M4, qa[i][c].y & M4, qb[i][c].y & M4, bf.x, bf.y);
              (void)c1; (void)c3;
              const uint32_t wsa = c < 2 ? sa.sc03 : sa.sc47, wsb = c < 2 ? sb_.sc03 : sb_.sc47;
              accA += (int)__byte_perm(wsa, 0u, 0x4440u + (uint32_t)((2 * c) & 3)) * c0;
              accB += (int)__byte_perm(wsb, 0u, 0x4440u + (uint32_t)((2 * c) & 3)) * c2;
              int h0, h1, h2, h3;
              dl_mma_u8s8(h0, h1, h2, h3, qa[i][c].x & M4H, qb[i][c].x & M4H, qa[i][c].y & M4H, qb[i][c].y & M4H, bf.x, bf.y);
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
        if (!ok) continue;
        // sum the eight warps' partial rows through a ring of reduction slots
        resA += __shfl_xor_sync(0xffffffffu, resA, 1);
        resA += __shfl_xor_sync(0xffffffffu, resA, 2);
        resB += __shfl_xor_sync(0xffffffffu, resB, 1);
        resB += __shfl_xor_sync(0xffffffffu, resB, 2);
        const int slot = (int)(tile_no % DL_RED_SLOTS);
        float *rs = red + slot * DL_CONSUMERS * 16;
        if (t == 0) { rs[warp * 16 + g] = resA; rs[warp * 16 + g + 8] = resB; }
        __syncwarp();
        if (lane == 0) mbar_arrive(red_bar(slot));
        // The reducing warp of group g is warp g+1: with 17 warps on four schedulers the producer (warp 16)
        // shares scheduler 0 with consumer warps 0, 4, 8, 12; the extra work goes to other schedulers.
        if (warp == group + 1) {
          if (!__all_sync(0xffffffffu, mbar_wait_bounded(red_bar(slot), (tile_no / DL_RED_SLOTS) & 1u, abort_flag))) continue;
          float v = 0.0f;
          if (lane < 16) {
#pragma unroll
            for (int w = 0; w < DL_CONSUMERS; w++) v += rs[w * 16 + lane];
          }
          const int row = rt * 16 + lane;
          if (ph.out == DL_OUT_PUSH) {  // this rank's partial of the row, with its ticket, into its slot on every rank
            if (lane < 16) {
              const size_t off = dp_tp_slot_offset((unsigned)ph.parity, rank) + (size_t)row;
              for (int r = 0; r < nr; r++) dl_put(P.area[r] + off, v, ticket_out);
            }
          } else if (ph.out == DL_OUT_SILU) {  // lanes 0-7 hold gate rows, lanes 8-15 the matching up rows
            const float up = __shfl_down_sync(0xffffffffu, v, 8);
            if (lane < 8) {
              const float cl = fminf(fmaxf(v, -15.0f), 15.0f);
              dl_put(P.act + rt * 8 + lane, (v * (1.0f / (1.0f + expf(-cl)))) * up, ticket_out);
            }
          } else if (lane < 16) {
            ph.y[row] = v;
          }
        }
      }
  return local;
}

__global__ void __launch_bounds__((DL_NW + 1) * 32, 1) decode_layer_kernel(const __grid_constant__ DlParams P) {
  uint8_t *smem = dl_smem;
  const DlLayout L = dl_layout(P.digit_bytes, (uint32_t)P.hidden * 4u, P.slot_bytes, P.stages);
  const int tid = threadIdx.x, lane = tid & 31, warp_all = tid >> 5;
  const int group = warp_all / DL_CONSUMERS;  // producer: group == DL_GROUPS
  const int stages = P.stages;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L.abort_flag);
  const uint32_t bars = smem_u32(smem + L.bars);
  auto full_bar = [&](int s) { return bars + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return bars + 8u * (uint32_t)(stages + s); };
  auto red_bar = [&](int s) { return bars + 8u * (uint32_t)(2 * stages + s); };

  if (tid == 0) {
    for (int s = 0; s < stages; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), DL_CONSUMERS); }
    for (int s = 0; s < DL_RED_SLOTS; s++) mbar_init(red_bar(s), DL_CONSUMERS);
    *abort_flag = 0;
    mbar_fence_init();
  }
  pdl_launch();
  __syncthreads();

  if (group == DL_GROUPS) {
    // ---------------- producer: the weight rows of every phase, in order, through one ring ----------------
    // (weights are written by no kernel of the step, so this starts before griddepcontrol.wait)
    uint32_t u = 0;
    bool ok = true;
    for (int p = 0; p < P.n_phases && ok; p++) {
      const DlPhase &ph = P.ph[p];
      const int tiles = ph.N / 16, bpr = ph.K / QK_K, cb = ph.cb, chunks = cb ? bpr / cb : 0;
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
            const uint8_t *src = ph.W + ((size_t)(rt * 16 + lane) * bpr + (size_t)ch * cb) * Q4K_BLOCK_BYTES;
            const uint32_t row_stride = (uint32_t)cb * Q4K_BLOCK_BYTES + DL_ROW_PAD;
            bulk_g2s(smem_u32(smem + L.stages + (uint32_t)s * P.slot_bytes + (uint32_t)lane * row_stride), src, (uint32_t)cb * Q4K_BLOCK_BYTES,
                     full_bar(s));
          }
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
    pdl_wait();  // everything below reads or writes what earlier kernels of the step produce
    const unsigned ticket_base = *reinterpret_cast<const volatile unsigned *>(P.ticket_step) * P.ticket_stride + 1u;
    float *h_s = reinterpret_cast<float *>(smem + L.h);
    const int cw = tid >> 5;  // consumer warp 0..15
    // pull the norm weights of the later phases into L2 now (128-byte lines, one per thread)
    for (int p = 1; p < P.n_phases; p++) {
      const float *w = P.ph[p].norm_w;
      if (w && tid * 32 < P.ph[p].K) asm volatile("prefetch.global.L2 [%0];" ::"l"(w + tid * 32));
    }
    // Thread (cw, lane) owns elements lane*8 .. lane*8+7 of the 256-blocks cw and cw + 16 of the residual
    // stream, in every phase: it alone reads and writes them in h_s, so they need no CTA barrier.
    if (P.h_in) {
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int off = (cw + DL_NW * i) * QK_K + lane * 8;
        if (off < P.hidden) {
          float v[8];
          dl_load8(P.h_in + off, v);
          dl_store8(h_s + off, v);
        }
      }
    }
    uint32_t tile_no = 0;  // row tiles of this CTA so far, over all phases (ring order)
    uint32_t u_base = 0;   // ring units before the current phase

    for (int p = 0; p < P.n_phases; p++) {
      // (warp-uniform: the digit builders shuffle across the whole warp)
      const bool live = __shfl_sync(0xffffffffu, *abort_flag, 0) == 0;
      dl_prologue(P, p, L.red, L.h, ticket_base, L.abort_flag, live);
      asm volatile("bar.sync 1, %0;" ::"r"(DL_CT) : "memory");  // digits complete (and `red` free again)

      {
        DlTileCtx X;
        X.stages_off = L.stages; X.bars = bars; X.red_off = L.red; X.slot_bytes = P.slot_bytes; X.stages = stages;
        X.abort_off = L.abort_flag; X.ticket_base = ticket_base;
        const uint32_t local = dl_phase_tiles(P, p, X, tile_no, u_base);
        tile_no += local;
        const DlPhase &phx = P.ph[p];
        u_base += local * (uint32_t)(phx.cb ? (phx.K / QK_K) / phx.cb : 0);
      }
      // every warp is done with this phase's digits before the next prologue overwrites them
      asm volatile("bar.sync 1, %0;" ::"r"(DL_CT) : "memory");
    }
  }
  __syncthreads();
  if (*abort_flag && tid == 0) atomicExch(P.err, 4);
}

// ---- host side --------------------------------------------------------------------------------
bool dpk_decode_layer_plan(dp_ctx *ctx, DlParams *P) {
  uint32_t digit_bytes = 0, slot = 0;
  for (int p = 0; p < P->n_phases; p++) {
    DlPhase &ph = P->ph[p];
    if (ph.K <= 0 || ph.K % QK_K || ph.N % 16) return false;
    if (ph.src == DL_SRC_RMSNORM || ph.src == DL_SRC_XCHG_RMSNORM) {
      if (ph.K > 2 * DL_NW * QK_K || ph.K != P->hidden) return false;  // two blocks per warp in registers
      if (ph.src == DL_SRC_XCHG_RMSNORM && ph.K > DP_TP_SLOT_FLOATS) return false;
    }
    if (ph.out == DL_OUT_PUSH && ph.N > DP_TP_SLOT_FLOATS) return false;
    if (ph.out == DL_OUT_SILU && (ph.N % 16 || !P->act)) return false;
    if (ph.src == DL_SRC_ACT && !P->act) return false;
    const uint32_t db = dl_digit_bytes(ph.K);
    if (db > digit_bytes) digit_bytes = db;
    ph.cb = 0;
    if (ph.N == 0) continue;
    const int bpr = ph.K / QK_K;
    // chunk = the largest divisor of the row's block count whose stage (16 padded row pieces) stays
    // under 56 KB: long per-row copies keep the number of bulk-copy requests per byte low
    for (int c = bpr; c >= 1; c--)
      if (bpr % c == 0 && c <= DL_MAX_BW * DL_CONSUMERS && 16 * (c * Q4K_BLOCK_BYTES + DL_ROW_PAD) <= 56 * 1024) { ph.cb = c; break; }
    if (!ph.cb) return false;
    const uint32_t sb = 16u * ((uint32_t)ph.cb * Q4K_BLOCK_BYTES + DL_ROW_PAD);
    if (sb > slot) slot = sb;
  }
  if (!slot) slot = 16u * (Q4K_BLOCK_BYTES + DL_ROW_PAD);
  size_t budget = (size_t)227 * 1024;
  if (budget > ctx->smem_optin) budget = ctx->smem_optin;
  int stages = 12;
  while (stages >= 2 && dl_layout(digit_bytes, (uint32_t)P->hidden * 4u, slot, stages).total > budget) stages--;
  if (stages < 2) return false;
  P->digit_bytes = digit_bytes;
  P->slot_bytes = slot;
  P->stages = stages;
  return true;
}

dp_status dpk_decode_layer(dp_ctx *ctx, const DlParams &P) {
  static bool attr_set = false;
  if (!attr_set) {
    DP_CUDA(ctx, cudaFuncSetAttribute(decode_layer_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set = true;
  }
  const uint32_t smem = dl_layout(P.digit_bytes, (uint32_t)P.hidden * 4u, P.slot_bytes, P.stages).total;
  DP_LAUNCH(ctx, decode_layer_kernel, ctx->sm_count, (DL_NW + 1) * 32, smem, P);
  return DP_OK;
}
