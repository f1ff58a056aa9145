// tcgen05 / tensor-memory / TMA helpers in inline PTX shared by the tensor-core GEMM kernels (sm_100a).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mbar.cuh"

namespace umma {

constexpr int BK = 64;  // K step: 64 f16 = one 128-byte swizzled line per row

__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  // K-major operand, 128-byte swizzle: 8-row groups are 1024 bytes apart (SBO); LBO unused
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);       // start address
  d |= (uint64_t)0 << 16;                             // leading byte offset
  d |= (uint64_t)(1024u >> 4) << 32;                  // stride byte offset
  d |= (uint64_t)1 << 46;                             // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                             // layout: SWIZZLE_128B
  return d;
}

__device__ __forceinline__ uint32_t umma_idesc_f16(int M, int N) {
  // D = f32, A = B = f16, both K-major
  return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(map), "r"(x), "r"(y), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,"
      "%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// ---- two-CTA cluster helpers (two-SM kernel) ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {  // same offset in another CTA of the cluster
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {  // acquire at cluster scope
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  for (uint32_t i = 0; i < (1u << 20); i++) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((i & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Output scale: alpha, times an optional factor per output row (f32 activations are brought into f16 range
// row by row with a power of two, which the epilogue multiplies back)
struct TcAlpha {
  float value;
  const float *row_scale;
  int k_splits;  // one-SM kernel: parts of K per output tile (grid.z); part z writes its f32 sums to C + z * M * N
  // f32 output, k_splits == 1: the columns are gate|up pairs (eight gate columns, then their eight up columns, per
  // group of sixteen) and the epilogue stores silu(gate) * up, N / 2 columns per row, instead of the N raw ones
  int silu_out;
};

// silu(gate) * up of one group of sixteen accumulator columns (silu.wgsl:30-37,98-104: sigmoid argument clamped to +-15)
__device__ __forceinline__ void tc_silu_group(const uint32_t *r, float arow, float *o) {
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const float g = __uint_as_float(r[j]) * arow, u = __uint_as_float(r[8 + j]) * arow;
    const float cl = fminf(fmaxf(g, -15.0f), 15.0f);
    o[j] = (g * (1.0f / (1.0f + expf(-cl)))) * u;
  }
}

// Two dequantised weights as f16, and (NPROD >= 2) their f16 rounding residues w - f16(w): the part of each
// weight that the rounding drops, which a second product adds back.
__device__ __forceinline__ uint32_t tc_pack_hi(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}
__device__ __forceinline__ uint32_t tc_pack_lo(float a, float b, uint32_t hi) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&hi));
  const __half2 h = __floats2half2_rn(a - f.x, b - f.y);
  return *reinterpret_cast<const uint32_t *>(&h);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn get_encode() {
  // resolved once per process (initialisation of a function-local static is thread safe)
  static const EncodeTiledFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      return (EncodeTiledFn)p;
    return (EncodeTiledFn) nullptr;
  }();
  return fn;
}

}  // namespace umma
