// Fixed-point activation digits for the fast Q4_K decode GEMV (see gemv_q4k_fast.cu).
//
// One warp turns one 256-element block of an f32 activation vector into
//   limbs  int8 [8 sub-blocks][4][32]   three signed base-256 digits per value (column 3 zero)
//   xscale f32                           2^(e - 22), e = exponent of the block's max magnitude
//   ssum   f32 [8]                       sum of the fixed-point integers of each sub-block
// Lane l holds elements 8l .. 8l+7 of the block.  Buffer layout for K = 256*bpr values:
//   [limbs: K*4 bytes][xscale: bpr floats][ssum: K/32 floats]
#pragma once
#include <stdint.h>

__device__ __forceinline__ void actq_emit_block(const float v[8], int lane, int b, int bpr, void *actq) {
  int8_t *limbs = reinterpret_cast<int8_t *>(actq);
  float *xscale = reinterpret_cast<float *>(limbs + (size_t)bpr * 256 * 4);
  float *ssum = xscale + bpr;
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  int e = 0;
  if (amax > 0.0f) frexpf(amax, &e);  // amax < 2^e
  if (e < -100) e = -100;
  const float up = ldexpf(1.0f, 22 - e);
  int s = 0;
  uint32_t d[3][2] = {{0, 0}, {0, 0}, {0, 0}};
#pragma unroll
  for (int i = 0; i < 8; i++) {
    int r = __float2int_rn(v[i] * up);
    s += r;
    const int l0 = ((r + 128) & 255) - 128;
    r = (r - l0) >> 8;
    const int l1 = ((r + 128) & 255) - 128;
    const int l2 = (r - l1) >> 8;
    d[0][i >> 2] |= (uint32_t)(l0 & 255) << (8 * (i & 3));
    d[1][i >> 2] |= (uint32_t)(l1 & 255) << (8 * (i & 3));
    d[2][i >> 2] |= (uint32_t)(l2 & 255) << (8 * (i & 3));
  }
  // Digit layout per block (1024 bytes): four chunks (sub-block pairs) of eight 32-byte columns; column
  // 2*limb + (sub-block & 1) holds that limb of that sub-block, columns 6 and 7 are never read.  A lane of
  // the GEMV that loads column g of a chunk once has the B operand of both MMAs of the chunk.
  const int sbl = lane >> 2;
  const int sb = b * 8 + sbl;
  uint2 *dst = reinterpret_cast<uint2 *>(limbs + (size_t)b * 1024 + (size_t)(sbl >> 1) * 256 + (size_t)(sbl & 1) * 32) + (lane & 3);
  dst[0] = make_uint2(d[0][0], d[0][1]);
  dst[8] = make_uint2(d[1][0], d[1][1]);
  dst[16] = make_uint2(d[2][0], d[2][1]);
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  if ((lane & 3) == 0) ssum[sb] = (float)s;
  float sc = ldexpf(1.0f, e - 22);
  if (!(amax <= 3.0e38f)) sc = __int_as_float(0x7fc00000);  // inf / nan activations poison the block
  if (lane == 0) xscale[b] = sc;
}
