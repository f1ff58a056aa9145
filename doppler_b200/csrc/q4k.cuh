// Device-side helpers for the Q4_K super-block (256 weights in 144 bytes).
//
// Layout (identical to the reference's Q4KBlock, src/gpu/kernels/fused_matmul_q4.wgsl:37-41,
// writer src/converter/quantizer.js:137-163):
//   bytes 0-1  d    (f16)      bytes 2-3  dmin (f16)
//   bytes 4-15 twelve scale bytes: b[4+i] = sc_i | (sc_{i+4}>>4)<<6, b[8+i] = m_i | (m_{i+4}>>4)<<6,
//              b[12+i] = (sc_{i+4}&15) | (m_{i+4}&15)<<4        (i = 0..3)
//   bytes 16-143 qs: chunk c (32 bytes) byte i: low nibble = element 64c+i (sub-block 2c),
//              high nibble = element 64c+32+i (sub-block 2c+1)
//   weight = (d*sc_s)*q - (dmin*m_s),  s = element/32
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#define Q4K_BLOCK_BYTES 144
#define Q4K_BLOCK_WORDS 36
#define QK_K 256

struct Q4KScales {
  uint32_t sc03, sc47, mn03, mn47;  // one 6-bit code per byte
};

// u0,u1,u2 = words 1..3 of the block (bytes 4..15)
__device__ __forceinline__ Q4KScales q4k_unpack_scales(uint32_t u0, uint32_t u1, uint32_t u2) {
  Q4KScales s;
  s.sc03 = u0 & 0x3f3f3f3fu;
  s.mn03 = u1 & 0x3f3f3f3fu;
  s.sc47 = (u2 & 0x0f0f0f0fu) | ((u0 >> 2) & 0x30303030u);
  s.mn47 = ((u2 >> 4) & 0x0f0f0f0fu) | ((u1 >> 2) & 0x30303030u);
  return s;
}

__device__ __forceinline__ uint32_t q4k_byte(uint32_t w, int i) { return (w >> (8 * i)) & 0xffu; }

// code of sub-block s (0..7)
__device__ __forceinline__ uint32_t q4k_sc(const Q4KScales &s, int sb) {
  return sb < 4 ? q4k_byte(s.sc03, sb) : q4k_byte(s.sc47, sb - 4);
}
__device__ __forceinline__ uint32_t q4k_mn(const Q4KScales &s, int sb) {
  return sb < 4 ? q4k_byte(s.mn03, sb) : q4k_byte(s.mn47, sb - 4);
}

__device__ __forceinline__ float2 q4k_d_dmin(uint32_t w0) {
  __half2 h = *reinterpret_cast<__half2 *>(&w0);
  return __half22float2(h);
}

// exact small-integer -> float without the conversion pipe: 0x4B000000 is 2^23
__device__ __forceinline__ float q4k_u8_to_float(uint32_t v) {
  return __uint_as_float(0x4B000000u | v) - 8388608.0f;
}
