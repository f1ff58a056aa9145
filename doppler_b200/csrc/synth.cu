// Seeded synthetic inputs, generated on the host: packed Q4_K weight blocks,
// normal f32/f16 tensors and token ids.  Counter based (element i of stream
// `key` depends only on (key, i)), so any shard of a tensor can be produced on
// its own and every rank of a tensor-parallel run sees the same model.
//
// These stand in for real checkpoints: Q4_K blocks get d, dmin = f16(|N(0,0.02)|),
// uniform 6-bit scale/min codes and uniform 4-bit quants.
#include "common.h"

#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

static inline uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ULL;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}
static inline uint64_t stream_word(uint64_t key, uint64_t i) { return mix64(key + i * 0x9E3779B97F4A7C15ULL); }
static inline float normal_from_word(uint64_t h) {
  const float u1 = (float)((h >> 40) + 1u) * (1.0f / 16777216.0f);
  const float u2 = (float)((h >> 16) & 0xFFFFFFu) * (1.0f / 16777216.0f);
  return sqrtf(-2.0f * logf(u1)) * cosf(6.2831853071795864f * u2);
}
static inline uint16_t f16_bits(float v) {
  __half h = __float2half_rn(v);
  uint16_t u;
  memcpy(&u, &h, 2);
  return u;
}

template <typename F>
static void parallel_for(size_t n, F f) {
  unsigned hw = std::thread::hardware_concurrency();
  size_t nt = hw ? hw : 4;
  if (nt > 32) nt = 32;
  if (n < 65536 || nt == 1) { f(0, n); return; }
  std::vector<std::thread> th;
  const size_t chunk = (n + nt - 1) / nt;
  for (size_t t = 0; t < nt; t++) {
    const size_t lo = t * chunk, hi = lo + chunk < n ? lo + chunk : n;
    if (lo >= hi) break;
    th.emplace_back([=] { f(lo, hi); });
  }
  for (auto &t : th) t.join();
}

extern "C" uint64_t dp_synth_key(uint64_t seed, uint64_t tensor_id) { return mix64(seed * 0x100000001B3ULL + tensor_id); }

extern "C" void dp_synth_normal_f32(uint64_t key, uint64_t first, size_t n, float sigma, float mean, float *out) {
  parallel_for(n, [=](size_t lo, size_t hi) {
    for (size_t i = lo; i < hi; i++) out[i] = mean + sigma * normal_from_word(stream_word(key, first + i));
  });
}

extern "C" void dp_synth_normal_f16(uint64_t key, uint64_t first, size_t n, float sigma, void *out) {
  uint16_t *o = (uint16_t *)out;
  parallel_for(n, [=](size_t lo, size_t hi) {
    for (size_t i = lo; i < hi; i++) o[i] = f16_bits(sigma * normal_from_word(stream_word(key, first + i)));
  });
}

extern "C" void dp_synth_q4k_blocks(uint64_t key, uint64_t first_block, size_t n_blocks, void *out) {
  uint8_t *o = (uint8_t *)out;
  parallel_for(n_blocks, [=](size_t lo, size_t hi) {
    for (size_t b = lo; b < hi; b++) {
      const uint64_t base = (first_block + b) * 20u;
      uint8_t *blk = o + b * DP_Q4K_BLOCK_BYTES;
      const uint16_t d = f16_bits(fabsf(0.02f * normal_from_word(stream_word(key, base))));
      const uint16_t dm = f16_bits(fabsf(0.02f * normal_from_word(stream_word(key, base + 1))));
      memcpy(blk, &d, 2);
      memcpy(blk + 2, &dm, 2);
      uint8_t bytes[144];
      for (int j = 0; j < 18; j++) {
        const uint64_t w = stream_word(key, base + 2 + (uint64_t)j);
        memcpy(bytes + j * 8, &w, 8);
      }
      memcpy(blk + 4, bytes, 140);
    }
  });
}

extern "C" void dp_synth_tokens(uint64_t key, size_t n, int vocab, int32_t *out) {
  for (size_t i = 0; i < n; i++) out[i] = (int32_t)(stream_word(key, i) % (uint64_t)vocab);
}
