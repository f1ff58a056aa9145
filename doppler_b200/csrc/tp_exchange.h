// Layout of the peer-memory exchange area used by the one-shot allreduce (tp.cu, model.cu).
#pragma once
#include <stddef.h>
#include <stdint.h>

#define DP_TP_MAX_RANKS 8
#define DP_TP_SLOT_FLOATS 8192  // largest vector the one-shot path carries (one token of hidden state)

// area (floats): [parity 0..1][source rank 0..7][DP_TP_SLOT_FLOATS], then flags u32 [parity][source rank]
#ifdef __CUDACC__
#define DP_HD __host__ __device__
#else
#define DP_HD
#endif
DP_HD static inline size_t dp_tp_flags_offset_floats() { return (size_t)2 * DP_TP_MAX_RANKS * DP_TP_SLOT_FLOATS; }
static inline size_t dp_tp_area_bytes() { return (dp_tp_flags_offset_floats() + 2 * DP_TP_MAX_RANKS + 64) * sizeof(float); }

struct dp_tp_exchange {
  int rank, size;
  float *area[DP_TP_MAX_RANKS];  // every rank's area, mapped into this process
  unsigned epoch;                // number of exchanges done so far (device side)
};
