// Layout of the peer-memory exchange area (tp.cu) used by the decode-step kernels
// (gemv_q4k_fast.cu, model.cu; helpers in handoff.cuh).  No counterpart in the reference, which has no collective backend.
//
// Every rank owns one area in its own HBM, mapped into every other rank with CUDA IPC.  A rank PUSHES
// its data into its own slot of every rank's area with ordinary stores over NVLink; a consumer reads
// slots in its OWN memory only.  Nothing is ever loaded from a peer, and no bulk/TMA copy touches peer
// memory.
//
// Hand-off without fences or counters: every element travels as one aligned 8-byte word
// (value, ticket).  An 8-byte store is a single transaction, so a reader that sees the ticket it is
// waiting for also sees the value that was stored with it; it simply re-reads (with a bound) until the
// ticket matches.  Tickets are numbers that grow from exchange to exchange and never repeat.
//
//   vector slots   (f32, u32) [2 parities][DP_TP_MAX_RANKS][DP_TP_SLOT_FLOATS]   partial output vectors of
//                  the row-parallel projections: parity 0 after o_proj, parity 1 after down_proj
//   argmax slots   (f32, u32) [2 parities][DP_TP_MAX_RANKS][DP_TP_MAX_BATCH][2]  best logit / global index
// Two parities of slots: a rank finishes reading exchange x only when every rank has pushed x, and it
// pushes x + 2 (the same parity) only after it has read x + 1 from every rank, which every rank pushes
// after it has finished reading x.  So a push never overwrites what a slower rank still has to read.
#pragma once
#include <stddef.h>
#include <stdint.h>

#define DP_TP_MAX_RANKS 8
#define DP_TP_SLOT_FLOATS 8192  // largest vector the exchange carries (one token of hidden state)
#define DP_TP_MAX_BATCH 256

#ifdef __CUDACC__
#define DP_HD __host__ __device__
#else
#define DP_HD
#endif
// offsets in 8-byte words from the start of an area
DP_HD static inline size_t dp_tp_slot_offset(unsigned parity, int rank) {
  return ((size_t)(parity & 1u) * DP_TP_MAX_RANKS + (size_t)rank) * DP_TP_SLOT_FLOATS;
}
DP_HD static inline size_t dp_tp_am_slot_offset(unsigned parity, int rank) {
  return (size_t)2 * DP_TP_MAX_RANKS * DP_TP_SLOT_FLOATS + ((size_t)(parity & 1u) * DP_TP_MAX_RANKS + (size_t)rank) * DP_TP_MAX_BATCH * 2;
}
static inline size_t dp_tp_area_bytes() { return ((size_t)2 * DP_TP_MAX_RANKS * DP_TP_SLOT_FLOATS + (size_t)2 * DP_TP_MAX_RANKS * DP_TP_MAX_BATCH * 2 + 64) * 8; }

// Descriptor handed to kernels; lives in this rank's device memory.
struct dp_tp_exchange {
  int rank, size;
  uint2 *area[DP_TP_MAX_RANKS];  // every rank's area as seen from this process (area[rank] is local)
  unsigned am_ticket;            // argmax exchanges done so far (device side)
};
