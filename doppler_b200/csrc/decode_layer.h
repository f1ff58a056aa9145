// Parameters of the persistent per-layer decode kernel (decode_layer.cu).
#pragma once
#include <stdint.h>
#include <vector_types.h>

struct dp_ctx;

#define DL_MAX_PHASES 4
#define DL_MAX_RANKS 8

// where a phase's input vector comes from
enum {
  DL_SRC_RMSNORM = 1,       // rmsnorm(h) * w, h = the residual stream as the launch found it
  DL_SRC_XCHG_RMSNORM = 2,  // h += sum over ranks of the partial vectors pushed by the previous phase, then rmsnorm(h) * w
  DL_SRC_ACT = 3,           // silu(gate) * up, written element by element by the previous phase's epilogue
  DL_SRC_COMBINE = 4,       // merge of the split-K attention partials (layout of attention.cu)
  DL_SRC_VECTOR = 5,        // an f32 vector an earlier kernel left in memory (the merged attention output)
};
// where its output rows go
enum {
  DL_OUT_STORE = 0,  // y[row]: read after the launch
  DL_OUT_PUSH = 1,   // (value, ticket) into this rank's slot of every rank's exchange area
  DL_OUT_SILU = 2,   // rows come as eight gate rows then their eight up rows: silu(gate) * up as (value, ticket) into act[]
};

struct DlPhase {
  const uint8_t *W;     // packed Q4_K [N, K]; N == 0: the phase only runs its prologue
  int N, K, cb;         // cb (super-blocks per ring stage and row) is filled in by the planner
  int src;              // DL_SRC_*
  int out;              // DL_OUT_*
  unsigned ticket_in;   // XCHG_RMSNORM / ACT: ticket offset (within the step) of the hand-off this phase reads
  unsigned ticket_out;  // PUSH / SILU: ticket offset of the hand-off this phase writes
  int parity;           // XCHG_RMSNORM reads / PUSH writes this parity of the exchange slots
  const float *x;       // COMBINE: attention split partials; VECTOR: the vector
  const float *norm_w;  // RMSNORM / XCHG_RMSNORM
  float *h_out;         // XCHG_RMSNORM, optional: the updated residual stream (every CTA writes its share)
  float *n_out;         // optional: the normalised vector in f32 (written by CTA 0)
  float *y;             // DL_OUT_STORE target [N]
};

struct DlParams {
  DlPhase ph[DL_MAX_PHASES];
  int n_phases;
  float eps;
  int D, splits;               // DL_SRC_COMBINE: head_dim and number of KV splits
  const float *h_in;           // residual stream at the start of the launch (f32 [hidden]) or null
  int hidden;
  int rank, nr;                // exchange group (one rank on a single GPU)
  uint2 *area[DL_MAX_RANKS];   // every rank's exchange area (area[rank] is local memory)
  uint2 *act;                  // local (value, ticket) buffer of the SiLU hand-off, [inter]
  const unsigned *ticket_step; // device counter: tickets of this step start at *ticket_step * ticket_stride
  unsigned ticket_stride;
  int stages;                  // ring depth, slot size and digit area: filled in by the planner
  uint32_t slot_bytes, digit_bytes;
  unsigned wait_limit;         // polls before a wait on another CTA / rank gives up
  int *err;
};

// fills cb / stages / slot_bytes / digit_bytes; false when a phase's shape has no plan
bool dpk_decode_layer_plan(dp_ctx *ctx, DlParams *P);
