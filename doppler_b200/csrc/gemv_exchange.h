// Tensor-parallel exchange hooks of the decode GEMV kernel (gemv_q4k_fast.cu): what its prologue reads
// from, and its epilogue pushes into, the peer-memory exchange areas (tp_exchange.h, handoff.cuh).
#pragma once
#include <stdint.h>
#include <vector_types.h>

struct GemvExchange {
  int rank = 0, nr = 0;                 // nr == 0: no exchange on this launch
  uint2 *area[8] = {};                  // every rank's exchange area (area[rank] is local memory)
  const uint2 *mine = nullptr;          // area[rank]
  const unsigned *ticket_step = nullptr;  // device counter of decode steps: tickets of a step start at *ticket_step * ticket_stride + 1
  unsigned ticket_stride = 0;
  unsigned ticket_in = 0, ticket_out = 0;  // offsets (within the step) of the hand-off read by the prologue / written by the epilogue
  int parity_in = 0, parity_out = 0;    // slot parity of those hand-offs
  int push = 0;                         // 1: output rows go into the exchange areas instead of y
  float *h_out = nullptr;               // SRC_XCHG_RMSNORM: the updated residual stream (every CTA writes its share)
  unsigned wait_limit = 0;              // polls before the prologue's wait for the other ranks gives up
};
