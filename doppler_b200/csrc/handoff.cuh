// Ticketed 8-byte hand-off between CTAs and between ranks (layout and rationale: tp_exchange.h).
// A writer stores (value, ticket) as ONE aligned 8-byte word; a reader re-reads, with a bound, until the
// ticket is the one it waits for.  An 8-byte store is a single transaction, so a matching ticket proves
// the value next to it, and neither side needs a fence.  Reads go to L2 (volatile), never to a stale L1 line.
#pragma once
#include <stdint.h>

__device__ __forceinline__ void handoff_put(uint2 *p, float v, unsigned ticket) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(ticket) : "memory");
}
__device__ __forceinline__ uint4 handoff_peek2(const uint2 *p) {  // two words
  uint4 r;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
  return r;
}
// Eight consecutive words: re-read until all carry `ticket`, at most `limit` times, or until another thread of
// the CTA has given up (abort flag in shared memory).  false: gave up (the abort flag is then set).
__device__ __forceinline__ bool handoff_take8(const uint2 *p, unsigned ticket, float (&v)[8], unsigned limit, volatile int *abort_flag) {
  for (unsigned it = 0; it < limit; it++) {
    const uint4 a = handoff_peek2(p), b = handoff_peek2(p + 2), c = handoff_peek2(p + 4), d = handoff_peek2(p + 6);
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
