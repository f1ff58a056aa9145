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

// Two slots at once (two ranks' words of the same elements): the eight 16-byte reads are in flight together, so a
// gather over R ranks costs R / 2 round trips to L2 instead of R.  Same give-up rules as handoff_take8.
__device__ __forceinline__ bool handoff_take8x2(const uint2 *p0, const uint2 *p1, unsigned ticket, float (&v0)[8], float (&v1)[8], unsigned limit,
                                                volatile int *abort_flag) {
  for (unsigned it = 0; it < limit; it++) {
    const uint4 a = handoff_peek2(p0), b = handoff_peek2(p0 + 2), c = handoff_peek2(p0 + 4), d = handoff_peek2(p0 + 6);
    const uint4 e = handoff_peek2(p1), f = handoff_peek2(p1 + 2), g = handoff_peek2(p1 + 4), h = handoff_peek2(p1 + 6);
    const bool ok0 = a.y == ticket && a.w == ticket && b.y == ticket && b.w == ticket && c.y == ticket && c.w == ticket && d.y == ticket && d.w == ticket;
    const bool ok1 = e.y == ticket && e.w == ticket && f.y == ticket && f.w == ticket && g.y == ticket && g.w == ticket && h.y == ticket && h.w == ticket;
    if (ok0 && ok1) {
      v0[0] = __uint_as_float(a.x); v0[1] = __uint_as_float(a.z); v0[2] = __uint_as_float(b.x); v0[3] = __uint_as_float(b.z);
      v0[4] = __uint_as_float(c.x); v0[5] = __uint_as_float(c.z); v0[6] = __uint_as_float(d.x); v0[7] = __uint_as_float(d.z);
      v1[0] = __uint_as_float(e.x); v1[1] = __uint_as_float(e.z); v1[2] = __uint_as_float(f.x); v1[3] = __uint_as_float(f.z);
      v1[4] = __uint_as_float(g.x); v1[5] = __uint_as_float(g.z); v1[6] = __uint_as_float(h.x); v1[7] = __uint_as_float(h.z);
      return true;
    }
    if ((it & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
