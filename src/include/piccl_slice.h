// How one action's element range is divided among CTAs and FIFO segments.
// Shared by the device executor and the CPU validator so both sides of every
// connection agree on the number and size of FIFO entries.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define PICCL_HD __host__ __device__ __forceinline__
#else
#define PICCL_HD inline
#endif

namespace piccl {

struct Slice { int64_t lo, hi; int64_t seg_elems; int nseg; };

// Elements are grouped in 16-byte packs (relative to the start of the action);
// CTA c gets a contiguous run of packs; a segment is at most slot_bytes.
PICCL_HD Slice slice_of(int64_t count, int elem_size, int cta, int n_cta, int64_t slot_bytes) {
  int64_t pack = elem_size >= 16 ? 1 : 16 / elem_size;
  int64_t npack = (count + pack - 1) / pack;
  int64_t per = (npack + n_cta - 1) / n_cta;
  int64_t lo = (int64_t)cta * per; if (lo > npack) lo = npack;
  int64_t hi = lo + per; if (hi > npack) hi = npack;
  Slice s;
  s.lo = lo * pack; s.hi = hi * pack; if (s.hi > count) s.hi = count; if (s.lo > count) s.lo = count;
  s.seg_elems = (slot_bytes / 16) * pack;
  int64_t len = s.hi - s.lo;
  s.nseg = (int)((len + s.seg_elems - 1) / s.seg_elems);
  return s;
}

}  // namespace piccl
