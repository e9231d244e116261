// AllGather schedules.  Reference: src/coll/allgather.c — RING :3-46, K_RING
// :49-123, RD :126-171, RM :174-230, PRD :233-288, PRM :517-570.  The permuted
// variants place every incoming block at its final offset while it arrives, so
// the index kernel, the host synchronisation and the in-place permutation of
// the reference (:245-282) have no counterpart here.
#include "coll_internal.h"

namespace piccl {

static Program ag_ring(const CollArgs& a, int rank) {
  int n = a.nranks; int64_t st = a.block_stride ? a.block_stride : a.count;
  Builder b(rank, n);
  int right = (rank + 1) % n, left = mod(rank - 1, n);
  std::vector<int> sd; if (n > 1) sd.push_back(right);
  b.act(BUF_IN, 0, a.in_place ? BUF_NONE : BUF_OUT, rank * st, a.count, {}, sd);
  b.next_step();
  for (int i = 1; i < n; i++) {
    std::vector<int> fw; if (i < n - 1) fw.push_back(right);
    b.act(BUF_NONE, 0, BUF_OUT, mod(rank - i, n) * st, a.count, {left}, fw);
    b.next_step();
  }
  return b.finish();
}

static Program ag_k_ring(const CollArgs& a, int rank, int k) {
  int n = a.nranks, g = n / k, grp = rank / k, rel = rank % k;
  int64_t st = a.block_stride ? a.block_stride : a.count;
  Builder b(rank, n);
  int inter_next = (rank + k) % n, inter_prev = mod(rank - k, n);
  int intra_next = grp * k + (rel + 1) % k, intra_prev = grp * k + mod(rel - 1, k);
  // phase A: ring over the groups between ranks of equal position (allgather.c:78-90)
  {
    std::vector<int> sd; if (g > 1) sd.push_back(inter_next);
    b.act(BUF_IN, 0, a.in_place ? BUF_NONE : BUF_OUT, rank * st, a.count, {}, sd);
    b.next_step();
    for (int i = 1; i < g; i++) {
      std::vector<int> fw; if (i < g - 1) fw.push_back(inter_next);
      b.act(BUF_NONE, 0, BUF_OUT, mod(rank - i * k, n) * st, a.count, {inter_prev}, fw);
      b.next_step();
    }
  }
  // phase B: one ring per group of blocks inside my group (allgather.c:93-119)
  if (k > 1) for (int t = 0; t < g; t++) {
    int off = mod(grp - t, g) * k;
    if (t == 0) b.act(BUF_IN, 0, BUF_NONE, 0, a.count, {}, {intra_next});
    else b.act(BUF_OUT, (off + rel) * st, BUF_NONE, 0, a.count, {}, {intra_next});
    b.next_step();
    for (int j = 1; j < k; j++) {
      std::vector<int> fw; if (j < k - 1) fw.push_back(intra_next);
      b.act(BUF_NONE, 0, BUF_OUT, (off + mod(rel - j, k)) * st, a.count, {intra_prev}, fw);
      b.next_step();
    }
  }
  return b.finish();
}

static Program ag_recursive(const CollArgs& a, const Resolved& rs, int rank, bool permuted) {
  int n = a.nranks; int64_t st = a.block_stride ? a.block_stride : a.count;
  Builder b(rank, n);
  if (rs.radices.empty() && !a.in_place) b.act(BUF_IN, 0, BUF_OUT, rank * st, a.count, {}, {});
  for (size_t s = 0; s < rs.radices.size(); s++) {
    std::vector<int> peers = step_peers(rank, (int)s, rs.radices, n, permuted);
    std::vector<int> mine = held_blocks(rank, (int)s, rs.radices, n, permuted);
    std::vector<std::vector<int>> theirs;
    for (int p : peers) theirs.push_back(held_blocks(p, (int)s, rs.radices, n, permuted));
    if (s == 0) {
      b.act(BUF_IN, 0, a.in_place ? BUF_NONE : BUF_OUT, rank * st, a.count, {}, peers);
      for (size_t i = 0; i < peers.size(); i++) b.act(BUF_NONE, 0, BUF_OUT, theirs[i][0] * st, a.count, {peers[i]}, {});
    } else {
      // One action per block (never merged): every action that touches a block slices it
      // among CTAs and segments in the same way, so each CTA only ever depends on data it
      // handled itself.  Farthest-first (permuted) order stores each block straight at its
      // final offset.
      for (size_t q = 0; q < mine.size(); q++) {
        b.act(BUF_OUT, mine[q] * st, BUF_NONE, 0, a.count, {}, peers);
        for (size_t i = 0; i < peers.size(); i++) b.act(BUF_NONE, 0, BUF_OUT, theirs[i][q] * st, a.count, {peers[i]}, {});
      }
    }
    b.next_step();
  }
  return b.finish();
}

Program compile_allgather(const CollArgs& a, const Resolved& rs, int rank) {
  switch (rs.algo) {
    case ALGO_K_RING: return ag_k_ring(a, rank, rs.k);
    case ALGO_RD: case ALGO_RM: return ag_recursive(a, rs, rank, false);
    case ALGO_PRD: case ALGO_PRM: return ag_recursive(a, rs, rank, true);
    default: return ag_ring(a, rank);
  }
}

}  // namespace piccl
