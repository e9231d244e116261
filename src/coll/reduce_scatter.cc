// ReduceScatter schedules.  The reference only has stubs here
// (src/coll/reduce_scatter.c:3-29); these are the natural completions: RING and
// K_RING are the reduce-scatter halves of the allreduce variants, the recursive
// ones are the recursive allgathers run backwards with the reduction folded
// into each exchange (recursive halving / k-ary splitting).
#include "coll_internal.h"

namespace piccl {

static Program rsc_ring_like(const CollArgs& a, int rank, int k) {
  int n = a.nranks; int64_t st = a.block_stride ? a.block_stride : a.count;
  Builder b(rank, n);
  RsChain c = rs_chain(rank, n, k);
  for (size_t i = 0; i < c.chunk.size(); i++) {
    std::vector<int> rv; if (i > 0) rv.push_back(c.from[i]);
    b.act(BUF_IN, c.chunk[i] * st, BUF_NONE, 0, a.count, rv, {c.to[i]});
    b.next_step();
  }
  std::vector<int> rv; if (!c.chunk.empty()) rv.push_back(c.final_from);
  if (n > 1 || !a.in_place) b.act(BUF_IN, rank * st, BUF_OUT, 0, a.count, rv, {});
  b.next_step();
  return b.finish();
}

static Program rsc_recursive(const CollArgs& a, const Resolved& rs, int rank, bool permuted) {
  int n = a.nranks; int64_t st = a.block_stride ? a.block_stride : a.count;
  int p = (int)rs.radices.size();
  Builder b(rank, n);
  if (p == 0) { if (!a.in_place) b.act(BUF_IN, rank * st, BUF_OUT, 0, a.count, {}, {}); return b.finish(); }
  int64_t pack = a.elem_size >= 16 ? 1 : 16 / a.elem_size;
  int64_t slot_stride = (a.count + pack - 1) / pack * pack;
  std::vector<int> kept = held_blocks(rank, p - 1, rs.radices, n, permuted);   // blocks that get a scratch slot
  std::vector<int> slot_of(n, -1), in_scratch(n, 0);
  for (size_t i = 0; i < kept.size(); i++) slot_of[kept[i]] = (int)i;
  if (p >= 2) b.prog.scratch_elems = (int64_t)kept.size() * slot_stride;
  auto acc_buf = [&](int blk) { return in_scratch[blk] ? BUF_SCRATCH : BUF_IN; };
  auto acc_off = [&](int blk) { return in_scratch[blk] ? slot_of[blk] * slot_stride : blk * st; };
  for (int s = p - 1; s >= 0; s--) {
    std::vector<int> peers = step_peers(rank, s, rs.radices, n, permuted);
    std::vector<int> mine = held_blocks(rank, s, rs.radices, n, permuted);
    std::vector<std::vector<int>> theirs;
    for (int pr : peers) theirs.push_back(held_blocks(pr, s, rs.radices, n, permuted));
    for (size_t q = 0; q < mine.size(); q++) {
      for (size_t i = 0; i < peers.size(); i++) { int blk = theirs[i][q]; b.act(acc_buf(blk), acc_off(blk), BUF_NONE, 0, a.count, {}, {peers[i]}); }
      int blk = mine[q];
      if (s == 0) b.act(acc_buf(blk), acc_off(blk), BUF_OUT, 0, a.count, peers, {});
      else { Buf sb = acc_buf(blk); int64_t so = acc_off(blk); in_scratch[blk] = 1; b.act(sb, so, BUF_SCRATCH, acc_off(blk), a.count, peers, {}); }
    }
    b.next_step();
  }
  return b.finish();
}

Program compile_reduce_scatter(const CollArgs& a, const Resolved& rs, int rank) {
  switch (rs.algo) {
    case ALGO_K_RING: return rsc_ring_like(a, rank, rs.k);
    case ALGO_RD: case ALGO_RM: return rsc_recursive(a, rs, rank, false);
    case ALGO_PRD: case ALGO_PRM: return rsc_recursive(a, rs, rank, true);
    default: return rsc_ring_like(a, rank, a.nranks);
  }
}

}  // namespace piccl
