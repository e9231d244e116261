// AllReduce schedules.  Reference: src/coll/allreduce.c — RING :97-155,
// K_RING :157-280, RD :282-348, RM :350-449, PRD :451-522, PRM :524-614.
// Differences: the partial sum travels from FIFO to FIFO and is reduced with
// the local operand while it is forwarded, so the ring variants are a chain
// of 2(n-1) fused hops per rank, and the recursive variants reduce all k-1
// incoming buffers in one pass.
#include "coll_internal.h"

namespace piccl {

static Program ar_ring_like(const CollArgs& a, int rank, int k) {
  int n = a.nranks;
  Builder b(rank, n);
  std::vector<int64_t> displ, cnt; ar_chunks(a.count, n, a.elem_size, displ, cnt);
  RsChain c = rs_chain(rank, n, k);
  int right = (rank + 1) % n, left = mod(rank - 1, n);
  // reduce-scatter: hop i forwards chunk[i] (+ my contribution) towards its owner
  for (size_t i = 0; i < c.chunk.size(); i++) {
    int ch = c.chunk[i];
    std::vector<int> rv; if (i > 0) rv.push_back(c.from[i]);
    b.act(BUF_IN, displ[ch], BUF_NONE, 0, cnt[ch], rv, {c.to[i]});
    b.next_step();
  }
  // the last partial arrives: chunk `rank` is complete; it starts the ring allgather
  // (the reference's allgather phase is the plain ring for both variants, allreduce.c:279)
  {
    std::vector<int> rv; if (!c.chunk.empty()) rv.push_back(c.final_from);
    std::vector<int> sd; if (n > 1) sd.push_back(right);
    if (n > 1 || !a.in_place) b.act(BUF_IN, displ[rank], BUF_OUT, displ[rank], cnt[rank], rv, sd);
    b.next_step();
  }
  for (int j = 1; j < n; j++) {
    int ch = mod(rank - j, n);
    std::vector<int> sd; if (j < n - 1) sd.push_back(right);
    b.act(BUF_NONE, 0, BUF_OUT, displ[ch], cnt[ch], {left}, sd);
    b.next_step();
  }
  return b.finish();
}

static Program ar_recursive(const CollArgs& a, const Resolved& rs, int rank, bool permuted) {
  int n = a.nranks, core = rs.core;
  Builder b(rank, n);
  if (rank >= core) {                      // follower: hand over, then wait for the result
    int leader = rank % core;
    b.act(BUF_IN, 0, BUF_NONE, 0, a.count, {}, {leader});
    b.step = (int)rs.radices.size() + 1;
    b.act(BUF_NONE, 0, BUF_OUT, 0, a.count, {leader}, {});
    b.next_step();
    return b.finish();
  }
  std::vector<int> followers;
  for (int f = rank + core; f < n; f += core) followers.push_back(f);
  Buf cur = BUF_IN;
  if (!followers.empty()) { b.act(BUF_IN, 0, BUF_OUT, 0, a.count, followers, {}); cur = BUF_OUT; }
  if (core < n) b.next_step();
  for (size_t s = 0; s < rs.radices.size(); s++) {
    std::vector<int> peers = step_peers(rank, (int)s, rs.radices, core, permuted);
    b.act(cur, 0, BUF_NONE, 0, a.count, {}, peers);        // my current value to every partner
    b.act(cur, 0, BUF_OUT, 0, a.count, peers, {});         // all partners' values + mine, in rank order
    cur = BUF_OUT;
    b.next_step();
  }
  if (cur == BUF_IN && !a.in_place) b.act(BUF_IN, 0, BUF_OUT, 0, a.count, {}, {});
  if (!followers.empty()) { b.act(BUF_OUT, 0, BUF_NONE, 0, a.count, {}, followers); b.next_step(); }
  return b.finish();
}

// DIRECT: every rank owns one chunk.  Step 0 hands each owner my contribution to its chunk, step 1
// reduces my chunk (the peers' contributions and mine, in rank order) and sends the sum to everybody
// while it is stored, step 2 stores the peers' sums.  Per rank 2(n-1)/n of the vector crosses the
// switch, as with the ring, but in three steps.
static Program ar_direct(const CollArgs& a, int rank) {
  int n = a.nranks;
  Builder b(rank, n);
  std::vector<int64_t> displ, cnt; ar_chunks(a.count, n, a.elem_size, displ, cnt);
  std::vector<int> others;
  for (int j = 1; j < n; j++) others.push_back((rank + j) % n);
  for (int p : others) b.act(BUF_IN, displ[p], BUF_NONE, 0, cnt[p], {}, {p});
  b.next_step();
  if (n > 1 || !a.in_place) b.act(BUF_IN, displ[rank], BUF_OUT, displ[rank], cnt[rank], others, others);
  b.next_step();
  for (int j = 1; j < n; j++) { int p = mod(rank - j, n); b.act(BUF_NONE, 0, BUF_OUT, displ[p], cnt[p], {p}, {}); }
  b.next_step();
  return b.finish();
}

Program compile_allreduce(const CollArgs& a, const Resolved& rs, int rank) {
  switch (rs.algo) {
    case ALGO_DIRECT: return ar_direct(a, rank);
    case ALGO_K_RING: return ar_ring_like(a, rank, rs.k);
    case ALGO_RD: case ALGO_RM: return ar_recursive(a, rs, rank, false);
    case ALGO_PRD: case ALGO_PRM: return ar_recursive(a, rs, rank, true);
    default: return ar_ring_like(a, rank, a.nranks);
  }
}

}  // namespace piccl
