// Reduce schedules.  Reference: src/coll/reduce.c — RING :4-46 (chain
// root+1 -> ... -> root with a reduction at every hop); K_RING/PRD/PRM are stubs
// there (:48-67) and are defined here as the broadcast trees with the arrows
// reversed.  One action per rank: receive the children's partial sums, add the
// local operand, pass the result to the parent (the root stores it instead).
#include "coll_internal.h"

namespace piccl {

// DIRECT: the vector is cut into n-1 slices, one per non-root rank.  Everybody (the root too) sends
// each owner its contribution to that slice; the owner adds its own, in rank order, and sends the sum
// to the root.  Two steps; the root receives the vector once.
static Program rd_direct(const CollArgs& a, int rank) {
  int n = a.nranks, root = a.root;
  Builder b(rank, n);
  if (n == 1) { if (!a.in_place) b.act(BUF_IN, 0, BUF_OUT, 0, a.count, {}, {}); b.next_step(); return b.finish(); }
  std::vector<int64_t> displ, cnt; ar_chunks(a.count, n - 1, a.elem_size, displ, cnt);
  auto owner = [&](int s) { return (root + 1 + s) % n; };
  int mine = rank == root ? -1 : mod(rank - root - 1, n);
  for (int j = 1; j < n; j++) {
    int p = (rank + j) % n;
    if (p == root) continue;
    int s = mod(p - root - 1, n);
    b.act(BUF_IN, displ[s], BUF_NONE, 0, cnt[s], {}, {p});
  }
  b.next_step();
  if (rank == root) {
    for (int s = 0; s < n - 1; s++) b.act(BUF_NONE, 0, BUF_OUT, displ[s], cnt[s], {owner(s)}, {});
  } else {
    std::vector<int> from;
    for (int p = 0; p < n; p++) if (p != rank) from.push_back(p);
    b.act(BUF_IN, displ[mine], BUF_NONE, 0, cnt[mine], from, {root});
  }
  b.next_step();
  return b.finish();
}

Program compile_reduce(const CollArgs& a, const Resolved& rs, int rank) {
  if (rs.algo == ALGO_DIRECT) return rd_direct(a, rank);
  Builder b(rank, a.nranks);
  Tree t = reduce_tree(rs.algo, rs.k, a.nranks, a.root, rank);
  b.step = t.depth;
  if (rank == a.root) {
    if (!t.children.empty() || !a.in_place) b.act(BUF_IN, 0, BUF_OUT, 0, a.count, t.children, {});
  } else {
    b.act(BUF_IN, 0, BUF_NONE, 0, a.count, t.children, {t.parent});
  }
  b.next_step();
  return b.finish();
}

}  // namespace piccl
