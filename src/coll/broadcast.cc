// Broadcast schedules.  Reference: src/coll/broadcast.c — RING :3-35 (a chain,
// whole message per hop), K_RING :37-92 (leader chain + chains inside the
// groups); PRD/PRM are stubs there (:94-106) and are defined here as k-nomial
// trees over root-relative ranks (farthest child first; RD/RM nearest first).
// Every rank runs one action — receive from the parent, store, forward to all
// children — and the FIFO segments pipeline the message down the tree.
#include "coll_internal.h"

namespace piccl {

// DIRECT: the message is cut into n-1 slices, one per non-root rank.  The root sends every rank its
// slice; each rank stores its slice while it passes it on to the other non-root ranks, and stores
// theirs.  The root sends the message once, every other rank receives it once: two steps, and no
// link carries more than the message size.
static Program bc_direct(const CollArgs& a, int rank) {
  int n = a.nranks, root = a.root;
  Builder b(rank, n);
  if (n == 1) { if (!a.in_place) b.act(BUF_IN, 0, BUF_OUT, 0, a.count, {}, {}); b.next_step(); return b.finish(); }
  std::vector<int64_t> displ, cnt; ar_chunks(a.count, n - 1, a.elem_size, displ, cnt);
  auto owner = [&](int s) { return (root + 1 + s) % n; };          // slice s belongs to this rank
  if (rank == root) {
    for (int s = 0; s < n - 1; s++) b.act(BUF_IN, displ[s], a.in_place ? BUF_NONE : BUF_OUT, displ[s], cnt[s], {}, {owner(s)});
    b.next_step();
    return b.finish();
  }
  int mine = mod(rank - root - 1, n);
  std::vector<int> others;
  for (int s = 0; s < n - 1; s++) if (s != mine) others.push_back(owner(s));
  b.step = 1;
  b.act(BUF_NONE, 0, BUF_OUT, displ[mine], cnt[mine], {root}, others);
  b.next_step();
  for (int j = 1; j < n - 1; j++) { int s = mod(mine - j, n - 1); b.act(BUF_NONE, 0, BUF_OUT, displ[s], cnt[s], {owner(s)}, {}); }
  b.next_step();
  return b.finish();
}

Program compile_broadcast(const CollArgs& a, const Resolved& rs, int rank) {
  if (rs.algo == ALGO_DIRECT) return bc_direct(a, rank);
  Builder b(rank, a.nranks);
  Tree t = bcast_tree(rs.algo, rs.k, a.nranks, a.root, rank);
  b.step = t.depth;
  if (rank == a.root) b.act(BUF_IN, 0, a.in_place ? BUF_NONE : BUF_OUT, 0, a.count, {}, t.children);
  else b.act(BUF_NONE, 0, BUF_OUT, 0, a.count, {t.parent}, t.children);
  b.next_step();
  return b.finish();
}

}  // namespace piccl
