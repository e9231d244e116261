// Broadcast schedules.  Reference: src/coll/broadcast.c — RING :3-35 (a chain,
// whole message per hop), K_RING :37-92 (leader chain + chains inside the
// groups); PRD/PRM are stubs there (:94-106) and are defined here as k-nomial
// trees over root-relative ranks (farthest child first; RD/RM nearest first).
// Every rank runs one action — receive from the parent, store, forward to all
// children — and the FIFO segments pipeline the message down the tree.
#include "coll_internal.h"

namespace piccl {

Program compile_broadcast(const CollArgs& a, const Resolved& rs, int rank) {
  Builder b(rank, a.nranks);
  Tree t = bcast_tree(rs.algo, rs.k, a.nranks, a.root, rank);
  b.step = t.depth;
  if (rank == a.root) b.act(BUF_IN, 0, a.in_place ? BUF_NONE : BUF_OUT, 0, a.count, {}, t.children);
  else b.act(BUF_NONE, 0, BUF_OUT, 0, a.count, {t.parent}, t.children);
  b.next_step();
  return b.finish();
}

}  // namespace piccl
