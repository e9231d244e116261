// Reduce schedules.  Reference: src/coll/reduce.c — RING :4-46 (chain
// root+1 -> ... -> root with a reduction at every hop); K_RING/PRD/PRM are stubs
// there (:48-67) and are defined here as the broadcast trees with the arrows
// reversed.  One action per rank: receive the children's partial sums, add the
// local operand, pass the result to the parent (the root stores it instead).
#include "coll_internal.h"

namespace piccl {

Program compile_reduce(const CollArgs& a, const Resolved& rs, int rank) {
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
