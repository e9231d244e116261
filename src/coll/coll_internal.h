// Helpers shared by the per-collective schedule compilers.
#pragma once
#include <algorithm>
#include <initializer_list>
#include "../include/piccl_sched.h"

namespace piccl {

inline int mod(int a, int n) { int m = a % n; return m < 0 ? m + n : m; }

struct Builder {
  Program prog;
  int step = 0;
  Builder(int rank, int n) { prog.rank = rank; prog.nranks = n; }

  // value = reduce(src?, recv...) -> dst?, send...
  void act(Buf src, int64_t src_off, Buf dst, int64_t dst_off, int64_t count,
           std::vector<int> recv, std::vector<int> send, uint8_t flags = 0) {
    if (count <= 0) return;                       // zero-size transfers do not exist on either side
    if (src == BUF_NONE && recv.empty()) return;
    if (dst == BUF_NONE && send.empty()) return;
    Action a;
    a.src_buf = src; a.dst_buf = dst; a.src_off = src_off; a.dst_off = dst_off; a.count = count;
    std::sort(recv.begin(), recv.end());
    a.n_recv = (uint8_t)recv.size(); a.n_send = (uint8_t)send.size();
    int pos = 0;
    for (size_t i = 0; i < recv.size(); i++) { a.recv_peer[i] = (uint8_t)recv[i]; if (recv[i] < prog.rank) pos++; }
    for (size_t i = 0; i < send.size(); i++) a.send_peer[i] = (uint8_t)send[i];
    a.self_pos = (uint8_t)pos;
    a.flags = (src == BUF_IN) ? (flags | ACT_SCALE_SRC) : flags;
    a.step = (uint8_t)std::min(step, 255);
    prog.actions.push_back(a);
  }
  void next_step() { step++; }
  Program finish() { prog.nsteps = step; return prog; }
};

// Tree shapes for broadcast / reduce (root-relative virtual ranks).
struct Tree { int parent = -1; std::vector<int> children; int depth = 0; };
Tree bcast_tree(Algo algo, int k, int nranks, int root, int rank);
Tree reduce_tree(Algo algo, int k, int nranks, int root, int rank);

Program compile_allgather(const CollArgs& a, const Resolved& rs, int rank);
Program compile_allreduce(const CollArgs& a, const Resolved& rs, int rank);
Program compile_broadcast(const CollArgs& a, const Resolved& rs, int rank);
Program compile_reduce(const CollArgs& a, const Resolved& rs, int rank);
Program compile_reduce_scatter(const CollArgs& a, const Resolved& rs, int rank);

// Reduce-scatter hop chain shared by allreduce/reduce_scatter RING and K_RING:
// hop i sends chunk[i] to to[i]; hop i>0 first receives that chunk's partial from from[i].
struct RsChain { std::vector<int> chunk, to, from; int final_chunk = 0, final_from = 0; };
RsChain rs_chain(int rank, int nranks, int k);

}  // namespace piccl
