// CPU data-flow executor: runs the programs of all ranks against each other
// exactly as the device kernel would (same CTA slicing, same per-step segment
// interleaving, bounded FIFOs) and compares the buffers with a serial
// reduction.  The reference has no such check (it relies on the external OSU
// validation flag, README.md:40-44).
#include <cmath>
#include <cstdio>
#include <deque>
#include <random>
#include "coll_internal.h"
#include "../include/piccl_slice.h"

namespace piccl {

namespace {

template <class T> T apply(int op, T a, T b) {
  switch (op) { case 0: return a + b; case 1: return a * b; case 2: return a > b ? a : b; default: return a < b ? a : b; }
}

struct Cursor { int seg = 0, maxseg = 0; size_t act = 0; bool done = false; };

struct Sizes { int64_t in_elems, out_elems; };
Sizes buffer_sizes(const CollArgs& a) {
  int64_t st = a.block_stride ? a.block_stride : a.count;
  switch (a.coll) {
    case COLL_ALLGATHER: return {a.count, (a.nranks - 1) * st + a.count};
    case COLL_REDUCE_SCATTER: return {(a.nranks - 1) * st + a.count, a.count};
    default: return {a.count, a.count};
  }
}

template <class T>
ValidateResult run(const CollArgs& a, int op, bool with_data, int fifo_cap, int64_t seg_elems_req, int n_cta, bool defer) {
  ValidateResult res;
  int n = a.nranks;
  int64_t st = a.block_stride ? a.block_stride : a.count;
  Sizes sz = buffer_sizes(a);
  std::vector<Program> progs; for (int r = 0; r < n; r++) progs.push_back(compile(a, r));
  int64_t slot_bytes = std::max<int64_t>(16, seg_elems_req * a.elem_size / 16 * 16);

  const int64_t guard = with_data ? 8 : 0;
  const T canary = (T)7777;
  // storage: per rank one arena holding IN and OUT (aliased when in place) with guards
  std::vector<std::vector<T>> arena(n), scratch(n), in_copy(n);
  std::vector<T*> in(n, nullptr), out(n, nullptr);
  std::vector<std::vector<uint8_t>> out_written(n);
  if (with_data) {
    std::mt19937 gen(0);
    std::uniform_real_distribution<float> fd(-1.f, 1.f);
    std::uniform_int_distribution<int> id(-1000, 1000);
    for (int r = 0; r < n; r++) {
      int64_t total = sz.in_elems + sz.out_elems + 3 * guard;
      arena[r].assign(total, canary);
      if (a.in_place) {
        if (a.coll == COLL_ALLGATHER) { out[r] = arena[r].data() + guard; in[r] = out[r] + r * st; }
        else if (a.coll == COLL_REDUCE_SCATTER) { in[r] = arena[r].data() + guard; out[r] = in[r] + r * st; }
        else { in[r] = out[r] = arena[r].data() + guard; }
      } else { in[r] = arena[r].data() + guard; out[r] = in[r] + sz.in_elems + guard; }
      for (int64_t i = 0; i < sz.in_elems; i++) {
        T v;
        if (std::is_floating_point<T>::value) v = (T)fd(gen); else v = (T)id(gen);
        if (op == 1) v = std::is_floating_point<T>::value ? (T)(1.0 + 0.01 * (double)v) : (T)((i + r) % 3 == 0 ? 2 : 1);
        in[r][i] = v;
      }
      in_copy[r].assign(in[r], in[r] + sz.in_elems);
      scratch[r].assign(progs[r].scratch_elems + 1, canary);
    }
  }
  for (int r = 0; r < n; r++) out_written[r].assign(with_data ? 0 : 0, 0);

  // symbolic coverage: count of writes per OUT pack is too big for 1 GiB; track per (rank) intervals
  std::vector<std::vector<std::pair<int64_t, int64_t>>> cover(n);

  int64_t entries = 0; int maxdepth = 0; std::vector<int64_t> sent_bytes(n, 0);
  for (int cta = 0; cta < n_cta; cta++) {
    struct Entry { std::vector<T> data; int64_t n; };
    std::vector<std::deque<Entry>> fifo((size_t)n * n);   // [src*n+dst]
    std::vector<Cursor> cur(n);
    // Deferred publishing (the executor's DEFER variant): a push is visible to the consumer, and a pop to the producer, only
    // once the rank that made it has published it, which it does when it is about to block and when its program ends.
    std::vector<int64_t> pushed((size_t)n * n, 0), popped((size_t)n * n, 0), pub_push((size_t)n * n, 0), pub_pop((size_t)n * n, 0);
    auto flush = [&](int r) {
      bool any = false;
      for (int o = 0; o < n; o++) {
        size_t out_c = (size_t)r * n + o, in_c = (size_t)o * n + r;
        if (pub_push[out_c] != pushed[out_c]) { pub_push[out_c] = pushed[out_c]; any = true; }
        if (pub_pop[in_c] != popped[in_c]) { pub_pop[in_c] = popped[in_c]; any = true; }
      }
      return any;
    };
    // device order: outer loop over segments, inner loop over all actions of the program
    for (int r = 0; r < n; r++) {
      for (auto& ac : progs[r].actions) cur[r].maxseg = std::max(cur[r].maxseg, slice_of(ac.count, a.elem_size, cta, n_cta, slot_bytes).nseg);
      cur[r].done = cur[r].maxseg == 0;
    }
    bool progress = true;
    auto all_done = [&] { for (auto& c : cur) if (!c.done) return false; return true; };
    while (!all_done()) {
      if (!progress) {
        char buf[256]; int r0 = 0; for (int r = 0; r < n; r++) if (!cur[r].done) { r0 = r; break; }
        snprintf(buf, sizeof buf, "deadlock: cta %d, rank %d stuck at action %zu seg %d", cta, r0, cur[r0].act, cur[r0].seg);
        res.error = buf; return res;
      }
      progress = false;
      for (int r = 0; r < n; r++) {
        Cursor& c = cur[r]; const Program& p = progs[r];
        while (!c.done) {
          const Action& ac = p.actions[c.act];
          Slice sl = slice_of(ac.count, a.elem_size, cta, n_cta, slot_bytes);
          bool advance = true;
          if (c.seg < sl.nseg) {
            bool ready = true;
            for (int i = 0; i < ac.n_send; i++) {
              size_t cn = (size_t)r * n + ac.send_peer[i];
              if ((defer ? pushed[cn] - pub_pop[cn] : (int64_t)fifo[cn].size()) >= fifo_cap) ready = false;
            }
            for (int i = 0; i < ac.n_recv; i++) {
              size_t cn = (size_t)ac.recv_peer[i] * n + r;
              if (defer ? pub_push[cn] - popped[cn] <= 0 : fifo[cn].empty()) ready = false;
            }
            if (!ready) { advance = false; if (defer && flush(r)) progress = true; }
            else {
              int64_t lo = sl.lo + (int64_t)c.seg * sl.seg_elems, hi = std::min(sl.hi, lo + sl.seg_elems), len = hi - lo;
              std::vector<T> val;
              if (with_data) {
                val.resize(len);
                const T* src = ac.src_buf == BUF_IN ? in[r] : ac.src_buf == BUF_OUT ? out[r] : ac.src_buf == BUF_SCRATCH ? scratch[r].data() : nullptr;
                int64_t src_lim = ac.src_buf == BUF_IN ? sz.in_elems : ac.src_buf == BUF_OUT ? sz.out_elems : p.scratch_elems;
                if (src && ac.src_off + hi > src_lim) { res.error = "source range out of bounds"; return res; }
                // rank order: recv peers below me, me, recv peers above me
                bool first = true; int pos = 0;
                auto fold = [&](const T* x) { for (int64_t i = 0; i < len; i++) val[i] = first ? x[i] : apply<T>(op, val[i], x[i]); first = false; };
                for (int i = 0; i <= ac.n_recv; i++) {
                  if (i == ac.self_pos && src) fold(src + ac.src_off + lo);
                  if (i < ac.n_recv) {
                    Entry& e = fifo[(size_t)ac.recv_peer[i] * n + r].front();
                    if (e.n != len) { res.error = "fifo entry size mismatch"; return res; }
                    fold(e.data.data()); pos++;
                  }
                }
              } else {
                for (int i = 0; i < ac.n_recv; i++) if (fifo[(size_t)ac.recv_peer[i] * n + r].front().n != len) { res.error = "fifo entry size mismatch"; return res; }
              }
              for (int i = 0; i < ac.n_recv; i++) { fifo[(size_t)ac.recv_peer[i] * n + r].pop_front(); popped[(size_t)ac.recv_peer[i] * n + r]++; }
              if (ac.dst_buf != BUF_NONE) {
                int64_t lim = ac.dst_buf == BUF_OUT ? sz.out_elems : p.scratch_elems;
                if (ac.dst_buf == BUF_IN || ac.dst_off + hi > lim || ac.dst_off + lo < 0) { res.error = "destination range out of bounds"; return res; }
                if (with_data) { T* d = ac.dst_buf == BUF_OUT ? out[r] : scratch[r].data(); for (int64_t i = 0; i < len; i++) d[ac.dst_off + lo + i] = val[i]; }
                if (ac.dst_buf == BUF_OUT) cover[r].push_back({ac.dst_off + lo, ac.dst_off + hi});
              }
              for (int i = 0; i < ac.n_send; i++) {
                auto& q = fifo[(size_t)r * n + ac.send_peer[i]];
                q.push_back(Entry{val, len}); entries++; sent_bytes[r] += len * a.elem_size; pushed[(size_t)r * n + ac.send_peer[i]]++;
                maxdepth = std::max<int>(maxdepth, (int)q.size());
              }
              progress = true;
            }
          }
          if (!advance) break;
          c.act++;
          if (c.act >= p.actions.size()) { c.act = 0; c.seg++; if (c.seg >= c.maxseg) { c.done = true; progress = true; if (defer) flush(r); } }
        }
      }
    }
    for (size_t i = 0; i < fifo.size(); i++) if (!fifo[i].empty()) { res.error = "fifo not drained at the end"; return res; }
  }
  res.fifo_entries = entries; res.max_fifo_depth = maxdepth;
  for (int r = 0; r < n; r++) res.bytes_sent_max_rank = std::max(res.bytes_sent_max_rank, sent_bytes[r]);

  // coverage: every expected OUT element written at least once on every rank that has an output
  for (int r = 0; r < n; r++) {
    bool has_out = !(a.coll == COLL_REDUCE && r != a.root);
    if (!has_out) { if (!cover[r].empty()) { res.error = "non-root rank wrote its receive buffer"; return res; } continue; }
    std::vector<std::pair<int64_t, int64_t>> need;
    if (a.coll == COLL_ALLGATHER) { for (int b = 0; b < n; b++) if (!(a.in_place && b == r)) need.push_back({b * st, b * st + a.count}); }
    else if (a.in_place && (a.coll == COLL_BROADCAST) && r == a.root) {}
    else if (a.in_place && n == 1) {}
    else need.push_back({0, a.count});
    auto cv = cover[r]; std::sort(cv.begin(), cv.end());
    for (auto& nd : need) {
      int64_t pos = nd.first;
      for (auto& iv : cv) { if (iv.second <= pos) continue; if (iv.first > pos) break; pos = std::max(pos, iv.second); if (pos >= nd.second) break; }
      if (pos < nd.second) { char buf[128]; snprintf(buf, sizeof buf, "rank %d: output [%lld,%lld) not fully written", r, (long long)nd.first, (long long)nd.second); res.error = buf; return res; }
    }
    if (a.coll == COLL_ALLGATHER && st > a.count)
      for (auto& iv : cv) { int64_t b = iv.first / st; if (iv.second > b * st + a.count) { res.error = "write into the gap between blocks"; return res; } }
  }
  if (!with_data) { res.ok = true; return res; }

  // data check
  double maxerr = 0;
  auto expect_reduce = [&](int64_t idx_in) { T v = in_copy[0][idx_in]; for (int r = 1; r < n; r++) v = apply<T>(op, v, in_copy[r][idx_in]); return v; };
  auto check = [&](int r, int64_t oi, T want, double tol) {
    double e = std::fabs((double)out[r][oi] - (double)want);
    maxerr = std::max(maxerr, e);
    return e <= tol;
  };
  for (int r = 0; r < n; r++) {
    if (a.coll == COLL_REDUCE && r != a.root) continue;
    for (int64_t i = 0; i < a.count; i++) {
      bool good = true;
      double tol = std::is_floating_point<T>::value ? 1e-5 * n : 0.0;
      switch (a.coll) {
        case COLL_ALLREDUCE: case COLL_REDUCE: good = check(r, i, expect_reduce(i), tol); break;
        case COLL_BROADCAST: good = check(r, i, in_copy[a.root][i], 0); break;
        case COLL_REDUCE_SCATTER: good = check(r, i, expect_reduce(r * st + i), tol); break;
        case COLL_ALLGATHER: for (int b = 0; b < n && good; b++) good = check(r, b * st + i, in_copy[b][i], 0); break;
        default: break;
      }
      if (!good) { char buf[160]; snprintf(buf, sizeof buf, "rank %d element %lld wrong (max err %g)", r, (long long)i, maxerr); res.error = buf; res.max_abs_err = maxerr; return res; }
    }
    // guards and untouched input
    T* base = arena[r].data(); int64_t total = (int64_t)arena[r].size();
    for (int64_t g = 0; g < guard; g++) if (base[g] != canary || base[total - 1 - g] != canary) { res.error = "guard zone overwritten"; return res; }
    if (!a.in_place) {
      for (int64_t g = 0; g < guard; g++) if (in[r][sz.in_elems + g] != canary) { res.error = "guard zone between buffers overwritten"; return res; }
      for (int64_t i = 0; i < sz.in_elems; i++) if (in[r][i] != in_copy[r][i]) { res.error = "send buffer modified"; return res; }
    }
    if (scratch[r].back() != canary) { res.error = "scratch overrun"; return res; }
  }
  res.max_abs_err = maxerr; res.ok = true;
  return res;
}

}  // namespace

ValidateResult validate(const CollArgs& a, int op, bool integer, int fifo_cap, int64_t seg_elems, int n_cta, bool defer_publish) {
  if (integer) return run<int32_t>(a, op, true, fifo_cap, seg_elems, n_cta, defer_publish);
  return run<float>(a, op, true, fifo_cap, seg_elems, n_cta, defer_publish);
}

ValidateResult validate_symbolic(const CollArgs& a, int fifo_cap, int n_cta, bool defer_publish) {
  return run<float>(a, 0, false, fifo_cap, (int64_t)(256 * 1024) / a.elem_size, n_cta, defer_publish);
}

}  // namespace piccl
