// Algorithm / radix selection for requests that name no algorithm (AUTO).
// PICCL_TUNE_FILE points to the table written by tools/selector (CSV:
// collective,nranks,max_bytes,algorithm,k — first row whose max_bytes is not
// below the message wins).  Without a table the built-in rule is used: one
// exchange step with every rank (PRM, k = n) while the message is latency
// bound, the bandwidth-optimal ring above that.  The reference has no
// selector: the user picks through the environment (src/piccl.c:257-285).
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>
#include "comm.h"
#include "nvls.h"

namespace piccl {

static std::vector<TuneRow> g_rows;
static std::once_flag g_once;

static void load_table() {
  const std::string& path = env().tune_file;
  if (path.empty()) return;
  FILE* f = fopen(path.c_str(), "r");
  if (!f) { log_msg(1, "tuning table %s not readable", path.c_str()); return; }
  char line[256];
  while (fgets(line, sizeof line, f)) {
    char coll[32], algo[32]; int n, k; long long mb;
    if (line[0] == '#' || sscanf(line, "%31[^,],%d,%lld,%31[^,],%d", coll, &n, &mb, algo, &k) != 5) continue;
    int ci = -1;
    for (int c = 0; c < COLL_COUNT; c++) if (!strcmp(coll, coll_name((Coll)c))) ci = c;
    Algo a = algo_from_string(algo);
    if (ci < 0 || a == ALGO_DEFAULT_NCCL || a == ALGO_AUTO) continue;
    g_rows.push_back(TuneRow{ci, n, mb, a, k});
  }
  fclose(f);
  log_msg(1, "tuning table %s: %zu rows", path.c_str(), g_rows.size());
}

Algo select_algo_n(int n, Coll coll, size_t bytes, int* k, bool window) {
  std::call_once(g_once, load_table);
  for (auto& r : g_rows)
    if (r.coll == coll && r.nranks == n && (long long)bytes <= r.max_bytes && (window || r.algo != ALGO_NVLS)) { if (k) *k = r.k; return r.algo; }
  // With a multicast window (four ranks or more; on two ranks the peer-to-peer schedules are ahead at every size: 609 vs 310
  // GB/s at 1 GiB).  Measured on 8 B200, bus bandwidth in GB/s, in-switch / best peer-to-peer schedule / stock NCCL:
  //   all-reduce      4 MiB 171 / 104 / 123, 16 MiB 368 / 222 / 279, 64 MiB 517 / 357 / 415, 1 GiB 789 / 617 / 727; up to 1 MiB the
  //                   low-latency kernel is ahead (27 us against 37 us at 1 MiB)
  //   all-gather      (per rank) 1 MiB 184 / 74 / 146, 4 MiB 369 / 232 / 361, 16 MiB 490 / 464 / 549, 64 MiB 529 / 598 / 601
  //   reduce-scatter  (per rank) 1 MiB 200 / 80 / 153, 4 MiB 400 / 239 / 373, 16 MiB 542 / 466 / 550, 64 MiB 590 / 601 / 602
  //   broadcast, reduce   the root's multicast stores / load-reduces are the bottleneck (340 GB/s): the pipelined chain stays
  // `bytes` is the whole vector for all-reduce / broadcast / reduce and one rank's block for all-gather / reduce-scatter.
  if (window && n >= 4) {
    const size_t lo = (size_t)env().nvls_auto_kb << 10;
    if (coll == COLL_ALLREDUCE && bytes > lo) { if (k) *k = -1; return ALGO_NVLS; }
    if ((coll == COLL_ALLGATHER || coll == COLL_REDUCE_SCATTER) && bytes * (size_t)n > lo / 4 && bytes > ((size_t)env().llx_kb << 10) && bytes <= ((size_t)32 << 20)) { if (k) *k = -1; return ALGO_NVLS; }
  }
  // Built-in rule, from sweeps on 2, 4 and 8 B200 (fp32 and bf16 sum):
  //   all-reduce      <= 4 KiB one exchange with every rank (PRM, k = n: 8 us on 8 GPUs); up to 32 MiB (8 MiB on two
  //                   ranks) recursive doubling, whose few steps beat the ring's 2(n-1) (222 vs 154 GB/s at 16 MiB on 8
  //                   GPUs); above that the bandwidth-optimal ring (600 vs 290 GB/s at 256 MiB)
  //   all-gather / reduce-scatter   one exchange with every rank while a rank's block is small (flag-in-data lines, one launch),
  //                   the ring otherwise
  //   broadcast / reduce   the segment-pipelined chain at every size (8.5 us at 1 KiB, 581 GB/s at 256 MiB on 8 GPUs,
  //                   the trees 8.8 us and 225 GB/s)
  int kk = n < 8 ? n : 8;
  switch (coll) {
    case COLL_ALLREDUCE:
      if (bytes <= (size_t)4 << 10) { if (k) *k = kk; return ALGO_PRM; }
      if (bytes <= ((size_t)(n <= 2 ? 8 : 32) << 20)) { if (k) *k = 2; return ALGO_PRD; }
      return ALGO_RING;
    case COLL_ALLGATHER: case COLL_REDUCE_SCATTER:
      // one exchange with every rank in the low-latency kernel while a rank's block is small (up to 8 ranks: the radix is the rank count)
      if (bytes <= ((size_t)(n <= 8 ? std::max(16, env().llx_kb) : 16) << 10)) { if (k) *k = kk; return ALGO_PRM; }
      return ALGO_RING;
    default:
      return ALGO_RING;
  }
}

Algo select_algo(piccl_comm* c, Coll coll, size_t bytes, int* k) { return select_algo_n(c->nranks, coll, bytes, k, nvls_ready(c)); }
Algo select_algo_p2p(piccl_comm* c, Coll coll, size_t bytes, int* k) { return select_algo_n(c->nranks, coll, bytes, k, false); }

}  // namespace piccl

// What AUTO resolves to for a communicator of `nranks` ranks (tuning table first, then the built-in rule).
// Returns the algorithm (PICCL_ALGO_*) and, through *k, the radix or group size (-1 / 2 / n as the rule says).
// piccl_select_algorithm answers for a communicator without a multicast window, the _ex form for either.
extern "C" int piccl_select_algorithm_ex(int nranks, int coll, unsigned long long bytes, int have_window, int* k) {
  int kk = -1;
  if (coll < 0 || coll >= piccl::COLL_COUNT || nranks < 1) return 0;
  piccl::Algo a = piccl::select_algo_n(nranks, (piccl::Coll)coll, (size_t)bytes, &kk, have_window != 0);
  if (k) *k = kk;
  return (int)a;
}
extern "C" int piccl_select_algorithm(int nranks, int coll, unsigned long long bytes, int* k) { return piccl_select_algorithm_ex(nranks, coll, bytes, 0, k); }
