// piccl_sched: command line front end of the schedule layer.
//   piccl_sched xml      --collective C --algorithm A [--k K] --nodes N --buffer-size BYTES [--root R]
//   piccl_sched json     ... --rank R
//   piccl_sched validate ... [--int] [--op sum|prod|max|min] [--in-place] [--cta N] [--fifo N] [--seg ELEMS] [--symbolic] [--defer]
// `--buffer-size` is the whole buffer in bytes, as in the reference's generator
// (tools/schedule_generator/main.py:15-21): for allgather / reduce_scatter each
// rank contributes buffer_size / nodes.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include "../include/piccl_sched.h"

using namespace piccl;

static Coll coll_from(const std::string& s) {
  if (s == "allgather") return COLL_ALLGATHER;
  if (s == "allreduce") return COLL_ALLREDUCE;
  if (s == "bcast" || s == "broadcast") return COLL_BROADCAST;
  if (s == "reduce") return COLL_REDUCE;
  if (s == "reduce_scatter") return COLL_REDUCE_SCATTER;
  fprintf(stderr, "unknown collective %s\n", s.c_str()); exit(2);
}
static Algo algo_from(std::string s) {
  for (auto& c : s) c = (char)toupper(c);
  Algo a = algo_from_string(s.c_str());
  if (a == ALGO_DEFAULT_NCCL) { fprintf(stderr, "unknown algorithm %s\n", s.c_str()); exit(2); }
  return a;
}

int main(int argc, char** argv) {
  if (argc < 2) { fprintf(stderr, "usage: piccl_sched xml|json|validate --collective C --algorithm A [--k K] --nodes N --buffer-size B\n"); return 2; }
  std::string cmd = argv[1];
  // fifo = 2: the smallest FIFO depth the runtime allows (a fused receive + forward needs two entries in flight)
  CollArgs a; a.elem_size = 4; int rank = 0, op = 0, fifo = 2, cta = 1; bool integer = false, symbolic = false, defer = false; int64_t seg = 0, bytes = 0;
  for (int i = 2; i < argc; i++) {
    std::string f = argv[i];
    auto val = [&]() -> const char* { if (i + 1 >= argc) { fprintf(stderr, "missing value for %s\n", f.c_str()); exit(2); } return argv[++i]; };
    if (f == "--collective") a.coll = coll_from(val());
    else if (f == "--algorithm") a.algo = algo_from(val());
    else if (f == "--k") a.k = atoi(val());
    else if (f == "--nodes" || f == "--num_nodes") a.nranks = atoi(val());
    else if (f == "--buffer-size" || f == "--buffer_size") bytes = atoll(val());
    else if (f == "--elem-size") a.elem_size = atoi(val());
    else if (f == "--root") a.root = atoi(val());
    else if (f == "--rank") rank = atoi(val());
    else if (f == "--int") integer = true;
    else if (f == "--in-place") a.in_place = true;
    else if (f == "--symbolic") symbolic = true;
    else if (f == "--defer") defer = true;
    else if (f == "--cta") cta = atoi(val());
    else if (f == "--fifo") fifo = atoi(val());
    else if (f == "--seg") seg = atoll(val());
    else if (f == "--op") { std::string o = val(); op = o == "sum" ? 0 : o == "prod" ? 1 : o == "max" ? 2 : 3; }
    else { fprintf(stderr, "unknown flag %s\n", f.c_str()); return 2; }
  }
  if (a.nranks < 1 || bytes < 0) { fprintf(stderr, "need --nodes >= 1 and --buffer-size >= 0\n"); return 2; }
  int64_t elems = bytes / a.elem_size;
  a.count = (a.coll == COLL_ALLGATHER || a.coll == COLL_REDUCE_SCATTER) ? elems / a.nranks : elems;
  if (cmd == "xml") { fputs(dump_xml(a).c_str(), stdout); return 0; }
  if (cmd == "json") { puts(dump_json(a, rank).c_str()); return 0; }
  if (cmd == "validate") {
    if (!seg) seg = std::max<int64_t>(4, a.count / 3 / (16 / std::min(16, a.elem_size)) * (16 / std::min(16, a.elem_size)));
    ValidateResult v = symbolic ? validate_symbolic(a, fifo, cta, defer) : validate(a, op, integer, fifo, seg, cta, defer);
    printf("%s entries=%lld max_fifo_depth=%d max_abs_err=%g bytes_sent_max_rank=%lld %s\n", v.ok ? "OK" : "FAIL",
           (long long)v.fifo_entries, v.max_fifo_depth, v.max_abs_err, (long long)v.bytes_sent_max_rank, v.error.c_str());
    return v.ok ? 0 : 1;
  }
  fprintf(stderr, "unknown command %s\n", cmd.c_str());
  return 2;
}
