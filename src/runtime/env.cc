#include "env.h"
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unistd.h>

namespace piccl {

static Env g_env;
static std::once_flag g_once;

static int env_int(const char* name, int def, bool* was_set = nullptr) {
  const char* v = getenv(name);
  if (was_set) *was_set = v && *v;
  if (!v || !*v) return def;
  return atoi(v);
}

static void load() {
  static const char* cn[COLL_COUNT] = {"ALLGATHER", "ALLREDUCE", "BROADCAST", "REDUCE", "REDUCE_SCATTER"};
  Env e;
  for (int c = 0; c < COLL_COUNT; c++) {
    char name[64];
    snprintf(name, sizeof name, "PICCL_%s_ALGO", cn[c]);
    e.algo[c] = algo_from_string(getenv(name));
    snprintf(name, sizeof name, "PICCL_%s_K", cn[c]);
    e.k[c] = env_int(name, -1);
  }
  e.block_size = env_int("PICCL_BLOCK_SIZE", 1024, &e.block_size_set);
  e.max_grid = env_int("PICCL_MAX_GRID_SIZE", 1024, &e.max_grid_set);
  e.min_grid = env_int("PICCL_MIN_GRID_SIZE", 1, &e.min_grid_set);
  e.timeout_ms = env_int("PICCL_TIMEOUT_MS", 10000);
  e.scratch_mb = env_int("PICCL_SCRATCH_MB", 64);
  e.slot_kb = env_int("PICCL_SLOT_KB", 512);
  e.nslot = env_int("PICCL_NSLOT", 4);
  e.max_cta = env_int("PICCL_MAX_CTA", 64);
  e.ll_kb = env_int("PICCL_LL_KB", 1024);         // largest all-reduce taken by the low-latency kernel; 0 turns it off
  e.llf_kb = env_int("PICCL_LLF_KB", 64);        // largest message (any collective) on the low-latency executor; 0 turns it off
  e.llx_kb = env_int("PICCL_LLX_KB", 64);        // largest block per rank of an all-gather / reduce-scatter taken by the one-exchange low-latency kernel
  e.tp_mb = env_int("PICCL_TP_MB", 0);           // heap space for the fused tensor-parallel kernels (0: none)
  e.tp_feeders = env_int("PICCL_TP_FEEDERS", 24); // CTAs that push the local shard in all-gather -> GEMM
  e.exec_defer = env_int("PICCL_EXEC_DEFER", 0);
  e.nvls = env_int("PICCL_NVLS", 1);            // 0: no NVLink multicast window (algorithm NVLS then runs the peer-to-peer schedules)
  e.nvls_chunk_kb = env_int("PICCL_NVLS_CHUNK_KB", 256);   // largest chunk = one part of a CTA's slot
  e.nvls_depth = env_int("PICCL_NVLS_DEPTH", 5);           // parts per slot (2 .. 8): chunks a CTA has in flight in its stages
  e.nvls_cta = env_int("PICCL_NVLS_CTA", 128);             // CTAs (= slots of the window) of an in-switch collective
  e.nvls_auto_kb = env_int("PICCL_NVLS_AUTO_KB", 1024);    // AUTO sends all-reduces above this size (all-gathers / reduce-scatters above a quarter of it in total) through the switch
  e.nvls_min_kb = env_int("PICCL_NVLS_MIN_KB", 64);        // a mid-size message is cut into chunks of at least this size before more CTAs are used
  { const char* g = getenv("PICCL_NVLS_GRAN"); e.nvls_gran_min = !(g && !strcmp(g, "recommended")); }
  e.nvls_bulk = env_int("PICCL_NVLS_BULK", 1);             // 0: copies between user buffers and the window use the threads' loads and stores, not the bulk-copy engine
  { const char* f = getenv("PICCL_NVLS_FENCE"); e.nvls_strict_fences = f && !strcmp(f, "sys"); }   // sys: a system-wide fence before every counter update of the in-switch kernels
  e.nvls_sub = env_int("PICCL_NVLS_SUB", 0);               // 1 / 3: groups of the stage that talks to the switch; 0: 3 for large all-reduces on four ranks or more, else 1
  e.nvls_profile = env_int("PICCL_NVLS_PROFILE", 0);       // 1: the kernels sum the time of every phase; printed when the communicator is destroyed
  // PICCL_PROTO narrows the choice of data path that is otherwise made per call by message size:
  //   auto    (default) low-latency kernels for small messages, the FIFO executor otherwise
  //   simple  FIFO executor only
  //   ll      low-latency executor up to 1 MiB for every collective
  //   nvls    every eligible collective goes through the switch, whatever its size
  e.proto = 0;
  if (const char* p = getenv("PICCL_PROTO")) {
    if (!strcmp(p, "ll")) { e.proto = 1; e.llf_kb = std::max(e.llf_kb, 1024); }
    else if (!strcmp(p, "simple")) { e.proto = 2; e.ll_kb = 0; e.llf_kb = 0; }
    else if (!strcmp(p, "nvls")) { e.proto = 3; e.nvls = 1; }
  }
  e.log_level = env_int("PICCL_LOG", 0);
  e.debug = env_int("PICCL_DEBUG", 0);
  { const char* l = getenv("PICCL_LAUNCH"); e.launch_persistent = l && !strcmp(l, "persistent"); }
  e.persist_idle_us = env_int("PICCL_PERSIST_IDLE_US", 500);
  const char* t = getenv("PICCL_TRACE"); e.trace_file = t ? t : "";
  const char* tf = getenv("PICCL_TUNE_FILE"); e.tune_file = tf ? tf : "";
  e.fault_rank = -1; e.fault_call = -1; e.fault_delay_ms = 0; e.fault_skip = false;
  if (const char* f = getenv("PICCL_FAULT")) {
    int r = -1, c = -1; char what[64] = {0};
    if (sscanf(f, "%d:%d:%63s", &r, &c, what) == 3) {
      e.fault_rank = r; e.fault_call = c;
      if (!strcmp(what, "skip_call")) e.fault_skip = true;
      else if (!strncmp(what, "delay_ms=", 9)) e.fault_delay_ms = atoi(what + 9);
    }
  }
  g_env = e;
}

const Env& env() { std::call_once(g_once, load); return g_env; }
void env_reload() { std::call_once(g_once, [] {}); load(); }

void log_msg(int level, const char* fmt, ...) {
  if (env().log_level < level) return;
  char buf[1024];
  va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof buf, fmt, ap); va_end(ap);
  fprintf(stderr, "[PICCL %d] %s\n", (int)getpid(), buf);
}

}  // namespace piccl

// Reads the PICCL_* environment again (benchmarks that switch the algorithm inside one process; all ranks must do it at the
// same point between collectives).  Geometry that a communicator fixed at creation (heap, window) keeps its old values.
extern "C" void piccl_env_reload(void) { piccl::env_reload(); }

// The effective configuration as "key=value" pairs separated by blanks (for logs and tests).
// Returns the length needed, like snprintf.
extern "C" int piccl_env_describe(char* buf, int len) {
  const piccl::Env& e = piccl::env();
  static const char* proto[] = {"auto", "ll", "simple", "nvls"};
  return snprintf(buf, len > 0 ? (size_t)len : 0,
                  "proto=%s ll_kb=%d llf_kb=%d nvls=%d nvls_chunk_kb=%d nvls_cta=%d nvls_min_kb=%d max_cta=%d slot_kb=%d nslot=%d timeout_ms=%d "
                  "launch=%s allreduce=%s/%d allgather=%s/%d broadcast=%s/%d reduce=%s/%d reduce_scatter=%s/%d",
                  proto[e.proto & 3], e.ll_kb, e.llf_kb, e.nvls, e.nvls_chunk_kb, e.nvls_cta, e.nvls_min_kb, e.max_cta, e.slot_kb, e.nslot, e.timeout_ms,
                  e.launch_persistent ? "persistent" : "direct", piccl::algo_name(e.algo[piccl::COLL_ALLREDUCE]), e.k[piccl::COLL_ALLREDUCE],
                  piccl::algo_name(e.algo[piccl::COLL_ALLGATHER]), e.k[piccl::COLL_ALLGATHER], piccl::algo_name(e.algo[piccl::COLL_BROADCAST]), e.k[piccl::COLL_BROADCAST],
                  piccl::algo_name(e.algo[piccl::COLL_REDUCE]), e.k[piccl::COLL_REDUCE], piccl::algo_name(e.algo[piccl::COLL_REDUCE_SCATTER]), e.k[piccl::COLL_REDUCE_SCATTER]);
}
