#include "env.h"
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
  e.timeout_ms = env_int("PICCL_TIMEOUT_MS", 120000);
  e.scratch_mb = env_int("PICCL_SCRATCH_MB", 64);
  e.slot_kb = env_int("PICCL_SLOT_KB", 512);
  e.nslot = env_int("PICCL_NSLOT", 4);
  e.max_cta = env_int("PICCL_MAX_CTA", 64);
  e.ll_kb = env_int("PICCL_LL_KB", 1024);         // largest all-reduce taken by the low-latency kernel; 0 turns it off
  e.llf_kb = env_int("PICCL_LLF_KB", 64);        // largest message (any collective) on the low-latency executor; 0 turns it off
  e.tp_mb = env_int("PICCL_TP_MB", 0);           // heap space for the fused tensor-parallel kernels (0: none)
  e.tp_feeders = env_int("PICCL_TP_FEEDERS", 24); // CTAs that push the local shard in all-gather -> GEMM
  e.nvls = env_int("PICCL_NVLS", 0);            // 1: build an NVLink multicast window per communicator (algorithm NVLS)
  e.nvls_chunk_kb = env_int("PICCL_NVLS_CHUNK_KB", 256);
  e.nvls_cta = env_int("PICCL_NVLS_CTA", 64);
  e.nvls_pipe = env_int("PICCL_NVLS_PIPE", 0);   // 1: the pipelined kernel (two half slots per CTA)
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
