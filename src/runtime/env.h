// Environment configuration, read once per process.
//
// Same variables, values and defaults as the reference
// (README.md:46-68; parsing src/piccl.c:224-334): PICCL_<COLL>_ALGO in
// {RING,K_RING,RD,RM,PRD,PRM} (anything else or unset: real NCCL), PICCL_<COLL>_K
// (default -1), PICCL_BLOCK_SIZE (1024), PICCL_MAX_GRID_SIZE (1024),
// PICCL_MIN_GRID_SIZE (1).  Additions that do not change those semantics: the
// value AUTO, PICCL_TIMEOUT_MS, PICCL_SCRATCH_MB, PICCL_SLOT_KB, PICCL_NSLOT,
// PICCL_MAX_CTA, PICCL_LL_KB, PICCL_LLF_KB, PICCL_LLX_KB, PICCL_TP_MB, PICCL_TP_FEEDERS, PICCL_LAUNCH, PICCL_PERSIST_IDLE_US, PICCL_PROTO, PICCL_EXEC_DEFER, PICCL_NVLS, PICCL_NVLS_CHUNK_KB, PICCL_NVLS_DEPTH, PICCL_NVLS_CTA, PICCL_NVLS_MIN_KB, PICCL_NVLS_AUTO_KB, PICCL_NVLS_GRAN, PICCL_NVLS_PROFILE, PICCL_NVLS_BULK, PICCL_NVLS_FENCE, PICCL_NVLS_SUB, PICCL_LOG, PICCL_TRACE, PICCL_FAULT, PICCL_TUNE_FILE, PICCL_DEBUG.
#pragma once
#include <string>
#include "../include/piccl_sched.h"

namespace piccl {

struct Env {
  Algo algo[COLL_COUNT];
  int k[COLL_COUNT];
  int block_size, max_grid, min_grid;          // reference knobs (now size the fused executor)
  bool block_size_set, max_grid_set, min_grid_set;
  int timeout_ms, scratch_mb, slot_kb, nslot, max_cta, ll_kb, llf_kb, llx_kb, tp_mb, tp_feeders;
  int log_level, debug;
  int exec_defer;                                // PICCL_EXEC_DEFER=1: the FIFO executor publishes counters lazily (exec_impl.cuh)
  int proto;                                     // PICCL_PROTO: 0 auto, 1 ll, 2 simple, 3 nvls (see env.cc)
  int nvls, nvls_chunk_kb, nvls_depth, nvls_cta, nvls_min_kb, nvls_auto_kb, nvls_gran_min, nvls_profile, nvls_bulk, nvls_strict_fences, nvls_sub;           // PICCL_NVLS=0: no multicast window; half-slot size, CTA count and smallest chunk of the in-switch collectives
  bool launch_persistent; int persist_idle_us;   // PICCL_LAUNCH=persistent, PICCL_PERSIST_IDLE_US
  std::string trace_file, tune_file;
  // host-side fault injection: rank:call:{skip_call|delay_ms=N}
  int fault_rank, fault_call, fault_delay_ms; bool fault_skip;
};

const Env& env();
void env_reload();                 // tests only
void log_msg(int level, const char* fmt, ...);

}  // namespace piccl
