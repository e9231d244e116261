// Internal definitions of the communicator runtime.
#pragma once
#include <cuda_runtime.h>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>
#include "../include/piccl.h"
#include "../include/piccl_sched.h"
#include "../kernels/exec.cuh"
#include "env.h"

namespace piccl {

constexpr unsigned kHandleMagic = 0x5049434cu;   // "PICL"

struct HandleBlob {
  unsigned magic; int rank, nranks, pid, device; int max_cta, nslot, ipc_ok;   // ipc_ok bit 0: heap exported; bit 1: wants and can use an NVLink multicast window; bits 8-15: CTAs of the in-switch collectives
  unsigned long long host_id, heap_bytes, raw_ptr, slot_bytes;
  cudaIpcMemHandle_t ipc;
};

struct ProgKey {
  int coll, algo, k, root, elem_size, in_place; long long count, stride;
  bool operator==(const ProgKey& o) const {
    return coll == o.coll && algo == o.algo && k == o.k && root == o.root && elem_size == o.elem_size && in_place == o.in_place && count == o.count && stride == o.stride;
  }
};
struct ProgKeyHash {
  size_t operator()(const ProgKey& k) const {
    unsigned long long h = 1469598103934665603ull;
    auto mix = [&](unsigned long long v) { h ^= v; h *= 1099511628211ull; };
    mix(k.coll); mix(k.algo); mix((unsigned)k.k); mix(k.root); mix(k.elem_size); mix(k.in_place); mix((unsigned long long)k.count); mix((unsigned long long)k.stride);
    return (size_t)h;
  }
};
struct ProgEntry { const Action* dev = nullptr; int n_actions = 0; long long scratch_elems = 0; cudaEvent_t ready = nullptr; cudaStream_t origin = nullptr; bool synced = false; };
struct ProgChunk { char* dev = nullptr; char* host = nullptr; size_t cap = 0, used = 0; };

struct TraceRec { int coll, algo, k, n_cta; long long bytes; double host_us; cudaEvent_t start = nullptr, stop = nullptr; };

struct TuneRow { int coll, nranks; long long max_bytes; Algo algo; int k; };

}  // namespace piccl

struct piccl_comm {
  int rank = 0, nranks = 1, device = 0, sm_count = 148;
  piccl_config_t cfg{};
  unsigned long long host_id = 0;
  char* heap = nullptr; long long heap_bytes = 0;
  piccl::RankCtx h_ctx{}; piccl::RankCtx* d_ctx = nullptr;
  unsigned long long *d_sent = nullptr, *d_rcvd = nullptr, *d_sent_ll = nullptr, *d_rcvd_ll = nullptr; int* d_abort = nullptr;
  long long llf_max_bytes = 0;         // largest message the low-latency executor takes (0: off)
  piccl_status_t* h_status = nullptr; piccl_status_t* d_status = nullptr;
  bool ipc_opened[piccl::kMaxRanks] = {false};
  bool connected = false, broken = false;
  unsigned long long call_index = 0;
  unsigned tp_epoch_rs = 0, tp_epoch_ag = 0;   // epochs of the fused tensor-parallel kernels
  int* d_tp_status = nullptr;
  void* persist = nullptr;             // state of the persistent launcher (runtime/persistent.cu)
  void* nvls = nullptr;                // multicast window of the in-switch all-reduce (runtime/nvls.cu)
  unsigned ll_epoch = 0;               // epoch of the last low-latency all-reduce (same on all ranks)
  long long ll_max_bytes = 0;          // largest message the low-latency path takes (0: off)
  piccl_stats_t stats{};
  std::unordered_map<piccl::ProgKey, piccl::ProgEntry, piccl::ProgKeyHash> cache;
  std::vector<piccl::ProgChunk> chunks;
  std::vector<piccl::TraceRec> trace;
  std::mutex mu;
};

namespace piccl {
int fail(int code, const char* fmt, ...);
TraceRec* trace_begin(piccl_comm* c, Coll coll, Algo algo, int k, long long bytes, int n_cta, cudaStream_t s);
void trace_end(piccl_comm* c, TraceRec* r, cudaStream_t s);
void trace_dump(piccl_comm* c);
// Algorithm choice for AUTO / unspecified requests: PICCL_TUNE_FILE table if given, else built-in thresholds.
Algo select_algo(piccl_comm* c, Coll coll, size_t bytes, int* k);
Algo select_algo_n(int nranks, Coll coll, size_t bytes, int* k, bool window);
// the rule for a communicator without a multicast window (what an NVLS request falls back to)
Algo select_algo_p2p(piccl_comm* c, Coll coll, size_t bytes, int* k);
// persistent launcher (PICCL_LAUNCH=persistent): PICCL_OK if enqueued through the server, PICCL_UNSUPPORTED: launch directly
int persist_allreduce(piccl_comm** cs, int n, const LLArgs& la, const void* const* in, void* const* out, long long count, int dtype, int op, int avg,
                      int algo, int k, cudaStream_t stream);
void persist_destroy(piccl_comm* c);
}  // namespace piccl
