// Communicator runtime: symmetric heap, peer mapping, program cache and the
// launcher of the fused executor.
//
// The reference's counterpart is the scratch-buffer manager inside its
// ncclCommInitRank hook (src/piccl.c:175-199: three process-global buffers,
// 16 GiB per process, no error checks).  Here every communicator owns one heap
// of a few hundred MiB that peers map through CUDA IPC; the handles travel by
// whatever the caller has (real NCCL in the preload shim, torch.distributed
// in the Python package, a pipe in the benchmark).
#include "comm.h"
#include "nvls.h"
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>
#include <algorithm>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <thread>
#include <unistd.h>

namespace piccl {

thread_local std::string g_last_error;
int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof buf, fmt, ap); va_end(ap);
  g_last_error = buf;
  log_msg(1, "error: %s", buf);
  return code;
}

#define CUDA_TRY(expr)                                                                              \
  do {                                                                                              \
    cudaError_t e_ = (expr);                                                                        \
    if (e_ != cudaSuccess) return fail(PICCL_CUDA_ERROR, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), __FILE__, __LINE__); \
  } while (0)

static unsigned long long host_hash() {
  char h[256] = {0}; gethostname(h, sizeof h - 1);
  unsigned long long x = 1469598103934665603ull;
  for (char* p = h; *p; p++) { x ^= (unsigned char)*p; x *= 1099511628211ull; }
  // CUDA IPC needs one PID namespace as well as one host: the boot id tells hosts apart,
  // the host name tells containers apart
  if (FILE* f = fopen("/proc/sys/kernel/random/boot_id", "r")) { int c; while ((c = fgetc(f)) != EOF) { x ^= (unsigned char)c; x *= 1099511628211ull; } fclose(f); }
  return x;
}

static long long round_up(long long v, long long a) { return (v + a - 1) / a * a; }

struct DevGuard {
  int prev = -1; bool changed = false;
  explicit DevGuard(int dev) { if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) { cudaSetDevice(dev); changed = true; } }
  ~DevGuard() { if (changed) cudaSetDevice(prev); }
};

}  // namespace piccl

using namespace piccl;

extern "C" {

const char* piccl_last_error(void) { return g_last_error.c_str(); }

int piccl_comm_create(int rank, int nranks, int device, const piccl_config_t* user_cfg, piccl_comm_t** out) {
  if (!out || nranks < 1 || nranks > kMaxRanks || rank < 0 || rank >= nranks) return fail(PICCL_INVALID_ARGUMENT, "bad rank/nranks %d/%d", rank, nranks);
  const Env& e = env();
  piccl_config_t cfg; memset(&cfg, 0, sizeof cfg);
  if (user_cfg) cfg = *user_cfg;
  if (cfg.max_cta <= 0) cfg.max_cta = e.max_cta;
  if (cfg.nslot <= 0) cfg.nslot = e.nslot;
  if (cfg.nslot < 2) cfg.nslot = 2;                        // fused receive+forward needs two entries in flight
  if (cfg.slot_bytes <= 0) cfg.slot_bytes = (long long)e.slot_kb * 1024;
  cfg.slot_bytes = round_up(cfg.slot_bytes, 16);
  if (cfg.scratch_bytes <= 0) cfg.scratch_bytes = (long long)e.scratch_mb << 20;
  if (cfg.block_size <= 0) cfg.block_size = e.block_size_set ? e.block_size : 512;
  if (cfg.block_size > kMaxBlock) cfg.block_size = kMaxBlock;
  if (cfg.block_size < 64) cfg.block_size = 64;
  cfg.block_size = cfg.block_size / 32 * 32;
  if (cfg.timeout_ms <= 0) cfg.timeout_ms = e.timeout_ms;
  if (cfg.max_cta > 128) cfg.max_cta = 128;
  if (cfg.nvls_cta <= 0) cfg.nvls_cta = e.nvls_cta;

  DevGuard g(device);
  piccl_comm* c = new piccl_comm();
  c->rank = rank; c->nranks = nranks; c->device = device; c->cfg = cfg;
  c->host_id = host_hash();
  RankCtx& x = c->h_ctx; memset(&x, 0, sizeof x);
  x.rank = rank; x.nranks = nranks; x.max_cta = cfg.max_cta; x.nslot = cfg.nslot; x.slot_bytes = cfg.slot_bytes;
  long long flags = round_up((long long)nranks * cfg.max_cta * kFlagStride, 4096);
  // low-latency slots: [parity][step][source rank], each 2 x the largest payload (line = 8 B data + 8 B flags)
  long long ll_payload = (long long)e.ll_kb * 1024;
  x.ll_slot_bytes = round_up(2 * ll_payload, 4096);
  long long ll_bytes = ll_payload > 0 ? 2LL * kLLMaxSteps * nranks * x.ll_slot_bytes : 0;
  if (cfg.tp_bytes <= 0) cfg.tp_bytes = (long long)e.tp_mb << 20;
  c->cfg.tp_bytes = cfg.tp_bytes;
  const long long tp_flags = cfg.tp_bytes > 0 ? (1 << 20) : 0;
  x.tail_off = 0; x.head_off = flags; x.ll_off = 2 * flags; x.tp_flag_off = x.ll_off + ll_bytes;
  // low-latency FIFO of the executor (all collectives, small messages): head counters, then the lines
  x.llf_head_off = x.tp_flag_off + tp_flags;
  x.llf_off = x.llf_head_off + round_up((long long)nranks * kLLFifoCta * kFlagStride, 4096);
  x.scratch_off = x.llf_off + (long long)nranks * kLLFifoCta * kLLFifoSlots * kLLFifoSlotBytes; x.scratch_bytes = round_up(cfg.scratch_bytes, 4096);
  c->llf_max_bytes = (long long)e.llf_kb * 1024;
  c->ll_max_bytes = ll_payload;
  x.fifo_off = x.scratch_off + x.scratch_bytes;
  x.tp_data_off = round_up(x.fifo_off + (long long)nranks * cfg.max_cta * cfg.nslot * cfg.slot_bytes, 4096);
  x.tp_bytes = round_up(cfg.tp_bytes, 4096);
  x.heap_bytes = x.tp_data_off + x.tp_bytes;
  c->heap_bytes = x.heap_bytes;

  cudaError_t err;
#define CREATE_TRY(expr) if ((err = (expr)) != cudaSuccess) { int rc = fail(PICCL_CUDA_ERROR, "%s failed: %s", #expr, cudaGetErrorString(err)); piccl_comm_destroy(c); return rc; }
  CREATE_TRY(cudaMalloc(&c->heap, c->heap_bytes));
  CREATE_TRY(cudaMemset(c->heap, 0, x.scratch_off));          // counters start at zero; payload needs no clearing
  size_t cnt_bytes = (size_t)nranks * cfg.max_cta * sizeof(unsigned long long);
  CREATE_TRY(cudaMalloc(&c->d_sent, cnt_bytes)); CREATE_TRY(cudaMemset(c->d_sent, 0, cnt_bytes));
  CREATE_TRY(cudaMalloc(&c->d_rcvd, cnt_bytes)); CREATE_TRY(cudaMemset(c->d_rcvd, 0, cnt_bytes));
  size_t cnt_ll = (size_t)nranks * kLLFifoCta * sizeof(unsigned long long);
  CREATE_TRY(cudaMalloc(&c->d_sent_ll, cnt_ll)); CREATE_TRY(cudaMemset(c->d_sent_ll, 0, cnt_ll));
  CREATE_TRY(cudaMalloc(&c->d_rcvd_ll, cnt_ll)); CREATE_TRY(cudaMemset(c->d_rcvd_ll, 0, cnt_ll));
  CREATE_TRY(cudaMalloc(&c->d_abort, sizeof(int))); CREATE_TRY(cudaMemset(c->d_abort, 0, sizeof(int)));
  CREATE_TRY(cudaHostAlloc(&c->h_status, sizeof(piccl_status_t), cudaHostAllocMapped));
  memset(c->h_status, 0, sizeof(piccl_status_t));
  CREATE_TRY(cudaHostGetDevicePointer((void**)&c->d_status, c->h_status, 0));
  CREATE_TRY(cudaMalloc(&c->d_ctx, sizeof(RankCtx)));
  CREATE_TRY(cudaDeviceSynchronize());
#undef CREATE_TRY
  x.sent = c->d_sent; x.rcvd = c->d_rcvd; x.sent_ll = c->d_sent_ll; x.rcvd_ll = c->d_rcvd_ll; x.abort_flag = c->d_abort; x.status = c->d_status;
  int sms = 0; cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device); c->sm_count = sms > 0 ? sms : 148;
  log_msg(2, "comm %p: rank %d/%d dev %d heap %.1f MiB (max_cta %d nslot %d slot %lld KiB scratch %lld MiB)", (void*)c, rank, nranks, device,
          c->heap_bytes / 1048576.0, cfg.max_cta, cfg.nslot, cfg.slot_bytes >> 10, x.scratch_bytes >> 20);
  *out = c;
  return PICCL_OK;
}

int piccl_comm_local_handle(piccl_comm_t* c, piccl_handle_t* out) {
  if (!c || !out) return fail(PICCL_INVALID_ARGUMENT, "null argument");
  DevGuard g(c->device);
  HandleBlob b; memset(&b, 0, sizeof b);
  b.magic = kHandleMagic; b.rank = c->rank; b.nranks = c->nranks; b.pid = (int)getpid(); b.device = c->device;
  b.host_id = c->host_id; b.heap_bytes = (unsigned long long)c->heap_bytes; b.raw_ptr = (unsigned long long)(uintptr_t)c->heap;
  b.max_cta = c->cfg.max_cta; b.nslot = c->cfg.nslot; b.slot_bytes = (unsigned long long)c->cfg.slot_bytes;
  cudaError_t e = cudaIpcGetMemHandle(&b.ipc, c->heap);
  b.ipc_ok = (e == cudaSuccess) ? 1 : 0;
  if (env().nvls && nvls_device_capable(c->device)) b.ipc_ok |= 2;
  b.ipc_ok |= (c->cfg.nvls_cta & 0xff) << 8;                 // the window geometry must agree on all ranks
  if (e != cudaSuccess) { cudaGetLastError(); log_msg(1, "cudaIpcGetMemHandle: %s (peers in other processes cannot map this rank)", cudaGetErrorString(e)); }
  static_assert(sizeof(HandleBlob) <= sizeof(piccl_handle_t), "handle blob too large");
  memset(out, 0, sizeof *out); memcpy(out->bytes, &b, sizeof b);
  return PICCL_OK;
}

int piccl_comm_connect(piccl_comm_t* c, const piccl_handle_t* all) {
  if (!c || !all) return fail(PICCL_INVALID_ARGUMENT, "null argument");
  if (c->connected) return fail(PICCL_INVALID_USAGE, "communicator already connected");
  DevGuard g(c->device);
  for (int p = 0; p < c->nranks; p++) {
    HandleBlob b; memcpy(&b, all[p].bytes, sizeof b);
    if (b.magic != kHandleMagic || b.rank != p || b.nranks != c->nranks) return fail(PICCL_INVALID_ARGUMENT, "handle %d is not a handle of rank %d of this communicator", p, p);
    if (b.max_cta != c->cfg.max_cta || b.nslot != c->cfg.nslot || (long long)b.slot_bytes != c->cfg.slot_bytes || (long long)b.heap_bytes != c->heap_bytes)
      return fail(PICCL_INVALID_USAGE, "rank %d uses a different heap layout (PICCL_MAX_CTA/NSLOT/SLOT_KB/SCRATCH_MB must agree)", p);
    if (((b.ipc_ok >> 8) & 0xff) != (c->cfg.nvls_cta & 0xff)) return fail(PICCL_INVALID_USAGE, "rank %d uses a different number of in-switch CTAs (nvls_cta / PICCL_NVLS_CTA must agree)", p);
    if (p == c->rank) { c->h_ctx.heap[p] = c->heap; continue; }
    if (b.host_id != c->host_id) return fail(PICCL_UNSUPPORTED, "rank %d is on another host: peer memory is not reachable", p);
    if (b.pid == (int)getpid()) {
      // same process: the pointer itself is valid; another device needs peer access
      if (b.device != c->device) {
        int can = 0; cudaDeviceCanAccessPeer(&can, c->device, b.device);
        if (!can) return fail(PICCL_UNSUPPORTED, "no peer access from device %d to %d", c->device, b.device);
        cudaError_t e = cudaDeviceEnablePeerAccess(b.device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return fail(PICCL_CUDA_ERROR, "cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(e));
        cudaGetLastError();
      }
      c->h_ctx.heap[p] = (char*)(uintptr_t)b.raw_ptr;
    } else {
      if (!(b.ipc_ok & 1)) return fail(PICCL_UNSUPPORTED, "rank %d could not export its heap", p);
      void* ptr = nullptr;
      cudaError_t e = cudaIpcOpenMemHandle(&ptr, b.ipc, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) { cudaGetLastError(); return fail(PICCL_UNSUPPORTED, "cudaIpcOpenMemHandle(rank %d): %s", p, cudaGetErrorString(e)); }
      c->h_ctx.heap[p] = (char*)ptr; c->ipc_opened[p] = true;
    }
  }
  CUDA_TRY(cudaMemcpy(c->d_ctx, &c->h_ctx, sizeof(RankCtx), cudaMemcpyHostToDevice));
  c->connected = true;
  if (c->nranks >= 2) {
    // In-switch collectives: a multicast window if every rank asked for it and can do it, and no two ranks share a process
    // (each rank binds its own device to the multicast object, and the set-up blocks until all ranks take part).
    // All ranks inside this process on this device (virtual ranks): a plain window each, the kernels emulate the switch.
    bool want = true, one_process = true; int root_pid = 0; unsigned long long root_id = 0;
    for (int p = 0; p < c->nranks; p++) {
      HandleBlob b; memcpy(&b, all[p].bytes, sizeof b);
      want &= (b.ipc_ok & 2) != 0;
      one_process &= b.pid == (int)getpid() && b.device == c->device;
      if (p == 0) { root_pid = b.pid; root_id = b.raw_ptr; }
      for (int q = 0; q < p; q++) { HandleBlob o; memcpy(&o, all[q].bytes, sizeof o); if (o.pid == b.pid) want = false; }
    }
    if (one_process) { if (env().nvls && c->nranks <= kMaxVRanks) nvls_setup_emulated(c); }
    else if (want) nvls_setup(c, root_pid, root_id);
  }
  return PICCL_OK;
}

// A consumer's kernel acknowledges the last entries this rank sent by writing head counters into THIS rank's heap, and that
// can happen after this rank's own kernels have ended.  Before the heap is freed: wait on the host, with a limit, until every
// entry sent has been acknowledged.  (Everything peers sent to this rank was consumed by kernels that have ended.)
static void quiesce_fifos(piccl_comm* c) {
  if (!c->connected || !c->heap || c->nranks < 2 || c->broken || (c->h_status && c->h_status->aborted)) return;
  const RankCtx& x = c->h_ctx;
  const int n = c->nranks, mc = c->cfg.max_cta;
  std::vector<unsigned long long> sent((size_t)n * mc), sent_ll((size_t)n * kLLFifoCta);
  const size_t head_bytes = (size_t)n * mc * kFlagStride, llh_bytes = (size_t)n * kLLFifoCta * kFlagStride;
  std::vector<char> head(head_bytes), llh(llh_bytes);
  if (cudaMemcpy(sent.data(), c->d_sent, sent.size() * 8, cudaMemcpyDeviceToHost) != cudaSuccess ||
      cudaMemcpy(sent_ll.data(), c->d_sent_ll, sent_ll.size() * 8, cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return; }
  for (int tries = 0; tries < 200; tries++) {
    if (cudaMemcpy(head.data(), c->heap + x.head_off, head_bytes, cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(llh.data(), c->heap + x.llf_head_off, llh_bytes, cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return; }
    bool done = true;
    for (int p = 0; p < n && done; p++) {
      if (p == c->rank) continue;
      for (int b = 0; b < mc && done; b++) { unsigned long long h; memcpy(&h, &head[(size_t)(p * mc + b) * kFlagStride], 8); if (h < sent[(size_t)p * mc + b]) done = false; }
      for (int b = 0; b < kLLFifoCta && done; b++) { unsigned long long h; memcpy(&h, &llh[(size_t)(p * kLLFifoCta + b) * kFlagStride], 8); if (h < sent_ll[(size_t)p * kLLFifoCta + b]) done = false; }
    }
    if (done) return;
    usleep(5000);
  }
  log_msg(1, "rank %d: peers did not acknowledge everything this rank sent within 1 s", c->rank);
}

int piccl_comm_destroy(piccl_comm_t* c) {
  if (!c) return PICCL_OK;
  DevGuard g(c->device);
  cudaDeviceSynchronize();
  quiesce_fifos(c);
  persist_destroy(c);
  nvls_destroy(c);
  if (!env().trace_file.empty()) trace_dump(c);
  if (env().log_level >= 1) {
    const piccl_stats_t& s = c->stats;
    log_msg(1, "comm rank %d: calls ag %llu ar %llu bc %llu rd %llu rs %llu, launches %llu, cache hit/miss %llu/%llu, fallbacks %llu, timeouts %llu", c->rank,
            s.calls[0], s.calls[1], s.calls[2], s.calls[3], s.calls[4], s.launches, s.program_cache_hits, s.program_cache_misses, s.fallbacks, s.timeouts);
  }
  for (int p = 0; p < c->nranks; p++) if (c->ipc_opened[p]) cudaIpcCloseMemHandle(c->h_ctx.heap[p]);
  for (auto& ch : c->chunks) { cudaFree(ch.dev); cudaFreeHost(ch.host); }
  for (auto& kv : c->cache) if (kv.second.ready) cudaEventDestroy(kv.second.ready);
  for (auto& t : c->trace) { if (t.start) cudaEventDestroy(t.start); if (t.stop) cudaEventDestroy(t.stop); }
  if (c->d_tp_status) cudaFree(c->d_tp_status);
  cudaFree(c->d_sent_ll); cudaFree(c->d_rcvd_ll);
  cudaFree(c->heap); cudaFree(c->d_sent); cudaFree(c->d_rcvd); cudaFree(c->d_abort); cudaFree(c->d_ctx);
  if (c->h_status) cudaFreeHost(c->h_status);
  cudaGetLastError();
  delete c;
  return PICCL_OK;
}

int piccl_comm_abort(piccl_comm_t* c) {
  if (!c) return PICCL_OK;
  DevGuard g(c->device);
  int one = 1;
  // a blocking copy on the legacy stream would wait for the very kernel we want to stop
  cudaStream_t s; if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) return fail(PICCL_CUDA_ERROR, "stream create failed");
  cudaMemcpyAsync(c->d_abort, &one, sizeof one, cudaMemcpyHostToDevice, s);
  cudaStreamSynchronize(s); cudaStreamDestroy(s);
  if (!c->h_status->aborted) { c->h_status->code = 3; c->h_status->rank = c->rank; c->h_status->aborted = 1; }
  c->broken = true;
  return PICCL_OK;
}

int piccl_comm_status(piccl_comm_t* c, piccl_status_t* out) {
  if (!c || !out) return fail(PICCL_INVALID_ARGUMENT, "null argument");
  memcpy(out, (const void*)c->h_status, sizeof *out);
  return PICCL_OK;
}
int piccl_get_stats(piccl_comm_t* c, piccl_stats_t* out) {
  if (!c || !out) return fail(PICCL_INVALID_ARGUMENT, "null argument");
  std::lock_guard<std::mutex> l(c->mu); *out = c->stats; out->timeouts += c->h_status->aborted && c->h_status->code != 3 ? 1 : 0; return PICCL_OK;
}
int piccl_comm_rank(piccl_comm_t* c) { return c ? c->rank : -1; }
int piccl_comm_nranks(piccl_comm_t* c) { return c ? c->nranks : -1; }

}  // extern "C"

// ------------------------------------------------------------------ program cache
namespace piccl {

static int upload_program(piccl_comm* c, const Program& p, cudaStream_t stream, ProgEntry& e) {
  size_t bytes = std::max<size_t>(p.actions.size(), 1) * sizeof(Action);
  bytes = (bytes + 255) / 256 * 256;
  if (c->chunks.empty() || c->chunks.back().used + bytes > c->chunks.back().cap) {
    ProgChunk ch; ch.cap = std::max<size_t>(1 << 20, bytes); ch.used = 0;
    CUDA_TRY(cudaMalloc(&ch.dev, ch.cap));
    cudaError_t er = cudaHostAlloc(&ch.host, ch.cap, cudaHostAllocDefault);
    if (er != cudaSuccess) { cudaFree(ch.dev); return fail(PICCL_CUDA_ERROR, "cudaHostAlloc: %s", cudaGetErrorString(er)); }
    c->chunks.push_back(ch);
  }
  ProgChunk& ch = c->chunks.back();
  memcpy(ch.host + ch.used, p.actions.data(), p.actions.size() * sizeof(Action));
  e.dev = reinterpret_cast<const Action*>(ch.dev + ch.used);
  e.n_actions = (int)p.actions.size(); e.scratch_elems = p.scratch_elems; e.origin = stream; e.synced = false;
  if (!p.actions.empty()) CUDA_TRY(cudaMemcpyAsync(ch.dev + ch.used, ch.host + ch.used, p.actions.size() * sizeof(Action), cudaMemcpyHostToDevice, stream));
  CUDA_TRY(cudaEventCreateWithFlags(&e.ready, cudaEventDisableTiming));
  CUDA_TRY(cudaEventRecord(e.ready, stream));
  ch.used += bytes;
  return PICCL_OK;
}

// PICCL_DEBUG=1: every action of a freshly compiled program is checked against the extents of the
// buffers of the call before it is ever given to the device (ranges, peers, scratch capacity).
static const char* check_program(const Program& p, const CollArgs& a, long long scratch_cap_elems) {
  const long long st = a.block_stride ? a.block_stride : a.count;
  long long in_elems = a.count, out_elems = a.count;
  if (a.coll == COLL_ALLGATHER) out_elems = (a.nranks - 1) * st + a.count;
  if (a.coll == COLL_REDUCE_SCATTER) in_elems = (a.nranks - 1) * st + a.count;
  for (const Action& ac : p.actions) {
    if (ac.count <= 0 || ac.n_recv > kMaxActionPeers || ac.n_send > kMaxActionPeers) return "bad operand count";
    for (int i = 0; i < ac.n_recv; i++) if (ac.recv_peer[i] >= a.nranks || ac.recv_peer[i] == p.rank) return "bad receive peer";
    for (int i = 0; i < ac.n_send; i++) if (ac.send_peer[i] >= a.nranks || ac.send_peer[i] == p.rank) return "bad send peer";
    const long long slim = ac.src_buf == BUF_IN ? in_elems : ac.src_buf == BUF_OUT ? out_elems : scratch_cap_elems;
    if (ac.src_buf != BUF_NONE && (ac.src_off < 0 || ac.src_off + ac.count > slim)) return "source range outside its buffer";
    const long long dlim = ac.dst_buf == BUF_OUT ? out_elems : scratch_cap_elems;
    if (ac.dst_buf == BUF_IN) return "write to the send buffer";
    if (ac.dst_buf != BUF_NONE && (ac.dst_off < 0 || ac.dst_off + ac.count > dlim)) return "destination range outside its buffer";
  }
  return nullptr;
}

static int get_program(piccl_comm* c, const CollArgs& a, cudaStream_t stream, const ProgEntry** out) {
  ProgKey k{(int)a.coll, (int)a.algo, a.k, a.root, a.elem_size, a.in_place ? 1 : 0, a.count, a.block_stride};
  auto it = c->cache.find(k);
  if (it == c->cache.end()) {
    // A new program needs device and pinned memory and an upload on the caller's stream: not inside a stream capture (an
    // allocation ends a capture in the global mode, and the upload's event would belong to the graph).  The caller runs
    // the call once before capturing, or, in the preload library, the call goes to NCCL.
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cs) == cudaSuccess && cs != cudaStreamCaptureStatusNone) {
      c->stats.fallbacks++;
      return fail(PICCL_UNSUPPORTED, "%s %s of %lld elements was never run outside a stream capture: its program cannot be built while capturing", coll_name(a.coll), algo_name(a.algo), a.count);
    }
    cudaGetLastError();
    // programs are kept for the life of the communicator (kernels in flight may read them): bound what they may take
    size_t held = 0;
    for (const auto& ch : c->chunks) held += ch.cap;
    if (held > ((size_t)256 << 20)) {
      c->stats.fallbacks++;
      return fail(PICCL_UNSUPPORTED, "program cache full (%zu MiB for %zu distinct calls)", held >> 20, c->cache.size());
    }
    c->stats.program_cache_misses++;
    Program p = compile(a, c->rank);
    if (env().debug) {
      if (const char* why = check_program(p, a, c->h_ctx.scratch_bytes / std::max(1, a.elem_size)))
        return fail(PICCL_INTERNAL_ERROR, "program check failed (%s %s, rank %d): %s", coll_name(a.coll), algo_name(a.algo), c->rank, why);
    }
    ProgEntry e;
    int rc = upload_program(c, p, stream, e); if (rc) return rc;
    it = c->cache.emplace(k, e).first;
  } else {
    c->stats.program_cache_hits++;
    ProgEntry& e = it->second;
    if (!e.synced) {
      if (e.origin != stream) CUDA_TRY(cudaStreamWaitEvent(stream, e.ready, 0));
      if (cudaEventQuery(e.ready) == cudaSuccess) e.synced = true; else cudaGetLastError();
    }
  }
  *out = &it->second;
  return PICCL_OK;
}

// CTAs for one collective: enough to fill NVLink for large messages, one for tiny ones.
// All ranks compute the same number from the same arguments.  The reference's grid formula
// grid = clamp(count / block, MIN, MAX) (src/kernels/permutation_kernel.cu:76-77) is kept when
// PICCL_MIN/MAX_GRID_SIZE are set; the result is capped by the FIFO channel count.
static int choose_cta(const piccl_comm* c, const CollArgs& a, int n_vrank) {
  long long bytes = a.count * a.elem_size;
  if (a.coll == COLL_ALLREDUCE && (a.algo == ALGO_RING || a.algo == ALGO_K_RING)) bytes /= std::max(1, a.nranks);
  if (a.algo == ALGO_DIRECT && a.coll != COLL_ALLGATHER && a.coll != COLL_REDUCE_SCATTER) bytes /= std::max(1, a.coll == COLL_ALLREDUCE ? a.nranks : a.nranks - 1);
  const Env& e = env();
  long long n = (bytes + 32767) / 32768;
  if (e.min_grid_set || e.max_grid_set) {
    long long g = a.count / std::max(1, c->cfg.block_size);
    n = std::max<long long>(e.min_grid_set ? e.min_grid : 1, std::min<long long>(e.max_grid_set ? e.max_grid : g, g));
  }
  n = std::max<long long>(1, std::min<long long>(n, c->cfg.max_cta));
  if (n_vrank > 1) n = std::min<long long>(n, std::max(1, c->sm_count / n_vrank));
  return (int)n;
}

static bool fault_now(piccl_comm* c) {
  const Env& e = env();
  if (e.fault_rank != c->rank) return false;
  unsigned long long call = c->call_index;
  if ((long long)call != e.fault_call) return false;
  if (e.fault_delay_ms > 0) { log_msg(1, "fault injection: delaying call %llu by %d ms", call, e.fault_delay_ms); std::this_thread::sleep_for(std::chrono::milliseconds(e.fault_delay_ms)); return false; }
  if (e.fault_skip) { log_msg(1, "fault injection: skipping call %llu", call); return true; }
  return false;
}

struct CallDesc { Coll coll; const void* send; void* recv; size_t count; int dtype, op, root; Algo algo; int k; };

// Runs one collective over `n` communicators of this process (n == 1: the normal case).
static int run(piccl_comm** comms, int n, const CallDesc* calls, cudaStream_t stream) {
  piccl_comm* c0 = comms[0];
  const CallDesc& d0 = calls[0];
  if (n > kMaxVRanks) return fail(PICCL_INVALID_ARGUMENT, "at most %d communicators per group launch", kMaxVRanks);
  for (int i = 0; i < n; i++) {
    if (!comms[i]->connected) return fail(PICCL_INVALID_USAGE, "communicator is not connected");
    if (comms[i]->broken || comms[i]->h_status->aborted) { comms[i]->broken = true; return fail(PICCL_REMOTE_ERROR, "communicator aborted earlier (code %d, peer %d)", comms[i]->h_status->code, comms[i]->h_status->peer); }
    if (comms[i]->device != c0->device) return fail(PICCL_INVALID_ARGUMENT, "group launch needs one device");
  }
  const int esz_real = dtype_size(d0.dtype);
  if (!esz_real) { c0->stats.fallbacks++; return fail(PICCL_UNSUPPORTED, "unsupported data type %d", d0.dtype); }
  const bool reducing = d0.coll == COLL_ALLREDUCE || d0.coll == COLL_REDUCE || d0.coll == COLL_REDUCE_SCATTER;
  int op = d0.op; bool avg = false;
  if (reducing) {
    if (op == 4) { avg = true; op = 0; if (!(d0.dtype == DT_F32 || d0.dtype == DT_F16 || d0.dtype == DT_BF16 || d0.dtype == DT_F64)) { c0->stats.fallbacks++; return fail(PICCL_UNSUPPORTED, "avg on integer types"); } }
    if (op < 0 || op > 3) { c0->stats.fallbacks++; return fail(PICCL_UNSUPPORTED, "unsupported reduction op %d", d0.op); }
  }
  if (d0.root < 0 || d0.root >= c0->nranks) return fail(PICCL_INVALID_ARGUMENT, "root %d out of range", d0.root);
  if (d0.count == 0) return PICCL_OK;
  DevGuard g(c0->device);

  // data-moving collectives run the byte-wise instantiation
  const int esz = reducing ? esz_real : 1;
  const long long count = reducing ? (long long)d0.count : (long long)d0.count * esz_real;
  // small messages of every collective run the low-latency variant of the executor (flags inside the data lines)
  const bool use_llf = c0->llf_max_bytes > 0 && (long long)d0.count * esz_real <= c0->llf_max_bytes;
  const bool defer = env().exec_defer != 0;
  ExecKernelFn fn = use_llf ? (reducing ? exec_ll_kernel_for(d0.dtype, op) : exec_ll_copy_kernel())
                   : defer ? (reducing ? exec_defer_kernel_for(d0.dtype, op) : exec_defer_copy_kernel())
                           : (reducing ? exec_kernel_for(d0.dtype, op) : exec_copy_kernel());
  if (!fn) return fail(PICCL_INTERNAL_ERROR, "no kernel for dtype %d op %d", d0.dtype, op);

  // small exchange-type all-reduces take the low-latency kernel (flags travel inside the data lines)
  // (not while the stream is being captured: the call epoch is a launch argument, a replay would reuse it)
  cudaStreamCaptureStatus cap_state = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap_state) != cudaSuccess) { cudaGetLastError(); cap_state = cudaStreamCaptureStatusNone; }
  if (cap_state == cudaStreamCaptureStatusNone && d0.coll == COLL_ALLREDUCE && c0->ll_max_bytes > 0 && (long long)d0.count * esz_real <= c0->ll_max_bytes &&
      (d0.algo == ALGO_RD || d0.algo == ALGO_RM || d0.algo == ALGO_PRD || d0.algo == ALGO_PRM)) {
    Resolved rs = resolve(COLL_ALLREDUCE, d0.algo, d0.k, c0->nranks);
    LLKernelFn lf = ll_kernel_for(d0.dtype, op);
    if (rs.core == c0->nranks && !rs.radices.empty() && (int)rs.radices.size() <= kLLMaxSteps && rs.algo == d0.algo && lf) {
      const bool permuted = d0.algo == ALGO_PRD || d0.algo == ALGO_PRM;
      LLArgs la; memset(&la, 0, sizeof la);
      la.n_vrank = n; la.nsteps = (int)rs.radices.size(); la.avg = avg ? 1 : 0; la.scale = avg ? 1.0f / (float)c0->nranks : 1.0f;
      la.count = (long long)d0.count; la.timeout_ns = (unsigned long long)c0->cfg.timeout_ms * 1000000ull;
      const int E = 8 / esz_real;
      long long nlines = ((long long)d0.count + E - 1) / E;
      la.n_cta = (int)((nlines + ll_lines_per_cta() - 1) / ll_lines_per_cta());
      if (n * la.n_cta <= c0->sm_count) {
        bool skip = false;
        for (int i = 0; i < n; i++) {
          piccl_comm* c = comms[i];
          std::lock_guard<std::mutex> l(c->mu);
          for (int s = 0; s < la.nsteps; s++) {
            std::vector<int> pe = step_peers(c->rank, s, rs.radices, c->nranks, permuted);
            std::sort(pe.begin(), pe.end());
            la.npeers[s] = (uint8_t)pe.size();
            int below = 0;
            for (size_t j = 0; j < pe.size(); j++) { la.peers[i][s][j] = (uint8_t)pe[j]; if (pe[j] < c->rank) below++; }
            la.self_pos[i][s] = (uint8_t)below;
          }
          la.r[i].ctx = c->d_ctx; la.r[i].in = calls[i].send; la.r[i].out = calls[i].recv;
          la.epoch = ++c->ll_epoch;
          c->stats.launches++; c->stats.calls[COLL_ALLREDUCE]++; c->stats.bytes[COLL_ALLREDUCE] += (unsigned long long)d0.count * esz_real;
          skip |= fault_now(c); c->call_index++;
        }
        if (skip) return PICCL_OK;
        if (env().launch_persistent) {
          const void* ins[kMaxVRanks]; void* outs[kMaxVRanks];
          for (int i = 0; i < n; i++) { ins[i] = calls[i].send; outs[i] = calls[i].recv; }
          if (persist_allreduce(comms, n, la, ins, outs, (long long)d0.count, d0.dtype, op, avg ? 1 : 0, (int)d0.algo, d0.k, stream) == PICCL_OK) { c0->stats.persistent_calls++; return PICCL_OK; }
        }
        nvtxRangePushA("allreduce_ll");
        void* args[] = {&la};
        cudaError_t e;
        if (n > 1) e = cudaLaunchCooperativeKernel((const void*)lf, dim3(n * la.n_cta), dim3(kLLBlock), args, 0, stream);
        else e = cudaLaunchKernel((const void*)lf, dim3(la.n_cta), dim3(kLLBlock), args, 0, stream);
        nvtxRangePop();
        if (e != cudaSuccess) return fail(PICCL_CUDA_ERROR, "low-latency launch failed: %s", cudaGetErrorString(e));
        return PICCL_OK;
      }
    }
  }

  // small all-gather / reduce-scatter whose schedule is one exchange with every rank (DIRECT, or RM / PRM with a radix of at least
  // the rank count): the low-latency exchange kernel.  (Not while capturing: the epoch is a launch argument.)
  if (cap_state == cudaStreamCaptureStatusNone && (d0.coll == COLL_ALLGATHER || d0.coll == COLL_REDUCE_SCATTER) && c0->ll_max_bytes > 0 && c0->nranks >= 2 &&
      (long long)d0.count * esz_real <= std::min<long long>(c0->ll_max_bytes, (long long)env().llx_kb * 1024) &&
      (d0.algo == ALGO_DIRECT || ((d0.algo == ALGO_RM || d0.algo == ALGO_PRM) && d0.k >= c0->nranks))) {
    LLXKernelFn xf = d0.coll == COLL_ALLGATHER ? llx_allgather_kernel() : llx_reduce_scatter_kernel_for(d0.dtype, op);
    LLXArgs xa; memset(&xa, 0, sizeof xa);
    xa.n_vrank = n; xa.avg = avg ? 1 : 0; xa.scale = avg ? 1.0f / (float)c0->nranks : 1.0f;
    xa.count = d0.coll == COLL_ALLGATHER ? (long long)d0.count * esz_real : (long long)d0.count;
    xa.timeout_ns = (unsigned long long)c0->cfg.timeout_ms * 1000000ull;
    const long long nlines = d0.coll == COLL_ALLGATHER ? (xa.count + 7) / 8 : ((long long)d0.count + (8 / esz_real) - 1) / (8 / esz_real);
    xa.n_cta = (int)((nlines + llx_lines_per_cta() - 1) / llx_lines_per_cta());
    if (xf && esz_real <= 8 && n * xa.n_cta <= c0->sm_count) {
      bool skip = false;
      for (int i = 0; i < n; i++) {
        piccl_comm* c = comms[i];
        std::lock_guard<std::mutex> l(c->mu);
        xa.r[i].ctx = c->d_ctx; xa.r[i].in = calls[i].send; xa.r[i].out = calls[i].recv;
        xa.epoch = ++c->ll_epoch;
        c->stats.launches++; c->stats.calls[d0.coll]++; c->stats.bytes[d0.coll] += (unsigned long long)d0.count * esz_real;
        skip |= fault_now(c); c->call_index++;
      }
      if (skip) return PICCL_OK;
      nvtxRangePushA("exchange_ll");
      void* args[] = {&xa};
      cudaError_t e;
      if (n > 1) e = cudaLaunchCooperativeKernel((const void*)xf, dim3(n * xa.n_cta), dim3(kLLBlock), args, 0, stream);
      else e = cudaLaunchKernel((const void*)xf, dim3(xa.n_cta), dim3(kLLBlock), args, 0, stream);
      nvtxRangePop();
      if (e != cudaSuccess) return fail(PICCL_CUDA_ERROR, "low-latency exchange launch failed: %s", cudaGetErrorString(e));
      return PICCL_OK;
    }
  }

  // through the switch: all ranks of the communicator in this launch (one real rank, or every virtual rank of an emulated group)
  if (d0.algo == ALGO_NVLS || env().proto == 3) {
    bool can = (op == 0 || op == 2 || op == 3 || !reducing) && (n == 1 ? !nvls_emulated(c0) : nvls_emulated(c0) && n == c0->nranks);
    for (int i = 0; i < n && can; i++) can = nvls_eligible(comms[i], d0.coll, d0.dtype, op, d0.count);
    if (can) {
      bool skip = false;
      for (int i = 0; i < n; i++) { std::lock_guard<std::mutex> l(comms[i]->mu); skip |= fault_now(comms[i]); comms[i]->call_index++; }
      if (skip) return PICCL_OK;
      const void* ins[kMaxVRanks]; void* outs[kMaxVRanks];
      for (int i = 0; i < n; i++) { ins[i] = calls[i].send; outs[i] = calls[i].recv; }
      TraceRec* tr = trace_begin(c0, d0.coll, ALGO_NVLS, 0, (long long)d0.count * esz_real, 0, stream);
      nvtxRangePushA("in_switch");
      int rc = nvls_collective(comms, n, d0.coll, ins, outs, d0.count, d0.dtype, op, avg, d0.root, stream);
      nvtxRangePop();
      trace_end(c0, tr, stream);
      if (rc == PICCL_OK) {
        for (int i = 0; i < n; i++) { piccl_comm* c = comms[i]; c->stats.launches++; c->stats.nvls_calls++; c->stats.calls[d0.coll]++; c->stats.bytes[d0.coll] += (unsigned long long)d0.count * esz_real; }
        return rc;
      }
      if (rc != PICCL_UNSUPPORTED) return rc;
    }
  }
  if (d0.algo == ALGO_NVLS) {
    // no window, or a type / operator / size the switch path does not take: what AUTO picks without a window
    CallDesc alt[kMaxVRanks];
    int k2 = d0.k;
    const Algo a2 = select_algo_p2p(c0, d0.coll, d0.count * (size_t)esz_real, &k2);
    for (int i = 0; i < n; i++) { alt[i] = calls[i]; alt[i].algo = a2; alt[i].k = k2; }
    return run(comms, n, alt, stream);
  }

  // slabs: bound the local scratch of the recursive reduce-scatters
  long long slab = count, stride = 0;
  if (d0.coll == COLL_REDUCE_SCATTER) {
    CollArgs probe; probe.coll = d0.coll; probe.algo = d0.algo; probe.k = d0.k; probe.nranks = c0->nranks; probe.count = count; probe.elem_size = esz;
    Program p = compile(probe, 0);
    if (p.scratch_elems * esz > c0->h_ctx.scratch_bytes) {
      long long blocks = (p.scratch_elems + count - 1) / count + 1;
      slab = c0->h_ctx.scratch_bytes / esz / blocks / 64 * 64;
      if (slab <= 0) return fail(PICCL_UNSUPPORTED, "scratch too small");
      stride = count;
    }
  }

  nvtxRangePushA(coll_name(d0.coll));
  int rc = PICCL_OK;
  for (long long done = 0; done < count && rc == PICCL_OK; done += slab) {
    long long cur = std::min(slab, count - done);
    KernelArgs ka; memset(&ka, 0, sizeof ka);
    ka.n_vrank = n; ka.elem_size = esz; ka.avg = avg ? 1 : 0; ka.scale = avg ? 1.0f / (float)c0->nranks : 1.0f;
    int n_cta = 0;
    for (int i = 0; i < n && rc == PICCL_OK; i++) {
      piccl_comm* c = comms[i]; const CallDesc& d = calls[i];
      std::lock_guard<std::mutex> l(c->mu);
      CollArgs a; a.coll = d.coll; a.algo = d.algo; a.k = d.k; a.nranks = c->nranks; a.root = d.root; a.count = cur; a.block_stride = stride; a.elem_size = esz;
      const char* s = (const char*)d.send; char* r = (char*)d.recv;
      switch (d.coll) {
        case COLL_ALLGATHER: a.in_place = (s == r + (long long)c->rank * count); s += done; r += done; if (stride == 0 && slab != count) a.block_stride = count; break;
        case COLL_REDUCE_SCATTER: a.in_place = (r == s + (long long)c->rank * count * esz); s += done * esz; r += done * esz; break;
        default: a.in_place = (s == r); break;
      }
      if (d.coll == COLL_REDUCE && c->rank != d.root) a.in_place = false;
      const ProgEntry* pe = nullptr;
      rc = get_program(c, a, stream, &pe); if (rc) break;
      if (i == 0) {
        n_cta = choose_cta(c, a, n);
        if (use_llf) {   // 4 KiB of payload per CTA and segment, at most kLLFifoCta CTAs
          long long ab = a.count * a.elem_size;
          if (a.coll == COLL_ALLREDUCE && (a.algo == ALGO_RING || a.algo == ALGO_K_RING)) ab /= std::max(1, a.nranks);
          if (a.algo == ALGO_DIRECT && a.coll != COLL_ALLGATHER && a.coll != COLL_REDUCE_SCATTER) ab /= std::max(1, a.coll == COLL_ALLREDUCE ? a.nranks : a.nranks - 1);
          n_cta = (int)std::max<long long>(1, std::min<long long>((ab + 4095) / 4096, kLLFifoCta));
          if (n > 1) n_cta = std::min(n_cta, std::max(1, c->sm_count / n));
        }
        ka.n_cta = n_cta; ka.timeout_ns = (unsigned long long)c->cfg.timeout_ms * 1000000ull;
      }
      ka.r[i].ctx = c->d_ctx; ka.r[i].actions = pe->dev; ka.r[i].n_actions = pe->n_actions; ka.r[i].in = s; ka.r[i].out = r;
      c->stats.launches++;
    }
    if (rc) break;
    bool skip = false;
    for (int i = 0; i < n; i++) skip |= fault_now(comms[i]);
    for (int i = 0; i < n; i++) comms[i]->call_index++;
    if (skip) continue;
    TraceRec* tr = trace_begin(c0, d0.coll, d0.algo, d0.k, cur * esz, n_cta, stream);
    void* args[] = {&ka};
    cudaError_t e;
    const int block = use_llf ? kLLBlock : c0->cfg.block_size;
    if (n > 1) e = cudaLaunchCooperativeKernel((const void*)fn, dim3(n * n_cta), dim3(block), args, 0, stream);
    else e = cudaLaunchKernel((const void*)fn, dim3(n_cta), dim3(block), args, 0, stream);
    if (e != cudaSuccess) rc = fail(PICCL_CUDA_ERROR, "executor launch failed: %s", cudaGetErrorString(e));
    trace_end(c0, tr, stream);
  }
  nvtxRangePop();
  if (rc == PICCL_OK) for (int i = 0; i < n; i++) { comms[i]->stats.calls[d0.coll]++; comms[i]->stats.bytes[d0.coll] += (unsigned long long)d0.count * esz_real; }
  return rc;
}

}  // namespace piccl

extern "C" {

static int one(piccl_comm_t* c, CallDesc d, void* stream) {
  if (!c) return fail(PICCL_INVALID_ARGUMENT, "null communicator");
  if (d.algo == ALGO_DEFAULT_NCCL || d.algo == ALGO_AUTO) d.algo = select_algo(c, d.coll, d.count * (size_t)dtype_size(d.dtype), &d.k);
  piccl_comm* cs[1] = {c};
  return run(cs, 1, &d, (cudaStream_t)stream);
}

int piccl_allreduce(piccl_comm_t* c, const void* send, void* recv, size_t count, int dtype, int op, int algo, int k, void* stream) {
  return one(c, CallDesc{COLL_ALLREDUCE, send, recv, count, dtype, op, 0, (Algo)algo, k}, stream);
}
int piccl_allgather(piccl_comm_t* c, const void* send, void* recv, size_t sendcount, int dtype, int algo, int k, void* stream) {
  return one(c, CallDesc{COLL_ALLGATHER, send, recv, sendcount, dtype, 0, 0, (Algo)algo, k}, stream);
}
int piccl_reduce_scatter(piccl_comm_t* c, const void* send, void* recv, size_t recvcount, int dtype, int op, int algo, int k, void* stream) {
  return one(c, CallDesc{COLL_REDUCE_SCATTER, send, recv, recvcount, dtype, op, 0, (Algo)algo, k}, stream);
}
int piccl_reduce(piccl_comm_t* c, const void* send, void* recv, size_t count, int dtype, int op, int root, int algo, int k, void* stream) {
  return one(c, CallDesc{COLL_REDUCE, send, recv, count, dtype, op, root, (Algo)algo, k}, stream);
}
int piccl_broadcast(piccl_comm_t* c, const void* send, void* recv, size_t count, int dtype, int root, int algo, int k, void* stream) {
  return one(c, CallDesc{COLL_BROADCAST, send, recv, count, dtype, 0, root, (Algo)algo, k}, stream);
}

int piccl_group_collective(piccl_comm_t** comms, int ncomms, int coll, const void* const* send, void* const* recv,
                           size_t count, int dtype, int op, int root, int algo, int k, void* stream) {
  if (!comms || ncomms < 1 || ncomms > kMaxVRanks) return fail(PICCL_INVALID_ARGUMENT, "bad group size %d", ncomms);
  CallDesc d[kMaxVRanks];
  Algo al = (Algo)algo;
  if (al == ALGO_DEFAULT_NCCL || al == ALGO_AUTO) al = select_algo(comms[0], (Coll)coll, count * (size_t)dtype_size(dtype), &k);
  for (int i = 0; i < ncomms; i++) d[i] = CallDesc{(Coll)coll, send[i], recv[i], count, dtype, op, root, al, k};
  return run(comms, ncomms, d, (cudaStream_t)stream);
}

int piccl_test_unmatched_wait(piccl_comm_t* c, int timeout_ms, void* stream) {
  if (!c || !c->connected) return fail(PICCL_INVALID_USAGE, "communicator is not connected");
  DevGuard g(c->device);
  // one action: receive 16 bytes from the next rank (or from myself), which never sends
  Program p; p.rank = c->rank; p.nranks = c->nranks;
  Action a; a.n_recv = 1; a.recv_peer[0] = (uint8_t)((c->rank + 1) % c->nranks); a.dst_buf = BUF_SCRATCH; a.dst_off = 0; a.count = 16;
  p.actions.push_back(a);
  ProgEntry e;
  int rc = upload_program(c, p, (cudaStream_t)stream, e); if (rc) return rc;
  c->cache.emplace(ProgKey{-1, 0, 0, 0, 1, 0, (long long)c->cache.size(), 0}, e);
  KernelArgs ka; memset(&ka, 0, sizeof ka);
  ka.n_vrank = 1; ka.n_cta = 1; ka.elem_size = 1; ka.scale = 1.f; ka.timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
  ka.r[0].ctx = c->d_ctx; ka.r[0].actions = e.dev; ka.r[0].n_actions = 1;
  void* args[] = {&ka};
  CUDA_TRY(cudaLaunchKernel((const void*)exec_copy_kernel(), dim3(1), dim3(c->cfg.block_size), args, 0, (cudaStream_t)stream));
  return PICCL_OK;
}

}  // extern "C"
