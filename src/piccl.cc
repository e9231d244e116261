// LD_PRELOAD interposer: exports the NCCL entry points and hands each
// collective either to the fused executor or to the real NCCL.
//
// Reference behaviour kept (src/piccl.c): the load banner (:202), the
// PICCL_<COLL>_ALGO / PICCL_<COLL>_K environment (:241-308), "algorithm unset or
// unknown -> real NCCL" (:53-57,87-90,113-116,140-143,166-169), in-place
// conventions, stream-ordered asynchronous calls.
// Differences:
//  * real symbols are resolved lazily with dlsym(RTLD_NEXT) at first use, never by a
//    dlopen in a constructor (reference :206-211): a preloaded constructor that opens
//    "libnccl.so" pins whichever build the loader finds first and breaks applications
//    that ship their own NCCL (PyTorch).  Nothing links against libnccl.
//  * per-communicator state is created lazily on the first eligible collective, so it
//    works for communicators made by ncclCommInitRankConfig / Split / InitAll as well
//    (the reference only hooks ncclCommInitRank, :181-189).
//  * return codes are real; collectives inside an application ncclGroupStart/End pair,
//    during stream capture before the communicator is set up, with custom reduction
//    operators or unsupported types go to the real NCCL.
//  * the set-up of a communicator is itself a collective (handles travel over the real
//    NCCL), so whether and when it runs depends only on what is the same on every rank:
//    it is started by the first intercepted collective of ANY kind, count and type
//    outside a group and outside a stream capture, as soon as any algorithm variable is
//    set; whether that very call then runs here or in NCCL is decided afterwards.
//  * ncclCommFinalize / Split / Shrink / InitRankConfig / InitAll are hooked so that the registry never
//    keeps state for a communicator handle that NCCL has given away again.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <atomic>
#include <nccl.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <unistd.h>
#include "include/piccl.h"
#include "kernels/exec.cuh"
#include "runtime/comm.h"
#include "runtime/env.h"

using namespace piccl;

// ------------------------------------------------------------------ real NCCL
namespace {

void* real_sym(const char* name) {
  void* p = dlsym(RTLD_NEXT, name);
  if (p) return p;
  static void* handle = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    handle = dlopen("libnccl.so.2", RTLD_LAZY | RTLD_GLOBAL);
    if (!handle) handle = dlopen("libnccl.so", RTLD_LAZY | RTLD_GLOBAL);
    if (!handle) fprintf(stderr, "[PICCL] no NCCL library found: %s\n", dlerror());
  });
  return handle ? dlsym(handle, name) : nullptr;
}

#define REAL(name) \
  static auto real_##name = reinterpret_cast<decltype(&name)>(real_sym(#name)); \
  if (!real_##name) { fprintf(stderr, "[PICCL] real %s not found\n", #name); return ncclSystemError; }

struct ShimComm {
  piccl_comm_t* pc = nullptr;
  bool tried = false, usable = false;
  int rank = -1, nranks = 0;
  std::mutex mu;
};

std::mutex g_mu;
std::map<ncclComm_t, ShimComm*> g_comms;
thread_local int g_group_depth = 0;
std::atomic<unsigned long long> g_passthrough[COLL_COUNT], g_native[COLL_COUNT];

ShimComm* shim_of(ncclComm_t comm) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_comms.find(comm);
  if (it != g_comms.end()) return it->second;
  ShimComm* s = new ShimComm();
  g_comms[comm] = s;
  return s;
}

void drop(ncclComm_t comm) {
  ShimComm* s = nullptr;
  { std::lock_guard<std::mutex> l(g_mu); auto it = g_comms.find(comm); if (it != g_comms.end()) { s = it->second; g_comms.erase(it); } }
  if (s) { if (s->pc) piccl_comm_destroy(s->pc); delete s; }
}

// Collective set-up over the application's communicator: every rank publishes its heap
// handle with a real ncclAllGather on a private stream, then a second round agrees on
// whether everybody managed to map everybody.  Any failure anywhere => all ranks use NCCL.
bool bootstrap(ShimComm* s, ncclComm_t comm) {
  static auto real_count = reinterpret_cast<decltype(&ncclCommCount)>(real_sym("ncclCommCount"));
  static auto real_rank = reinterpret_cast<decltype(&ncclCommUserRank)>(real_sym("ncclCommUserRank"));
  static auto real_dev = reinterpret_cast<decltype(&ncclCommCuDevice)>(real_sym("ncclCommCuDevice"));
  static auto real_ag = reinterpret_cast<decltype(&ncclAllGather)>(real_sym("ncclAllGather"));
  if (!real_count || !real_rank || !real_dev || !real_ag) return false;
  int n = 0, r = -1, dev = -1;
  if (real_count(comm, &n) != ncclSuccess || real_rank(comm, &r) != ncclSuccess || real_dev(comm, &dev) != ncclSuccess) return false;
  s->rank = r; s->nranks = n;
  if (n < 2 || n > kMaxRanks) { log_msg(1, "communicator with %d ranks: NCCL is used", n); return false; }
  int prev = -1; cudaGetDevice(&prev); if (prev != dev) cudaSetDevice(dev);
  bool ok = false;
  cudaStream_t st = nullptr; char* dbuf = nullptr;
  piccl_handle_t* all = (piccl_handle_t*)calloc(n, sizeof(piccl_handle_t));
  do {
    if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) break;
    if (cudaMalloc(&dbuf, (size_t)n * sizeof(piccl_handle_t)) != cudaSuccess) break;
    piccl_handle_t mine; memset(&mine, 0, sizeof mine);
    piccl_comm_t* pc = nullptr;
    bool created = piccl_comm_create(r, n, dev, nullptr, &pc) == PICCL_OK && piccl_comm_local_handle(pc, &mine) == PICCL_OK;
    if (!created) memset(&mine, 0, sizeof mine);            // an all-zero blob tells the peers
    cudaMemcpyAsync(dbuf + (size_t)r * sizeof mine, &mine, sizeof mine, cudaMemcpyHostToDevice, st);
    if (real_ag(dbuf + (size_t)r * sizeof mine, dbuf, sizeof mine, ncclChar, comm, st) != ncclSuccess) { if (pc) piccl_comm_destroy(pc); break; }
    cudaMemcpyAsync(all, dbuf, (size_t)n * sizeof mine, cudaMemcpyDeviceToHost, st);
    if (cudaStreamSynchronize(st) != cudaSuccess) { if (pc) piccl_comm_destroy(pc); break; }
    char good = created && piccl_comm_connect(pc, all) == PICCL_OK ? 1 : 0;
    // second exchange: one byte per rank
    cudaMemcpyAsync(dbuf + r, &good, 1, cudaMemcpyHostToDevice, st);
    if (real_ag(dbuf + r, dbuf, 1, ncclChar, comm, st) != ncclSuccess) { if (pc) piccl_comm_destroy(pc); break; }
    char flags[kMaxRanks];
    cudaMemcpyAsync(flags, dbuf, n, cudaMemcpyDeviceToHost, st);
    if (cudaStreamSynchronize(st) != cudaSuccess) { if (pc) piccl_comm_destroy(pc); break; }
    bool all_good = true; for (int i = 0; i < n; i++) all_good &= flags[i] == 1;
    if (!all_good) { log_msg(1, "rank %d: peer memory not available on every rank (%s): NCCL is used", r, piccl_last_error()); if (pc) piccl_comm_destroy(pc); break; }
    s->pc = pc; ok = true;
  } while (0);
  if (dbuf) cudaFree(dbuf);
  if (st) cudaStreamDestroy(st);
  free(all);
  cudaGetLastError();
  if (prev != dev && prev >= 0) cudaSetDevice(prev);
  return ok;
}

bool any_algorithm_set() {
  const Env& e = env();
  for (int c = 0; c < COLL_COUNT; c++) if (e.algo[c] != ALGO_DEFAULT_NCCL) return true;
  return false;
}

// Decides whether this call runs natively; sets up the communicator on first use.
piccl_comm_t* native_comm(Coll coll, ncclComm_t comm, cudaStream_t stream, size_t count, ncclDataType_t dt, int op, Algo* algo, int* k) {
  const Env& e = env();
  *algo = e.algo[coll]; *k = e.k[coll];
  if (!any_algorithm_set()) return nullptr;                             // the reference's default path: nothing is ever set up
  if (g_group_depth > 0) return nullptr;
  ShimComm* s = shim_of(comm);
  std::lock_guard<std::mutex> l(s->mu);
  if (!s->tried) {
    // Every rank reaches this point with the same call of the same communicator, whatever the call's count, type or operator.
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    cudaError_t ce = cudaStreamIsCapturing(stream, &cs);
    if (ce != cudaSuccess) {
      cudaGetLastError();
      s->tried = true; s->usable = false;
      log_msg(1, "communicator %p: no usable CUDA device (%s) at the first intercepted call (%s, count %zu): NCCL is used", (void*)comm, cudaGetErrorString(ce), coll_name(coll), count);
      return nullptr;
    }
    if (cs != cudaStreamCaptureStatusNone) return nullptr;              // set up at the first call outside a capture
    s->tried = true;
    s->usable = bootstrap(s, comm);
    log_msg(1, "communicator %p rank %d/%d: %s (set up at the first intercepted call: %s, count %zu)", (void*)comm, s->rank, s->nranks,
            s->usable ? "fused executor ready" : "using NCCL", coll_name(coll), count);
  }
  if (!s->usable) return nullptr;
  // what this particular call needs
  if (*algo == ALGO_DEFAULT_NCCL || count == 0) return nullptr;
  if (!dtype_size((int)dt)) return nullptr;                              // fp8 and future types
  const bool reducing = coll == COLL_ALLREDUCE || coll == COLL_REDUCE || coll == COLL_REDUCE_SCATTER;
  if (reducing) {
    if (op < 0 || op > 4) return nullptr;                                // ncclRedOpCreatePreMulSum handles
    if (op == 4 && !(dt == ncclFloat32 || dt == ncclFloat16 || dt == ncclBfloat16 || dt == ncclFloat64)) return nullptr;
  }
  return s->pc;
}

ncclResult_t to_nccl(int rc) {
  switch (rc) {
    case PICCL_OK: return ncclSuccess;
    case PICCL_CUDA_ERROR: return ncclUnhandledCudaError;
    case PICCL_INVALID_ARGUMENT: return ncclInvalidArgument;
    case PICCL_INVALID_USAGE: return ncclInvalidUsage;
    case PICCL_REMOTE_ERROR: return ncclRemoteError;
    case PICCL_SYSTEM_ERROR: return ncclSystemError;
    default: return ncclInternalError;
  }
}

__attribute__((constructor)) void piccl_loaded() {
  fprintf(stderr, "[PICCL] loaded (PID %d).\n", (int)getpid());
  const Env& e = env();
  static const char* cn[COLL_COUNT] = {"ALLGATHER", "ALLREDUCE", "BROADCAST", "REDUCE", "REDUCE_SCATTER"};
  if (e.log_level >= 1)
    for (int c = 0; c < COLL_COUNT; c++) fprintf(stderr, "[PICCL] %s_ALGO=%s K=%d\n", cn[c], algo_name(e.algo[c]), e.k[c]);
}

__attribute__((destructor)) void piccl_unloaded() {
  if (env().log_level >= 1)
    for (int c = 0; c < COLL_COUNT; c++)
      if (g_native[c] || g_passthrough[c]) fprintf(stderr, "[PICCL %d] %s: %llu fused, %llu passed to NCCL\n", (int)getpid(), coll_name((Coll)c), g_native[c].load(), g_passthrough[c].load());
}

}  // namespace

// ------------------------------------------------------------------ exported NCCL ABI
extern "C" {

ncclResult_t ncclAllReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream) {
  Algo algo; int k;
  if (piccl_comm_t* pc = native_comm(COLL_ALLREDUCE, comm, stream, count, datatype, (int)op, &algo, &k)) {
    int rc = piccl_allreduce(pc, sendbuff, recvbuff, count, (int)datatype, (int)op, (int)algo, k, stream);
    if (rc != PICCL_UNSUPPORTED) { g_native[COLL_ALLREDUCE]++; return to_nccl(rc); }
  }
  g_passthrough[COLL_ALLREDUCE]++;
  REAL(ncclAllReduce);
  return real_ncclAllReduce(sendbuff, recvbuff, count, datatype, op, comm, stream);
}

ncclResult_t ncclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount, ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream) {
  Algo algo; int k;
  if (piccl_comm_t* pc = native_comm(COLL_ALLGATHER, comm, stream, sendcount, datatype, 0, &algo, &k)) {
    int rc = piccl_allgather(pc, sendbuff, recvbuff, sendcount, (int)datatype, (int)algo, k, stream);
    if (rc != PICCL_UNSUPPORTED) { g_native[COLL_ALLGATHER]++; return to_nccl(rc); }
  }
  g_passthrough[COLL_ALLGATHER]++;
  REAL(ncclAllGather);
  return real_ncclAllGather(sendbuff, recvbuff, sendcount, datatype, comm, stream);
}

ncclResult_t ncclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream) {
  Algo algo; int k;
  if (piccl_comm_t* pc = native_comm(COLL_REDUCE_SCATTER, comm, stream, recvcount, datatype, (int)op, &algo, &k)) {
    int rc = piccl_reduce_scatter(pc, sendbuff, recvbuff, recvcount, (int)datatype, (int)op, (int)algo, k, stream);
    if (rc != PICCL_UNSUPPORTED) { g_native[COLL_REDUCE_SCATTER]++; return to_nccl(rc); }
  }
  g_passthrough[COLL_REDUCE_SCATTER]++;
  REAL(ncclReduceScatter);
  return real_ncclReduceScatter(sendbuff, recvbuff, recvcount, datatype, op, comm, stream);
}

ncclResult_t ncclReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, int root, ncclComm_t comm, cudaStream_t stream) {
  Algo algo; int k;
  if (piccl_comm_t* pc = native_comm(COLL_REDUCE, comm, stream, count, datatype, (int)op, &algo, &k)) {
    int rc = piccl_reduce(pc, sendbuff, recvbuff, count, (int)datatype, (int)op, root, (int)algo, k, stream);
    if (rc != PICCL_UNSUPPORTED) { g_native[COLL_REDUCE]++; return to_nccl(rc); }
  }
  g_passthrough[COLL_REDUCE]++;
  REAL(ncclReduce);
  return real_ncclReduce(sendbuff, recvbuff, count, datatype, op, root, comm, stream);
}

ncclResult_t ncclBroadcast(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream) {
  Algo algo; int k;
  if (piccl_comm_t* pc = native_comm(COLL_BROADCAST, comm, stream, count, datatype, 0, &algo, &k)) {
    int rc = piccl_broadcast(pc, sendbuff, recvbuff, count, (int)datatype, root, (int)algo, k, stream);
    if (rc != PICCL_UNSUPPORTED) { g_native[COLL_BROADCAST]++; return to_nccl(rc); }
  }
  g_passthrough[COLL_BROADCAST]++;
  REAL(ncclBroadcast);
  return real_ncclBroadcast(sendbuff, recvbuff, count, datatype, root, comm, stream);
}

// legacy in-place broadcast
ncclResult_t ncclBcast(void* buff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream) {
  return ncclBroadcast(buff, buff, count, datatype, root, comm, stream);
}

// Communicator creation: per-communicator state is made lazily, at the first collective.  A handle that NCCL hands out may be
// the address of a communicator that was freed earlier without passing through a hook: whatever the registry still holds for
// it belongs to that dead communicator and goes away.
ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId commId, int rank) {
  REAL(ncclCommInitRank);
  ncclResult_t rc = real_ncclCommInitRank(comm, nranks, commId, rank);
  if (rc == ncclSuccess && comm && *comm) drop(*comm);
  return rc;
}

ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId commId, int rank, ncclConfig_t* config) {
  REAL(ncclCommInitRankConfig);
  ncclResult_t rc = real_ncclCommInitRankConfig(comm, nranks, commId, rank, config);
  if ((rc == ncclSuccess || rc == ncclInProgress) && comm && *comm) drop(*comm);
  return rc;
}

ncclResult_t ncclCommInitAll(ncclComm_t* comms, int ndev, const int* devlist) {
  REAL(ncclCommInitAll);
  ncclResult_t rc = real_ncclCommInitAll(comms, ndev, devlist);
  if (rc == ncclSuccess && comms) for (int i = 0; i < ndev; i++) if (comms[i]) drop(comms[i]);
  return rc;
}

ncclResult_t ncclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm, ncclConfig_t* config) {
  REAL(ncclCommSplit);
  ncclResult_t rc = real_ncclCommSplit(comm, color, key, newcomm, config);
  if ((rc == ncclSuccess || rc == ncclInProgress) && newcomm && *newcomm) drop(*newcomm);
  return rc;
}

ncclResult_t ncclCommShrink(ncclComm_t comm, int* excludeRanksList, int excludeRanksCount, ncclComm_t* newcomm, ncclConfig_t* config, int shrinkFlags) {
  REAL(ncclCommShrink);
  ncclResult_t rc = real_ncclCommShrink(comm, excludeRanksList, excludeRanksCount, newcomm, config, shrinkFlags);
  if ((rc == ncclSuccess || rc == ncclInProgress) && newcomm && *newcomm) drop(*newcomm);
  return rc;
}

// After ncclCommFinalize a communicator takes no more collectives: its heap and window go now, while the peers are still there.
ncclResult_t ncclCommFinalize(ncclComm_t comm) {
  drop(comm);
  REAL(ncclCommFinalize);
  return real_ncclCommFinalize(comm);
}

ncclResult_t ncclCommDestroy(ncclComm_t comm) {
  drop(comm);
  REAL(ncclCommDestroy);
  return real_ncclCommDestroy(comm);
}

ncclResult_t ncclCommAbort(ncclComm_t comm) {
  { std::lock_guard<std::mutex> l(g_mu); auto it = g_comms.find(comm); if (it != g_comms.end() && it->second->pc) piccl_comm_abort(it->second->pc); }
  drop(comm);
  REAL(ncclCommAbort);
  return real_ncclCommAbort(comm);
}

ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* asyncError) {
  REAL(ncclCommGetAsyncError);
  ncclResult_t rc = real_ncclCommGetAsyncError(comm, asyncError);
  if (rc == ncclSuccess && asyncError && *asyncError == ncclSuccess) {
    std::lock_guard<std::mutex> l(g_mu);
    auto it = g_comms.find(comm);
    if (it != g_comms.end() && it->second->pc) { piccl_status_t st; piccl_comm_status(it->second->pc, &st); if (st.aborted) *asyncError = ncclSystemError; }
  }
  return rc;
}

ncclResult_t ncclGroupStart() {
  REAL(ncclGroupStart);
  ncclResult_t rc = real_ncclGroupStart();
  if (rc == ncclSuccess) g_group_depth++;
  return rc;
}

ncclResult_t ncclGroupEnd() {
  REAL(ncclGroupEnd);
  if (g_group_depth > 0) g_group_depth--;
  return real_ncclGroupEnd();
}

// Counters of the shim itself (calls run by the fused executor / handed to NCCL).
void piccl_shim_counters(unsigned long long* native, unsigned long long* passthrough) {
  for (int c = 0; c < COLL_COUNT; c++) { if (native) native[c] = g_native[c].load(); if (passthrough) passthrough[c] = g_passthrough[c].load(); }
}

}  // extern "C"
