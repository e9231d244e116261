// Host side of the in-switch collectives (kernels: kernels/nvls_coll.cu): the multicast
// window of a communicator and the launch geometry.  PICCL_NVLS=0 turns the window off;
// the algorithm name is NVLS and AUTO picks it for large messages when a window exists.
//
// Set-up, inside piccl_comm_connect once every rank's handle is known:
//   rank 0 creates the multicast object and exports it as a file descriptor; the
//   descriptor travels to the peers over a Unix socket (fdshare.h); every rank adds
//   its device; barrier; every rank creates device memory of the window size, binds it
//   to the object at offset 0, maps its own copy (uc) and the multicast view (mc),
//   clears the counters; barrier.  A failure on any rank makes all ranks drop
//   the window again (the barriers carry the verdict) and the communicator works
//   without it: NVLS requests then run the peer-to-peer schedules.
// When all ranks of a communicator are virtual ranks of one process on one device the window is
// plain device memory and the kernels emulate the switch (tests on one GPU).
// The driver entry points are fetched at run time, so the library links against the
// CUDA runtime only.  The reference has no counterpart.
#include <cuda.h>
#include <cuda_runtime.h>
#include <fcntl.h>
#include <unistd.h>
#include <algorithm>
#include <cstdio>
#include <cstring>
#include "comm.h"
#include "fdshare.h"
#include "nvls.h"
#include "../kernels/nvls.cuh"

namespace piccl {

namespace {

struct Drv {
  decltype(&cuCtxGetDevice) CtxGetDevice = nullptr;
  decltype(&cuDeviceGetAttribute) DeviceGetAttribute = nullptr;
  decltype(&cuMulticastCreate) MulticastCreate = nullptr;
  decltype(&cuMulticastGetGranularity) MulticastGetGranularity = nullptr;
  decltype(&cuMulticastAddDevice) MulticastAddDevice = nullptr;
  decltype(&cuMulticastBindMem) MulticastBindMem = nullptr;
  decltype(&cuMulticastUnbind) MulticastUnbind = nullptr;
  decltype(&cuMemCreate) MemCreate = nullptr;
  decltype(&cuMemRelease) MemRelease = nullptr;
  decltype(&cuMemGetAllocationGranularity) MemGetAllocationGranularity = nullptr;
  decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
  decltype(&cuMemAddressFree) MemAddressFree = nullptr;
  decltype(&cuMemMap) MemMap = nullptr;
  decltype(&cuMemUnmap) MemUnmap = nullptr;
  decltype(&cuMemSetAccess) MemSetAccess = nullptr;
  decltype(&cuMemExportToShareableHandle) MemExportToShareableHandle = nullptr;
  decltype(&cuMemImportFromShareableHandle) MemImportFromShareableHandle = nullptr;
  bool ok = false;
};

template <typename F> bool resolve_one(const char* name, F& fn) {
  void* p = nullptr; cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) { cudaGetLastError(); return false; }
  fn = reinterpret_cast<F>(p);
  return true;
}

const Drv& drv() {
  static Drv d; static bool tried = false;
  if (!tried) {
    tried = true;
    bool ok = true;
#define R(x) ok &= resolve_one("cu" #x, d.x)
    R(CtxGetDevice); R(DeviceGetAttribute); R(MulticastCreate); R(MulticastGetGranularity); R(MulticastAddDevice); R(MulticastBindMem); R(MulticastUnbind);
    R(MemCreate); R(MemRelease); R(MemGetAllocationGranularity); R(MemAddressReserve); R(MemAddressFree); R(MemMap); R(MemUnmap); R(MemSetAccess);
    R(MemExportToShareableHandle); R(MemImportFromShareableHandle);
#undef R
    d.ok = ok;
  }
  return d;
}

struct NvlsState {
  bool ready = false;
  CUdevice dev = 0;
  CUmemGenericAllocationHandle mc = 0, mem = 0;
  bool have_mc = false, have_mem = false, added = false, bound = false, uc_mapped = false, mc_mapped = false;
  CUdeviceptr uc_va = 0, mc_va = 0;
  size_t win = 0;
  long long slot_bytes = 0; int max_cta = 0;
  unsigned long long* d_used = nullptr;      // uses of every part of every slot so far (kernels/nvls.cuh)
  int depth = 2;                             // parts per slot
  unsigned long long* d_prof = nullptr;      // PICCL_NVLS_PROFILE=1: phase times summed by the kernels
  bool emulated = false; char* emu_win = nullptr;
};

void teardown(NvlsState* s) {
  const Drv& d = drv();
  if (s->mc_mapped) { d.MemUnmap(s->mc_va, s->win); s->mc_mapped = false; }
  if (s->mc_va) { d.MemAddressFree(s->mc_va, s->win); s->mc_va = 0; }
  if (s->bound) { d.MulticastUnbind(s->mc, s->dev, 0, s->win); s->bound = false; }
  if (s->uc_mapped) { d.MemUnmap(s->uc_va, s->win); s->uc_mapped = false; }
  if (s->uc_va) { d.MemAddressFree(s->uc_va, s->win); s->uc_va = 0; }
  if (s->have_mem) { d.MemRelease(s->mem); s->have_mem = false; }
  if (s->have_mc) { d.MemRelease(s->mc); s->have_mc = false; }
  if (s->d_used) { cudaFree(s->d_used); s->d_used = nullptr; }
  if (s->d_prof) { cudaFree(s->d_prof); s->d_prof = nullptr; }
  if (s->emu_win) { cudaFree(s->emu_win); s->emu_win = nullptr; }
  s->ready = false;
}

const char* cu_name(CUresult r) {
  switch (r) {
    case CUDA_SUCCESS: return "success";
    case CUDA_ERROR_NOT_SUPPORTED: return "not supported";
    case CUDA_ERROR_NOT_PERMITTED: return "not permitted";
    case CUDA_ERROR_OUT_OF_MEMORY: return "out of memory";
    case CUDA_ERROR_INVALID_VALUE: return "invalid value";
    case CUDA_ERROR_INVALID_DEVICE: return "invalid device";
    default: return "driver error";
  }
}

}  // namespace

bool nvls_device_capable(int device) {
  const Drv& d = drv();
  if (!d.ok) return false;
  int cur = -1; cudaGetDevice(&cur);
  if (cur != device) cudaSetDevice(device);
  cudaFree(0);                                   // the primary context exists and is current
  CUdevice dev; int v = 0;
  bool ok = d.CtxGetDevice(&dev) == CUDA_SUCCESS && d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) == CUDA_SUCCESS && v != 0;
  if (cur != device && cur >= 0) cudaSetDevice(cur);
  return ok;
}

bool nvls_ready(const piccl_comm* c) { return c->nvls && static_cast<const NvlsState*>(c->nvls)->ready; }
bool nvls_emulated(const piccl_comm* c) { return nvls_ready(c) && static_cast<const NvlsState*>(c->nvls)->emulated; }

static void window_geometry(const piccl_comm* c, NvlsState* s, bool emulated) {
  const Env& e = env();
  s->max_cta = std::max(1, std::min(c->cfg.nvls_cta > 0 ? c->cfg.nvls_cta : e.nvls_cta, emulated ? 32 : kNvlsMaxCta));
  s->depth = std::max(2, std::min(e.nvls_depth, kNvlsMaxDepth));
  const long long part = (std::max<long long>(1, e.nvls_chunk_kb) * 1024 + 255) / 256 * 256;     // one part = one chunk of at most PICCL_NVLS_CHUNK_KB
  s->slot_bytes = s->depth * part;
}

// All ranks are virtual ranks of this process on this device: plain memory, the kernels loop over the ranks' windows.
void nvls_setup_emulated(piccl_comm* c) {
  NvlsState* s = new NvlsState();
  c->nvls = s;
  window_geometry(c, s, true);
  s->emulated = true;
  s->win = (size_t)kNvlsFlagBytes + (size_t)s->max_cta * (size_t)s->slot_bytes;
  cudaError_t ce = cudaMalloc(&s->emu_win, s->win);
  if (ce == cudaSuccess) ce = cudaMemset(s->emu_win, 0, kNvlsFlagBytes);
  if (ce == cudaSuccess) ce = cudaMalloc(&s->d_used, (size_t)kNvlsMaxCta * kNvlsUsedPerCta * sizeof(unsigned long long));
  if (ce == cudaSuccess) ce = cudaMemset(s->d_used, 0, (size_t)kNvlsMaxCta * kNvlsUsedPerCta * sizeof(unsigned long long));
  if (ce == cudaSuccess) ce = cudaDeviceSynchronize();
  if (ce != cudaSuccess) { cudaGetLastError(); log_msg(1, "rank %d: no emulated window (%s)", c->rank, cudaGetErrorString(ce)); teardown(s); return; }
  s->uc_va = (CUdeviceptr)(uintptr_t)s->emu_win;
  s->ready = true;
}

// Before the window goes away: arrivals of the peers for this rank's last uses of each part of a slot may still be on their
// way (they are the last thing a peer's kernel does).  Waits on the host, with a limit, until every CONSUMED counter shows
// all ranks; nothing writes into the window after that.
static void quiesce(piccl_comm* c, NvlsState* s) {
  if (!s->ready || s->emulated || !s->d_used) return;
  const size_t nu = (size_t)kNvlsMaxCta * kNvlsUsedPerCta;
  std::vector<unsigned long long> used(nu), flags(kNvlsFlagBytes / sizeof(unsigned long long));
  if (cudaMemcpy(used.data(), s->d_used, nu * sizeof(unsigned long long), cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return; }
  for (int tries = 0; tries < 200; tries++) {
    if (cudaMemcpy(flags.data(), (const void*)s->uc_va, kNvlsFlagBytes, cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return; }
    bool done = true;
    for (int b = 0; b < kNvlsMaxCta && done; b++)
      for (int h = 0; h < kNvlsMaxDepth; h++) {
        const unsigned long long want = used[(size_t)b * kNvlsUsedPerCta + h] * (unsigned long long)c->nranks;
        const unsigned long long have = flags[(size_t)(((b * kNvlsMaxDepth + h) * 3 + NVC_CONSUMED) * 128) / sizeof(unsigned long long)];
        if (have < want) { done = false; break; }
      }
    if (done) return;
    usleep(5000);
  }
  log_msg(1, "rank %d: peers did not finish with the multicast window within 1 s", c->rank);
}

void nvls_destroy(piccl_comm* c) {
  if (!c->nvls) return;
  NvlsState* s = static_cast<NvlsState*>(c->nvls);
  if (s->d_prof) {
    // where thread 0 of the CTAs spent its time, per chunk, averaged over every CTA of every in-switch call of this communicator
    unsigned long long h[kNvlsProfSlots] = {0};
    if (cudaMemcpy(h, s->d_prof, sizeof h, cudaMemcpyDeviceToHost) == cudaSuccess && h[NVP_CHUNKS]) {
      const double ch = (double)h[NVP_CHUNKS];
      fprintf(stderr, "[PICCL %d] rank %d in-switch profile: %llu CTAs, %llu chunks; per chunk us: fill %.1f wait-filled %.1f switch %.1f wait-reduced %.1f out %.1f wait-consumed %.1f; per CTA us: %.1f\n",
              (int)getpid(), c->rank, h[NVP_CTAS], h[NVP_CHUNKS], h[NVP_FILL] / ch / 1e3, h[NVP_WAIT_FILLED] / ch / 1e3, h[NVP_SWITCH] / ch / 1e3, h[NVP_WAIT_REDUCED] / ch / 1e3,
              h[NVP_OUT] / ch / 1e3, h[NVP_WAIT_CONSUMED] / ch / 1e3, h[NVP_TOTAL] / (double)h[NVP_CTAS] / 1e3);
    } else cudaGetLastError();
  }
  quiesce(c, s);
  teardown(s);
  delete s;
  c->nvls = nullptr;
}

// Caller: piccl_comm_connect, device current, every rank of the communicator calls it (or none does).
void nvls_setup(piccl_comm* c, int root_pid, unsigned long long root_id) {
  const Drv& d = drv();
  const Env& e = env();
  NvlsState* s = new NvlsState();
  c->nvls = s;
  const int n = c->nranks;
  bool ok = d.ok;
  char why[160] = "driver entry points missing";
#define STEP(expr) do { if (ok) { CUresult r_ = (expr); if (r_ != CUDA_SUCCESS) { ok = false; snprintf(why, sizeof why, "%s: %s (%d)", #expr, cu_name(r_), (int)r_); } } } while (0)
  cudaFree(0);
  STEP(d.CtxGetDevice(&s->dev));

  // window geometry: the same arithmetic on every rank
  window_geometry(c, s, false);
  size_t want = (size_t)kNvlsFlagBytes + (size_t)s->max_cta * (size_t)s->slot_bytes;
  CUmulticastObjectProp mp; memset(&mp, 0, sizeof mp);
  mp.numDevices = (unsigned)n; mp.size = want; mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemAllocationProp ap; memset(&ap, 0, sizeof ap);
  ap.type = CU_MEM_ALLOCATION_TYPE_PINNED; ap.location.type = CU_MEM_LOCATION_TYPE_DEVICE; ap.location.id = c->device;
  ap.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t g_mc = 0, g_mem = 0;
  // the smallest granularity the driver accepts (a 66 MiB window with the defaults on B200); PICCL_NVLS_GRAN=recommended: the
  // recommended one, which makes every window 512 MiB
  const bool gran_min = e.nvls_gran_min != 0;
  STEP(d.MulticastGetGranularity(&g_mc, &mp, gran_min ? CU_MULTICAST_GRANULARITY_MINIMUM : CU_MULTICAST_GRANULARITY_RECOMMENDED));
  STEP(d.MemGetAllocationGranularity(&g_mem, &ap, gran_min ? CU_MEM_ALLOC_GRANULARITY_MINIMUM : CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  size_t gran = std::max<size_t>(std::max(g_mc, g_mem), 4096);
  s->win = (want + gran - 1) / gran * gran;
  mp.size = s->win;

  // the multicast object: created by rank 0, imported by the others
  int fd = -1;
  if (c->rank == 0) {
    STEP(d.MulticastCreate(&s->mc, &mp));
    if (ok) s->have_mc = true;
    if (n > 1) {
      STEP(d.MemExportToShareableHandle(&fd, s->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
      if (!ok || fd < 0) fd = open("/dev/null", O_RDONLY | O_CLOEXEC);   // the peers still get an answer; the vote below says no
    }
  }
  FdShare sh; sh.rank = c->rank; sh.nranks = n; sh.timeout_ms = std::max(1000, std::min(c->cfg.timeout_ms, 30000));
  char name[96]; snprintf(name, sizeof name, "piccl-nvls-%d-%llx", root_pid, root_id);
  int got = -1;
  bool talk = fdshare_open(sh, name, fd, &got);
  if (!talk) { ok = false; snprintf(why, sizeof why, "descriptor exchange: %s", sh.error.c_str()); }
  if (c->rank != 0 && talk) {
    STEP(d.MemImportFromShareableHandle(&s->mc, (void*)(uintptr_t)got, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
    if (ok) s->have_mc = true;
  }
  if (c->rank == 0 ? fd >= 0 : got >= 0) close(c->rank == 0 ? fd : got);
  STEP(d.MulticastAddDevice(s->mc, s->dev));
  if (ok) s->added = true;
  bool all = ok;
  if (talk && !fdshare_barrier(sh, ok, &all)) all = false;
  if (ok && !all) { ok = false; snprintf(why, sizeof why, "another rank could not join the multicast object"); }

  // the window: physical memory, bound to the object, two mappings
  STEP(d.MemCreate(&s->mem, s->win, &ap, 0));
  if (ok) s->have_mem = true;
  STEP(d.MulticastBindMem(s->mc, 0, s->mem, 0, s->win, 0));
  if (ok) s->bound = true;
  CUmemAccessDesc acc; memset(&acc, 0, sizeof acc);
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE; acc.location.id = c->device; acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  STEP(d.MemAddressReserve(&s->uc_va, s->win, gran, 0, 0));
  STEP(d.MemMap(s->uc_va, s->win, 0, s->mem, 0));
  if (ok) s->uc_mapped = true;
  STEP(d.MemSetAccess(s->uc_va, s->win, &acc, 1));
  STEP(d.MemAddressReserve(&s->mc_va, s->win, gran, 0, 0));
  STEP(d.MemMap(s->mc_va, s->win, 0, s->mc, 0));
  if (ok) s->mc_mapped = true;
  STEP(d.MemSetAccess(s->mc_va, s->win, &acc, 1));
#undef STEP
  if (ok) {
    cudaError_t ce = cudaMemset((void*)s->uc_va, 0, kNvlsFlagBytes);
    if (ce == cudaSuccess) ce = cudaMalloc(&s->d_used, (size_t)kNvlsMaxCta * kNvlsUsedPerCta * sizeof(unsigned long long));
    if (ce == cudaSuccess) ce = cudaMemset(s->d_used, 0, (size_t)kNvlsMaxCta * kNvlsUsedPerCta * sizeof(unsigned long long));
    if (ce == cudaSuccess) ce = cudaDeviceSynchronize();
    if (ce != cudaSuccess) { cudaGetLastError(); ok = false; snprintf(why, sizeof why, "clearing the window: %s", cudaGetErrorString(ce)); }
  }
  all = ok;
  if (talk && !fdshare_barrier(sh, ok, &all)) all = false;
  if (ok && !all) { ok = false; snprintf(why, sizeof why, "another rank could not bind its window"); }
  fdshare_close(sh);
  if (!ok) {
    log_msg(1, "rank %d: no multicast window (%s); NVLS requests run the peer-to-peer schedules", c->rank, why);
    teardown(s);
    return;
  }
  s->ready = true;
  log_msg(1, "rank %d: multicast window of %.1f MiB (%d slots of %d x %lld KiB)", c->rank, s->win / 1048576.0, s->max_cta, s->depth, (s->slot_bytes / s->depth) >> 10);
}

// What the kernels take: sum of fp32, sum / max / min of fp16 and bf16 (what the switch can reduce), any type for the
// collectives that only move data; messages (blocks) of a multiple of 16 bytes except for all-reduce, which stages through
// typed copies.  Only what is the same on every rank may decide (never a buffer address): all ranks must take the same path.
bool nvls_eligible(const piccl_comm* c, int coll, int dtype, int op, size_t count) {
  if (!nvls_ready(c) || count == 0) return false;
  const long long es = dtype_size(dtype);
  if (!es) return false;
  const bool reducing = coll == COLL_ALLREDUCE || coll == COLL_REDUCE || coll == COLL_REDUCE_SCATTER;
  if (reducing && !nvls_kernel_exists(dtype, op)) return false;
  const long long bytes = (long long)count * es;
  if (bytes >= (1LL << 40)) return false;
  if (coll == COLL_ALLREDUCE) return true;
  return (bytes & 15) == 0;
}

// Enqueues one collective on `n` communicators: n == 1, the normal case, or all virtual ranks of an emulated group.
// op: 0 sum, 2 max, 3 min (avg: sum with `avg` set).  count: elements of the message, or of one rank's block for
// all-gather / reduce-scatter.  Callers check nvls_eligible first.
int nvls_collective(piccl_comm** comms, int n, int coll, const void* const* in, void* const* out, size_t count, int dtype, int op, bool avg, int root, cudaStream_t stream) {
  piccl_comm* c0 = comms[0];
  NvlsState* s0 = static_cast<NvlsState*>(c0->nvls);
  const bool emu = s0->emulated;
  if (emu ? n != c0->nranks : n != 1) return PICCL_UNSUPPORTED;
  const int nr = c0->nranks;
  const long long es = dtype_size(dtype), bytes = (long long)count * es, half = s0->slot_bytes / s0->depth;
  const bool blocks = coll == COLL_ALLGATHER || coll == COLL_REDUCE_SCATTER;      // the message is one block per rank
  const bool reducing = coll == COLL_ALLREDUCE || coll == COLL_REDUCE || coll == COLL_REDUCE_SCATTER;
  NvlsArgs a; memset(&a, 0, sizeof a);
  a.coll = coll; a.nranks = nr; a.n_vrank = n; a.avg = (avg && reducing) ? 1 : 0; a.root = root; a.scale = a.avg ? 1.0f / (float)nr : 1.0f;
  a.bytes = bytes; a.slot_bytes = s0->slot_bytes; a.depth = s0->depth; a.use_bulk = env().nvls_bulk ? 1 : 0; a.strict_fences = env().nvls_strict_fences ? 1 : 0;

  a.timeout_ns = (unsigned long long)c0->cfg.timeout_ms * 1000000ull;
  // chunks: spread a mid-size message over all CTAs (at least PICCL_NVLS_MIN_KB of traffic per chunk), fill the parts of the slots for a large one
  const long long unit = coll == COLL_ALLREDUCE ? 16LL * nr : 16;
  const long long room = blocks ? (half / nr) / 16 * 16 : half / unit * unit;       // largest chunk (per rank block for all-gather / reduce-scatter)
  if (room < unit) return PICCL_UNSUPPORTED;
  a.sub_stride = blocks ? room : 0;
  int max_cta = s0->max_cta;
  if (emu) max_cta = std::max(1, std::min(max_cta, nvls_max_resident_ctas(true) / n));
  const long long total = blocks ? bytes * nr : bytes;
  const long long min_chunk = std::max<long long>(1, env().nvls_min_kb) * 1024;
  const long long want_cta = std::max<long long>(1, std::min<long long>((total + min_chunk - 1) / min_chunk, max_cta));
  long long chunk = (bytes + want_cta - 1) / want_cta;
  chunk = (chunk + unit - 1) / unit * unit;
  a.chunk_bytes = std::min(chunk, room);
  const long long nchunks = (bytes + a.chunk_bytes - 1) / a.chunk_bytes;
  a.n_cta = (int)std::min<long long>(nchunks, max_cta);
  // The switch stage of an all-reduce in three groups that take the chunks in turn: pays from four ranks on (a rank's share of a
  // chunk is then small enough for a third of the threads) and when every group gets chunks to work on.  Measured on 8 GPUs: 714 vs
  // 632 GB/s at 1 GiB; the stages of the other collectives that talk to the switch lose with it (all-gather 476 vs 542 GB/s).
  a.n_sub = 1;
  if (env().nvls_sub > 0) a.n_sub = env().nvls_sub >= 3 ? 3 : 1;
  else if (coll == COLL_ALLREDUCE && nr >= 4 && nchunks >= 3LL * a.n_cta) a.n_sub = 3;
  for (int i = 0; i < n; i++) {
    piccl_comm* c = comms[i];
    NvlsState* s = static_cast<NvlsState*>(c->nvls);
    if (!s || !s->ready || s->emulated != emu || s->slot_bytes != s0->slot_bytes || s->depth != s0->depth) return PICCL_UNSUPPORTED;
    NvlsRank& r = a.r[i];
    if (env().nvls_profile && !s->d_prof) {
      if (cudaMalloc(&s->d_prof, kNvlsProfSlots * sizeof(unsigned long long)) == cudaSuccess) cudaMemset(s->d_prof, 0, kNvlsProfSlots * sizeof(unsigned long long));
      else { cudaGetLastError(); s->d_prof = nullptr; }
    }
    r.prof = s->d_prof;
    r.uc = (char*)s->uc_va; r.mc = (char*)s->mc_va; r.in = in[i]; r.out = out[i]; r.used = s->d_used; r.abort_flag = c->d_abort; r.status = c->d_status; r.rank = c->rank;
  }
  // copy-only collectives run any instantiation
  const int kdt = reducing ? dtype : DT_F32, kop = reducing ? op : 0;
  cudaError_t e = (cudaError_t)nvls_launch(a, kdt, kop, emu, stream);
  if (e != cudaSuccess) return fail(PICCL_CUDA_ERROR, "in-switch %s launch failed: %s", coll_name((Coll)coll), cudaGetErrorString(e));
  return PICCL_OK;
}

}  // namespace piccl
