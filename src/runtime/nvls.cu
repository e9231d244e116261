// Host side of the in-switch all-reduce (kernel: kernels/nvls_allreduce.cu): the
// multicast window of a communicator.  Opt-in (PICCL_NVLS=1); the algorithm name is NVLS.
//
// Set-up, inside piccl_comm_connect once every rank's handle is known:
//   rank 0 creates the multicast object and exports it as a file descriptor; the
//   descriptor travels to the peers over a Unix socket (fdshare.h); every rank adds
//   its device; barrier; every rank creates device memory of the window size, binds it
//   to the object at offset 0, maps its own copy (uc) and the multicast view (mc),
//   clears the barrier counters; barrier.  A failure on any rank makes all ranks drop
//   the window again (the barriers carry the verdict) and the communicator works
//   without it: NVLS requests then run the ring.
// The driver entry points are fetched at run time, so the library links against the
// CUDA runtime only.  The reference has no counterpart.
#include <cuda.h>
#include <cuda_runtime.h>
#include <fcntl.h>
#include <unistd.h>
#include <algorithm>
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
  unsigned long long* d_bar = nullptr;
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
  if (s->d_bar) { cudaFree(s->d_bar); s->d_bar = nullptr; }
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

void nvls_destroy(piccl_comm* c) {
  if (!c->nvls) return;
  NvlsState* s = static_cast<NvlsState*>(c->nvls);
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
  s->max_cta = std::max(1, std::min(e.nvls_cta, kNvlsMaxCta));
  s->slot_bytes = std::max<long long>(1, e.nvls_chunk_kb) * 1024;
  s->slot_bytes = (s->slot_bytes + 16LL * n - 1) / (16LL * n) * (16LL * n);
  size_t want = (size_t)kNvlsFlagBytes + (size_t)s->max_cta * (size_t)s->slot_bytes;
  CUmulticastObjectProp mp; memset(&mp, 0, sizeof mp);
  mp.numDevices = (unsigned)n; mp.size = want; mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemAllocationProp ap; memset(&ap, 0, sizeof ap);
  ap.type = CU_MEM_ALLOCATION_TYPE_PINNED; ap.location.type = CU_MEM_LOCATION_TYPE_DEVICE; ap.location.id = c->device;
  ap.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t g_mc = 0, g_mem = 0;
  // PICCL_NVLS_GRAN=min: the smallest granularity the driver accepts instead of the recommended one (512 MiB per window on B200)
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
    if (ce == cudaSuccess) ce = cudaMalloc(&s->d_bar, kNvlsBarCounts * sizeof(unsigned long long));
    if (ce == cudaSuccess) ce = cudaMemset(s->d_bar, 0, kNvlsBarCounts * sizeof(unsigned long long));
    if (ce == cudaSuccess) ce = cudaDeviceSynchronize();
    if (ce != cudaSuccess) { cudaGetLastError(); ok = false; snprintf(why, sizeof why, "clearing the window: %s", cudaGetErrorString(ce)); }
  }
  all = ok;
  if (talk && !fdshare_barrier(sh, ok, &all)) all = false;
  if (ok && !all) { ok = false; snprintf(why, sizeof why, "another rank could not bind its window"); }
  fdshare_close(sh);
  if (!ok) {
    log_msg(1, "rank %d: no multicast window (%s); NVLS requests run the ring", c->rank, why);
    teardown(s);
    return;
  }
  s->ready = true;
  log_msg(1, "rank %d: multicast window of %.1f MiB (%d slots of %lld KiB)", c->rank, s->win / 1048576.0, s->max_cta, s->slot_bytes >> 10);
}

int nvls_allreduce(piccl_comm* c, const void* in, void* out, size_t count, int dtype, bool avg, cudaStream_t stream) {
  if (!nvls_ready(c) || !nvls_dtype_supported(dtype)) return PICCL_UNSUPPORTED;
  NvlsState* s = static_cast<NvlsState*>(c->nvls);
  const long long bytes = (long long)count * dtype_size(dtype);
  const long long unit = 16LL * c->nranks;
  NvlsArgs a; memset(&a, 0, sizeof a);
  a.uc = (char*)s->uc_va; a.mc = (char*)s->mc_va; a.in = in; a.out = out; a.bytes = bytes;
  // mid-size messages are spread over all CTAs instead of filling a few slots
  long long chunk = (bytes + s->max_cta - 1) / s->max_cta;
  chunk = std::max<long long>(chunk, 16384);
  chunk = (chunk + unit - 1) / unit * unit;
  a.pipelined = env().nvls_pipe ? 1 : 0;
  const int max_cta = a.pipelined ? std::min(s->max_cta, kNvlsPipeMaxCta) : s->max_cta;
  const long long room = a.pipelined ? (s->slot_bytes / 2) / unit * unit : s->slot_bytes;      // a chunk fills a slot, or half of it
  if (room < unit) return PICCL_UNSUPPORTED;
  a.chunk_bytes = std::min(chunk, room);
  a.slot_bytes = s->slot_bytes;
  const long long nchunks = (bytes + a.chunk_bytes - 1) / a.chunk_bytes;
  a.rank = c->rank; a.nranks = c->nranks; a.n_cta = (int)std::min<long long>(nchunks, max_cta);
  a.avg = avg ? 1 : 0; a.scale = avg ? 1.0f / (float)c->nranks : 1.0f;
  a.timeout_ns = (unsigned long long)c->cfg.timeout_ms * 1000000ull;
  a.bar_count = s->d_bar; a.abort_flag = c->d_abort; a.status = c->d_status;
  cudaError_t e = (cudaError_t)nvls_launch(a, dtype, stream);
  if (e != cudaSuccess) return fail(PICCL_CUDA_ERROR, "in-switch all-reduce launch failed: %s", cudaGetErrorString(e));
  return PICCL_OK;
}

}  // namespace piccl
