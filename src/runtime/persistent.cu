// Persistent launcher for small all-reduces (PICCL_LAUNCH=persistent).
//
// Instead of one kernel launch per collective, a resident "server" kernel of one
// CTA per rank waits for a doorbell.  A call becomes a single batch of stream memory
// operations on the caller's stream: write the call descriptor (buffers, count, type, epoch)
// and the doorbell value into device memory, then wait until the server has written the
// matching completion value.  Stream order is therefore kept exactly as with a launch.
//
// The server never stays resident without bound: after PICCL_PERSIST_IDLE_US without work it
// leaves, and the next call starts it again.  Leaving and posting can race, so they use a
// two-sided handshake through pinned host memory: the host publishes `posted` BEFORE it looks at
// `exiting`; the server raises `exiting`, fences, and re-reads `posted` BEFORE it leaves.  At
// least one side sees the other.  A doorbell that does not come within the communicator's time
// limit although a call was posted makes the server release the waiting stream (completion value
// written), mark the communicator aborted and leave — a stream never waits for a dead server.
//
// Only the low-latency path is served (exchange-type algorithms, <= 8 KiB, fp32 / bf16 / fp16 /
// int32); everything else takes the direct launch.  The reference has no counterpart.
#include <cuda.h>
#include <cuda_runtime.h>
#include <atomic>
#include <chrono>
#include <cstring>
#include <thread>
#include "../kernels/ll_impl.cuh"
#include "comm.h"

namespace piccl {

struct PDesc { unsigned long long in, out, meta; unsigned epoch; unsigned pad; };   // meta: count | dtype << 40 | op << 48 | avg << 56
struct PHost {                           // pinned, mapped host memory
  volatile unsigned posted;              // last call the host has enqueued (written before `exiting` is read)
  volatile unsigned exiting;             // server: "about to leave"
  volatile unsigned alive;               // 1 from launch until the server has decided to leave for good
};
struct PServer {                         // device memory
  unsigned doorbell;                     // written by the stream: sequence number of the newest call
  unsigned done;                         // written by the server: newest completed call (the stream waits on it)
  unsigned cmd;                          // CTA 0 -> other CTAs: (seq << 1) | leave
  unsigned done_cta[kMaxVRanks];
  unsigned start_seq;                    // first sequence number this server instance will see is start_seq + 1
  unsigned long long idle_ns, stuck_ns;
  PHost* host;
  PDesc desc[kMaxVRanks];
  LLArgs tmpl;                           // peers tables, contexts, step count: fixed per server instance
};

__device__ __forceinline__ unsigned ld_acq_u32(const unsigned* p) { unsigned v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ void st_rel_u32(unsigned* p, unsigned v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }

template <typename T>
__device__ __forceinline__ void serve_ops(const LLArgs& a, int op, int vr, char** s_heap) {
  switch (op) {
    case 0: ll_allreduce_body<T, 0>(a, vr, 0, s_heap); break;
    case 1: ll_allreduce_body<T, 1>(a, vr, 0, s_heap); break;
    case 2: ll_allreduce_body<T, 2>(a, vr, 0, s_heap); break;
    default: ll_allreduce_body<T, 3>(a, vr, 0, s_heap); break;
  }
}

__global__ void __launch_bounds__(kLLBlock) ll_server_kernel(PServer* sv) {
  const int vr = blockIdx.x, tid = threadIdx.x;
  __shared__ char* s_heap[kMaxRanks];
  __shared__ LLArgs s_args;
  __shared__ unsigned s_cmd;
  for (int i = tid; i < (int)(sizeof(LLArgs) / 4); i += blockDim.x) reinterpret_cast<unsigned*>(&s_args)[i] = reinterpret_cast<const unsigned*>(&sv->tmpl)[i];
  __syncthreads();
  unsigned last = sv->start_seq;
  unsigned long long idle0 = globaltimer_ns();
  for (;;) {
    if (tid == 0) {
      unsigned cmd = 0;
      if (vr == 0) {
        for (unsigned it = 1;; it++) {
          const unsigned v = ld_acq_u32(&sv->doorbell);
          if (v != last) { cmd = (last + 1) << 1; break; }
          if ((it & 255u) == 0) {                      // host memory is far away: look rarely
            const unsigned long long now = globaltimer_ns();
            PHost* h = sv->host;
            const unsigned posted = h->posted;
            if (posted == last) {
              if (now - idle0 > sv->idle_ns) {
                // nothing outstanding: announce, fence, look again, then leave
                h->exiting = 1;
                asm volatile("fence.sc.sys;" ::: "memory");
                if (h->posted == last) { cmd = 1; break; }
                h->exiting = 0;
                asm volatile("fence.sc.sys;" ::: "memory");
                idle0 = now;
              }
            } else if (now - idle0 > sv->stuck_ns) {
              // a call was posted but its doorbell never came: release whoever waits and give up
              RankCtx* ctx = s_args.r[0].ctx;
              if (atomicCAS(ctx->abort_flag, 0, 1) == 0) { ctx->status->code = 4; ctx->status->rank = ctx->rank; __threadfence_system(); ctx->status->aborted = 1; }
              st_rel_u32(&sv->done, posted);
              h->exiting = 1;
              cmd = 1; break;
            }
          }
        }
        st_rel_u32(&sv->cmd, cmd);
      } else {
        unsigned long long t0 = globaltimer_ns();
        for (unsigned it = 1;; it++) {
          cmd = ld_acq_u32(&sv->cmd);
          if (cmd == 1 || (cmd >> 1) == last + 1) break;
          if ((it & 255u) == 0 && globaltimer_ns() - t0 > sv->stuck_ns + sv->idle_ns + 1000000000ull) { cmd = 1; break; }   // CTA 0 is gone
        }
      }
      s_cmd = cmd;
    }
    __syncthreads();
    const unsigned cmd = s_cmd;
    if (cmd & 1u) break;
    const unsigned seq = cmd >> 1;
    // ---- serve call `seq`
    if (tid == 0) {
      const PDesc d = sv->desc[vr];
      s_args.r[vr].in = reinterpret_cast<const void*>(d.in);
      s_args.r[vr].out = reinterpret_cast<void*>(d.out);
      s_args.count = (long long)(d.meta & 0xFFFFFFFFFFull);
      s_args.avg = (int)((d.meta >> 56) & 1);
      s_args.epoch = d.epoch;
      s_args.n_cta = 1;
    }
    __syncthreads();
    const int dtype = (int)((sv->desc[vr].meta >> 40) & 0xFF), op = (int)((sv->desc[vr].meta >> 48) & 0xFF);
    switch (dtype) {
      case DT_F32: serve_ops<float>(s_args, op, vr, s_heap); break;
      case DT_BF16: serve_ops<__nv_bfloat16>(s_args, op, vr, s_heap); break;
      case DT_F16: serve_ops<__half>(s_args, op, vr, s_heap); break;
      default: serve_ops<int32_t>(s_args, op, vr, s_heap); break;
    }
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      st_rel_u32(&sv->done_cta[vr], seq);
      if (vr == 0) {
        unsigned long long t0 = globaltimer_ns();
        for (int o = 1; o < (int)gridDim.x; o++)
          for (unsigned it = 1; ld_acq_u32(&sv->done_cta[o]) != seq; it++)
            if ((it & 255u) == 0 && globaltimer_ns() - t0 > sv->stuck_ns) break;
        st_rel_u32(&sv->done, seq);      // the caller's stream proceeds
      }
    }
    last = seq;
    idle0 = globaltimer_ns();
  }
  __syncthreads();
  if (vr == 0 && tid == 0) { __threadfence_system(); sv->host->alive = 0; __threadfence_system(); }
}

// ------------------------------------------------------------------ host
typedef CUresult (*BatchMemOpFn)(CUstream, unsigned, CUstreamBatchMemOpParams*, unsigned);
static BatchMemOpFn batch_fn() {
  static BatchMemOpFn fn = nullptr; static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr; cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamBatchMemOp", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (BatchMemOpFn)p;
  }
  return fn;
}

struct PersistState {
  PServer* dev = nullptr; PHost* host = nullptr; cudaStream_t stream = nullptr;
  unsigned seq = 0; int algo = -1, k = 0, n = 0; bool failed = false;
};

void persist_destroy(piccl_comm* c) {
  PersistState* ps = static_cast<PersistState*>(c->persist);
  if (!ps) return;
  if (ps->stream) { cudaStreamSynchronize(ps->stream); cudaStreamDestroy(ps->stream); }   // the server leaves by itself after its idle limit
  if (ps->dev) cudaFree(ps->dev);
  if (ps->host) cudaFreeHost(ps->host);
  delete ps; c->persist = nullptr;
}

static bool start_server(piccl_comm** cs, int n, PersistState* ps, const LLArgs& tmpl) {
  PServer h; memset(&h, 0, sizeof h);
  h.doorbell = ps->seq; h.done = ps->seq; h.cmd = 0; h.start_seq = ps->seq;
  h.idle_ns = (unsigned long long)env().persist_idle_us * 1000ull;
  h.stuck_ns = (unsigned long long)cs[0]->cfg.timeout_ms * 1000000ull;
  PHost* hd = nullptr; cudaHostGetDevicePointer((void**)&hd, ps->host, 0);
  h.host = hd; h.tmpl = tmpl;
  if (cudaMemcpyAsync(ps->dev, &h, sizeof h, cudaMemcpyHostToDevice, ps->stream) != cudaSuccess) return false;
  if (cudaStreamSynchronize(ps->stream) != cudaSuccess) return false;
  ps->host->exiting = 0; ps->host->alive = 1;
  std::atomic_thread_fence(std::memory_order_seq_cst);
  void* args[] = {&ps->dev};
  cudaError_t e = n > 1 ? cudaLaunchCooperativeKernel((const void*)ll_server_kernel, dim3(n), dim3(kLLBlock), args, 0, ps->stream)
                        : cudaLaunchKernel((const void*)ll_server_kernel, dim3(1), dim3(kLLBlock), args, 0, ps->stream);
  if (e != cudaSuccess) { ps->host->alive = 0; cudaGetLastError(); return false; }
  return true;
}

// Returns PICCL_OK if the call was enqueued through the server, PICCL_UNSUPPORTED if the caller should launch directly.
int persist_allreduce(piccl_comm** cs, int n, const LLArgs& la, const void* const* in, void* const* out, long long count, int dtype, int op, int avg,
                      int algo, int k, cudaStream_t stream) {
  if (!(dtype == DT_F32 || dtype == DT_BF16 || dtype == DT_F16 || dtype == DT_I32) || la.n_cta != 1) return PICCL_UNSUPPORTED;
  BatchMemOpFn bm = batch_fn();
  if (!bm) return PICCL_UNSUPPORTED;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) { cudaGetLastError(); return PICCL_UNSUPPORTED; }
  piccl_comm* c0 = cs[0];
  PersistState* ps = static_cast<PersistState*>(c0->persist);
  if (!ps) {
    ps = new PersistState(); c0->persist = ps;
    if (cudaMalloc(&ps->dev, sizeof(PServer)) != cudaSuccess || cudaHostAlloc((void**)&ps->host, sizeof(PHost), cudaHostAllocMapped) != cudaSuccess ||
        cudaStreamCreateWithFlags(&ps->stream, cudaStreamNonBlocking) != cudaSuccess) { ps->failed = true; cudaGetLastError(); }
    else memset((void*)ps->host, 0, sizeof(PHost));
  }
  if (ps->failed) return PICCL_UNSUPPORTED;
  // one server instance serves one (algorithm, k, group); a change waits for the old one to leave
  const bool config_changed = ps->algo != algo || ps->k != k || ps->n != n;
  const unsigned seq = ps->seq + 1;
  ps->host->posted = seq;
  std::atomic_thread_fence(std::memory_order_seq_cst);
  bool need_start = !ps->host->alive;
  if (!need_start && (ps->host->exiting || config_changed)) {
    if (config_changed) { ps->host->posted = ps->seq; std::atomic_thread_fence(std::memory_order_seq_cst); }   // let it idle out
    const auto t0 = std::chrono::steady_clock::now();
    while (ps->host->alive && (ps->host->exiting || config_changed)) {
      if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(5)) { ps->failed = true; return PICCL_UNSUPPORTED; }
      std::this_thread::yield();
    }
    if (config_changed) { ps->host->posted = seq; std::atomic_thread_fence(std::memory_order_seq_cst); }
    need_start = !ps->host->alive;
  }
  if (need_start) {
    cudaStreamSynchronize(ps->stream);                     // the previous instance has fully left
    LLArgs tmpl = la; tmpl.n_cta = 1; tmpl.n_vrank = n; tmpl.scale = 1.0f / (float)cs[0]->nranks;   // used only by avg calls
    ps->algo = algo; ps->k = k; ps->n = n;
    if (!start_server(cs, n, ps, tmpl)) { ps->failed = true; return PICCL_UNSUPPORTED; }
  }
  // descriptor + doorbell + completion wait, one batch on the caller's stream
  CUstreamBatchMemOpParams ops[4 * kMaxVRanks + 2]; memset(ops, 0, sizeof ops);
  int m = 0;
  auto w64 = [&](void* addr, unsigned long long v) { ops[m].operation = CU_STREAM_MEM_OP_WRITE_VALUE_64; ops[m].writeValue.address = (CUdeviceptr)(uintptr_t)addr; ops[m].writeValue.value64 = v; ops[m].writeValue.flags = CU_STREAM_WRITE_VALUE_DEFAULT; m++; };
  auto w32 = [&](void* addr, unsigned v) { ops[m].operation = CU_STREAM_MEM_OP_WRITE_VALUE_32; ops[m].writeValue.address = (CUdeviceptr)(uintptr_t)addr; ops[m].writeValue.value = v; ops[m].writeValue.flags = CU_STREAM_WRITE_VALUE_DEFAULT; m++; };
  const unsigned long long meta = (unsigned long long)count | ((unsigned long long)dtype << 40) | ((unsigned long long)op << 48) | ((unsigned long long)(avg ? 1 : 0) << 56);
  for (int i = 0; i < n; i++) {
    w64(&ps->dev->desc[i].in, (unsigned long long)(uintptr_t)in[i]);
    w64(&ps->dev->desc[i].out, (unsigned long long)(uintptr_t)out[i]);
    w64(&ps->dev->desc[i].meta, meta);
    w32(&ps->dev->desc[i].epoch, la.epoch);
  }
  w32(&ps->dev->doorbell, seq);
  ops[m].operation = CU_STREAM_MEM_OP_WAIT_VALUE_32; ops[m].waitValue.address = (CUdeviceptr)(uintptr_t)&ps->dev->done; ops[m].waitValue.value = seq;
  ops[m].waitValue.flags = CU_STREAM_WAIT_VALUE_GEQ; m++;
  if (bm((CUstream)stream, (unsigned)m, ops, 0) != CUDA_SUCCESS) {
    // nothing was enqueued: take the call back so that the server can idle out
    ps->host->posted = ps->seq; std::atomic_thread_fence(std::memory_order_seq_cst);
    ps->failed = true;
    return PICCL_UNSUPPORTED;
  }
  ps->seq = seq;
  return PICCL_OK;
}

}  // namespace piccl
