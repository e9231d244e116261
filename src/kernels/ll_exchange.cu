// Low-latency all-gather and reduce-scatter for small blocks: ONE exchange with every rank in ONE launch, data and
// flag in the same 16-byte line (8 bytes of payload and two copies of the call's epoch, written with one store), so a
// receiver that sees both flags has the data: no fence, no counter, no credit round trip.  The lines go to the slots
// [parity of the epoch][step 0][source rank] of the peers' heaps, the same slots and the same epoch sequence as the
// low-latency all-reduce (ll_allreduce.cu), which makes calls of the three kernels safe in any order: a rank can only
// write epoch e + 2 into a slot after it finished call e + 1, and every one of these calls needs data from EVERY
// other rank, which that rank sends after it finished reading call e.  (Broadcast and reduce move data in one
// direction only and have no such back pressure; they stay on the executor.)
// The reference runs an all-gather as n - 1 (ring) or log n (recursive) ncclSend/ncclRecv groups plus a permutation
// kernel (src/coll/allgather.c:3-123,233-288,517-570) and has no reduce-scatter (src/coll/reduce_scatter.c:3-29).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "ll_impl.cuh"

namespace piccl {

namespace {

constexpr int kLLXLines = 4;              // lines per thread and peer

// Polls one line until both flags show `epoch`.  false: gave up (time limit or abort); the status is recorded once.
__device__ __forceinline__ bool llx_poll(const char* src, unsigned epoch, RankCtx* ctx, unsigned long long timeout_ns, unsigned long long& t0, int cta, int peer,
                                         long long line_index, uint4& line) {
  for (unsigned spins = 1;; spins++) {
    line = ld_slot(src);
    if (line.y == epoch && line.w == epoch) return true;
    if ((spins & 63u) == 0) {
      if (*(volatile int*)ctx->abort_flag) return false;
      unsigned long long now = globaltimer_ns();
      if (!t0) t0 = now;
      else if (now - t0 > timeout_ns) {
        if (atomicCAS(ctx->abort_flag, 0, 1) == 0) {
          piccl_status_t* st = ctx->status;
          st->code = 2; st->rank = ctx->rank; st->cta = cta; st->action = 0; st->peer = peer; st->segment = (int)line_index;
          st->want = epoch; st->have = line.y;
          __threadfence_system(); st->aborted = 1; __threadfence_system();
        }
        return false;
      }
    }
  }
}

__device__ __forceinline__ void st_line(char* dst, unsigned lo, unsigned hi, unsigned epoch) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(lo), "r"(epoch), "r"(hi), "r"(epoch) : "memory");
}

// 8 bytes of a user buffer of which `valid` (1..8) exist; the buffer need not be aligned
__device__ __forceinline__ uint2 ld8(const char* p, int valid, bool aligned) {
  if (aligned && valid == 8) return *reinterpret_cast<const uint2*>(p);
  union { uint2 v; unsigned char b[8]; } u; u.v = make_uint2(0, 0);
  for (int k = 0; k < valid; k++) u.b[k] = reinterpret_cast<const unsigned char*>(p)[k];
  return u.v;
}
__device__ __forceinline__ void st8(char* p, uint2 v, int valid, bool aligned) {
  if (aligned && valid == 8) { *reinterpret_cast<uint2*>(p) = v; return; }
  union { uint2 v; unsigned char b[8]; } u; u.v = v;
  for (int k = 0; k < valid; k++) reinterpret_cast<unsigned char*>(p)[k] = u.b[k];
}

}  // namespace

// All-gather of `count` BYTES per rank.
__global__ void __launch_bounds__(kLLBlock) ll_allgather_kernel(const LLXArgs a) {
  __shared__ char* s_heap[kMaxRanks];
  const int vr = blockIdx.x / a.n_cta, cta = blockIdx.x % a.n_cta;
  RankCtx* __restrict__ ctx = a.r[vr].ctx;
  const char* in = static_cast<const char*>(a.r[vr].in);
  char* out = static_cast<char*>(a.r[vr].out);
  const int rank = ctx->rank, n = ctx->nranks;
  if (threadIdx.x < n) s_heap[threadIdx.x] = ctx->heap[threadIdx.x];
  __syncthreads();
  const unsigned epoch = a.epoch;
  const long long slot_bytes = ctx->ll_slot_bytes;
  const long long base = ctx->ll_off + ((long long)((epoch & 1) * kLLMaxSteps) * n) * slot_bytes;       // step 0 of this parity
  const long long bytes = a.count, nlines = (bytes + 7) / 8;
  const long long stride = (long long)a.n_cta * blockDim.x, first = (long long)cta * blockDim.x + threadIdx.x;
  const bool in_al = (reinterpret_cast<uintptr_t>(in) & 7) == 0, out_al = ((reinterpret_cast<uintptr_t>(out) | (uintptr_t)bytes) & 7) == 0;
  // push my block to every peer, nearest rank above me first, and put it into my own output
#pragma unroll
  for (int j = 0; j < kLLXLines; j++) {
    const long long i = first + j * stride;
    if (i < nlines) {
      const int valid = (int)(bytes - i * 8 < 8 ? bytes - i * 8 : 8);
      const uint2 v = ld8(in + i * 8, valid, in_al);
      for (int d = 1; d < n; d++) {
        const int p = (rank + d) % n;
        st_line(s_heap[p] + base + (long long)rank * slot_bytes + i * 16, v.x, v.y, epoch);
      }
      if (in != out + (long long)rank * bytes) st8(out + (long long)rank * bytes + i * 8, v, valid, out_al);
    }
  }
  // collect the others' blocks
  unsigned long long t0 = 0;
  for (int d = 1; d < n; d++) {
    const int q = (rank - d + n) % n;
    const char* slot = s_heap[rank] + base + (long long)q * slot_bytes;
#pragma unroll
    for (int j = 0; j < kLLXLines; j++) {
      const long long i = first + j * stride;
      if (i < nlines) {
        uint4 line;
        if (!llx_poll(slot + i * 16, epoch, ctx, a.timeout_ns, t0, cta, q, i, line)) return;
        const int valid = (int)(bytes - i * 8 < 8 ? bytes - i * 8 : 8);
        st8(out + (long long)q * bytes + i * 8, make_uint2(line.x, line.z), valid, out_al);
      }
    }
  }
}

// Reduce-scatter: rank r ends with the reduction over all ranks of block r (`count` elements) of their send buffers.
template <typename T, int OP>
__global__ void __launch_bounds__(kLLBlock) ll_reduce_scatter_kernel(const LLXArgs a) {
  typedef typename AccOf<T>::type A;
  constexpr int E = LLLine<T>::E;
  __shared__ char* s_heap[kMaxRanks];
  const int vr = blockIdx.x / a.n_cta, cta = blockIdx.x % a.n_cta;
  RankCtx* __restrict__ ctx = a.r[vr].ctx;
  const T* in = static_cast<const T*>(a.r[vr].in);
  T* out = static_cast<T*>(a.r[vr].out);
  const int rank = ctx->rank, n = ctx->nranks;
  if (threadIdx.x < n) s_heap[threadIdx.x] = ctx->heap[threadIdx.x];
  __syncthreads();
  const unsigned epoch = a.epoch;
  const long long slot_bytes = ctx->ll_slot_bytes;
  const long long base = ctx->ll_off + ((long long)((epoch & 1) * kLLMaxSteps) * n) * slot_bytes;
  const long long count = a.count, nlines = (count + E - 1) / E;
  const long long stride = (long long)a.n_cta * blockDim.x, first = (long long)cta * blockDim.x + threadIdx.x;
  // a line of block `blk` of my send buffer as the element type, scaled for avg, missing elements zero
  auto load_line = [&](int blk, long long i, typename LLLine<T>::U& u) {
#pragma unroll
    for (int e = 0; e < E; e++) {
      const long long idx = i * E + e;
      A v = A();
      if (idx < count) { v = Cvt<T>::up(in[(long long)blk * count + idx]); if (a.avg) v = scale_val<A>(v, a.scale); }
      u.t[e] = Cvt<T>::down(v);
    }
  };
  // push block p of my buffer to rank p
  for (int d = 1; d < n; d++) {
    const int p = (rank + d) % n;
#pragma unroll
    for (int j = 0; j < kLLXLines; j++) {
      const long long i = first + j * stride;
      if (i < nlines) {
        typename LLLine<T>::U u; load_line(p, i, u);
        st_line(s_heap[p] + base + (long long)rank * slot_bytes + i * 16, u.v.x, u.v.y, epoch);
      }
    }
  }
  // reduce block `rank` in rank order: contributions of the ranks below me, mine, the ranks above me
  unsigned long long t0 = 0;
#pragma unroll
  for (int j = 0; j < kLLXLines; j++) {
    const long long i = first + j * stride;
    if (i >= nlines) continue;
    A res[E];
    for (int q = 0; q < n; q++) {
      typename LLLine<T>::U u;
      if (q == rank) load_line(rank, i, u);
      else {
        uint4 line;
        if (!llx_poll(s_heap[rank] + base + (long long)q * slot_bytes + i * 16, epoch, ctx, a.timeout_ns, t0, cta, q, i, line)) return;
        u.v = make_uint2(line.x, line.z);
      }
#pragma unroll
      for (int e = 0; e < E; e++) { const A x = Cvt<T>::up(u.t[e]); res[e] = q == 0 ? x : red<OP, A>(res[e], x); }
    }
#pragma unroll
    for (int e = 0; e < E; e++) { const long long idx = i * E + e; if (idx < count) out[idx] = Cvt<T>::down(res[e]); }
  }
}

#define LLX_ROW(T) {ll_reduce_scatter_kernel<T, 0>, ll_reduce_scatter_kernel<T, 1>, ll_reduce_scatter_kernel<T, 2>, ll_reduce_scatter_kernel<T, 3>}
static LLXKernelFn g_llx_table[DT_COUNT][4] = {LLX_ROW(int8_t), LLX_ROW(uint8_t), LLX_ROW(int32_t), LLX_ROW(uint32_t), LLX_ROW(long long), LLX_ROW(unsigned long long),
                                               LLX_ROW(__half), LLX_ROW(float), LLX_ROW(double), LLX_ROW(__nv_bfloat16)};

LLXKernelFn llx_reduce_scatter_kernel_for(int dtype, int op) {
  if (dtype < 0 || dtype >= DT_COUNT || op < 0 || op > 3) return nullptr;
  return g_llx_table[dtype][op];
}
LLXKernelFn llx_allgather_kernel() { return ll_allgather_kernel; }
int llx_lines_per_cta() { return kLLBlock * kLLXLines; }

}  // namespace piccl
