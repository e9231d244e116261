// Device body of the low-latency all-reduce, shared by the directly launched
// kernel (ll_allreduce.cu) and the persistent server (runtime/persistent.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "exec_impl.cuh"

namespace piccl {

constexpr int kLLLinesPerThread = 4;

template <typename T> struct LLLine {
  static constexpr int E = 8 / sizeof(T);
  union U { uint2 v; T t[E]; };
};

// One CTA's share of a low-latency all-reduce.  `s_heap` is a shared-memory table the caller owns.
template <typename T, int OP>
__device__ __forceinline__ void ll_allreduce_body(const LLArgs& a, int vr, int cta, char** s_heap) {
  typedef typename AccOf<T>::type A;
  constexpr int E = LLLine<T>::E;
  RankCtx* __restrict__ ctx = a.r[vr].ctx;
  const T* in = static_cast<const T*>(a.r[vr].in);
  T* out = static_cast<T*>(a.r[vr].out);
  const int rank = ctx->rank, nranks = ctx->nranks;
  const long long ll_off = ctx->ll_off, slot_bytes = ctx->ll_slot_bytes;
  __syncthreads();                                   // previous user of s_heap is done
  if (threadIdx.x < nranks) s_heap[threadIdx.x] = ctx->heap[threadIdx.x];
  __syncthreads();
  char* const my_heap = s_heap[rank];
  const unsigned epoch = a.epoch;
  const int parity = epoch & 1;
  const long long nlines = (a.count + E - 1) / E;
  const long long stride = (long long)a.n_cta * blockDim.x;
  const long long first = (long long)cta * blockDim.x + threadIdx.x;

  A acc[kLLLinesPerThread][E];
#pragma unroll
  for (int j = 0; j < kLLLinesPerThread; j++) {
    const long long i = first + j * stride;
#pragma unroll
    for (int e = 0; e < E; e++) {
      const long long idx = i * E + e;
      A v = A();
      if (i < nlines && idx < a.count) { v = Cvt<T>::up(in[idx]); if (a.avg) v = scale_val<A>(v, a.scale); }
      acc[j][e] = v;
    }
  }

  unsigned long long t0 = 0;
  bool failed = false;
  for (int s = 0; s < a.nsteps && !failed; s++) {
    const int np = a.npeers[s];
    const long long step_base = ll_off + ((long long)(parity * kLLMaxSteps + s) * nranks) * slot_bytes;
    // push: my value, rounded to the element type exactly as the partners will see it
#pragma unroll
    for (int j = 0; j < kLLLinesPerThread; j++) {
      const long long i = first + j * stride;
      if (i < nlines) {
        typename LLLine<T>::U u;
#pragma unroll
        for (int e = 0; e < E; e++) { u.t[e] = Cvt<T>::down(acc[j][e]); acc[j][e] = Cvt<T>::up(u.t[e]); }
        const uint4 line = make_uint4(u.v.x, epoch, u.v.y, epoch);
        for (int p = 0; p < np; p++) {
          char* dst = s_heap[a.peers[vr][s][p]] + step_base + (long long)rank * slot_bytes + i * 16;
          asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(line.x), "r"(line.y), "r"(line.z), "r"(line.w) : "memory");
        }
      }
    }
    // pull and reduce in rank order (partners are listed in ascending rank; self_pos of them are below me)
#pragma unroll
    for (int j = 0; j < kLLLinesPerThread; j++) {
      const long long i = first + j * stride;
      if (i < nlines && !failed) {
        A mine[E], res[E];
#pragma unroll
        for (int e = 0; e < E; e++) mine[e] = acc[j][e];
        bool have = false;
        for (int p = 0; p <= np; p++) {
          if (p == a.self_pos[vr][s]) {
#pragma unroll
            for (int e = 0; e < E; e++) res[e] = have ? red<OP, A>(res[e], mine[e]) : mine[e];
            have = true;
          }
          if (p == np) break;
          const char* src = my_heap + step_base + (long long)a.peers[vr][s][p] * slot_bytes + i * 16;
          uint4 line;
          for (unsigned spins = 1;; spins++) {
            line = ld_slot(src);
            if (line.y == epoch && line.w == epoch) break;
            if ((spins & 63u) == 0) {
              if (*(volatile int*)ctx->abort_flag) { failed = true; break; }
              unsigned long long now = globaltimer_ns();
              if (!t0) t0 = now;
              else if (now - t0 > a.timeout_ns) {
                if (atomicCAS(ctx->abort_flag, 0, 1) == 0) {
                  piccl_status_t* st = ctx->status;
                  st->code = 2; st->rank = rank; st->cta = cta; st->action = s; st->peer = a.peers[vr][s][p]; st->segment = (int)i;
                  st->want = epoch; st->have = line.y;
                  __threadfence_system(); st->aborted = 1; __threadfence_system();
                }
                failed = true; break;
              }
            }
          }
          if (failed) break;
          typename LLLine<T>::U u; u.v = make_uint2(line.x, line.z);
#pragma unroll
          for (int e = 0; e < E; e++) { A x = Cvt<T>::up(u.t[e]); res[e] = have ? red<OP, A>(res[e], x) : x; }
          have = true;
        }
#pragma unroll
        for (int e = 0; e < E; e++) acc[j][e] = res[e];
      }
    }
  }
  if (failed) return;
#pragma unroll
  for (int j = 0; j < kLLLinesPerThread; j++) {
    const long long i = first + j * stride;
#pragma unroll
    for (int e = 0; e < E; e++) {
      const long long idx = i * E + e;
      if (i < nlines && idx < a.count) out[idx] = Cvt<T>::down(acc[j][e]);
    }
  }
}

}  // namespace piccl
