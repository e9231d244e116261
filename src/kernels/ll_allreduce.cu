// Low-latency all-reduce for small messages and the exchange-type algorithms
// (RD / RM / PRD / PRM): every 16-byte line carries 8 bytes of payload and two
// copies of the call's epoch, written with one store, so a receiver that sees
// both flags has the data — no fence, no separate counter, no credit
// round trip.  A rank pushes its current value to all partners of the step,
// then polls the lines its partners pushed, reduces in rank order and moves on;
// every thread owns the same lines in all steps, so the kernel needs no barrier.
//
// Slot reuse is safe with two buffers (epoch parity) because each step is a
// symmetric exchange: a partner can only write epoch e+2 into a slot after it
// finished call e+1, which needed my data of call e+1, which I send after I
// finished reading call e.
// The reference runs these steps as ncclSend/ncclRecv groups plus a reduce
// kernel per step (src/coll/allreduce.c:282-614).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "exec_impl.cuh"

namespace piccl {

constexpr int kLLLinesPerThread = 4;

template <typename T> struct LLLine {
  static constexpr int E = 8 / sizeof(T);
  union U { uint2 v; T t[E]; };
};

template <typename T, int OP>
__global__ void __launch_bounds__(kLLBlock) ll_allreduce_kernel(const LLArgs a) {
  typedef typename AccOf<T>::type A;
  constexpr int E = LLLine<T>::E;
  const int vr = blockIdx.x / a.n_cta, cta = blockIdx.x % a.n_cta;
  RankCtx* __restrict__ ctx = a.r[vr].ctx;
  const T* in = static_cast<const T*>(a.r[vr].in);
  T* out = static_cast<T*>(a.r[vr].out);
  const int rank = ctx->rank, nranks = ctx->nranks;
  const long long ll_off = ctx->ll_off, slot_bytes = ctx->ll_slot_bytes;
  __shared__ char* s_heap[kMaxRanks];
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

#define LL_ROW(T) {ll_allreduce_kernel<T, 0>, ll_allreduce_kernel<T, 1>, ll_allreduce_kernel<T, 2>, ll_allreduce_kernel<T, 3>}
static LLKernelFn g_ll_table[DT_COUNT][4] = {LL_ROW(int8_t), LL_ROW(uint8_t), LL_ROW(int32_t), LL_ROW(uint32_t), LL_ROW(long long), LL_ROW(unsigned long long),
                                             LL_ROW(__half), LL_ROW(float), LL_ROW(double), LL_ROW(__nv_bfloat16)};

LLKernelFn ll_kernel_for(int dtype, int op) {
  if (dtype < 0 || dtype >= DT_COUNT || op < 0 || op > 3) return nullptr;
  return g_ll_table[dtype][op];
}
int ll_lines_per_cta() { return kLLBlock * kLLLinesPerThread; }

}  // namespace piccl
