// Low-latency variant of the fused executor for small messages of ANY collective
// and algorithm: the same action programs, but FIFO entries are 16-byte lines of
// {4 B data, 4 B sequence, 4 B data, 4 B sequence} in a separate small FIFO.  A line
// is complete when both sequence words equal the entry's number, so the producer
// needs neither a fence nor a tail counter and the consumer polls the data itself.
// Slot reuse is guarded by a head counter the consumer advances with a plain
// store once its reads are done (the producer only looks at it when the ring of
// kLLFifoSlots entries is about to wrap).  Entry numbers never repeat for a slot,
// and the region is zero at start, so stale lines can never look complete.
#pragma once
#include "exec_impl.cuh"

namespace piccl {

template <typename T> struct LLUnit {
  static constexpr int E = 8 / sizeof(T);
  union U { uint2 v; T t[E]; };
};

template <typename T, int OP>
__global__ void __launch_bounds__(kLLBlock) exec_ll_kernel(const KernelArgs ka) {
  typedef typename AccOf<T>::type A;
  constexpr int E = LLUnit<T>::E;
  constexpr int esz = (int)sizeof(T);
  const int vr = blockIdx.x / ka.n_cta, cta = blockIdx.x % ka.n_cta;
  const LaunchRank& L = ka.r[vr];
  RankCtx* __restrict__ ctx = L.ctx;
  const int tid = threadIdx.x;

  __shared__ unsigned s_send_seq[kMaxRanks], s_recv_seq[kMaxRanks];
  __shared__ char* s_heap[kMaxRanks];
  __shared__ int s_fail, s_maxseg;

  const int rank = ctx->rank, nranks = ctx->nranks;
  const long long llf_off = ctx->llf_off, llf_head_off = ctx->llf_head_off, scratch_off = ctx->scratch_off;
  unsigned long long my_sent = 0, my_rcvd = 0;
  if (tid < nranks) { s_heap[tid] = ctx->heap[tid]; my_sent = ctx->sent_ll[tid * kLLFifoCta + cta]; my_rcvd = ctx->rcvd_ll[tid * kLLFifoCta + cta]; }
  if (tid == 0) { s_fail = 0; s_maxseg = 0; }
  __syncthreads();
  constexpr long long kPayload = kLLFifoSlotBytes / 2;
  const long long seg_elems = (kPayload / 16) * (16 / esz);
  {
    int m = 0;
    for (int ai = tid; ai < L.n_actions; ai += blockDim.x) m = max(m, slice_of(L.actions[ai].count, esz, cta, ka.n_cta, kPayload).nseg);
    if (m) atomicMax(&s_maxseg, m);
  }
  __syncthreads();
  const int maxseg = s_maxseg;
  char* const my_heap = s_heap[rank];
  WaitCtx w; w.ctx = ctx; w.timeout_ns = ka.timeout_ns; w.cta = cta;
  bool failed = false;
  unsigned long long t0 = 0;

  for (int seg = 0; seg < maxseg && !failed; seg++) {
    for (int ai = 0; ai < L.n_actions; ai++) {
      const Action ac = L.actions[ai];
      const Slice sl = slice_of(ac.count, esz, cta, ka.n_cta, kPayload);
      const long long lo = sl.lo + (long long)seg * seg_elems;
      if (lo >= sl.hi) continue;
      const long long hi = (lo + seg_elems < sl.hi) ? lo + seg_elems : sl.hi;
      const long long len = hi - lo;

      if (tid < nranks) {
        bool ok = true;
        w.action = ai; w.segment = seg;
        for (int j = 0; j < ac.n_send; j++) if (ac.send_peer[j] == tid) {
          s_send_seq[tid] = (unsigned)(my_sent + 1);
          if (my_sent + 1 > (unsigned long long)kLLFifoSlots)
            ok = wait_counter(reinterpret_cast<const unsigned long long*>(my_heap + llf_head_off + (long long)(tid * kLLFifoCta + cta) * kFlagStride),
                              my_sent + 1 - kLLFifoSlots, w, 1, tid);
        }
        for (int j = 0; j < ac.n_recv; j++) if (ac.recv_peer[j] == tid) s_recv_seq[tid] = (unsigned)(my_rcvd + 1);
        if (!ok) s_fail = 1;
      }
      __syncthreads();
      if (s_fail) { failed = true; break; }

      const bool has_src = ac.src_buf != BUF_NONE;
      const T* lsrc = nullptr; T* ldst = nullptr;
      if (has_src) lsrc = reinterpret_cast<const T*>(ac.src_buf == BUF_IN ? (const char*)L.in : ac.src_buf == BUF_OUT ? (const char*)L.out : my_heap + scratch_off) + ac.src_off + lo;
      if (ac.dst_buf != BUF_NONE) ldst = reinterpret_cast<T*>(ac.dst_buf == BUF_OUT ? (char*)L.out : my_heap + scratch_off) + ac.dst_off + lo;
      const bool do_scale = ka.avg && (ac.flags & ACT_SCALE_SRC) && has_src;
      const long long nunits = (len + E - 1) / E;

      for (long long u = tid; u < nunits && !failed; u += blockDim.x) {
        A acc[E];
        bool have = false;
        for (int j = 0; j <= ac.n_recv; j++) {
          if (j == ac.self_pos && has_src) {
#pragma unroll
            for (int e = 0; e < E; e++) {
              const long long idx = u * E + e;
              A x = A();
              if (idx < len) { x = Cvt<T>::up(lsrc[idx]); if (do_scale) x = scale_val<A>(x, ka.scale); }
              acc[e] = have ? red<OP, A>(acc[e], x) : x;
            }
            have = true;
          }
          if (j == ac.n_recv) break;
          const int p = ac.recv_peer[j];
          const unsigned seq = s_recv_seq[p];
          const char* src = my_heap + llf_off + ((long long)(p * kLLFifoCta + cta) * kLLFifoSlots + (seq - 1) % kLLFifoSlots) * kLLFifoSlotBytes + u * 16;
          uint4 line;
          for (unsigned spins = 1;; spins++) {
            line = ld_slot(src);
            if (line.y == seq && line.w == seq) break;
            if ((spins & 63u) == 0) {
              if (*(volatile int*)ctx->abort_flag) { failed = true; break; }
              unsigned long long now = globaltimer_ns();
              if (!t0) t0 = now;
              else if (now - t0 > ka.timeout_ns) {
                if (atomicCAS(ctx->abort_flag, 0, 1) == 0) {
                  piccl_status_t* st = ctx->status;
                  st->code = 2; st->rank = rank; st->cta = cta; st->action = ai; st->peer = p; st->segment = seg; st->want = seq; st->have = line.y;
                  __threadfence_system(); st->aborted = 1; __threadfence_system();
                }
                failed = true; break;
              }
            }
          }
          if (failed) break;
          typename LLUnit<T>::U un; un.v = make_uint2(line.x, line.z);
#pragma unroll
          for (int e = 0; e < E; e++) { A x = Cvt<T>::up(un.t[e]); acc[e] = have ? red<OP, A>(acc[e], x) : x; }
          have = true;
        }
        if (failed) break;
        typename LLUnit<T>::U out;
#pragma unroll
        for (int e = 0; e < E; e++) out.t[e] = Cvt<T>::down(acc[e]);
        if (ldst) {
#pragma unroll
          for (int e = 0; e < E; e++) { const long long idx = u * E + e; if (idx < len) ldst[idx] = out.t[e]; }
        }
        for (int j = 0; j < ac.n_send; j++) {
          const int p = ac.send_peer[j];
          const unsigned seq = s_send_seq[p];
          char* dst = s_heap[p] + llf_off + ((long long)(rank * kLLFifoCta + cta) * kLLFifoSlots + (seq - 1) % kLLFifoSlots) * kLLFifoSlotBytes + u * 16;
          asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(out.v.x), "r"(seq), "r"(out.v.y), "r"(seq) : "memory");
        }
      }
      if (failed) s_fail = 1;
      __syncthreads();
      if (s_fail) { failed = true; break; }

      if (tid < nranks) {
        for (int j = 0; j < ac.n_send; j++) if (ac.send_peer[j] == tid) my_sent++;
        for (int j = 0; j < ac.n_recv; j++) if (ac.recv_peer[j] == tid) {
          my_rcvd++;
          // the slot is read (its data went through registers): a plain store frees it for the producer
          *reinterpret_cast<volatile unsigned long long*>(s_heap[tid] + llf_head_off + (long long)(rank * kLLFifoCta + cta) * kFlagStride) = my_rcvd;
        }
      }
    }
  }
  if (tid < nranks) { ctx->sent_ll[tid * kLLFifoCta + cta] = my_sent; ctx->rcvd_ll[tid * kLLFifoCta + cta] = my_rcvd; }
}

}  // namespace piccl

#define PICCL_INSTANTIATE_EXEC(T, DT)                                                              \
  namespace piccl {                                                                                \
  ExecKernelFn exec_table_##DT[4] = {exec_kernel<T, 0, false>, exec_kernel<T, 1, false>, exec_kernel<T, 2, false>, exec_kernel<T, 3, false>}; \
  ExecKernelFn exec_defer_table_##DT[4] = {exec_kernel<T, 0, true>, exec_kernel<T, 1, true>, exec_kernel<T, 2, true>, exec_kernel<T, 3, true>}; \
  ExecKernelFn exec_ll_table_##DT[4] = {exec_ll_kernel<T, 0>, exec_ll_kernel<T, 1>, exec_ll_kernel<T, 2>, exec_ll_kernel<T, 3>}; \
  }
