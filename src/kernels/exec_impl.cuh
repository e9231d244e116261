// The fused collective executor: ONE kernel runs a whole collective.  Each CTA
// owns a fixed slice of every action; for each FIFO segment it walks the
// action program, and every action is a single pass
//     wait (bounded) -> load local + incoming slots -> reduce in registers ->
//     store local + peers' slots -> publish counters
// so reduction (reference: src/kernels/reduce_kernel.cu, one launch per step)
// and block placement (reference: src/kernels/permutation_kernel.cu) never
// exist as separate passes, and no ncclSend/ncclRecv is issued.
//
// Peer traffic is plain 16-byte stores into the peer's mapped heap (NVLink /
// NVSwitch P2P); ordering is fence.acq_rel.sys + st.release.sys on the
// producer and ld.acquire.sys on the consumer.  Every wait has a time limit;
// on expiry the CTA records where it gave up, raises the abort flag that all
// other waits poll, and the kernel returns.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "exec.cuh"
#include "../include/piccl_slice.h"

namespace piccl {

// ---------------------------------------------------------------- memory primitives
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// FIFO payload written by another GPU: read past L1.
__device__ __forceinline__ uint4 ld_slot(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_local(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st_vec(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }

// ---------------------------------------------------------------- element-wise maths
template <int OP, typename A> __device__ __forceinline__ A red(A x, A y) {
  if (OP == 0) return x + y;
  if (OP == 1) return x * y;
  if (OP == 2) return x > y ? x : y;
  return x < y ? x : y;
}

template <typename T> struct AccOf { typedef T type; };
template <> struct AccOf<__half> { typedef float type; };
template <> struct AccOf<__nv_bfloat16> { typedef float type; };

template <typename T> struct Cvt {
  typedef typename AccOf<T>::type A;
  static __device__ __forceinline__ A up(T v) { return (A)v; }
  static __device__ __forceinline__ T down(A v) { return (T)v; }
};
template <> struct Cvt<__half> {
  static __device__ __forceinline__ float up(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half down(float v) { return __float2half_rn(v); }
};
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 down(float v) { return __float2bfloat16_rn(v); }
};

template <typename T> struct Pack {
  static constexpr int N = 16 / sizeof(T);
  typedef typename AccOf<T>::type A;
  union U { uint4 v; T t[N]; };
  static __device__ __forceinline__ void up(const uint4& v, A (&a)[N]) {
    U u; u.v = v;
#pragma unroll
    for (int i = 0; i < N; i++) a[i] = Cvt<T>::up(u.t[i]);
  }
  static __device__ __forceinline__ uint4 down(const A (&a)[N]) {
    U u;
#pragma unroll
    for (int i = 0; i < N; i++) u.t[i] = Cvt<T>::down(a[i]);
    return u.v;
  }
};

template <typename A> __device__ __forceinline__ A scale_val(A v, float s) { return v; }
template <> __device__ __forceinline__ float scale_val<float>(float v, float s) { return v * s; }
template <> __device__ __forceinline__ double scale_val<double>(double v, float s) { return v * (double)s; }

// ---------------------------------------------------------------- bounded wait
struct WaitCtx { RankCtx* ctx; unsigned long long timeout_ns; int cta, action, segment; };

// Returns false if the wait was given up (time limit or abort raised elsewhere).
static __device__ __noinline__ bool wait_counter(const unsigned long long* flag, unsigned long long want, const WaitCtx& w, int code, int peer) {
  unsigned long long t0 = 0, have = 0;
  for (unsigned spins = 1;; spins++) {
    have = ld_acquire_sys(flag);
    if (have >= want) return true;
    if ((spins & 31u) == 0) {
      if (*(volatile int*)w.ctx->abort_flag) return false;
      unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > w.timeout_ns) break;
    }
  }
  // first CTA to give up records where; everybody else just leaves
  if (atomicCAS(w.ctx->abort_flag, 0, 1) == 0) {
    piccl_status_t* s = w.ctx->status;
    s->code = code; s->rank = w.ctx->rank; s->cta = w.cta; s->action = w.action; s->peer = peer; s->segment = w.segment;
    s->want = want; s->have = have;
    __threadfence_system();
    s->aborted = 1;
    __threadfence_system();
  }
  return false;
}

// ---------------------------------------------------------------- data movement
// value = reduce(src[0..NSRC)) -> dst[0..NDST); `local_src` (index or -1) is the
// user-buffer operand (plain loads, optional scaling); the other sources are FIFO slots.
// NSRC / NDST > 0: compile-time operand counts (pointers stay in registers, loops unroll);
// 0: run-time counts (generic path for wide radices).
// Both loops run an unpredicated main part (all U packs of a thread in range) and finish the
// remainder one pack at a time, which keeps the register count of the main part low.
template <int U, int NDST>
__device__ __forceinline__ void copy_vec(const char* src, bool src_local, int ndst_rt, char* const* dst, long long first, long long npack) {
  const int ndst = NDST ? NDST : ndst_rt;
  const long long nt = blockDim.x;
  // whole super-blocks of nt * U packs; the rest is done one pack per thread at a time
  const long long done = (U == 1) ? npack : first + ((npack - first) / (nt * U)) * (nt * U);
  for (long long base = first + threadIdx.x; base < done; base += nt * U) {
    uint4 v[U];
    const char* sp = src + base * 16;
#pragma unroll
    for (int u = 0; u < U; u++) v[u] = src_local ? ld_local(sp + u * nt * 16) : ld_slot(sp + u * nt * 16);
#pragma unroll
    for (int d = 0; d < (NDST ? NDST : kMaxActionPeers + 1); d++) {
      if (d < ndst) {
        char* dp = dst[d] + base * 16;
#pragma unroll
        for (int u = 0; u < U; u++) st_vec(dp + u * nt * 16, v[u]);
      }
    }
  }
  if (U > 1 && done < npack) copy_vec<1, NDST>(src, src_local, ndst_rt, dst, done, npack);
}

template <typename T, int OP, int U, int NSRC, int NDST>
__device__ __forceinline__ void reduce_copy_vec(int nsrc_rt, const char* const* src, int local_src, int ndst_rt, char* const* dst,
                                                long long first, long long npack, bool do_scale, float scale) {
  typedef typename AccOf<T>::type A;
  constexpr int N = Pack<T>::N;
  const int nsrc = NSRC ? NSRC : nsrc_rt, ndst = NDST ? NDST : ndst_rt;
  const long long nt = blockDim.x;
  const long long done = (U == 1) ? npack : first + ((npack - first) / (nt * U)) * (nt * U);
  for (long long base = first + threadIdx.x; base < done; base += nt * U) {
    A acc[U][N];
    {
      const char* sp = src[0] + base * 16;
#pragma unroll
      for (int u = 0; u < U; u++) {
        uint4 v = (local_src == 0) ? ld_local(sp + u * nt * 16) : ld_slot(sp + u * nt * 16);
        Pack<T>::up(v, acc[u]);
        if (do_scale && local_src == 0) {
#pragma unroll
          for (int e = 0; e < N; e++) acc[u][e] = scale_val<A>(acc[u][e], scale);
        }
      }
    }
#pragma unroll
    for (int s = 1; s < (NSRC ? NSRC : kMaxActionPeers + 1); s++) {
      if (s < nsrc) {
        uint4 v[U];
        const char* sp = src[s] + base * 16;
#pragma unroll
        for (int u = 0; u < U; u++) v[u] = (local_src == s) ? ld_local(sp + u * nt * 16) : ld_slot(sp + u * nt * 16);
#pragma unroll
        for (int u = 0; u < U; u++) {
          A x[N]; Pack<T>::up(v[u], x);
#pragma unroll
          for (int e = 0; e < N; e++) {
            A xv = (do_scale && local_src == s) ? scale_val<A>(x[e], scale) : x[e];
            acc[u][e] = red<OP, A>(acc[u][e], xv);
          }
        }
      }
    }
#pragma unroll
    for (int d = 0; d < (NDST ? NDST : kMaxActionPeers + 1); d++) {
      if (d < ndst) {
        char* dp = dst[d] + base * 16;
#pragma unroll
        for (int u = 0; u < U; u++) st_vec(dp + u * nt * 16, Pack<T>::down(acc[u]));
      }
    }
  }
  if (U > 1 && done < npack) reduce_copy_vec<T, OP, 1, NSRC, NDST>(nsrc_rt, src, local_src, ndst_rt, dst, done, npack, do_scale, scale);
}

// Picks the instantiation for the common operand counts of ring / pairwise schedules.
template <typename T, int OP>
__device__ __noinline__ void reduce_copy_dispatch(int nsrc, const char* const* src, int local_src, int ndst, char* const* dst,
                                                     long long npack, bool do_scale, float scale) {
  constexpr int N = Pack<T>::N;
  // 16-byte packs in flight per thread: 8 when only moving data; for reductions bounded by the accumulator registers
  constexpr int UR = (sizeof(typename AccOf<T>::type) * N * 4 <= 128) ? 4 : 2;
  if (nsrc == 1 && !do_scale) {
    if (ndst == 1) copy_vec<8, 1>(src[0], local_src == 0, 1, dst, 0, npack);
    else if (ndst == 2) copy_vec<8, 2>(src[0], local_src == 0, 2, dst, 0, npack);
    else copy_vec<4, 0>(src[0], local_src == 0, ndst, dst, 0, npack);
    return;
  }
  if (nsrc == 1 && ndst == 1) reduce_copy_vec<T, OP, UR, 1, 1>(1, src, local_src, 1, dst, 0, npack, do_scale, scale);
  else if (nsrc == 2 && ndst == 1) reduce_copy_vec<T, OP, UR, 2, 1>(2, src, local_src, 1, dst, 0, npack, do_scale, scale);
  else if (nsrc == 2 && ndst == 2) reduce_copy_vec<T, OP, UR, 2, 2>(2, src, local_src, 2, dst, 0, npack, do_scale, scale);
  else reduce_copy_vec<T, OP, (UR > 2 ? 2 : UR), 0, 0>(nsrc, src, local_src, ndst, dst, 0, npack, do_scale, scale);
}

// Element-wise path: unaligned user buffers and the last, partial pack of an action.
template <typename T, int OP>
__device__ __noinline__ void reduce_copy_elem(int nsrc, const char* const* src, int local_src, int ndst, char* const* dst,
                                                 long long first, long long nelem, bool do_scale, float scale) {
  typedef typename AccOf<T>::type A;
  for (long long i = first + threadIdx.x; i < nelem; i += blockDim.x) {
    A acc = A();
    for (int s = 0; s < nsrc; s++) {
      const T* p = reinterpret_cast<const T*>(src[s]) + i;
      T raw = (local_src == s) ? *p : *reinterpret_cast<const volatile T*>(p);
      A x = Cvt<T>::up(raw);
      if (do_scale && local_src == s) x = scale_val<A>(x, scale);
      acc = (s == 0) ? x : red<OP, A>(acc, x);
    }
    T o = Cvt<T>::down(acc);
    for (int d = 0; d < ndst; d++) reinterpret_cast<T*>(dst[d])[i] = o;
  }
}

// ---------------------------------------------------------------- the kernel
constexpr int kSliceCache = 192;      // actions whose CTA slice is precomputed in shared memory

// DEFER = true (PICCL_EXEC_DEFER=1) postpones the counter updates that end an action: a release store to another GPU waits
// for the action's data to be acknowledged (a round trip through the switch), and a chain of independent actions, such as the
// n-1 sends that open a DIRECT all-reduce, pays that once per action.  The deferred variant only bumps its private counters
// and publishes all of them together, with the fences of the owning threads running side by side, at the first point
// where the CTA is about to block (one probe of the flags it needs; somebody may be waiting for what was held back) and at
// the end of the kernel.  Nothing is ever held back across a wait, so progress is as in the plain variant.
template <typename T, int OP, bool DEFER>
__global__ void __launch_bounds__(kMaxBlock, 1) exec_kernel(const KernelArgs ka) {
  const int vr = blockIdx.x / ka.n_cta, cta = blockIdx.x % ka.n_cta;
  const LaunchRank& L = ka.r[vr];
  RankCtx* __restrict__ ctx = L.ctx;
  const int tid = threadIdx.x;
  constexpr int esz = (int)sizeof(T);

  __shared__ int s_send_slot[kMaxRanks], s_recv_slot[kMaxRanks];
  __shared__ char* s_heap[kMaxRanks];
  __shared__ long long s_lo[kSliceCache], s_hi[kSliceCache];
  __shared__ int s_fail, s_maxseg;

  // everything read from the context more than once is fetched once, in parallel
  const int rank = ctx->rank, nranks = ctx->nranks, max_cta = ctx->max_cta, nslot = ctx->nslot;
  const long long slot_bytes = ctx->slot_bytes, tail_off = ctx->tail_off, head_off = ctx->head_off, fifo_off = ctx->fifo_off, scratch_off = ctx->scratch_off;
  // thread p (< nranks) owns the two counters of the connections with peer p
  unsigned long long my_sent = 0, my_rcvd = 0;
  if (tid < nranks) { s_heap[tid] = ctx->heap[tid]; my_sent = ctx->sent[tid * max_cta + cta]; my_rcvd = ctx->rcvd[tid * max_cta + cta]; }
  if (tid == 0) { s_fail = 0; s_maxseg = 0; }
  __syncthreads();
  const long long seg_elems = (slot_bytes / 16) * (esz >= 16 ? 1 : 16 / esz);
  {
    int m = 0;
    for (int ai = tid; ai < L.n_actions; ai += blockDim.x) {
      const Slice sl = slice_of(L.actions[ai].count, esz, cta, ka.n_cta, slot_bytes);
      if (ai < kSliceCache) { s_lo[ai] = sl.lo; s_hi[ai] = sl.hi; }
      m = max(m, sl.nseg);
    }
    if (m) atomicMax(&s_maxseg, m);
  }
  __syncthreads();
  const int maxseg = s_maxseg;
  char* const my_heap = s_heap[rank];
  WaitCtx w; w.ctx = ctx; w.timeout_ns = ka.timeout_ns; w.cta = cta;
  bool failed = false;
  // DEFER: what peer `tid` has been told so far, and whether any update is held back (the same value in every thread)
  unsigned long long pub_sent = my_sent, pub_rcvd = my_rcvd;
  bool pending = false;
  auto flush = [&]() {
    if (tid < nranks) {
      if (pub_sent != my_sent) { st_release_sys(reinterpret_cast<unsigned long long*>(s_heap[tid] + tail_off + (long long)(rank * max_cta + cta) * kFlagStride), my_sent); pub_sent = my_sent; }
      if (pub_rcvd != my_rcvd) { st_release_sys(reinterpret_cast<unsigned long long*>(s_heap[tid] + head_off + (long long)(rank * max_cta + cta) * kFlagStride), my_rcvd); pub_rcvd = my_rcvd; }
    }
  };

  for (int seg = 0; seg < maxseg && !failed; seg++) {
    for (int ai = 0; ai < L.n_actions; ai++) {
      long long sl_lo, sl_hi;
      if (ai < kSliceCache) { sl_lo = s_lo[ai]; sl_hi = s_hi[ai]; }
      else { const Slice sl = slice_of(L.actions[ai].count, esz, cta, ka.n_cta, slot_bytes); sl_lo = sl.lo; sl_hi = sl.hi; }
      const long long lo = sl_lo + (long long)seg * seg_elems;
      if (lo >= sl_hi) continue;
      const long long hi = (lo + seg_elems < sl_hi) ? lo + seg_elems : sl_hi;
      const long long len = hi - lo;
      const Action ac = L.actions[ai];

      if (DEFER && pending) {
        // one probe of everything this action waits for; if anything is missing, tell the peers what was held back first
        bool block = false;
        if (tid < nranks) {
          for (int j = 0; j < ac.n_send; j++) if (ac.send_peer[j] == tid && my_sent + 1 > (unsigned long long)nslot)
            block |= ld_acquire_sys(reinterpret_cast<const unsigned long long*>(my_heap + head_off + (long long)(tid * max_cta + cta) * kFlagStride)) < my_sent + 1 - nslot;
          for (int j = 0; j < ac.n_recv; j++) if (ac.recv_peer[j] == tid)
            block |= ld_acquire_sys(reinterpret_cast<const unsigned long long*>(my_heap + tail_off + (long long)(tid * max_cta + cta) * kFlagStride)) < my_rcvd + 1;
        }
        if (__syncthreads_or(block)) { flush(); pending = false; }
      }
      // ---- wait: credit on every send connection, data on every receive connection
      if (tid < nranks) {
        bool ok = true;
        w.action = ai; w.segment = seg;
        for (int j = 0; j < ac.n_send; j++) if (ac.send_peer[j] == tid) {
          s_send_slot[tid] = (int)(my_sent % (unsigned)nslot);
          if (my_sent + 1 > (unsigned long long)nslot)
            ok = wait_counter(reinterpret_cast<const unsigned long long*>(my_heap + head_off + (long long)(tid * max_cta + cta) * kFlagStride),
                              my_sent + 1 - nslot, w, 1, tid);
        }
        for (int j = 0; j < ac.n_recv && ok; j++) if (ac.recv_peer[j] == tid) {
          s_recv_slot[tid] = (int)(my_rcvd % (unsigned)nslot);
          ok = wait_counter(reinterpret_cast<const unsigned long long*>(my_heap + tail_off + (long long)(tid * max_cta + cta) * kFlagStride),
                            my_rcvd + 1, w, 2, tid);
        }
        if (!ok) s_fail = 1;
      }
      __syncthreads();
      if (s_fail) { failed = true; break; }

      // ---- operands, in rank order: receive peers below me, my own buffer, receive peers above me
      const char* src[kMaxActionPeers + 1]; char* dst[kMaxActionPeers + 1];
      int nsrc = 0, ndst = 0, local_src = -1;
      bool aligned = true;
      const bool has_src = ac.src_buf != BUF_NONE;
#pragma unroll
      for (int j = 0; j <= kMaxActionPeers; j++) {
        if (j <= ac.n_recv) {
          if (j == ac.self_pos && has_src) {
            const char* base = ac.src_buf == BUF_IN ? (const char*)L.in : ac.src_buf == BUF_OUT ? (const char*)L.out : my_heap + scratch_off;
            src[nsrc] = base + (ac.src_off + lo) * esz;
            aligned &= ((reinterpret_cast<uintptr_t>(src[nsrc]) & 15) == 0);
            local_src = nsrc++;
          }
          if (j < ac.n_recv) {
            const int p = ac.recv_peer[j];
            src[nsrc++] = my_heap + fifo_off + ((long long)(p * max_cta + cta) * nslot + s_recv_slot[p]) * slot_bytes;
          }
        }
      }
      if (ac.dst_buf != BUF_NONE) {
        char* base = ac.dst_buf == BUF_OUT ? (char*)L.out : my_heap + scratch_off;
        dst[ndst] = base + (ac.dst_off + lo) * esz;
        aligned &= ((reinterpret_cast<uintptr_t>(dst[ndst]) & 15) == 0);
        ndst++;
      }
#pragma unroll
      for (int j = 0; j < kMaxActionPeers; j++) {
        if (j < ac.n_send) {
          const int p = ac.send_peer[j];
          dst[ndst++] = s_heap[p] + fifo_off + ((long long)(rank * max_cta + cta) * nslot + s_send_slot[p]) * slot_bytes;
        }
      }
      const bool do_scale = ka.avg && (ac.flags & ACT_SCALE_SRC) && local_src >= 0;

      // ---- one pass over the segment
      constexpr int N = Pack<T>::N;
      long long nfull = aligned ? len / N : 0;
      if (nfull) reduce_copy_dispatch<T, OP>(nsrc, src, local_src, ndst, dst, nfull, do_scale, ka.scale);
      if (nfull * N < len) reduce_copy_elem<T, OP>(nsrc, src, local_src, ndst, dst, nfull * N, len, do_scale, ka.scale);
      __syncthreads();

      // ---- publish: the data to the consumers, the freed slot to the producers
      if (DEFER) {
        if (tid < nranks) {
          for (int j = 0; j < ac.n_send; j++) if (ac.send_peer[j] == tid) my_sent++;
          for (int j = 0; j < ac.n_recv; j++) if (ac.recv_peer[j] == tid) my_rcvd++;
        }
        pending = true;
      } else if (tid < nranks) {
        for (int j = 0; j < ac.n_send; j++) if (ac.send_peer[j] == tid) {
          my_sent++;
          st_release_sys(reinterpret_cast<unsigned long long*>(s_heap[tid] + tail_off + (long long)(rank * max_cta + cta) * kFlagStride), my_sent);
        }
        for (int j = 0; j < ac.n_recv; j++) if (ac.recv_peer[j] == tid) {
          my_rcvd++;
          st_release_sys(reinterpret_cast<unsigned long long*>(s_heap[tid] + head_off + (long long)(rank * max_cta + cta) * kFlagStride), my_rcvd);
        }
      }
    }
  }
  if (DEFER && pending && !failed) flush();
  if (tid < nranks) { ctx->sent[tid * max_cta + cta] = my_sent; ctx->rcvd[tid * max_cta + cta] = my_rcvd; }
}


}  // namespace piccl
