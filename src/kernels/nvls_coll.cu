// Kernels of the in-switch collectives; protocol and window layout in nvls.cuh.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "exec.cuh"
#include "nvls.cuh"

namespace piccl {

namespace {

__device__ __forceinline__ unsigned long long nv_ld_acquire(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long nv_time_ns() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
// data that the switch (or another rank) wrote into this GPU's memory: read past L1
__device__ __forceinline__ uint4 nv_ld_volatile(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 nv_ld_plain(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void nv_st(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }

// ---------------------------------------------------------------- element maths (emulated switch, scaling)
template <typename T> __device__ __forceinline__ float nv_up(T v);
template <> __device__ __forceinline__ float nv_up<float>(float v) { return v; }
template <> __device__ __forceinline__ float nv_up<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float nv_up<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T nv_down(float v);
template <> __device__ __forceinline__ float nv_down<float>(float v) { return v; }
template <> __device__ __forceinline__ __half nv_down<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 nv_down<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <int OP> __device__ __forceinline__ float nv_red(float x, float y) { return OP == 0 ? x + y : OP == 2 ? (x > y ? x : y) : (x < y ? x : y); }

// A user buffer need not be 16-byte aligned, and for the collectives that only move data T is not the caller's element
// type, so the buffer need not even be aligned to T.  Alignment class of an address: 2 = 16 bytes, 1 = T, 0 = bytes.
template <typename T> __device__ __forceinline__ int align_class(const void* p) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  return (a & 15) == 0 ? 2 : (a & (sizeof(T) - 1)) == 0 ? 1 : 0;
}
template <typename T> __device__ __forceinline__ uint4 ld_user(const char* p, int al) {
  if (al == 2) return nv_ld_plain(p);
  constexpr int N = 16 / sizeof(T);
  union { uint4 v; T t[N]; unsigned char b[16]; } u;
  if (al == 1) {
#pragma unroll
    for (int e = 0; e < N; e++) u.t[e] = reinterpret_cast<const T*>(p)[e];
  } else {
#pragma unroll
    for (int e = 0; e < 16; e++) u.b[e] = reinterpret_cast<const unsigned char*>(p)[e];
  }
  return u.v;
}
template <typename T> __device__ __forceinline__ void st_user(char* p, const uint4& v, int al) {
  if (al == 2) { nv_st(p, v); return; }
  constexpr int N = 16 / sizeof(T);
  union { uint4 v; T t[N]; unsigned char b[16]; } u; u.v = v;
  if (al == 1) {
#pragma unroll
    for (int e = 0; e < N; e++) reinterpret_cast<T*>(p)[e] = u.t[e];
  } else {
#pragma unroll
    for (int e = 0; e < 16; e++) reinterpret_cast<unsigned char*>(p)[e] = u.b[e];
  }
}

// ---------------------------------------------------------------- the switch
// ld: OP over all copies of the 16 bytes at `mc`; st: 16 bytes written to all copies
template <typename T, int OP> struct Mm;
template <> struct Mm<float, 0> {
  static __device__ __forceinline__ uint4 ld(const char* mc) {
    float a, b, c, d;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(a), "=f"(b), "=f"(c), "=f"(d) : "l"(mc) : "memory");
    return make_uint4(__float_as_uint(a), __float_as_uint(b), __float_as_uint(c), __float_as_uint(d));
  }
};
#define PICCL_MM_HALF(T, OP, INSTR)                                                                                                         \
  template <> struct Mm<T, OP> {                                                                                                            \
    static __device__ __forceinline__ uint4 ld(const char* mc) {                                                                            \
      uint4 v;                                                                                                                              \
      asm volatile("multimem.ld_reduce.relaxed.sys.global." INSTR " {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory"); \
      return v;                                                                                                                             \
    }                                                                                                                                       \
  };
PICCL_MM_HALF(__nv_bfloat16, 0, "add.acc::f32.v4.bf16x2")
PICCL_MM_HALF(__nv_bfloat16, 2, "max.v4.bf16x2")
PICCL_MM_HALF(__nv_bfloat16, 3, "min.v4.bf16x2")
PICCL_MM_HALF(__half, 0, "add.acc::f32.v4.f16x2")
PICCL_MM_HALF(__half, 2, "max.v4.f16x2")
PICCL_MM_HALF(__half, 3, "min.v4.f16x2")
#undef PICCL_MM_HALF
// the store moves bits; the type in the instruction only names the width
__device__ __forceinline__ void mm_st(char* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)),
               "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)) : "memory");
}

// One (virtual) rank's view of the switch.  `off` is a byte offset into the window.
template <typename T, int OP, bool EMU> struct Switch {
  const NvlsArgs& a; const NvlsRank& R;
  __device__ __forceinline__ Switch(const NvlsArgs& a_, const NvlsRank& r_) : a(a_), R(r_) {}
  __device__ __forceinline__ uint4 ld_reduce(long long off) const {
    if (!EMU) return Mm<T, OP>::ld(R.mc + off);
    constexpr int N = 16 / sizeof(T);
    union U { uint4 v; T t[N]; };
    float acc[N];
    for (int q = 0; q < a.nranks; q++) {
      U u; u.v = nv_ld_volatile(a.r[q].uc + off);
#pragma unroll
      for (int e = 0; e < N; e++) acc[e] = q == 0 ? nv_up<T>(u.t[e]) : nv_red<OP>(acc[e], nv_up<T>(u.t[e]));
    }
    U o;
#pragma unroll
    for (int e = 0; e < N; e++) o.t[e] = nv_down<T>(acc[e]);
    return o.v;
  }
  __device__ __forceinline__ void st_all(long long off, const uint4& v) const {
    if (!EMU) { mm_st(R.mc + off, v); return; }
    for (int q = 0; q < a.nranks; q++) nv_st(a.r[q].uc + off, v);
  }
  // raises the counter at `off` by `inc` on every copy; everything this thread has observed is ordered before it
  __device__ __forceinline__ void add_all(long long off, unsigned long long inc) const {
    if (!EMU) { asm volatile("multimem.red.release.sys.global.add.u64 [%0], %1;" ::"l"(R.mc + off), "l"(inc) : "memory"); return; }
    for (int q = 0; q < a.nranks; q++) asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(a.r[q].uc + off), "l"(inc) : "memory");
  }
};

// ---------------------------------------------------------------- data movement inside one CTA
// nblk blocks of `len` bytes: block q from src + q * src_stride to dst + q * dst_stride.  With every address, stride and
// length a multiple of 16 the blocks are moved as one flat sequence of 16-byte packs, U in flight per thread; otherwise
// element by element.  `scale_on` multiplies by `scale` on the way (avg); src_volatile: the source was written by the switch.
// One group of warps of a CTA that works on its own stage of the pipeline: thread index inside the group, threads of the
// group, and the named barrier the group synchronises on.
struct Role { int tid, nthr, bar; };
__device__ __forceinline__ void role_sync(const Role& g) { asm volatile("bar.sync %0, %1;" ::"r"(g.bar), "r"(g.nthr) : "memory"); }

template <typename T, int U>
__device__ __forceinline__ void copy_blocks(const Role& g, char* dst, long long dst_stride, const char* src, long long src_stride, int nblk, long long len, bool src_volatile,
                                            bool scale_on, float scale) {
  constexpr int N = 16 / sizeof(T);
  const bool fast = (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | (uintptr_t)dst_stride | (uintptr_t)src_stride) & 15) == 0);
  const int nt = g.nthr, tid = g.tid;
  if (fast) {
    const int ppb = (int)(len >> 4);                    // whole packs per block
    const int total = ppb * nblk;
    // pack p of the flat sequence: block q = p / ppb, pack i = p % ppb of that block
    auto src_of = [&](int p) { const int q = nblk == 1 ? 0 : p / ppb; return src + (long long)q * src_stride + ((long long)(p - q * ppb) << 4); };
    auto dst_of = [&](int p) { const int q = nblk == 1 ? 0 : p / ppb; return dst + (long long)q * dst_stride + ((long long)(p - q * ppb) << 4); };
    auto scaled = [&](uint4 v) {
      union { uint4 v; T t[N]; } u; u.v = v;
#pragma unroll
      for (int e = 0; e < N; e++) u.t[e] = nv_down<T>(nv_up<T>(u.t[e]) * scale);
      return u.v;
    };
    const int done = (total / (nt * U)) * (nt * U);
    for (int base = tid; base < done; base += nt * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; u++) { const char* sp = src_of(base + u * nt); v[u] = src_volatile ? nv_ld_volatile(sp) : nv_ld_plain(sp); }
      if (scale_on) {
#pragma unroll
        for (int u = 0; u < U; u++) v[u] = scaled(v[u]);
      }
#pragma unroll
      for (int u = 0; u < U; u++) nv_st(dst_of(base + u * nt), v[u]);
    }
    for (int p = done + tid; p < total; p += nt) {
      const char* sp = src_of(p);
      uint4 v = src_volatile ? nv_ld_volatile(sp) : nv_ld_plain(sp);
      if (scale_on) v = scaled(v);
      nv_st(dst_of(p), v);
    }
    // the tail of each block that does not fill a pack
    const int tail0 = ppb * N, nelem = (int)(len / (long long)sizeof(T));
    if (tail0 < nelem) {
      const int per = nelem - tail0;
      for (int t = tid; t < per * nblk; t += nt) {
        const int q = t / per, i = tail0 + (t - q * per);
        T v = src_volatile ? reinterpret_cast<const volatile T*>(src + (long long)q * src_stride)[i] : reinterpret_cast<const T*>(src + (long long)q * src_stride)[i];
        reinterpret_cast<T*>(dst + (long long)q * dst_stride)[i] = scale_on ? nv_down<T>(nv_up<T>(v) * scale) : v;
      }
    }
  } else if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & (sizeof(T) - 1)) == 0) {
    const long long nelem = len / (long long)sizeof(T);
    for (int q = 0; q < nblk; q++) {
      const T* s = reinterpret_cast<const T*>(src + (long long)q * src_stride); T* d = reinterpret_cast<T*>(dst + (long long)q * dst_stride);
      for (long long i = tid; i < nelem; i += nt) {
        T v = src_volatile ? reinterpret_cast<const volatile T*>(s)[i] : s[i];
        d[i] = scale_on ? nv_down<T>(nv_up<T>(v) * scale) : v;
      }
    }
  } else {
    // not even aligned to T: only the collectives that move data get here (T is then not the caller's type), never with scaling
    for (int q = 0; q < nblk; q++) {
      const unsigned char* s = reinterpret_cast<const unsigned char*>(src + (long long)q * src_stride); unsigned char* d = reinterpret_cast<unsigned char*>(dst + (long long)q * dst_stride);
      for (long long i = tid; i < len; i += nt) d[i] = src_volatile ? reinterpret_cast<const volatile unsigned char*>(s)[i] : s[i];
    }
  }
}

// `len` bytes (a multiple of 16) from the user buffer `src` to window offset `off` of every copy
template <typename T, typename SW>
__device__ __forceinline__ void store_all(const SW& sw, const Role& g, long long off, const char* src, long long len) {
  constexpr int U = 8;
  const int al = align_class<T>(src);
  const int nt = g.nthr, tid = g.tid, total = (int)(len >> 4);
  const int done = (total / (nt * U)) * (nt * U);
  for (int base = tid; base < done; base += nt * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; u++) v[u] = ld_user<T>(src + ((long long)(base + u * nt) << 4), al);
#pragma unroll
    for (int u = 0; u < U; u++) sw.st_all(off + ((long long)(base + u * nt) << 4), v[u]);
  }
  for (int p = done + tid; p < total; p += nt) sw.st_all(off + ((long long)p << 4), ld_user<T>(src + ((long long)p << 4), al));
}

// packs [lo, hi) of the part of a slot at window offset `off`: reduced in the switch, the result to every copy
template <typename SW>
__device__ __forceinline__ void reduce_to_all(const SW& sw, const Role& g, long long off, int lo, int hi) {
  constexpr int U = 8;
  const int nt = g.nthr, tid = g.tid;
  const int done = lo + ((hi - lo) / (nt * U)) * (nt * U);
  for (int base = lo + tid; base < done; base += nt * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; u++) v[u] = sw.ld_reduce(off + ((long long)(base + u * nt) << 4));
#pragma unroll
    for (int u = 0; u < U; u++) sw.st_all(off + ((long long)(base + u * nt) << 4), v[u]);
  }
  for (int p = done + tid; p < hi; p += nt) { const long long o = off + ((long long)p << 4); sw.st_all(o, sw.ld_reduce(o)); }
}

// `len` bytes (a multiple of 16) at window offset `off`, reduced in the switch, to the user buffer `dst`
template <typename T, typename SW>
__device__ __forceinline__ void reduce_to_local(const SW& sw, const Role& g, long long off, char* dst, long long len) {
  constexpr int U = 8;
  const int al = align_class<T>(dst);
  const int nt = g.nthr, tid = g.tid, total = (int)(len >> 4);
  const int done = (total / (nt * U)) * (nt * U);
  for (int base = tid; base < done; base += nt * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; u++) v[u] = sw.ld_reduce(off + ((long long)(base + u * nt) << 4));
#pragma unroll
    for (int u = 0; u < U; u++) st_user<T>(dst + ((long long)(base + u * nt) << 4), v[u], al);
  }
  for (int p = done + tid; p < total; p += nt) st_user<T>(dst + ((long long)p << 4), sw.ld_reduce(off + ((long long)p << 4)), al);
}

// ---------------------------------------------------------------- counters
// The group's accesses so far are ordered before `inc` more arrivals on every copy of the counter.
template <typename SW>
__device__ __forceinline__ void nv_arrive(const SW& sw, const Role& g, long long flag_off, unsigned long long inc) {
  role_sync(g);
  if (g.tid == 0) {
    __threadfence_system();
    sw.add_all(flag_off, inc);
  }
}

// Bounded wait of the whole group until the own copy of the counter shows `target`.  false: the wait ran out or the communicator was aborted.
// `s_fail` belongs to the group: only its thread 0 writes it, and all its threads read it after the group's barrier.
__device__ __forceinline__ bool nv_wait(const NvlsArgs& a, const NvlsRank& R, const Role& g, int cta, long long flag_off, unsigned long long target, int stage, long long chunk,
                                        int* s_fail) {
  if (target == 0) return true;                       // first use of this part of the slot: nothing to wait for (the same in every thread)
  if (g.tid == 0) {
    const unsigned long long* flag = reinterpret_cast<const unsigned long long*>(R.uc + flag_off);
    unsigned long long t0 = 0, have = 0;
    bool ok = false, timed_out = false;
    for (unsigned spins = 1;; spins++) {
      have = nv_ld_acquire(flag);
      if (have >= target) { ok = true; break; }
      if ((spins & 31u) == 0) {
        if (*(volatile int*)R.abort_flag) break;
        unsigned long long now = nv_time_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > a.timeout_ns) { timed_out = true; break; }
      }
    }
    if (!ok) {
      if (timed_out && atomicCAS(R.abort_flag, 0, 1) == 0) {
        piccl_status_t* s = R.status;
        s->code = 5 + stage; s->rank = R.rank; s->cta = cta; s->action = stage; s->peer = -1; s->segment = (int)chunk;
        s->want = target; s->have = have;
        __threadfence_system();
        s->aborted = 1;
        __threadfence_system();
      }
      *s_fail = 1;
    }
  }
  role_sync(g);
  return *(volatile int*)s_fail == 0;
}

// ---------------------------------------------------------------- the kernel
// Three groups of warps per CTA, each looping over the CTA's chunks on its own and meeting the others only through the
// counters (which include this rank's own arrivals):
//   FILL    waits until the part of the slot is free (CONSUMED of its previous use), stages the chunk, raises FILLED
//   SWITCH  all-reduce only: waits for FILLED, sums its 1/n of the chunk in the switch and stores it to all copies, raises REDUCED
//   OUT     waits for REDUCED (all-reduce) or FILLED, moves the result to the receive buffer, raises CONSUMED
// With `depth` parts per slot the three stages of a CTA work on different chunks at the same time.
template <typename T, int OP, bool EMU>
__global__ void __launch_bounds__(kNvlsBlock, 1) nvls_coll_kernel(const __grid_constant__ NvlsArgs a) {
  __shared__ int s_fail[3];
  const int vr = blockIdx.x / a.n_cta, cta = blockIdx.x - vr * a.n_cta;
  const NvlsRank& R = a.r[vr];
  const Switch<T, OP, EMU> sw(a, R);
  if (threadIdx.x < 3) s_fail[threadIdx.x] = 0;
  __syncthreads();
  const int n = a.nranks, rank = R.rank, D = a.depth;
  const unsigned long long N = (unsigned long long)n;
  unsigned long long* const used = R.used + (long long)cta * kNvlsUsedPerCta;
  const long long part_bytes = a.slot_bytes / D;
  const long long slot0 = (long long)kNvlsFlagBytes + (long long)cta * a.slot_bytes;
  auto part = [&](int p) { return slot0 + (long long)p * part_bytes; };
  auto flag = [&](int p, int which) { return (long long)(((cta * kNvlsMaxDepth + p) * 3 + which) * 128); };
  const long long nchunks = (a.bytes + a.chunk_bytes - 1) / a.chunk_bytes;
  const long long m = cta < nchunks ? (nchunks - cta + a.n_cta - 1) / a.n_cta : 0;     // chunks of this CTA
  auto off_of = [&](long long j) { return (cta + j * a.n_cta) * a.chunk_bytes; };
  auto len_of = [&](long long j) { const long long o = off_of(j); return (a.bytes - o < a.chunk_bytes) ? a.bytes - o : a.chunk_bytes; };
  const char* const in = static_cast<const char*>(R.in);
  char* const out = static_cast<char*>(R.out);
  const bool scale_on = a.avg != 0;
  const bool allreduce = a.coll == COLL_ALLREDUCE;
  const bool filler = a.coll == COLL_BROADCAST ? rank == a.root : true;
  const bool consumer = a.coll == COLL_REDUCE ? rank == a.root : true;
  const unsigned long long fill_inc = a.coll == COLL_BROADCAST ? N : 1, cons_inc = a.coll == COLL_REDUCE ? N : 1;

  // threads per group (multiples of 32): in proportion to the bytes each stage moves per chunk
  int nF, nS = 0, nO;
  switch (a.coll) {
    case COLL_ALLREDUCE: if (n <= 2) { nF = 160; nS = 192; nO = 160; } else { nF = 192; nS = 128; nO = 192; } break;
    case COLL_ALLGATHER: nF = n <= 2 ? 192 : 128; nO = kNvlsBlock - nF; break;
    case COLL_REDUCE_SCATTER: nO = n <= 2 ? 192 : 128; nF = kNvlsBlock - nO; break;
    case COLL_BROADCAST: if (!filler) { nF = 0; nO = kNvlsBlock; } else if (in == out) { nO = 32; nF = kNvlsBlock - 32; } else { nF = 256; nO = 256; } break;
    default: if (!consumer) { nF = kNvlsBlock; nO = 0; } else { nF = 192; nO = 320; } break;      // reduce
  }
  const int t = threadIdx.x;
  int role; Role g;
  if (t < nF) { role = 0; g.tid = t; g.nthr = nF; g.bar = 1; }
  else if (t < nF + nS) { role = 1; g.tid = t - nF; g.nthr = nS; g.bar = 2; }
  else if (t < nF + nS + nO) { role = 2; g.tid = t - nF - nS; g.nthr = nO; g.bar = 3; }
  else { role = -1; g.tid = 1; g.nthr = 32; g.bar = 4; }

  // stopwatch of each group's thread 0 (PICCL_NVLS_PROFILE=1): the time since the last lap goes to one profile slot
  const bool prof = R.prof != nullptr && role >= 0 && g.tid == 0 && m > 0;
  unsigned long long t_last = prof ? nv_time_ns() : 0, t_first = t_last, acc[6] = {0, 0, 0, 0, 0, 0};
  auto lap = [&](int slot_id) { if (prof) { const unsigned long long now = nv_time_ns(); acc[slot_id] += now - t_last; t_last = now; } };

  if (role == 0 && filler) {
    for (long long j = 0; j < m; j++) {
      const int p = (int)(j % D);
      const unsigned long long u = used[p] + (unsigned long long)(j / D);
      const long long off = off_of(j), len = len_of(j);
      // nobody reads the previous use of this part any more
      if (!nv_wait(a, R, g, cta, flag(p, NVC_CONSUMED), N * u, NVC_CONSUMED, cta + j * a.n_cta, &s_fail[0])) break;
      lap(NVP_WAIT_CONSUMED);
      switch (a.coll) {
        case COLL_ALLGATHER: store_all<T>(sw, g, part(p) + (long long)rank * a.sub_stride, in + off, len); break;
        case COLL_BROADCAST: store_all<T>(sw, g, part(p), in + off, len); break;
        case COLL_REDUCE_SCATTER: copy_blocks<T, 8>(g, R.uc + part(p), a.sub_stride, in + off, a.bytes, n, len, false, scale_on, a.scale); break;
        default: copy_blocks<T, 8>(g, R.uc + part(p), 0, in + off, 0, 1, len, false, scale_on, a.scale); break;      // all-reduce, reduce
      }
      nv_arrive(sw, g, flag(p, NVC_FILLED), fill_inc);
      lap(NVP_FILL);
    }
  } else if (role == 1 && allreduce) {
    for (long long j = 0; j < m; j++) {
      const int p = (int)(j % D);
      const unsigned long long u = used[p] + (unsigned long long)(j / D);
      const long long len = len_of(j);
      // every rank has copied chunk j in
      if (!nv_wait(a, R, g, cta, flag(p, NVC_FILLED), N * (u + 1), NVC_FILLED, cta + j * a.n_cta, &s_fail[1])) break;
      lap(NVP_WAIT_FILLED);
      const int npack = (int)((len + 15) >> 4);          // the bytes past `len` in the last pack are summed too and never copied out
      const int per = (npack + n - 1) / n;
      int lo = rank * per; if (lo > npack) lo = npack;
      int hi = lo + per; if (hi > npack) hi = npack;
      reduce_to_all(sw, g, part(p), lo, hi);
      nv_arrive(sw, g, flag(p, NVC_REDUCED), 1);
      lap(NVP_SWITCH);
    }
  } else if (role == 2 && consumer) {
    for (long long j = 0; j < m; j++) {
      const int p = (int)(j % D);
      const unsigned long long u = used[p] + (unsigned long long)(j / D), uy = used[kNvlsMaxDepth + p] + (unsigned long long)(j / D);
      const long long off = off_of(j), len = len_of(j);
      if (allreduce) {
        // every rank has written its share of the sums of chunk j
        if (!nv_wait(a, R, g, cta, flag(p, NVC_REDUCED), N * (uy + 1), NVC_REDUCED, cta + j * a.n_cta, &s_fail[2])) break;
        lap(NVP_WAIT_REDUCED);
      } else {
        if (!nv_wait(a, R, g, cta, flag(p, NVC_FILLED), N * (u + 1), NVC_FILLED, cta + j * a.n_cta, &s_fail[2])) break;
        lap(NVP_WAIT_FILLED);
      }
      switch (a.coll) {
        case COLL_ALLGATHER: copy_blocks<T, 8>(g, out + off, a.bytes, R.uc + part(p), a.sub_stride, n, len, true, false, 1.0f); break;
        case COLL_BROADCAST: if (!(rank == a.root && in == out)) copy_blocks<T, 8>(g, out + off, 0, R.uc + part(p), 0, 1, len, true, false, 1.0f); break;
        case COLL_REDUCE_SCATTER: reduce_to_local<T>(sw, g, part(p) + (long long)rank * a.sub_stride, out + off, len); break;
        case COLL_REDUCE: reduce_to_local<T>(sw, g, part(p), out + off, len); break;
        default: copy_blocks<T, 8>(g, out + off, 0, R.uc + part(p), 0, 1, len, true, false, 1.0f); break;        // all-reduce
      }
      nv_arrive(sw, g, flag(p, NVC_CONSUMED), cons_inc);
      lap(NVP_OUT);
    }
  }
  if (prof) {
    for (int i = 0; i < 6; i++) if (acc[i]) atomicAdd(R.prof + i, acc[i]);
    if (role == 2 || (role == 0 && !consumer)) { atomicAdd(R.prof + NVP_CHUNKS, (unsigned long long)m); atomicAdd(R.prof + NVP_CTAS, 1ull); atomicAdd(R.prof + NVP_TOTAL, nv_time_ns() - t_first); }
  }
  __syncthreads();                                    // every group is done with `used`
  if (threadIdx.x == 0 && m > 0 && !(s_fail[0] | s_fail[1] | s_fail[2])) {
    for (int p = 0; p < D; p++) {
      const unsigned long long cnt = (unsigned long long)((m + D - 1 - p) / D);      // chunks j < m with j % D == p
      used[p] += cnt;
      if (allreduce) used[kNvlsMaxDepth + p] += cnt;
    }
  }
}

template <bool EMU> const void* kernel_of(int dtype, int op) {
  if (dtype == DT_F32) return op == 0 ? (const void*)nvls_coll_kernel<float, 0, EMU> : nullptr;
  if (dtype == DT_BF16) return op == 0 ? (const void*)nvls_coll_kernel<__nv_bfloat16, 0, EMU> : op == 2 ? (const void*)nvls_coll_kernel<__nv_bfloat16, 2, EMU>
                               : op == 3 ? (const void*)nvls_coll_kernel<__nv_bfloat16, 3, EMU> : nullptr;
  if (dtype == DT_F16) return op == 0 ? (const void*)nvls_coll_kernel<__half, 0, EMU> : op == 2 ? (const void*)nvls_coll_kernel<__half, 2, EMU>
                              : op == 3 ? (const void*)nvls_coll_kernel<__half, 3, EMU> : nullptr;
  return nullptr;
}

}  // namespace

bool nvls_kernel_exists(int dtype, int op) { return kernel_of<false>(dtype, op) != nullptr; }

int nvls_max_resident_ctas(bool emulate) {
  const void* fn = emulate ? kernel_of<true>(DT_F32, 0) : kernel_of<false>(DT_F32, 0);
  int per_sm = 0, dev = 0, sms = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kNvlsBlock, 0) != cudaSuccess) { cudaGetLastError(); per_sm = 1; }
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return (per_sm > 0 ? per_sm : 1) * (sms > 0 ? sms : 1);
}

int nvls_launch(const NvlsArgs& a, int dtype, int op, bool emulate, void* stream) {
  void* args[] = {const_cast<NvlsArgs*>(&a)};
  const void* fn = emulate ? kernel_of<true>(dtype, op) : kernel_of<false>(dtype, op);
  if (!fn) return (int)cudaErrorInvalidValue;
  if (emulate) return (int)cudaLaunchCooperativeKernel(fn, dim3(a.n_vrank * a.n_cta), dim3(kNvlsBlock), args, 0, (cudaStream_t)stream);
  return (int)cudaLaunchKernel(fn, dim3(a.n_cta), dim3(kNvlsBlock), args, 0, (cudaStream_t)stream);
}

}  // namespace piccl
