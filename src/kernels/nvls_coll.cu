// Kernels of the in-switch collectives; protocol and window layout in nvls.cuh.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <mutex>
#include <set>
#include <utility>
#include "exec.cuh"
#include "nvls.cuh"
#include "../include/sm100_ptx.cuh"

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
// avg: the sum of a pack times 1/n
template <typename T> __device__ __forceinline__ uint4 nv_scaled(const uint4& v, float scale) {
  constexpr int N = 16 / sizeof(T);
  union { uint4 v; T t[N]; } u; u.v = v;
#pragma unroll
  for (int e = 0; e < N; e++) u.t[e] = nv_down<T>(nv_up<T>(u.t[e]) * scale);
  return u.v;
}

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
  // raises the counter at `off` by `inc` on every copy; release: everything this thread has observed is ordered before it
  __device__ __forceinline__ void add_all(long long off, unsigned long long inc, bool release) const {
    if (!EMU) {
      if (release) asm volatile("multimem.red.release.sys.global.add.u64 [%0], %1;" ::"l"(R.mc + off), "l"(inc) : "memory");
      else asm volatile("multimem.red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(R.mc + off), "l"(inc) : "memory");
      return;
    }
    for (int q = 0; q < a.nranks; q++) {
      if (release) asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(a.r[q].uc + off), "l"(inc) : "memory");
      else asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(a.r[q].uc + off), "l"(inc) : "memory");
    }
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
__device__ __forceinline__ void copy_blocks(const Role& g, char* dst, long long dst_stride, const char* src, long long src_stride, int nblk, long long len, bool src_volatile) {
  constexpr int N = 16 / sizeof(T);
  const bool fast = (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | (uintptr_t)dst_stride | (uintptr_t)src_stride) & 15) == 0);
  const int nt = g.nthr, tid = g.tid;
  if (fast) {
    const int ppb = (int)(len >> 4);                    // whole packs per block
    const int total = ppb * nblk;
    // pack p of the flat sequence: block q = p / ppb, pack i = p % ppb of that block
    auto src_of = [&](int p) { const int q = nblk == 1 ? 0 : p / ppb; return src + (long long)q * src_stride + ((long long)(p - q * ppb) << 4); };
    auto dst_of = [&](int p) { const int q = nblk == 1 ? 0 : p / ppb; return dst + (long long)q * dst_stride + ((long long)(p - q * ppb) << 4); };
    const int done = (total / (nt * U)) * (nt * U);
    for (int base = tid; base < done; base += nt * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; u++) { const char* sp = src_of(base + u * nt); v[u] = src_volatile ? nv_ld_volatile(sp) : nv_ld_plain(sp); }
#pragma unroll
      for (int u = 0; u < U; u++) nv_st(dst_of(base + u * nt), v[u]);
    }
    for (int p = done + tid; p < total; p += nt) {
      const char* sp = src_of(p);
      nv_st(dst_of(p), src_volatile ? nv_ld_volatile(sp) : nv_ld_plain(sp));
    }
    // the tail of each block that does not fill a pack
    const int tail0 = ppb * N, nelem = (int)(len / (long long)sizeof(T));
    if (tail0 < nelem) {
      const int per = nelem - tail0;
      for (int t = tid; t < per * nblk; t += nt) {
        const int q = t / per, i = tail0 + (t - q * per);
        reinterpret_cast<T*>(dst + (long long)q * dst_stride)[i] =
            src_volatile ? reinterpret_cast<const volatile T*>(src + (long long)q * src_stride)[i] : reinterpret_cast<const T*>(src + (long long)q * src_stride)[i];
      }
    }
  } else if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & (sizeof(T) - 1)) == 0) {
    const long long nelem = len / (long long)sizeof(T);
    for (int q = 0; q < nblk; q++) {
      const T* sp = reinterpret_cast<const T*>(src + (long long)q * src_stride); T* d = reinterpret_cast<T*>(dst + (long long)q * dst_stride);
      for (long long i = tid; i < nelem; i += nt) d[i] = src_volatile ? reinterpret_cast<const volatile T*>(sp)[i] : sp[i];
    }
  } else {
    // not even aligned to T: only the collectives that move data get here (T is then not the caller's type)
    for (int q = 0; q < nblk; q++) {
      const unsigned char* sp = reinterpret_cast<const unsigned char*>(src + (long long)q * src_stride); unsigned char* d = reinterpret_cast<unsigned char*>(dst + (long long)q * dst_stride);
      for (long long i = tid; i < len; i += nt) d[i] = src_volatile ? reinterpret_cast<const volatile unsigned char*>(sp)[i] : sp[i];
    }
  }
}

// The same movement by the bulk-copy engine (TMA), for buffers that are 16-byte aligned: ONE thread streams the blocks through a
// ring of shared-memory stages, kBulkAhead loads in flight, each stage stored to its destination as soon as it has landed.
// Far more bytes are in flight than loads and stores of the group's threads could keep in flight, and the load/store units
// stay free for the multimem traffic of the switch stage.  Only whole 16-byte packs of each block are moved.
constexpr int kBulkPiece = 16384, kBulkStages = 6, kBulkAhead = 4;
struct BulkRing { unsigned char* smem; uint64_t* mbar; uint32_t phase; };    // phase: bit s = the parity the next wait on stage s looks for

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(sm100::smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes),
               "r"(sm100::smem_u32(bar)) : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }

// Called by one thread.  false: a load did not arrive within the limit (the ring is drained before returning either way).
__device__ __noinline__ bool bulk_copy_blocks(BulkRing& ring, char* dst, long long dst_stride, const char* src, long long src_stride, int nblk, long long len,
                                              unsigned long long limit_ns) {
  const long long len16 = len & ~15ll;
  const int ppb = (int)((len16 + kBulkPiece - 1) / kBulkPiece), np = ppb * nblk;      // pieces per block, pieces
  bool ok = true;
  volatile int never = 0;
  int issued = 0;
  for (int i = 0; i < np + kBulkAhead; i++) {
    if (i < np && ok) {
      issued = i + 1;
      const int st = i % kBulkStages, q = i / ppb, k = i - q * ppb;
      const long long off = (long long)k * kBulkPiece;
      const uint32_t bytes = (uint32_t)(len16 - off < kBulkPiece ? len16 - off : kBulkPiece);
      // the stage last held piece i - kBulkStages; all but the newest (kBulkStages - 1 - kBulkAhead) stores have been read out of shared memory
      if (i >= kBulkStages) bulk_wait_read<kBulkStages - 1 - kBulkAhead>();
      sm100::mbar_arrive_expect_tx(&ring.mbar[st], bytes);
      bulk_load(ring.smem + (size_t)st * kBulkPiece, src + (long long)q * src_stride + off, bytes, &ring.mbar[st]);
    }
    const int j = i - kBulkAhead;
    if (j >= 0 && j < issued) {
      const int st = j % kBulkStages, q = j / ppb, k = j - q * ppb;
      const long long off = (long long)k * kBulkPiece;
      const uint32_t bytes = (uint32_t)(len16 - off < kBulkPiece ? len16 - off : kBulkPiece);
      // every issued load is waited for, also after a failure: no copy may be in flight when the CTA ends
      const bool landed = sm100::mbar_wait(&ring.mbar[st], (ring.phase >> st) & 1u, &never, limit_ns);
      ring.phase ^= 1u << st;
      if (!landed) { ok = false; continue; }
      if (ok) { sm100::bulk_store(dst + (long long)q * dst_stride + off, ring.smem + (size_t)st * kBulkPiece, bytes); sm100::bulk_commit(); }
    }
  }
  sm100::bulk_wait_all();                              // the writes are performed
  asm volatile("fence.proxy.async;" ::: "memory");
  return ok;
}

// Packs [lo, hi) spread over the group, U per thread in flight: all loads of a round are issued before its stores, and every
// round is U wide (the last one guarded), so the number of dependent round trips is ceil((hi - lo) / (threads * U)).
template <int U, typename Load, typename Store>
__device__ __forceinline__ void for_packs(const Role& g, int lo, int hi, Load load, Store store) {
  const int nt = g.nthr;
  for (int base = lo + g.tid; base < hi; base += nt * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; u++) if (base + u * nt < hi) v[u] = load(base + u * nt);
#pragma unroll
    for (int u = 0; u < U; u++) if (base + u * nt < hi) store(base + u * nt, v[u]);
  }
}

// `len` bytes (a multiple of 16) from the user buffer `src` to window offset `off` of every copy
template <typename T, typename SW>
__device__ __forceinline__ void store_all(const SW& sw, const Role& g, long long off, const char* src, long long len) {
  const int al = align_class<T>(src);
  for_packs<8>(g, 0, (int)(len >> 4), [&](int p) { return ld_user<T>(src + ((long long)p << 4), al); }, [&](int p, const uint4& v) { sw.st_all(off + ((long long)p << 4), v); });
}

// packs [lo, hi) of the part of a slot at window offset `off`: reduced in the switch (times `scale` for avg), the result to every copy
template <typename T, typename SW>
__device__ __forceinline__ void reduce_to_all(const SW& sw, const Role& g, long long off, int lo, int hi, bool scale_on, float scale) {
  for_packs<8>(g, lo, hi, [&](int p) { const uint4 v = sw.ld_reduce(off + ((long long)p << 4)); return scale_on ? nv_scaled<T>(v, scale) : v; },
               [&](int p, const uint4& v) { sw.st_all(off + ((long long)p << 4), v); });
}

// `len` bytes (a multiple of 16) at window offset `off`, reduced in the switch (times `scale` for avg), to the user buffer `dst`
template <typename T, typename SW>
__device__ __forceinline__ void reduce_to_local(const SW& sw, const Role& g, long long off, char* dst, long long len, bool scale_on, float scale) {
  const int al = align_class<T>(dst);
  for_packs<8>(g, 0, (int)(len >> 4), [&](int p) { const uint4 v = sw.ld_reduce(off + ((long long)p << 4)); return scale_on ? nv_scaled<T>(v, scale) : v; },
               [&](int p, const uint4& v) { st_user<T>(dst + ((long long)p << 4), v, al); });
}

// ---------------------------------------------------------------- counters
// The group's accesses so far are ordered before `inc` more arrivals on every copy of the counter.  What has to be ordered
// decides the price (a system-wide fence waits for the acknowledgement of every store that went out over NVLink):
//   ARRIVE_REMOTE  the group stored into other GPUs' memory (multimem.st): system-wide fence, release
//   ARRIVE_LOCAL   the group only wrote this GPU's memory, which peers read through this GPU's L2: a fence of GPU scope
//                  puts the data there before the counter update leaves
//   ARRIVE_READ    the arrival only says "done reading": the loads have returned (their values were used), nothing to flush
// strict (PICCL_NVLS_FENCE=sys): the system-wide fence in every case.
enum ArriveKind : int { ARRIVE_REMOTE = 0, ARRIVE_LOCAL = 1, ARRIVE_READ = 2 };
template <typename SW>
__device__ __forceinline__ void nv_arrive(const SW& sw, const Role& g, long long flag_off, unsigned long long inc, int kind, bool strict) {
  role_sync(g);
  if (g.tid == 0) {
    if (strict || kind == ARRIVE_REMOTE) { __threadfence_system(); sw.add_all(flag_off, inc, true); }
    else if (kind == ARRIVE_LOCAL) { __threadfence(); sw.add_all(flag_off, inc, false); }
    else sw.add_all(flag_off, inc, false);
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
// Groups of warps per CTA, each looping over chunks of the CTA on its own and meeting the others only through the
// counters (which include this rank's own arrivals):
//   FILL    waits until the part of the slot is free (CONSUMED of its previous use), stages the chunk, raises FILLED
//   SWITCH  all-reduce only: waits for FILLED, sums its 1/n of the chunk in the switch and stores it to all copies, raises REDUCED
//   OUT     waits for REDUCED (all-reduce) or FILLED, moves the result to the receive buffer, raises CONSUMED
// With `depth` parts per slot the stages of a CTA work on different chunks at the same time, and the stage that talks to the
// switch (SWITCH; FILL of all-gather / broadcast; OUT of reduce-scatter / reduce) is itself split into groups that take the
// chunks in turn: each of them spends most of its time waiting for one round trip through the switch.
template <typename T, int OP, bool EMU>
__global__ void __launch_bounds__(kNvlsBlock, 1) nvls_coll_kernel(const __grid_constant__ NvlsArgs a) {
  __shared__ int s_fail[9];                        // one per group of warps (3 stages x up to 3 groups)
  extern __shared__ __align__(128) unsigned char nv_smem[];      // two rings of kBulkStages x kBulkPiece bytes (fill, out), then their mbarriers
  uint64_t* const nv_mbar = reinterpret_cast<uint64_t*>(nv_smem + 2 * kBulkStages * kBulkPiece);
  const int vr = blockIdx.x / a.n_cta, cta = blockIdx.x - vr * a.n_cta;
  const NvlsRank& R = a.r[vr];
  const Switch<T, OP, EMU> sw(a, R);
  if (threadIdx.x < 9) s_fail[threadIdx.x] = 0;
  if (threadIdx.x == 0 && a.use_bulk) {
    for (int i = 0; i < 2 * kBulkStages; i++) sm100::mbar_init(&nv_mbar[i], 1);
    sm100::fence_barrier_init();
  }
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
  // Threads per stage.  The stages that copy between a user buffer and the window are driven by one thread each (bulk copies)
  // when the buffers are 16-byte aligned, so they get few threads.  The stage that issues the multimem instructions is bound by
  // the round trip through the switch (its loads, then the acknowledgement of its stores before the counter may be raised), not
  // by the number of threads: it is split into kSub groups that take the chunks in turn, so that kSub chunks are in that stage
  // at the same time.
  // (On two or three ranks a rank's share of a chunk is too large for a third of the threads, and there is no gain: one group.)
  constexpr int kSub = 3, kSwitchThreads = 384;
  const int ksub = a.n_sub > 0 ? a.n_sub : 1;                 // 1 or kSub
  int nF = 64, nS = 0, nO = 64, subF = 1, subS = 1, subO = 1;
  switch (a.coll) {
    case COLL_ALLREDUCE: nS = kSwitchThreads; subS = ksub; break;
    case COLL_ALLGATHER: nF = kSwitchThreads; subF = ksub; nO = kNvlsBlock - nF; break;
    case COLL_REDUCE_SCATTER: nO = kSwitchThreads; subO = ksub; nF = kNvlsBlock - nO; break;
    case COLL_BROADCAST: if (!filler) { nF = 0; nO = kNvlsBlock; } else { nF = kSwitchThreads; subF = ksub; nO = kNvlsBlock - nF; } break;
    default: if (!consumer) { nF = kNvlsBlock; nO = 0; } else { nO = kSwitchThreads; subO = ksub; nF = kNvlsBlock - nO; } break;      // reduce
  }
  const int t = threadIdx.x;
  int role, sub = 0, nsub = 1; Role g;       // role: 0 fill, 1 switch, 2 out; group `sub` of `nsub` takes chunks sub, sub + nsub, ...
  if (t < nF) { role = 0; nsub = subF; g.nthr = nF / subF; sub = t / g.nthr; g.tid = t - sub * g.nthr; g.bar = 1 + sub; }
  else if (t < nF + nS) { role = 1; nsub = subS; g.nthr = nS / subS; sub = (t - nF) / g.nthr; g.tid = t - nF - sub * g.nthr; g.bar = 4 + sub; }
  else if (t < nF + nS + nO) { role = 2; nsub = subO; g.nthr = nO / subO; sub = (t - nF - nS) / g.nthr; g.tid = t - nF - nS - sub * g.nthr; g.bar = 7 + sub; }
  else { role = -1; g.tid = 1; g.nthr = 32; g.bar = 10; }
  int* const my_fail = &s_fail[role < 0 ? 0 : role * kSub + sub];

  // Moves nblk blocks of len bytes between a user buffer and the window: with the bulk-copy engine when everything is 16-byte
  // aligned (one thread drives it, the others go on to the group's barrier), with the group's loads and stores otherwise.
  BulkRing ring;
  ring.smem = nv_smem + (role == 2 ? kBulkStages * kBulkPiece : 0); ring.mbar = nv_mbar + (role == 2 ? kBulkStages : 0); ring.phase = 0;
  auto move = [&](char* dst, long long dst_stride, const char* src, long long src_stride, int nblk, long long len, bool from_window, long long chunk) {
    const bool aligned = (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | (uintptr_t)dst_stride | (uintptr_t)src_stride) & 15) == 0);
    if (!(aligned && a.use_bulk && len >= 16)) { copy_blocks<T, 8>(g, dst, dst_stride, src, src_stride, nblk, len, from_window); return; }
    if (g.tid != 0) return;
    // what other GPUs stored into the window was observed through a counter; the bulk-copy engine reads it through the asynchronous proxy
    if (from_window) asm volatile("fence.proxy.async;" ::: "memory");
    const bool landed = bulk_copy_blocks(ring, dst, dst_stride, src, src_stride, nblk, len, a.timeout_ns);
    for (long long b = len & ~15ll; b < len; b++)        // the bytes past the last whole pack (end of an all-reduce of an odd size)
      for (int q = 0; q < nblk; q++)
        dst[(long long)q * dst_stride + b] = from_window ? *reinterpret_cast<const volatile char*>(src + (long long)q * src_stride + b) : src[(long long)q * src_stride + b];
    if (!landed) {
      if (atomicCAS(R.abort_flag, 0, 1) == 0) {
        piccl_status_t* st = R.status;
        st->code = 8; st->rank = R.rank; st->cta = cta; st->action = role; st->peer = -1; st->segment = (int)chunk; st->want = 0; st->have = 0;
        __threadfence_system();
        st->aborted = 1;
        __threadfence_system();
      }
      *my_fail = 1;
    }
  };

  // stopwatch of each group's thread 0 (PICCL_NVLS_PROFILE=1): the time since the last lap goes to one profile slot
  const bool prof = R.prof != nullptr && role >= 0 && g.tid == 0 && m > 0;
  unsigned long long t_last = prof ? nv_time_ns() : 0, t_first = t_last, acc[6] = {0, 0, 0, 0, 0, 0};
  auto lap = [&](int slot_id) { if (prof) { const unsigned long long now = nv_time_ns(); acc[slot_id] += now - t_last; t_last = now; } };

  if (role == 0 && filler) {
    for (long long j = sub; j < m; j += nsub) {
      const int p = (int)(j % D);
      const unsigned long long u = used[p] + (unsigned long long)(j / D);
      const long long off = off_of(j), len = len_of(j);
      // nobody reads the previous use of this part any more
      if (!nv_wait(a, R, g, cta, flag(p, NVC_CONSUMED), N * u, NVC_CONSUMED, cta + j * a.n_cta, my_fail)) break;
      lap(NVP_WAIT_CONSUMED);
      switch (a.coll) {
        case COLL_ALLGATHER: store_all<T>(sw, g, part(p) + (long long)rank * a.sub_stride, in + off, len); break;
        case COLL_BROADCAST: store_all<T>(sw, g, part(p), in + off, len); break;
        case COLL_REDUCE_SCATTER: move(R.uc + part(p), a.sub_stride, in + off, a.bytes, n, len, false, cta + j * a.n_cta); break;
        default: move(R.uc + part(p), 0, in + off, 0, 1, len, false, cta + j * a.n_cta); break;      // all-reduce, reduce
      }
      nv_arrive(sw, g, flag(p, NVC_FILLED), fill_inc, (a.coll == COLL_ALLGATHER || a.coll == COLL_BROADCAST) ? ARRIVE_REMOTE : ARRIVE_LOCAL, a.strict_fences != 0);
      lap(NVP_FILL);
    }
  } else if (role == 1 && allreduce) {
    for (long long j = sub; j < m; j += nsub) {
      const int p = (int)(j % D);
      const unsigned long long u = used[p] + (unsigned long long)(j / D);
      const long long len = len_of(j);
      // every rank has copied chunk j in
      if (!nv_wait(a, R, g, cta, flag(p, NVC_FILLED), N * (u + 1), NVC_FILLED, cta + j * a.n_cta, my_fail)) break;
      lap(NVP_WAIT_FILLED);
      const int npack = (int)((len + 15) >> 4);          // the bytes past `len` in the last pack are summed too and never copied out
      const int per = (npack + n - 1) / n;
      int lo = rank * per; if (lo > npack) lo = npack;
      int hi = lo + per; if (hi > npack) hi = npack;
      reduce_to_all<T>(sw, g, part(p), lo, hi, scale_on, a.scale);
      nv_arrive(sw, g, flag(p, NVC_REDUCED), 1, ARRIVE_REMOTE, a.strict_fences != 0);
      lap(NVP_SWITCH);
    }
  } else if (role == 2 && consumer) {
    for (long long j = sub; j < m; j += nsub) {
      const int p = (int)(j % D);
      const unsigned long long u = used[p] + (unsigned long long)(j / D), uy = used[kNvlsMaxDepth + p] + (unsigned long long)(j / D);
      const long long off = off_of(j), len = len_of(j);
      if (allreduce) {
        // every rank has written its share of the sums of chunk j
        if (!nv_wait(a, R, g, cta, flag(p, NVC_REDUCED), N * (uy + 1), NVC_REDUCED, cta + j * a.n_cta, my_fail)) break;
        lap(NVP_WAIT_REDUCED);
      } else {
        if (!nv_wait(a, R, g, cta, flag(p, NVC_FILLED), N * (u + 1), NVC_FILLED, cta + j * a.n_cta, my_fail)) break;
        lap(NVP_WAIT_FILLED);
      }
      switch (a.coll) {
        case COLL_ALLGATHER: move(out + off, a.bytes, R.uc + part(p), a.sub_stride, n, len, true, cta + j * a.n_cta); break;
        case COLL_BROADCAST: if (!(rank == a.root && in == out)) move(out + off, 0, R.uc + part(p), 0, 1, len, true, cta + j * a.n_cta); break;
        case COLL_REDUCE_SCATTER: reduce_to_local<T>(sw, g, part(p) + (long long)rank * a.sub_stride, out + off, len, scale_on, a.scale); break;
        case COLL_REDUCE: reduce_to_local<T>(sw, g, part(p), out + off, len, scale_on, a.scale); break;
        default: move(out + off, 0, R.uc + part(p), 0, 1, len, true, cta + j * a.n_cta); break;        // all-reduce
      }
      nv_arrive(sw, g, flag(p, NVC_CONSUMED), cons_inc, ARRIVE_READ, a.strict_fences != 0);
      lap(NVP_OUT);
    }
  }
  if (prof) {
    for (int i = 0; i < 6; i++) if (acc[i]) atomicAdd(R.prof + i, acc[i]);
    if ((role == 2 && sub == 0) || (role == 0 && sub == 0 && !consumer)) { atomicAdd(R.prof + NVP_CHUNKS, (unsigned long long)m); atomicAdd(R.prof + NVP_CTAS, 1ull); atomicAdd(R.prof + NVP_TOTAL, nv_time_ns() - t_first); }
  }
  __syncthreads();                                    // every group is done with `used`
  int any_fail = 0;
  for (int i = 0; i < 9; i++) any_fail |= s_fail[i];
  if (threadIdx.x == 0 && m > 0 && !any_fail) {
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

constexpr size_t kNvlsSmemBytes = 2 * (size_t)kBulkStages * kBulkPiece + 2 * kBulkStages * sizeof(uint64_t) + 32;

// the kernels take more dynamic shared memory than the default limit allows: raised once per kernel (and per device: the attribute is per context)
static bool allow_smem(const void* fn) {
  static std::mutex mu; static std::set<std::pair<const void*, int>> done;
  int dev = 0; cudaGetDevice(&dev);
  std::lock_guard<std::mutex> l(mu);
  if (done.count({fn, dev})) return true;
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kNvlsSmemBytes) != cudaSuccess) { cudaGetLastError(); return false; }
  done.insert({fn, dev});
  return true;
}

int nvls_max_resident_ctas(bool emulate) {
  const void* fn = emulate ? kernel_of<true>(DT_F32, 0) : kernel_of<false>(DT_F32, 0);
  int per_sm = 0, dev = 0, sms = 0;
  allow_smem(fn);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kNvlsBlock, kNvlsSmemBytes) != cudaSuccess) { cudaGetLastError(); per_sm = 1; }
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return (per_sm > 0 ? per_sm : 1) * (sms > 0 ? sms : 1);
}

int nvls_launch(const NvlsArgs& a, int dtype, int op, bool emulate, void* stream) {
  void* args[] = {const_cast<NvlsArgs*>(&a)};
  const void* fn = emulate ? kernel_of<true>(dtype, op) : kernel_of<false>(dtype, op);
  if (!fn) return (int)cudaErrorInvalidValue;
  if (!allow_smem(fn)) return (int)cudaErrorInvalidValue;
  if (emulate) return (int)cudaLaunchCooperativeKernel(fn, dim3(a.n_vrank * a.n_cta), dim3(kNvlsBlock), args, kNvlsSmemBytes, (cudaStream_t)stream);
  return (int)cudaLaunchKernel(fn, dim3(a.n_cta), dim3(kNvlsBlock), args, kNvlsSmemBytes, (cudaStream_t)stream);
}

}  // namespace piccl
