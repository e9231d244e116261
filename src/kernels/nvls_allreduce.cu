// Kernel of the in-switch all-reduce; protocol and window layout in nvls.cuh.
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
// data that the switch wrote into this GPU's memory: read past L1
__device__ __forceinline__ uint4 nv_ld_volatile(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// ld: sum over all copies of the 16 bytes at `mc`; st: 16 bytes written to all copies
template <typename T> struct Mm;
template <> struct Mm<float> {
  static __device__ __forceinline__ uint4 ld(const char* mc) {
    float a, b, c, d;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(a), "=f"(b), "=f"(c), "=f"(d) : "l"(mc) : "memory");
    return make_uint4(__float_as_uint(a), __float_as_uint(b), __float_as_uint(c), __float_as_uint(d));
  }
  static __device__ __forceinline__ void st(char* mc, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)),
                 "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)) : "memory");
  }
};
template <> struct Mm<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld(const char* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
  static __device__ __forceinline__ void st(char* mc, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};
template <> struct Mm<__half> {
  static __device__ __forceinline__ uint4 ld(const char* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
  static __device__ __forceinline__ void st(char* mc, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};

// packs [lo, hi) of the slot: in-switch sum, then the sum to every copy; 4 loads in flight per thread
template <typename T>
__device__ __forceinline__ void reduce_bcast(char* mc_slot, long long lo, long long hi) {
  constexpr int U = 4;
  const long long nt = blockDim.x;
  const long long done = lo + ((hi - lo) / (nt * U)) * (nt * U);
  for (long long base = lo + threadIdx.x; base < done; base += nt * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; u++) v[u] = Mm<T>::ld(mc_slot + (base + u * nt) * 16);
#pragma unroll
    for (int u = 0; u < U; u++) Mm<T>::st(mc_slot + (base + u * nt) * 16, v[u]);
  }
  for (long long p = done + threadIdx.x; p < hi; p += nt) { uint4 v = Mm<T>::ld(mc_slot + p * 16); Mm<T>::st(mc_slot + p * 16, v); }
}

template <typename T> __device__ __forceinline__ float nv_up(T v);
template <> __device__ __forceinline__ float nv_up<float>(float v) { return v; }
template <> __device__ __forceinline__ float nv_up<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float nv_up<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T nv_down(float v);
template <> __device__ __forceinline__ float nv_down<float>(float v) { return v; }
template <> __device__ __forceinline__ __half nv_down<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 nv_down<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// user buffer -> slot.  `len` bytes, a multiple of sizeof(T); the slot is 16-byte aligned, the user buffer need not be.
template <typename T>
__device__ __forceinline__ void copy_in(char* slot, const char* src, long long len, bool scale_on, float scale) {
  constexpr int N = 16 / sizeof(T);
  const long long npack = len / 16;
  if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    for (long long p = threadIdx.x; p < npack; p += blockDim.x) {
      union { uint4 v; T t[N]; } u;
      u.v = *reinterpret_cast<const uint4*>(src + p * 16);
      if (scale_on) {
#pragma unroll
        for (int i = 0; i < N; i++) u.t[i] = nv_down<T>(nv_up<T>(u.t[i]) * scale);
      }
      *reinterpret_cast<uint4*>(slot + p * 16) = u.v;
    }
    const long long done = npack * N, nelem = len / (long long)sizeof(T);
    for (long long i = done + threadIdx.x; i < nelem; i += blockDim.x) {
      T v = reinterpret_cast<const T*>(src)[i];
      reinterpret_cast<T*>(slot)[i] = scale_on ? nv_down<T>(nv_up<T>(v) * scale) : v;
    }
  } else {
    const long long nelem = len / (long long)sizeof(T);
    for (long long i = threadIdx.x; i < nelem; i += blockDim.x) {
      T v = reinterpret_cast<const T*>(src)[i];
      reinterpret_cast<T*>(slot)[i] = scale_on ? nv_down<T>(nv_up<T>(v) * scale) : v;
    }
  }
}

// slot -> user buffer
template <typename T>
__device__ __forceinline__ void copy_out(char* dst, const char* slot, long long len) {
  constexpr int N = 16 / sizeof(T);
  const long long nelem = len / (long long)sizeof(T);
  if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    const long long npack = len / 16;
    for (long long p = threadIdx.x; p < npack; p += blockDim.x) *reinterpret_cast<uint4*>(dst + p * 16) = nv_ld_volatile(slot + p * 16);
    for (long long i = npack * N + threadIdx.x; i < nelem; i += blockDim.x) reinterpret_cast<T*>(dst)[i] = reinterpret_cast<const volatile T*>(slot)[i];
  } else {
    for (long long i = threadIdx.x; i < nelem; i += blockDim.x) reinterpret_cast<T*>(dst)[i] = reinterpret_cast<const volatile T*>(slot)[i];
  }
}

// Thread 0 announces this rank on every copy of the counter and waits until the own copy shows all ranks.
// Returns false (for the whole CTA) if the wait ran out or the communicator was aborted.
__device__ __forceinline__ bool nvls_barrier(const NvlsArgs& a, int cta, unsigned long long target, int phase, long long chunk, int* s_fail) {
  __syncthreads();                                   // the CTA's writes of the phase before are issued
  if (threadIdx.x == 0) {
    unsigned long long* mc_flag = reinterpret_cast<unsigned long long*>(a.mc + (long long)cta * 128);
    const unsigned long long* uc_flag = reinterpret_cast<const unsigned long long*>(a.uc + (long long)cta * 128);
    __threadfence_system();
    asm volatile("multimem.red.release.sys.global.add.u64 [%0], %1;" ::"l"(mc_flag), "l"(1ull) : "memory");
    unsigned long long t0 = 0, have = 0;
    bool ok = false, timed_out = false;
    for (unsigned spins = 1;; spins++) {
      have = nv_ld_acquire(uc_flag);
      if (have >= target) { ok = true; break; }
      if ((spins & 31u) == 0) {
        if (*(volatile int*)a.abort_flag) break;
        unsigned long long now = nv_time_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > a.timeout_ns) { timed_out = true; break; }
      }
    }
    if (!ok) {
      if (timed_out && atomicCAS(a.abort_flag, 0, 1) == 0) {
        piccl_status_t* s = a.status;
        s->code = 4 + phase; s->rank = a.rank; s->cta = cta; s->action = phase; s->peer = -1; s->segment = (int)chunk;
        s->want = target; s->have = have;
        __threadfence_system();
        s->aborted = 1;
        __threadfence_system();
      }
      *s_fail = 1;
    }
  }
  __syncthreads();
  return *s_fail == 0;
}

// ---------------------------------------------------------------- pipelined variant
// Two half slots per CTA and four counters (A0, A1, B0, B1: barrier before / after the in-switch phase, per half slot), so that
// the copy-in of chunk j+1 runs while the other ranks finish the in-switch phase of chunk j:
//   copy_in(0); arrive A
//   for each chunk j (half slot s = j & 1):
//     wait A[s];  ld_reduce + st of my 1/n;  arrive B[s]
//     copy_in(j+1) into the other half slot;  arrive A[s^1]
//     wait B[s];  copy_out(j)
// A counter of half slot s is only touched for use t+1 after every rank has passed its wait of use t (see the notes on
// the hazards in the kernel), so "counter >= n * t" is exact.
template <typename T, int U>
__device__ __forceinline__ void copy_packs(char* dst, const char* src, long long npack, bool src_volatile, bool scale_on, float scale) {
  constexpr int N = 16 / sizeof(T);
  const long long nt = blockDim.x;
  const long long done = (npack / (nt * U)) * (nt * U);
  for (long long base = threadIdx.x; base < done; base += nt * U) {
    union { uint4 v; T t[N]; } u[U];
#pragma unroll
    for (int i = 0; i < U; i++) u[i].v = src_volatile ? nv_ld_volatile(src + (base + i * nt) * 16) : *reinterpret_cast<const uint4*>(src + (base + i * nt) * 16);
    if (scale_on) {
#pragma unroll
      for (int i = 0; i < U; i++) {
#pragma unroll
        for (int e = 0; e < N; e++) u[i].t[e] = nv_down<T>(nv_up<T>(u[i].t[e]) * scale);
      }
    }
#pragma unroll
    for (int i = 0; i < U; i++) *reinterpret_cast<uint4*>(dst + (base + i * nt) * 16) = u[i].v;
  }
  for (long long p = done + threadIdx.x; p < npack; p += nt) {
    union { uint4 v; T t[N]; } u;
    u.v = src_volatile ? nv_ld_volatile(src + p * 16) : *reinterpret_cast<const uint4*>(src + p * 16);
    if (scale_on) {
#pragma unroll
      for (int e = 0; e < N; e++) u.t[e] = nv_down<T>(nv_up<T>(u.t[e]) * scale);
    }
    *reinterpret_cast<uint4*>(dst + p * 16) = u.v;
  }
}

// user buffer -> slot and slot -> user buffer with 8 packs in flight per thread when both sides are 16-byte aligned
template <typename T>
__device__ __noinline__ void copy_in_fast(char* slot, const char* src, long long len, bool scale_on, float scale) {
  if ((reinterpret_cast<uintptr_t>(src) & 15) != 0) { copy_in<T>(slot, src, len, scale_on, scale); return; }
  const long long npack = len / 16;
  copy_packs<T, 8>(slot, src, npack, false, scale_on, scale);
  const long long nelem = len / (long long)sizeof(T);
  for (long long i = npack * (16 / (long long)sizeof(T)) + threadIdx.x; i < nelem; i += blockDim.x) {
    T v = reinterpret_cast<const T*>(src)[i];
    reinterpret_cast<T*>(slot)[i] = scale_on ? nv_down<T>(nv_up<T>(v) * scale) : v;
  }
}
template <typename T>
__device__ __noinline__ void copy_out_fast(char* dst, const char* slot, long long len) {
  if ((reinterpret_cast<uintptr_t>(dst) & 15) != 0) { copy_out<T>(dst, slot, len); return; }
  const long long npack = len / 16;
  copy_packs<T, 8>(dst, slot, npack, true, false, 1.0f);
  const long long nelem = len / (long long)sizeof(T);
  for (long long i = npack * (16 / (long long)sizeof(T)) + threadIdx.x; i < nelem; i += blockDim.x) reinterpret_cast<T*>(dst)[i] = reinterpret_cast<const volatile T*>(slot)[i];
}

// The CTA's writes so far are ordered before one more arrival on every copy of the counter.
__device__ __forceinline__ void nvls_arrive(const NvlsArgs& a, long long flag_off) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    asm volatile("multimem.red.release.sys.global.add.u64 [%0], %1;" ::"l"(a.mc + flag_off), "l"(1ull) : "memory");
  }
}
// Bounded wait of the whole CTA for `target` arrivals on the own copy of the counter.
__device__ __forceinline__ bool nvls_wait(const NvlsArgs& a, int cta, long long flag_off, unsigned long long target, int phase, long long chunk, int* s_fail) {
  if (threadIdx.x == 0) {
    const unsigned long long* uc_flag = reinterpret_cast<const unsigned long long*>(a.uc + flag_off);
    unsigned long long t0 = 0, have = 0;
    bool ok = false, timed_out = false;
    for (unsigned spins = 1;; spins++) {
      have = nv_ld_acquire(uc_flag);
      if (have >= target) { ok = true; break; }
      if ((spins & 31u) == 0) {
        if (*(volatile int*)a.abort_flag) break;
        unsigned long long now = nv_time_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > a.timeout_ns) { timed_out = true; break; }
      }
    }
    if (!ok) {
      if (timed_out && atomicCAS(a.abort_flag, 0, 1) == 0) {
        piccl_status_t* s = a.status;
        s->code = 4 + phase; s->rank = a.rank; s->cta = cta; s->action = phase; s->peer = -1; s->segment = (int)chunk;
        s->want = target; s->have = have;
        __threadfence_system();
        s->aborted = 1;
        __threadfence_system();
      }
      *s_fail = 1;
    }
  }
  __syncthreads();
  return *s_fail == 0;
}

template <typename T>
__global__ void __launch_bounds__(kNvlsBlock, 2) nvls_allreduce_pipe_kernel(const NvlsArgs a) {
  __shared__ int s_fail;
  const int cta = blockIdx.x;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const long long nchunks = (a.bytes + a.chunk_bytes - 1) / a.chunk_bytes;
  const long long m = cta < nchunks ? (nchunks - cta + a.n_cta - 1) / a.n_cta : 0;          // chunks of this CTA
  const long long half = (a.slot_bytes / 2) / 16 * 16;        // second half slot, 16-byte aligned for any rank count
  char* const my0 = a.uc + kNvlsFlagBytes + (long long)cta * a.slot_bytes;
  char* const mc0 = a.mc + kNvlsFlagBytes + (long long)cta * a.slot_bytes;
  // counters of this CTA index: A0, A1, B0, B1
  const long long flag0 = kNvlsPipeFlagOff + (long long)cta * 4 * 128;
  unsigned long long* const used = a.bar_count + kNvlsMaxCta + cta * 2;                      // uses of half slot 0 / 1 so far
  const unsigned long long base[2] = {used[0], used[1]};
  const unsigned long long n = (unsigned long long)a.nranks;
  auto off_of = [&](long long j) { return (cta + j * a.n_cta) * a.chunk_bytes; };
  auto len_of = [&](long long j) { long long o = off_of(j); return (a.bytes - o < a.chunk_bytes) ? a.bytes - o : a.chunk_bytes; };
  if (m > 0) {
    copy_in_fast<T>(my0, static_cast<const char*>(a.in) + off_of(0), len_of(0), a.avg != 0, a.scale);
    nvls_arrive(a, flag0);
  }
  for (long long j = 0; j < m; j++) {
    const int s = (int)(j & 1);
    const unsigned long long target = n * (base[s] + (unsigned long long)(j >> 1) + 1);
    const long long len = len_of(j);
    // every rank has copied chunk j in.  (All threads are past copy_out(j-1): each wait ends with a CTA barrier.)
    if (!nvls_wait(a, cta, flag0 + s * 128, target, 1, cta + j * a.n_cta, &s_fail)) break;
    {
      const long long npack = (len + 15) / 16;
      const long long per = (npack + a.nranks - 1) / a.nranks;
      long long lo = (long long)a.rank * per; if (lo > npack) lo = npack;
      long long hi = lo + per; if (hi > npack) hi = npack;
      reduce_bcast<T>(mc0 + s * half, lo, hi);
    }
    nvls_arrive(a, flag0 + (2 + s) * 128);
    // The other half slot is free: this rank copied chunk j-1 out of it, and every rank's in-switch phase of chunk j-1
    // (which read it and wrote the sums into it) ended before that rank's arrival at B, which this rank waited for.
    if (j + 1 < m) {
      copy_in_fast<T>(my0 + (s ^ 1) * half, static_cast<const char*>(a.in) + off_of(j + 1), len_of(j + 1), a.avg != 0, a.scale);
      nvls_arrive(a, flag0 + (s ^ 1) * 128);
    }
    // every rank has written its share of the sums of chunk j
    if (!nvls_wait(a, cta, flag0 + (2 + s) * 128, target, 2, cta + j * a.n_cta, &s_fail)) break;
    copy_out_fast<T>(static_cast<char*>(a.out) + off_of(j), my0 + s * half, len);
  }
  if (threadIdx.x == 0 && m > 0) { used[0] = base[0] + (unsigned long long)((m + 1) / 2); used[1] = base[1] + (unsigned long long)(m / 2); }
}

template <typename T>
__global__ void __launch_bounds__(kNvlsBlock, 2) nvls_allreduce_kernel(const NvlsArgs a) {
  __shared__ int s_fail;
  const int cta = blockIdx.x;
  if (threadIdx.x == 0) s_fail = 0;
  unsigned long long nbar = a.bar_count[cta];
  char* const my_slot = a.uc + kNvlsFlagBytes + (long long)cta * a.slot_bytes;
  char* const mc_slot = a.mc + kNvlsFlagBytes + (long long)cta * a.slot_bytes;
  const long long nchunks = (a.bytes + a.chunk_bytes - 1) / a.chunk_bytes;
  const unsigned long long n = (unsigned long long)a.nranks;
  for (long long k = cta; k < nchunks; k += a.n_cta) {
    const long long off = k * a.chunk_bytes;
    const long long len = (a.bytes - off < a.chunk_bytes) ? a.bytes - off : a.chunk_bytes;
    copy_in<T>(my_slot, static_cast<const char*>(a.in) + off, len, a.avg != 0, a.scale);
    nbar++;
    if (!nvls_barrier(a, cta, nbar * n, 1, k, &s_fail)) break;
    {
      const long long npack = (len + 15) / 16;                   // the bytes past `len` in the last pack are summed too and never copied out
      const long long per = (npack + a.nranks - 1) / a.nranks;
      long long lo = (long long)a.rank * per; if (lo > npack) lo = npack;
      long long hi = lo + per; if (hi > npack) hi = npack;
      reduce_bcast<T>(mc_slot, lo, hi);
    }
    nbar++;
    if (!nvls_barrier(a, cta, nbar * n, 2, k, &s_fail)) break;
    copy_out<T>(static_cast<char*>(a.out) + off, my_slot, len);
    __syncthreads();                                             // the slot is free for the next chunk
  }
  if (threadIdx.x == 0) a.bar_count[cta] = nbar;
}

}  // namespace

bool nvls_dtype_supported(int dtype) { return dtype == DT_F32 || dtype == DT_F16 || dtype == DT_BF16; }

int nvls_launch(const NvlsArgs& a, int dtype, void* stream) {
  void* args[] = {const_cast<NvlsArgs*>(&a)};
  const void* fn = nullptr;
  if (a.pipelined) fn = dtype == DT_F32 ? (const void*)nvls_allreduce_pipe_kernel<float> : dtype == DT_F16 ? (const void*)nvls_allreduce_pipe_kernel<__half>
                      : dtype == DT_BF16 ? (const void*)nvls_allreduce_pipe_kernel<__nv_bfloat16> : nullptr;
  else fn = dtype == DT_F32 ? (const void*)nvls_allreduce_kernel<float> : dtype == DT_F16 ? (const void*)nvls_allreduce_kernel<__half>
          : dtype == DT_BF16 ? (const void*)nvls_allreduce_kernel<__nv_bfloat16> : nullptr;
  if (!fn) return (int)cudaErrorInvalidValue;
  return (int)cudaLaunchKernel(fn, dim3(a.n_cta), dim3(kNvlsBlock), args, 0, (cudaStream_t)stream);
}

}  // namespace piccl
