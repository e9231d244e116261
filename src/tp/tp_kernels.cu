// Fused tensor-parallel kernels: one launch does the tcgen05 GEMM AND the
// collective that follows or precedes it, tile by tile, over peer memory.
//
//  gemm_rs   C = A_r · B_r^T per rank, summed over ranks, row block r kept by rank r.
//            Every CTA runs the persistent GEMM; tiles owned by OTHER ranks come first and their
//            epilogue stores the bf16 partial tile straight into the owner's heap (plain peer
//            stores over NVLink) and raises a per-(source, tile) epoch flag.  The rank's OWN tiles
//            come last: their epilogue waits (bounded) for the n-1 partials of that tile, adds them
//            in rank order to the accumulator it just read from TMEM, and writes the final result.
//            No partial of an own tile ever goes to memory; transfer overlaps the remaining MMA work.
//  ag_gemm   A is row-sharded over ranks; C = concat(A_r) · B^T.  A few "feeder" CTAs push this
//            rank's shard, 128 rows at a time, into every peer's gathered buffer (nearest consumer
//            first) and raise per-(source, row block) flags; the GEMM CTAs start on the local shard
//            and gate the TMA loads of a remote row block on its flag.  TMA only ever reads LOCAL
//            memory (the local shard or the local gathered buffer), never a peer's.
//
// Buffers are double buffered by call parity, flags carry the call epoch, so nothing is reset
// between calls.  All waits are bounded; a wait that gives up is reported through
// piccl_tp_status().  The reference has no GEMM at all; the comparison is cuBLAS + NCCL.
#include <cuda_bf16.h>
#include <algorithm>
#include <cstring>
#include "../include/sm100_gemm.cuh"
#include "../runtime/comm.h"

namespace piccl {

using namespace sm100;
typedef __nv_bfloat16 bf16;
constexpr int TP_BN = 256, TP_STAGES = 4, TP_MAX_RANKS = 8;
constexpr int RS_STAGES = 3, RS_STAGING = GEMM_BM * TP_BN * 2;   // reduce-scatter: one ring stage gives way to a 64 KiB staging tile

__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ void st_release_sys_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait until *flag == epoch.
__device__ __forceinline__ bool wait_flag(const unsigned* flag, unsigned epoch, volatile int* abort_flag) {
  unsigned long long t0 = 0;
  for (unsigned it = 1;; it++) {
    if (ld_acquire_sys_u32(flag) == epoch) return true;
    if ((it & 63u) == 0) {
      if (*abort_flag) return false;
      unsigned long long now = gtime_ns();
      if (!t0) t0 = now; else if (now - t0 > kGemmWaitLimitNs) return false;
    }
  }
}

struct TpRank {
  CUtensorMap ta;            // gemm_rs: A [M, K_local];   ag_gemm: local shard [M/n, K]
  CUtensorMap ta2;           // ag_gemm: gathered buffer [2*M, K] in this rank's heap
  CUtensorMap tb;
  char* heap[TP_MAX_RANKS];  // all ranks' heaps as mapped here
  const bf16* a_shard;       // ag_gemm: the local shard (feeder source)
  bf16* out;
  int* status;
  int rank;
};
struct TpArgs {
  int n, M, N, K;            // gemm_rs: K = K_local, N full;  ag_gemm: N = N_local, K full
  int ctas_per_rank, n_feed;
  unsigned epoch;
  long long flag_off, data_off;
  TpRank r[TP_MAX_RANKS];    // one entry per virtual rank of the launch
};

// ------------------------------------------------------------------ GEMM -> reduce-scatter
struct RsPolicy {
  const TpRank* R; int n, rank, N, mb_per_owner, num_n, tiles_per_owner, parity; unsigned epoch;
  long long flag_off, data_off; int* s_ok; uint8_t* staging;
  static constexpr int STAGING = RS_STAGING;
  __device__ void set_staging(uint8_t* p) { staging = p; }
  // A tile travels as 128 rows of 512 bytes; inside every 128-byte group the 16-byte pieces are XOR-ed with the
  // row number, which makes the epilogue's shared-memory stores conflict free.  Writer and reader use the same map.
  __device__ static int piece_off(int row, int piece) { return row * (TP_BN * 2) + (((piece & ~7) | ((piece & 7) ^ (row & 7))) << 4); }
  __device__ int num_tiles() const { return n * tiles_per_owner; }
  // Order: panels of 16 column blocks (one panel of B stays in L2); inside a panel the owners (rank+1, rank+2, ..., myself
  // last); inside an owner's block rows fastest.  All ranks walk the panels in the same order, so the partials of my own
  // tiles of a panel are on their way while I still compute the other owners' tiles of that panel.
  __device__ void tile(int idx, int& m_blk, int& n_blk) const {
    constexpr int PN = 16;
    const int per_panel = PN * mb_per_owner * n;              // tiles of a full panel
    const int panel = idx / per_panel; int within = idx % per_panel;
    const int cols = min(PN, num_n - panel * PN);             // last panel may be narrower
    const int per_owner = cols * mb_per_owner;
    const int owner = (rank + 1 + within / per_owner) % n; within %= per_owner;
    m_blk = owner * mb_per_owner + within % mb_per_owner; n_blk = panel * PN + within / mb_per_owner;
  }
  __device__ const CUtensorMap* a_map(int m_blk, int& row0) const { row0 = m_blk * GEMM_BM; return &R->ta; }
  __device__ bool gate(int, volatile int*) const { return true; }
  __device__ int tile_id(int m_blk, int n_blk) const { return (m_blk % mb_per_owner) + n_blk * mb_per_owner; }
  __device__ unsigned* flag_ptr(int owner, int src, int tid_) const {
    return reinterpret_cast<unsigned*>(R->heap[owner] + flag_off) + ((size_t)(parity * n + src) * tiles_per_owner + tid_);
  }
  __device__ bf16* inbox(int owner, int src, int tid_) const {
    return reinterpret_cast<bf16*>(R->heap[owner] + data_off) + ((size_t)src * tiles_per_owner + tid_) * (size_t)(GEMM_BM * TP_BN);      // data_off: this call's half of the region
  }
  __device__ bool tile_begin(int m_blk, int n_blk, int et, volatile int* abort_flag) {
    if (m_blk / mb_per_owner != rank) return true;
    // own tile: all other ranks' partials of this tile must have landed
    if (et == 0) *s_ok = 1;
    epilogue_barrier();
    if (et < n && et != rank && !wait_flag(flag_ptr(rank, et, tile_id(m_blk, n_blk)), epoch, abort_flag)) *s_ok = 0;
    epilogue_barrier();
    return *s_ok != 0;
  }
  __device__ void store(int m_blk, int n_blk, int row, int col0, float (&v)[32]) {
    const int owner = m_blk / mb_per_owner, t = tile_id(m_blk, n_blk);
    if (owner != rank) {
      // remote tile: into the staging tile; tile_end ships it with one bulk store
#pragma unroll
      for (int j = 0; j < 4; j++) {
        uint4 o; __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int q = 0; q < 4; q++) o2[q] = __floats2bfloat162_rn(v[8 * j + 2 * q], v[8 * j + 2 * q + 1]);
        *reinterpret_cast<uint4*>(staging + piece_off(row, col0 / 8 + j)) = o;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // these stores must be visible to the bulk-copy engine
      return;
    }
    float sum[32];
#pragma unroll
    for (int i = 0; i < 32; i++) sum[i] = 0.f;
    for (int src = 0; src < n; src++) {            // rank order: the same result whatever the arrival order
      if (src == rank) {
#pragma unroll
        for (int i = 0; i < 32; i++) sum[i] += v[i];
      } else {
        const char* tile = reinterpret_cast<const char*>(inbox(rank, src, t));
#pragma unroll
        for (int j = 0; j < 4; j++) {
          uint4 b;
          asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(tile + piece_off(row, col0 / 8 + j)) : "memory");
          const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
          for (int q = 0; q < 4; q++) { float2 f = __bfloat1622float2(b2[q]); sum[8 * j + 2 * q] += f.x; sum[8 * j + 2 * q + 1] += f.y; }
        }
      }
    }
    store_row32_bf16(R->out + (size_t)((m_blk % mb_per_owner) * GEMM_BM + row) * N + (size_t)n_blk * TP_BN + col0, sum);
  }
  __device__ void tile_end(int m_blk, int n_blk, int et) {
    const int owner = m_blk / mb_per_owner;
    if (owner == rank) return;
    // all 128 threads have written the staging tile (barrier passed): one asynchronous bulk store moves the 64 KiB over NVLink
    if (et == 0) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      bulk_store(inbox(owner, rank, tile_id(m_blk, n_blk)), staging, RS_STAGING);
      bulk_commit();
      bulk_wait_all();                              // data written; then tell the owner
      asm volatile("fence.proxy.async;" ::: "memory");
      st_release_sys_u32(flag_ptr(owner, rank, tile_id(m_blk, n_blk)), epoch);
    }
    epilogue_barrier();                             // the staging tile is free again
  }
};

__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_rs_kernel(const __grid_constant__ TpArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ int s_abort, s_ok;
  const int vr = blockIdx.x / a.ctas_per_rank, cta = blockIdx.x % a.ctas_per_rank;
  const TpRank* R = &a.r[vr];
  if (threadIdx.x == 0) { s_abort = 0; s_ok = 1; tma_prefetch_desc(&R->ta); }
  RsPolicy pol{R, a.n, R->rank, a.N, a.M / a.n / GEMM_BM, a.N / TP_BN, (a.M / a.n / GEMM_BM) * (a.N / TP_BN), (int)(a.epoch & 1), a.epoch, a.flag_off, a.data_off, &s_ok, nullptr};
  gemm_persistent<TP_BN, RS_STAGES>(smem_raw, &R->tb, pol, a.K, cta, a.ctas_per_rank, R->status, &s_abort);
}

// ------------------------------------------------------------------ all-gather -> GEMM
struct AgPolicy {
  const TpRank* R; int n, rank, M, N, mb_per_shard, num_n, parity; unsigned epoch; long long flag_off;
  __device__ int num_tiles() const { return n * mb_per_shard * num_n; }
  __device__ void tile(int idx, int& m_blk, int& n_blk) const {
    const int per = mb_per_shard * num_n, src = (rank + idx / per) % n, within = idx % per;   // own shard first, then rank+1, ...
    m_blk = src * mb_per_shard + within / num_n; n_blk = within % num_n;
  }
  __device__ const CUtensorMap* a_map(int m_blk, int& row0) const {
    if (m_blk / mb_per_shard == rank) { row0 = (m_blk % mb_per_shard) * GEMM_BM; return &R->ta; }
    row0 = m_blk * GEMM_BM; return &R->ta2;             // ta2 covers this call's half of the region
  }
  __device__ bool gate(int m_blk, volatile int* abort_flag) const {
    const int src = m_blk / mb_per_shard;
    if (src == rank) return true;
    const unsigned* f = reinterpret_cast<const unsigned*>(R->heap[rank] + flag_off) + ((size_t)(parity * n + src) * mb_per_shard + m_blk % mb_per_shard);
    if (!wait_flag(f, epoch, abort_flag)) return false;
    asm volatile("fence.proxy.async;" ::: "memory");   // the rows were written with ordinary stores; TMA reads them through the async proxy
    return true;
  }
  static constexpr int STAGING = 0;
  __device__ void set_staging(uint8_t*) {}
  __device__ bool tile_begin(int, int, int, volatile int*) { return true; }
  __device__ void tile_end(int, int, int) {}
  __device__ void store(int m_blk, int n_blk, int row, int col0, float (&v)[32]) {
    store_row32_bf16(R->out + (size_t)(m_blk * GEMM_BM + row) * N + (size_t)n_blk * TP_BN + col0, v);
  }
};

// Feeder CTAs: copy row blocks of the local shard into the peers' gathered buffers.
__device__ void ag_feed(const TpArgs& a, const TpRank* R, int feeder, int n_feed) {
  const int n = a.n, rank = R->rank, mbs = a.M / n / GEMM_BM, parity = a.epoch & 1;
  const size_t block_bytes = (size_t)GEMM_BM * a.K * 2;
  const int pairs = (n - 1) * mbs;
  for (int p = feeder; p < pairs; p += n_feed) {
    const int d = 1 + p / mbs, mb = p % mbs;             // distance-major: the peer that needs my shard next comes first
    const int dest = (rank - d + n) % n;
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(R->a_shard) + (size_t)mb * block_bytes);
    uint4* dst = reinterpret_cast<uint4*>(R->heap[dest] + a.data_off + ((size_t)rank * (a.M / n) + (size_t)mb * GEMM_BM) * a.K * 2);
    const size_t nvec = block_bytes / 16;
    size_t i = threadIdx.x;
    for (; i + 7 * GEMM_THREADS < nvec; i += 8 * GEMM_THREADS) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; u++) v[u] = src[i + u * GEMM_THREADS];
#pragma unroll
      for (int u = 0; u < 8; u++) dst[i + u * GEMM_THREADS] = v[u];
    }
    for (; i < nvec; i += GEMM_THREADS) dst[i] = src[i];
    __syncthreads();
    if (threadIdx.x == 0)
      st_release_sys_u32(reinterpret_cast<unsigned*>(R->heap[dest] + a.flag_off) + ((size_t)(parity * n + rank) * mbs + mb), a.epoch);
  }
}

__global__ void __launch_bounds__(GEMM_THREADS, 1) ag_gemm_kernel(const __grid_constant__ TpArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ int s_abort;
  const int vr = blockIdx.x / a.ctas_per_rank, cta = blockIdx.x % a.ctas_per_rank;
  const TpRank* R = &a.r[vr];
  if (cta < a.n_feed) { ag_feed(a, R, cta, a.n_feed); return; }     // feeders come first in the grid so they start first
  if (threadIdx.x == 0) { s_abort = 0; tma_prefetch_desc(&R->ta); tma_prefetch_desc(&R->ta2); }
  AgPolicy pol{R, a.n, R->rank, a.M, a.N, a.M / a.n / GEMM_BM, a.N / TP_BN, (int)(a.epoch & 1), a.epoch, a.flag_off};
  gemm_persistent<TP_BN, TP_STAGES>(smem_raw, &R->tb, pol, a.K, cta - a.n_feed, a.ctas_per_rank - a.n_feed, R->status, &s_abort);
}

// ------------------------------------------------------------------ host
// The workspace is used in four quarters: [kernel: gemm_rs, ag_gemm][parity of that kernel's call count].
static long long tp_quarter(long long tp_bytes) { return tp_bytes / 4 / 1024 * 1024; }
static long long tp_need_per_call(int which, int nranks, int M, int N, int K) {
  if (which == 0) return (long long)nranks * ((long long)M / nranks / GEMM_BM) * (N / TP_BN) * (GEMM_BM * TP_BN * 2);     // [src][tile] bf16 tiles
  return (long long)M * K * 2;                                                                                              // [M][K] bf16
}

static int tp_common_checks(piccl_comm** cs, int n, int M, int N, int K, int which) {
  if (n < 1 || n > TP_MAX_RANKS) return fail(PICCL_INVALID_ARGUMENT, "1..%d communicators per launch", TP_MAX_RANKS);
  piccl_comm* c = cs[0];
  if (c->nranks > TP_MAX_RANKS) return fail(PICCL_UNSUPPORTED, "fused tensor-parallel kernels support up to %d ranks", TP_MAX_RANKS);
  for (int i = 0; i < n; i++) if (!cs[i]->connected || cs[i]->broken) return fail(PICCL_INVALID_USAGE, "communicator not usable");
  if (M <= 0 || M % (GEMM_BM * c->nranks) || N % TP_BN || K % GEMM_BK || N <= 0 || K <= 0) return fail(PICCL_INVALID_ARGUMENT, "shape: M %% (128*ranks), N %% 256, K %% 64 must be 0");
  const long long nflags = which == 0 ? 2LL * c->nranks * (M / c->nranks / GEMM_BM) * (N / TP_BN) : 2LL * c->nranks * (M / c->nranks / GEMM_BM);
  if (nflags * 4 > (512 << 10)) return fail(PICCL_UNSUPPORTED, "too many tiles for the flag area");
  long long need = piccl_tp_workspace_bytes(which, c->nranks, M, N, K);
  if (tp_quarter(c->h_ctx.tp_bytes) < tp_need_per_call(which, c->nranks, M, N, K)) return fail(PICCL_INVALID_USAGE, "tensor-parallel workspace too small: %lld bytes needed, %lld configured (tp_bytes / PICCL_TP_MB)", need, c->h_ctx.tp_bytes);
  return PICCL_OK;
}

static int tp_launch(piccl_comm** cs, int n, const void* const* A, const void* const* B, void* const* out, int M, int N, int K, int which, cudaStream_t stream) {
  int rc = tp_common_checks(cs, n, M, N, K, which); if (rc) return rc;
  piccl_comm* c0 = cs[0];
  const int nr = c0->nranks;
  int prev = -1; cudaGetDevice(&prev); if (prev != c0->device) cudaSetDevice(c0->device);
  TpArgs a; memset(&a, 0, sizeof a);
  a.n = nr; a.M = M; a.N = N; a.K = K;
  a.flag_off = c0->h_ctx.tp_flag_off + (which ? (512 << 10) : 0);   // the two kernels keep their flags apart
  // ... and their payload: each kernel owns one half of the workspace, and each call one half of that, chosen by the parity of
  // the kernel's own call count.  The strides do not depend on the shape: a rank that is one call ahead (the other kernel, or
  // the same kernel with another shape) never writes where a peer still reads the call before.
  const long long quarter = tp_quarter(c0->h_ctx.tp_bytes);
  const unsigned next_epoch = (which ? c0->tp_epoch_ag : c0->tp_epoch_rs) + 1;
  a.data_off = c0->h_ctx.tp_data_off + (which ? 2 * quarter : 0) + (long long)(next_epoch & 1) * quarter;
  a.ctas_per_rank = std::max(1, c0->sm_count / n);
  a.n_feed = which ? std::min(std::max(1, env().tp_feeders), a.ctas_per_rank / 2) : 0;
  if (nr == 1) a.n_feed = 0;
  bool ok = true;
  for (int i = 0; i < n && ok; i++) {
    piccl_comm* c = cs[i];
    TpRank& R = a.r[i];
    R.rank = c->rank; R.out = (bf16*)out[i]; R.a_shard = (const bf16*)A[i];
    for (int p = 0; p < nr; p++) R.heap[p] = c->h_ctx.heap[p];
    if (!c->d_tp_status) { if (cudaMalloc(&c->d_tp_status, sizeof(int)) != cudaSuccess) { ok = false; break; } cudaMemset(c->d_tp_status, 0, sizeof(int)); }
    R.status = c->d_tp_status;
    if (which == 0) {
      ok &= make_tmap_bf16_k64(&R.ta, A[i], (uint64_t)M, (uint64_t)K, (uint64_t)K, GEMM_BM);
      R.ta2 = R.ta;
      a.epoch = ++c->tp_epoch_rs;
    } else {
      ok &= make_tmap_bf16_k64(&R.ta, A[i], (uint64_t)(M / nr), (uint64_t)K, (uint64_t)K, GEMM_BM);
      ok &= make_tmap_bf16_k64(&R.ta2, c->heap + a.data_off, (uint64_t)M, (uint64_t)K, (uint64_t)K, GEMM_BM);
      a.epoch = ++c->tp_epoch_ag;
    }
    ok &= make_tmap_bf16_k64(&R.tb, B[i], (uint64_t)N, (uint64_t)K, (uint64_t)K, TP_BN);
  }
  if (!ok) { if (prev != c0->device && prev >= 0) cudaSetDevice(prev); return fail(PICCL_CUDA_ERROR, "tensor map or status set-up failed"); }
  const int smem_bytes = which ? GemmSmem<TP_BN, TP_STAGES>::DYNAMIC : GemmSmem<TP_BN, RS_STAGES, RS_STAGING>::DYNAMIC;
  const void* fn = which ? (const void*)ag_gemm_kernel : (const void*)gemm_rs_kernel;
  static bool attr[2] = {false, false};
  if (!attr[which]) { if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) return fail(PICCL_CUDA_ERROR, "cannot get %d bytes of shared memory", smem_bytes); attr[which] = true; }
  void* args[] = {&a};
  cudaError_t e;
  // ranks wait for one another inside the kernel: several virtual ranks on one device must be co-resident
  if (n > 1) e = cudaLaunchCooperativeKernel(fn, dim3(n * a.ctas_per_rank), dim3(GEMM_THREADS), args, smem_bytes, stream);
  else e = cudaLaunchKernel(fn, dim3(a.ctas_per_rank), dim3(GEMM_THREADS), args, smem_bytes, stream);
  if (prev != c0->device && prev >= 0) cudaSetDevice(prev);
  if (e != cudaSuccess) return fail(PICCL_CUDA_ERROR, "fused kernel launch failed: %s", cudaGetErrorString(e));
  for (int i = 0; i < n; i++) cs[i]->stats.launches++;
  return PICCL_OK;
}

}  // namespace piccl

using namespace piccl;

extern "C" {

long long piccl_tp_workspace_bytes(int which, int nranks, int M, int N, int K) {
  // four quarters (two kernels x two calls in flight), each large enough for one call of this shape
  return 4 * ((tp_need_per_call(which, nranks, M, N, K) + 1023) / 1024 * 1024);
}
int piccl_gemm_rs(piccl_comm_t* c, const void* A, const void* B, void* out, int M, int N, int K_local, void* stream) {
  if (!c) return fail(PICCL_INVALID_ARGUMENT, "null communicator");
  const void* as[1] = {A}; const void* bs[1] = {B}; void* os[1] = {out}; piccl_comm* cs[1] = {c};
  return tp_launch(cs, 1, as, bs, os, M, N, K_local, 0, (cudaStream_t)stream);
}
int piccl_ag_gemm(piccl_comm_t* c, const void* A_shard, const void* B, void* out, int M, int N_local, int K, void* stream) {
  if (!c) return fail(PICCL_INVALID_ARGUMENT, "null communicator");
  const void* as[1] = {A_shard}; const void* bs[1] = {B}; void* os[1] = {out}; piccl_comm* cs[1] = {c};
  return tp_launch(cs, 1, as, bs, os, M, N_local, K, 1, (cudaStream_t)stream);
}
int piccl_gemm_rs_group(piccl_comm_t** comms, int n, const void* const* A, const void* const* B, void* const* out, int M, int N, int K_local, void* stream) {
  return tp_launch(comms, n, A, B, out, M, N, K_local, 0, (cudaStream_t)stream);
}
int piccl_ag_gemm_group(piccl_comm_t** comms, int n, const void* const* A_shard, const void* const* B, void* const* out, int M, int N_local, int K, void* stream) {
  return tp_launch(comms, n, A_shard, B, out, M, N_local, K, 1, (cudaStream_t)stream);
}
int piccl_tp_status(piccl_comm_t* c) {
  if (!c || !c->d_tp_status) return 0;
  int v = 0; cudaMemcpy(&v, c->d_tp_status, sizeof v, cudaMemcpyDeviceToHost);
  return v;
}

}  // extern "C"
