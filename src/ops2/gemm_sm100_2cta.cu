// bf16 GEMM for sm_100a on CTA PAIRS:  C[M,N] = A[M,K] · B[N,K]^T (+ bias), fp32 accumulation in TMEM.
//
// Two CTAs of a cluster (two SMs) work on one 256 x 256 tile of C with `tcgen05.mma.cta_group::2`:
// CTA v (0 = leader, 1 = follower) loads rows [128 v, 128 v + 128) of the A tile and rows
// [128 v, 128 v + 128) of the B tile, and ends up with rows [128 v, 128 v + 128) of the tile in its own
// TMEM.  Each SM therefore stages half of B per k-block: 32 KiB instead of the 48 KiB a lone CTA needs for
// the same work per SM, so the shared-memory ring is 6 k-blocks deep instead of 4 and the operand traffic
// out of L2 drops by a third.  That is the remedy for what the profile of the one-CTA kernel
// (src/ops/gemm_sm100.cu) shows: the tensor pipe waits for operands.
//
// Protocol (one ring of STAGES stages, two TMEM accumulators of 256 columns):
//   warp 0, both CTAs   TMA producer.  Waits for its own `empty[s]`, loads its A and B halves with
//                       `cp.async.bulk.tensor ... .cta_group::2`, whose byte count lands on the LEADER's `full[s]`
//                       (the leader's producer announces the bytes of both CTAs there).
//   warp 1, leader      one lane issues the MMAs of a k-block (M = 256, N = 256, K = 16 each; the hardware reads
//                       both CTAs' stages at the same offsets), then `tcgen05.commit` to `empty[s]` of BOTH CTAs;
//                       after the last k-block of a tile, `tcgen05.commit` to `tmem_full[a]` of both CTAs.
//   warps 2-5, both     epilogue: wait for the own `tmem_full[a]`, `tcgen05.ld` the own 128 rows, bias, bf16,
//                       store; then every thread arrives on the LEADER's `tmem_empty[a]` (256 arrivals).
//   TMEM                allocated and freed with `.cta_group::2` by warp 1 of both CTAs.
// Every wait is bounded (status word, CTA-wide abort flag); the cluster barrier at the end keeps a CTA alive
// while its partner may still read its shared memory or signal its barriers.
// This file issues `tcgen05.commit` with a CTA mask; it is built into a library of its own that is kept out of
// runs on several GPUs.  The reference has no GEMM at all.
#include <cuda_bf16.h>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include "../include/sm100_ptx.cuh"

namespace piccl_ops2 {

using namespace sm100;
typedef __nv_bfloat16 bf16;

constexpr int BM = 128, BN = 256, BK = 64;          // per CTA: 128 rows of A and C, 128 rows of B; per pair: 256 x 256
constexpr int STAGES = 6, THREADS = 192;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int BAR_OFF = STAGES * STAGE_BYTES;
constexpr int SMEM_TOTAL = BAR_OFF + (2 * STAGES + 4) * 8 + 16;
constexpr int SMEM_DYNAMIC = SMEM_TOTAL + 1024;    // slack for the 1024-byte alignment of the tiles
constexpr uint32_t TMEM_COLS = 2 * BN;
constexpr uint32_t kLeaderMask = 0xFEFFFFFFu;      // clears the bit that tells the two CTAs of a pair apart in a shared::cluster address
constexpr unsigned long long kWaitLimitNs = 4000000000ull;

__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Tile load of a CTA pair: the bytes are counted on the mbarrier at the same offset in the LEADER's shared memory.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar) & kLeaderMask), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {      // whole warp, in both CTAs, same warp index, same address
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[both CTAs' smem] * B[both CTAs' smem]; issued by one thread of the leader
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
               ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// The mbarrier at this offset in BOTH CTAs gets one arrival once all MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)), "h"(both) : "memory");
}
// One arrival on the mbarrier at this offset in the LEADER's shared memory (from either CTA).
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & kLeaderMask) : "memory");
}

// 256-row tiles in bands of 16, inside a band column blocks outer / row blocks inner (the pairs that run together share a band of A)
__device__ __forceinline__ void tile_of(int idx, int num_m, int num_n, int& m_blk, int& n_blk) {
  constexpr int GM = 16;
  const int per_band = GM * num_n, band = idx / per_band, within = idx % per_band;
  const int rows = min(GM, num_m - band * GM);
  m_blk = band * GM + within % rows; n_blk = within / rows;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_bf16_nt_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, bf16* __restrict__ C,
                         const bf16* __restrict__ bias, int M, int N, int K, int* __restrict__ status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ int s_abort_store;
  volatile int* s_abort = &s_abort_store;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + BAR_OFF);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t v = cluster_ctarank();                     // 0: leader, 1: follower
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_m = M / (2 * BM), num_n = N / BN, num_tiles = num_m * num_n, num_kb = K / BK;

  if (threadIdx.x == 0) {
    s_abort_store = 0;
    for (int s = 0; s < STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; a++) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 2 * 128); }
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a); tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) { tmem_alloc_pair(tmem_slot, TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                       // the partner's barriers exist before anything is signalled across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      for (int t = pair; t < num_tiles && !*s_abort; t += num_pairs) {
        int m_blk, n_blk; tile_of(t, num_m, num_n, m_blk, n_blk);
        const int row_a = m_blk * 2 * BM + (int)v * BM, row_b = n_blk * BN + (int)v * (BN / 2);
        bool ok = true;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&empty[stage], phase ^ 1, s_abort, kWaitLimitNs)) { atomicExch(status, 1); ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES; uint8_t* sb = sa + A_BYTES;
          if (v == 0) mbar_arrive_expect_tx(&full[stage], 2 * STAGE_BYTES);      // the bytes of both CTAs land on the leader's barrier
          tma_load_2d_pair(sa, &tmap_a, kb * BK, row_a, &full[stage]);
          tma_load_2d_pair(sb, &tmap_b, kb * BK, row_b, &full[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && v == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN);
      int stage = 0; uint32_t phase = 0; int local = 0;
      for (int t = pair; t < num_tiles && !*s_abort; t += num_pairs, local++) {
        const int acc = local & 1; const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, s_abort, kWaitLimitNs)) { atomicExch(status, 2); break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&full[stage], phase, s_abort, kWaitLimitNs)) { atomicExch(status, 3); ok = false; break; }
          tc_fence_after();
          const uint8_t* sa = smem + stage * STAGE_BYTES; const uint8_t* sb = sa + A_BYTES;
          const uint64_t da = make_smem_desc_k128(sa), db = make_smem_desc_k128(sb);
#pragma unroll
          for (int k = 0; k < BK / 16; k++) umma_f16_pair(d_tmem, desc_advance(da, k * 32), desc_advance(db, k * 32), idesc, (kb | k) != 0);
          umma_commit_pair(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(&tmem_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;                 // the TMEM lane quarter this warp may read
    int local = 0;
    for (int t = pair; t < num_tiles; t += num_pairs, local++) {
      int m_blk, n_blk; tile_of(t, num_m, num_n, m_blk, n_blk);
      const int acc = local & 1; const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, s_abort, kWaitLimitNs)) { atomicExch(status, 4); break; }
      tc_fence_after();
      const int row = quarter * 32 + lane;        // row inside this CTA's half of the tile == TMEM lane
      bf16* crow = C + (size_t)(m_blk * 2 * BM + (int)v * BM + row) * N + (size_t)n_blk * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + c * 32, r);
        tmem_ld_wait();
        uint4 o[4];
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(o);
        if (bias) {
          const uint4* b4 = reinterpret_cast<const uint4*>(bias + (size_t)n_blk * BN + c * 32);
#pragma unroll
          for (int i = 0; i < 4; i++) {
            uint4 bb = b4[i];
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bb);
#pragma unroll
            for (int j = 0; j < 4; j++) {
              float2 f = __bfloat1622float2(b2[j]);
              o2[i * 4 + j] = __floats2bfloat162_rn(__uint_as_float(r[i * 8 + 2 * j]) + f.x, __uint_as_float(r[i * 8 + 2 * j + 1]) + f.y);
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; i++) o2[i] = __floats2bfloat162_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        }
#pragma unroll
        for (int i = 0; i < 4; i++) reinterpret_cast<uint4*>(crow + c * 32)[i] = o[i];
      }
      tc_fence_before();
      mbar_arrive_leader(&tmem_empty[acc]);       // this half of the accumulator may be overwritten
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                             // neither CTA leaves while the other may still touch its shared memory or barriers
  if (*s_abort) {
    unsigned long long t0 = gtime_ns();
    while (gtime_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc_pair(tmem_base, TMEM_COLS); }
}

// ------------------------------------------------------------------ host
struct MapKey { const void* p; long rows, cols; bool operator<(const MapKey& o) const { return std::tie(p, rows, cols) < std::tie(o.p, o.rows, o.cols); } };
static std::mutex g_mu;
static std::map<MapKey, CUtensorMap> g_maps;
static int* g_status[64] = {nullptr};

static bool get_map(const void* p, long rows, long cols, CUtensorMap* out) {
  std::lock_guard<std::mutex> l(g_mu);
  MapKey k{p, rows, cols};
  auto it = g_maps.find(k);
  if (it != g_maps.end()) { *out = it->second; return true; }
  CUtensorMap m;
  if (!make_tmap_bf16_k64(&m, p, (uint64_t)rows, (uint64_t)cols, (uint64_t)cols, 128)) return false;
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps[k] = m; *out = m;
  return true;
}

}  // namespace piccl_ops2

extern "C" {

// C = A · B^T (+ bias).  A [M,K], B [N,K], C [M,N], bf16 row-major and contiguous, 16-byte aligned; bias [N] bf16 or null.
// Requires M % 256 == 0, N % 256 == 0, K % 64 == 0.  Returns 0 on launch, a negative code if the shape is unsupported or set-up failed.
int piccl_ops2_gemm_bf16_nt(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, void* stream) {
  using namespace piccl_ops2;
  if (M <= 0 || N <= 0 || K <= 0 || M % (2 * BM) || N % BN || K % BK) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) | reinterpret_cast<uintptr_t>(bias)) & 15) return -2;
  int dev = 0; cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -6;
  if (!g_status[dev]) { if (cudaMalloc(&g_status[dev], sizeof(int)) != cudaSuccess) return -7; cudaMemset(g_status[dev], 0, sizeof(int)); }
  CUtensorMap ta, tb;
  if (!get_map(A, M, K, &ta) || !get_map(B, N, K, &tb)) return -3;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_bf16_nt_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DYNAMIC) != cudaSuccess) return -4;
    attr_set = true;
  }
  // pairs that can be resident at once (a pair needs two SMs of one GPC): the persistent grid is never larger
  static int max_pairs[64] = {0};
  if (!max_pairs[dev]) {
    int sms = 148; cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int n = sms / 2;
    cudaLaunchConfig_t cfg; memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(2 * n); cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = SMEM_DYNAMIC;
    cudaLaunchAttribute at; memset(&at, 0, sizeof at);
    at.id = cudaLaunchAttributeClusterDimension; at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at; cfg.numAttrs = 1;
    int active = 0;
    if (cudaOccupancyMaxActiveClusters(&active, gemm_bf16_nt_pair_kernel, &cfg) == cudaSuccess && active > 0) n = active < n ? active : n;
    else cudaGetLastError();
    max_pairs[dev] = n;
  }
  const int tiles = (M / (2 * BM)) * (N / BN);
  const int pairs = tiles < max_pairs[dev] ? tiles : max_pairs[dev];
  gemm_bf16_nt_pair_kernel<<<2 * pairs, THREADS, SMEM_DYNAMIC, (cudaStream_t)stream>>>(ta, tb, (bf16*)C, (const bf16*)bias, M, N, K, g_status[dev]);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// 0: no wait has run out on this device since the last call; otherwise the role that gave up
// (1 producer, 2 / 3 MMA issuer waiting for the accumulator / the operands, 4 epilogue).  Synchronises the device.
int piccl_ops2_gemm_status(void) {
  using namespace piccl_ops2;
  int dev = 0; cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !g_status[dev]) return 0;
  int h = 0;
  if (cudaMemcpy(&h, g_status[dev], sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (h) cudaMemset(g_status[dev], 0, sizeof(int));
  return h;
}

}  // extern "C"
