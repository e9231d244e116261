// bf16 GEMM for sm_100a:  C[M,N] = act(A[M,K] · B[N,K]^T + bias)
//
// Persistent, warp-specialised CTAs (one per SM):
//   warp 0      TMA producer: 128x64 A tiles and BNx64 B tiles -> 128B-swizzled shared memory,
//               STAGES-deep ring guarded by full/empty mbarriers
//   warp 1      allocates TMEM; one elected lane issues tcgen05.mma (128 x BN x 16 per instruction),
//               accumulating in TMEM; tcgen05.commit releases shared-memory stages and publishes
//               finished accumulators
//   warps 2-5   epilogue: tcgen05.ld (each warp its own 32-lane quarter) -> bias / GELU in fp32 ->
//               bf16 -> global.  Two TMEM accumulators, so the epilogue of tile i overlaps the
//               main loop of tile i+1.
// All mbarrier waits are bounded; a wait that runs out raises a CTA-wide flag, every role leaves its
// loop, TMEM is released and the kernel returns with a status word set.
#include <cuda_bf16.h>
#include <cstdio>
#include <map>
#include <mutex>
#include <tuple>
#include "../include/sm100_ptx.cuh"

namespace piccl_ops {

using namespace sm100;
typedef __nv_bfloat16 bf16;

constexpr int BM = 128, BK = 64;
constexpr unsigned long long kWaitLimitNs = 4000000000ull;   // 4 s

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFF = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFF + (2 * STAGES + 4) * 8 + 16;
};

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_nt_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, bf16* __restrict__ C, bf16* __restrict__ C_pre,
                    const bf16* __restrict__ bias, int M, int N, int K, int act_gelu, int* __restrict__ status) {
  typedef SmemLayout<BN, STAGES> L;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // the 128-byte swizzle needs 1024-byte aligned tiles
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = M / BM, num_n = N / BN, num_tiles = num_m * num_n, num_kb = K / BK;
  constexpr uint32_t TMEM_COLS = 2 * BN;           // 256 or 512: a power of two

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; a++) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 128); }
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmap_a); tma_prefetch_desc(&tmap_b); }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !s_abort; tile += gridDim.x) {
        const int m_blk = tile % num_m, n_blk = tile / num_m;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&empty[stage], phase ^ 1, &s_abort, kWaitLimitNs)) { atomicExch(status, 1); break; }
          uint8_t* sa = smem + stage * L::STAGE_BYTES; uint8_t* sb = sa + L::A_BYTES;
          mbar_arrive_expect_tx(&full[stage], L::STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, kb * BK, m_blk * BM, &full[stage]);
          tma_load_2d(sb, &tmap_b, kb * BK, n_blk * BN, &full[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN);
      int stage = 0; uint32_t phase = 0; int local = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !s_abort; tile += gridDim.x, local++) {
        const int acc = local & 1; const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, &s_abort, kWaitLimitNs)) { atomicExch(status, 2); break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&full[stage], phase, &s_abort, kWaitLimitNs)) { atomicExch(status, 3); ok = false; break; }
          tc_fence_after();
          const uint8_t* sa = smem + stage * L::STAGE_BYTES; const uint8_t* sb = sa + L::A_BYTES;
          const uint64_t da = make_smem_desc_k128(sa), db = make_smem_desc_k128(sb);
#pragma unroll
          for (int k = 0; k < BK / 16; k++) umma_f16(d_tmem, desc_advance(da, k * 32), desc_advance(db, k * 32), idesc, (kb | k) != 0);
          umma_commit(&empty[stage]);                 // stage reusable once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tmem_full[acc]);                 // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps = 128 TMEM lanes)
    const int quarter = warp & 3;                     // TMEM lane quarter this warp may access
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, local++) {
      const int m_blk = tile % num_m, n_blk = tile / num_m;
      const int acc = local & 1; const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, &s_abort, kWaitLimitNs)) { atomicExch(status, 4); break; }
      tc_fence_after();
      const int row = m_blk * BM + quarter * 32 + lane;
      bf16* crow = C + (size_t)row * N + (size_t)n_blk * BN;
      bf16* prow = C_pre ? C_pre + (size_t)row * N + (size_t)n_blk * BN : nullptr;
      const bf16* brow = bias ? bias + (size_t)n_blk * BN : nullptr;
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + c * 32, r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
        if (brow) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 bb = *reinterpret_cast<const uint4*>(brow + c * 32 + i);
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bb);
#pragma unroll
            for (int j = 0; j < 4; j++) { float2 f = __bfloat1622float2(b2[j]); v[i + 2 * j] += f.x; v[i + 2 * j + 1] += f.y; }
          }
        }
        if (prow) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 o; __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; j++) o2[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
            *reinterpret_cast<uint4*>(prow + c * 32 + i) = o;
          }
        }
        if (act_gelu) {
#pragma unroll
          for (int i = 0; i < 32; i++) {
            // activation of the value as stored (bf16), so that backward sees the same pre-activation
            float x = prow ? __bfloat162float(__float2bfloat16_rn(v[i])) : v[i];
            v[i] = gelu_tanh(x);
          }
        }
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 o; __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int j = 0; j < 4; j++) o2[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
          *reinterpret_cast<uint4*>(crow + c * 32 + i) = o;
        }
      }
      tc_fence_before();
      mbar_arrive(&tmem_empty[acc]);
    }
  }
  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (s_abort) {
    // give copies that may still be in flight time to land before the shared memory is handed on
    unsigned long long t0 = gtime_ns();
    while (gtime_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ------------------------------------------------------------------ host
struct MapKey { const void* p; long rows, cols; int box; bool operator<(const MapKey& o) const { return std::tie(p, rows, cols, box) < std::tie(o.p, o.rows, o.cols, o.box); } };
static std::mutex g_mu;
static std::map<MapKey, CUtensorMap> g_maps;
static int* g_status[64] = {nullptr};

static bool get_map(const void* p, long rows, long cols, int box, CUtensorMap* out) {
  std::lock_guard<std::mutex> l(g_mu);
  MapKey k{p, rows, cols, box};
  auto it = g_maps.find(k);
  if (it != g_maps.end()) { *out = it->second; return true; }
  CUtensorMap m;
  if (!make_tmap_bf16_k64(&m, p, (uint64_t)rows, (uint64_t)cols, (uint64_t)cols, (uint32_t)box)) return false;
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps[k] = m; *out = m;
  return true;
}

template <int BN, int STAGES>
static int launch(const void* A, const void* B, void* C, void* C_pre, const void* bias, int M, int N, int K, int gelu, int* status, cudaStream_t s) {
  typedef SmemLayout<BN, STAGES> L;
  CUtensorMap ta, tb;
  if (!get_map(A, M, K, BM, &ta) || !get_map(B, N, K, BN, &tb)) return -3;
  static bool attr_set = false;
  const int smem = L::TOTAL + 1024;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_bf16_nt_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
    attr_set = true;
  }
  int dev = 0, sms = 148; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int tiles = (M / BM) * (N / BN);
  int grid = tiles < sms ? tiles : sms;
  gemm_bf16_nt_kernel<BN, STAGES><<<grid, 192, smem, s>>>(ta, tb, (bf16*)C, (bf16*)C_pre, (const bf16*)bias, M, N, K, gelu, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace piccl_ops

extern "C" {

// C = act(A · B^T + bias).  A [M,K], B [N,K], C [M,N], all bf16 row-major and contiguous; bias [N] bf16 or null;
// c_pre (optional) receives the value before the activation.  Requires M % 128 == 0, N % 128 == 0, K % 64 == 0.
// Returns 0 on launch, a negative code if the shape is unsupported or set-up failed.
int piccl_ops_gemm_bf16_nt_ex(const void* A, const void* B, void* C, void* c_pre, const void* bias, int M, int N, int K, int gelu, void* stream) {
  using namespace piccl_ops;
  if (M <= 0 || N <= 0 || K <= 0 || M % BM || N % 128 || K % BK) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) | reinterpret_cast<uintptr_t>(bias) | reinterpret_cast<uintptr_t>(c_pre)) & 15) return -2;
  int dev = 0; cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -6;
  if (!g_status[dev]) { if (cudaMalloc(&g_status[dev], sizeof(int)) != cudaSuccess) return -7; cudaMemset(g_status[dev], 0, sizeof(int)); }
  cudaStream_t s = (cudaStream_t)stream;
  if (N % 256 == 0) return launch<256, 4>(A, B, C, c_pre, bias, M, N, K, gelu, g_status[dev], s);
  return launch<128, 6>(A, B, C, c_pre, bias, M, N, K, gelu, g_status[dev], s);
}
int piccl_ops_gemm_bf16_nt(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int gelu, void* stream) {
  return piccl_ops_gemm_bf16_nt_ex(A, B, C, nullptr, bias, M, N, K, gelu, stream);
}
// Non-zero if a GEMM on the current device gave up on a wait (1 producer, 2/3 MMA issuer, 4 epilogue).  Synchronises.
int piccl_ops_gemm_status(void) {
  using namespace piccl_ops;
  int dev = 0; cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !g_status[dev]) return 0;
  int v = 0; cudaMemcpy(&v, g_status[dev], sizeof v, cudaMemcpyDeviceToHost);
  return v;
}

}  // extern "C"
