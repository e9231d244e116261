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
#include "../include/sm100_gemm.cuh"

namespace piccl_ops {

using namespace sm100;
typedef __nv_bfloat16 bf16;

constexpr int BM = GEMM_BM, BK = GEMM_BK;
template <int BN, int STAGES> using SmemLayout = GemmSmem<BN, STAGES>;

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
}

// Plain GEMM: tiles in m-fastest order, nothing to wait for, bias / GELU epilogue.
template <int BN>
struct PlainPolicy {
  const CUtensorMap* ta; bf16* C; bf16* C_pre; const bf16* bias; int N, num_m, num_n, act_gelu;
  __device__ int num_tiles() const { return num_m * num_n; }
  // Bands of 32 row blocks, inside a band column blocks outer / row blocks inner: the CTAs that run together share a
  // band of A (about 30 MB at K = 3584) that stays in L2 while B streams through once per band.
  __device__ void tile(int idx, int& m_blk, int& n_blk) const {
    constexpr int GM = 32;
    const int per_band = GM * num_n, band = idx / per_band, within = idx % per_band;
    const int rows = min(GM, num_m - band * GM);
    m_blk = band * GM + within % rows; n_blk = within / rows;
  }
  __device__ const CUtensorMap* a_map(int m_blk, int& row0) const { row0 = m_blk * BM; return ta; }
  __device__ bool gate(int, volatile int*) const { return true; }
  static constexpr int STAGING = 0;
  __device__ void set_staging(uint8_t*) {}
  __device__ bool tile_begin(int, int, int, volatile int*) { return true; }
  __device__ void tile_end(int, int, int) {}
  __device__ void store(int m_blk, int n_blk, int row, int col0, float (&v)[32]) {
    const size_t off = (size_t)(m_blk * BM + row) * N + (size_t)n_blk * BN + col0;
    if (bias) {
      const bf16* brow = bias + (size_t)n_blk * BN + col0;
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 bb = *reinterpret_cast<const uint4*>(brow + i);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bb);
#pragma unroll
        for (int j = 0; j < 4; j++) { float2 f = __bfloat1622float2(b2[j]); v[i + 2 * j] += f.x; v[i + 2 * j + 1] += f.y; }
      }
    }
    if (C_pre) store_row32_bf16(C_pre + off, v);
    if (act_gelu) {
#pragma unroll
      for (int i = 0; i < 32; i++) {
        // activation of the value as stored (bf16), so that backward sees the same pre-activation
        float x = C_pre ? __bfloat162float(__float2bfloat16_rn(v[i])) : v[i];
        v[i] = gelu_tanh(x);
      }
    }
    store_row32_bf16(C + off, v);
  }
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_nt_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, bf16* __restrict__ C, bf16* __restrict__ C_pre,
                    const bf16* __restrict__ bias, int M, int N, int K, int act_gelu, int* __restrict__ status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  if (threadIdx.x == 0) tma_prefetch_desc(&tmap_a);
  PlainPolicy<BN> pol{&tmap_a, C, C_pre, bias, N, M / BM, N / BN, act_gelu};
  gemm_persistent<BN, STAGES>(smem_raw, &tmap_b, pol, K, blockIdx.x, gridDim.x, status, &s_abort);
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
  const int smem = L::DYNAMIC;
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
