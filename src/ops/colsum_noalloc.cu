// Allocation-free variant of the bias-gradient column sum (see colsum_noalloc.h).
// Same two-pass scheme as piccl_ops_colsum in elementwise.cu — per-block partial
// sums in fp32, then one pass that folds the partials — but the partials live in
// a fixed device array that is part of the library image.
#include <cstdint>
#include <cstdio>
#include <mutex>
#include "colsum_noalloc.h"
#include "ops_common.cuh"

namespace {

using namespace piccl_ops;

// 64 x 16384 floats = 4 MiB, resident on every GPU that loads this library.
static __device__ __align__(256) float g_colsum_scratch[PICCL_OPS_COLSUM_NOALLOC_MAX_PARTS * PICCL_OPS_COLSUM_NOALLOC_MAX_COLS];

// In host code the name above is only a stand-in for the symbol; the device address has to be
// asked for, once per device, with that device current.
constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mu;

// block (bx, by): rows [by*rpb, (by+1)*rpb) of the 256 columns starting at bx*256 -> part[by][c]
__global__ void __launch_bounds__(256) colsum_noalloc_partial_kernel(const bf16* __restrict__ x, float* __restrict__ part, int rows, int C, int rows_per_block) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int c8 = blockIdx.x * 32 + lane;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; e++) acc[e] = 0.f;
  int r0 = blockIdx.y * rows_per_block, r1 = min(rows, r0 + rows_per_block);
  if (c8 * 8 < C)
    for (int r = r0 + warp; r < r1; r += 8) {
      float v[8]; unpack8(reinterpret_cast<const bf16x8*>(x + (size_t)r * C)[c8], v);
#pragma unroll
      for (int e = 0; e < 8; e++) acc[e] += v[e];
    }
  __shared__ float sh[8][256];
#pragma unroll
  for (int e = 0; e < 8; e++) sh[warp][lane * 8 + e] = acc[e];
  __syncthreads();
  int c = blockIdx.x * 256 + threadIdx.x;
  if (c < C) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) s += sh[w][threadIdx.x];
    part[(size_t)blockIdx.y * C + c] = s;
  }
}

__global__ void colsum_noalloc_finish_kernel(const float* __restrict__ part, int nparts, int C, bf16* __restrict__ out, int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (int p = 0; p < nparts; p++) s += part[(size_t)p * C + c];
  if (accumulate) s += __bfloat162float(out[c]);
  out[c] = __float2bfloat16_rn(s);
}

}  // namespace

extern "C" int piccl_ops_colsum_noalloc(const void* x, void* out, int rows, int C, int accumulate, void* stream) {
  if (!x || !out) { fprintf(stderr, "piccl_ops_colsum_noalloc: null input or output pointer\n"); return -4; }
  if (C < 8 || C % 8) { fprintf(stderr, "piccl_ops_colsum_noalloc: C = %d must be a positive multiple of 8\n", C); return -1; }
  if (C > PICCL_OPS_COLSUM_NOALLOC_MAX_COLS) {
    fprintf(stderr, "piccl_ops_colsum_noalloc: C = %d exceeds the built-in workspace (at most %d columns); use piccl_ops_colsum with your own workspace\n", C,
            PICCL_OPS_COLSUM_NOALLOC_MAX_COLS);
    return -2;
  }
  if (rows < 1) { fprintf(stderr, "piccl_ops_colsum_noalloc: rows = %d must be at least 1\n", rows); return -3; }
  // x is read as 16-byte vectors (8 bf16 at a time); out is accessed element by element and needs no more than its natural alignment
  if (reinterpret_cast<uintptr_t>(x) & 15) { fprintf(stderr, "piccl_ops_colsum_noalloc: x = %p is not 16-byte aligned\n", x); return -7; }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { fprintf(stderr, "piccl_ops_colsum_noalloc: no usable current device\n"); return -5; }
  float* scratch;
  {
    std::lock_guard<std::mutex> l(g_setup_mu);
    if (!g_scratch_addr[dev]) {
      void* p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&p, g_colsum_scratch);     // address on the CURRENT device
      if (e != cudaSuccess || !p) { fprintf(stderr, "piccl_ops_colsum_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(e)); return -5; }
      g_scratch_addr[dev] = static_cast<float*>(p);
    }
    scratch = g_scratch_addr[dev];
  }
  // fold the rows into at most 64 partial sums
  int rows_per_block = (rows + PICCL_OPS_COLSUM_NOALLOC_MAX_PARTS - 1) / PICCL_OPS_COLSUM_NOALLOC_MAX_PARTS;
  if (rows_per_block < 64) rows_per_block = 64;
  int nparts = (rows + rows_per_block - 1) / rows_per_block;
  cudaStream_t s = (cudaStream_t)stream;
  colsum_noalloc_partial_kernel<<<dim3((C + 255) / 256, nparts), 256, 0, s>>>((const bf16*)x, scratch, rows, C, rows_per_block);
  colsum_noalloc_finish_kernel<<<(C + 255) / 256, 256, 0, s>>>(scratch, nparts, C, (bf16*)out, accumulate);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { fprintf(stderr, "piccl_ops_colsum_noalloc: launch failed: %s\n", cudaGetErrorString(e)); return -6; }
  return 0;
}
