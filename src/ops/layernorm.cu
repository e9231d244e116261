// Fused residual-add + LayerNorm, forward and backward (bf16 data, fp32 statistics).
// One warp per row, rows of C = 8*32*V elements held in registers, a single pass
// over HBM in each direction.  The residual sum is produced by the same kernel,
// so the x + f(x) tensors of a transformer block are never a separate pass.
#include "ops_common.cuh"

namespace piccl_ops {

// y = LN(x + res) * gamma + beta ; sum_out = x + res (optional)
template <int V>   // V 16-byte vectors per lane: C = 256 * V
__global__ void __launch_bounds__(128) ln_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res, const bf16* __restrict__ gamma,
                                                     const bf16* __restrict__ beta, bf16* __restrict__ sum_out, bf16* __restrict__ y,
                                                     float* __restrict__ mean, float* __restrict__ rstd, int rows, float eps) {
  const int C = 256 * V;
  int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const bf16x8* xp = reinterpret_cast<const bf16x8*>(x + (size_t)row * C);
  const bf16x8* rp = res ? reinterpret_cast<const bf16x8*>(res + (size_t)row * C) : nullptr;
  float v[V][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < V; i++) {
    unpack8(xp[lane + 32 * i], v[i]);
    if (rp) { float r[8]; unpack8(rp[lane + 32 * i], r);
#pragma unroll
      for (int e = 0; e < 8; e++) v[i][e] += r[e]; }
    if (sum_out) {
      bf16x8 p = pack8(v[i]);
      reinterpret_cast<bf16x8*>(sum_out + (size_t)row * C)[lane + 32 * i] = p;
      unpack8(p, v[i]);          // normalise exactly what was stored
    }
#pragma unroll
    for (int e = 0; e < 8; e++) s += v[i][e];
  }
  float mu = warp_sum(s) / C;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < V; i++)
#pragma unroll
    for (int e = 0; e < 8; e++) { float d = v[i][e] - mu; q += d * d; }
  float rs = rsqrtf(warp_sum(q) / C + eps);
  if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
#pragma unroll
  for (int i = 0; i < V; i++) {
    float g[8], b[8], o[8];
    unpack8(reinterpret_cast<const bf16x8*>(gamma)[lane + 32 * i], g);
    unpack8(reinterpret_cast<const bf16x8*>(beta)[lane + 32 * i], b);
#pragma unroll
    for (int e = 0; e < 8; e++) o[e] = (v[i][e] - mu) * rs * g[e] + b[e];
    reinterpret_cast<bf16x8*>(y + (size_t)row * C)[lane + 32 * i] = pack8(o);
  }
}

// dx = LN-backward(dy) + dres ; per-block partial dgamma / dbeta in fp32
template <int V>
__global__ void __launch_bounds__(128) ln_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ xin, const bf16* __restrict__ gamma,
                                                     const float* __restrict__ mean, const float* __restrict__ rstd, const bf16* __restrict__ dres,
                                                     bf16* __restrict__ dx, float* __restrict__ dgamma_part, float* __restrict__ dbeta_part,
                                                     int rows, int rows_per_block) {
  const int C = 256 * V;
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float dg[V][8], db[V][8];
#pragma unroll
  for (int i = 0; i < V; i++)
#pragma unroll
    for (int e = 0; e < 8; e++) { dg[i][e] = 0.f; db[i][e] = 0.f; }
  float g[V][8];
#pragma unroll
  for (int i = 0; i < V; i++) unpack8(reinterpret_cast<const bf16x8*>(gamma)[lane + 32 * i], g[i]);
  int row0 = blockIdx.x * rows_per_block;
  for (int r = row0 + warp; r < min(rows, row0 + rows_per_block); r += 4) {
    float mu = mean[r], rs = rstd[r];
    float xh[V][8], dyv[V][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < V; i++) {
      unpack8(reinterpret_cast<const bf16x8*>(xin + (size_t)r * C)[lane + 32 * i], xh[i]);
      unpack8(reinterpret_cast<const bf16x8*>(dy + (size_t)r * C)[lane + 32 * i], dyv[i]);
#pragma unroll
      for (int e = 0; e < 8; e++) {
        xh[i][e] = (xh[i][e] - mu) * rs;
        dg[i][e] += dyv[i][e] * xh[i][e]; db[i][e] += dyv[i][e];
        float t = dyv[i][e] * g[i][e];
        s1 += t; s2 += t * xh[i][e];
        dyv[i][e] = t;
      }
    }
    s1 = warp_sum(s1) / C; s2 = warp_sum(s2) / C;
#pragma unroll
    for (int i = 0; i < V; i++) {
      float o[8];
      if (dres) unpack8(reinterpret_cast<const bf16x8*>(dres + (size_t)r * C)[lane + 32 * i], o);
      else {
#pragma unroll
        for (int e = 0; e < 8; e++) o[e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < 8; e++) o[e] += rs * (dyv[i][e] - s1 - xh[i][e] * s2);
      reinterpret_cast<bf16x8*>(dx + (size_t)r * C)[lane + 32 * i] = pack8(o);
    }
  }
  // combine the 4 warps of the block, then one partial row per block
  __shared__ float sh[4][256 * V];   // reused for gamma then beta
  for (int pass = 0; pass < 2; pass++) {
#pragma unroll
    for (int i = 0; i < V; i++)
#pragma unroll
      for (int e = 0; e < 8; e++) sh[warp][(lane + 32 * i) * 8 + e] = pass == 0 ? dg[i][e] : db[i][e];
    __syncthreads();
    float* dst = (pass == 0 ? dgamma_part : dbeta_part) + (size_t)blockIdx.x * C;
    for (int c = threadIdx.x; c < C; c += 128) dst[c] = sh[0][c] + sh[1][c] + sh[2][c] + sh[3][c];
    __syncthreads();
  }
}

// out[c] (+)= sum over parts of part[p][c]   (bf16 output, fp32 partials)
__global__ void colsum_parts_kernel(const float* __restrict__ part, int nparts, int C, bf16* __restrict__ out, int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (int p = 0; p < nparts; p++) s += part[(size_t)p * C + c];
  if (accumulate) s += __bfloat162float(out[c]);
  out[c] = __float2bfloat16_rn(s);
}

}  // namespace piccl_ops

using namespace piccl_ops;

extern "C" {

// C must be 256, 512, 768, 1024, 1280, 1536 or 2048.  res / sum_out may be null.
int piccl_ops_ln_fwd(const void* x, const void* res, const void* gamma, const void* beta, void* sum_out, void* y, float* mean, float* rstd,
                     int rows, int C, float eps, void* stream) {
  dim3 grid((rows + 3) / 4), block(128);
  cudaStream_t s = (cudaStream_t)stream;
#define LN_CASE(V) case 256 * V: ln_fwd_kernel<V><<<grid, block, 0, s>>>((const bf16*)x, (const bf16*)res, (const bf16*)gamma, (const bf16*)beta, (bf16*)sum_out, (bf16*)y, mean, rstd, rows, eps); break;
  switch (C) { LN_CASE(1) LN_CASE(2) LN_CASE(3) LN_CASE(4) LN_CASE(5) LN_CASE(6) LN_CASE(8) default: return -1; }
#undef LN_CASE
  PICCL_OPS_CHECK_LAUNCH();
  return 0;
}

// workspace: 2 * nblocks * C floats, nblocks = ceil(rows / rows_per_block).  dgamma/dbeta are bf16 and accumulated if accumulate != 0.
int piccl_ops_ln_bwd(const void* dy, const void* xin, const void* gamma, const float* mean, const float* rstd, const void* dres, void* dx,
                     void* dgamma, void* dbeta, float* workspace, int rows, int C, int rows_per_block, int accumulate, void* stream) {
  int nblocks = (rows + rows_per_block - 1) / rows_per_block;
  cudaStream_t s = (cudaStream_t)stream;
  float* pg = workspace; float* pb = workspace + (size_t)nblocks * C;
#define LN_CASE(V) case 256 * V: ln_bwd_kernel<V><<<nblocks, 128, 0, s>>>((const bf16*)dy, (const bf16*)xin, (const bf16*)gamma, mean, rstd, (const bf16*)dres, (bf16*)dx, pg, pb, rows, rows_per_block); break;
  switch (C) { LN_CASE(1) LN_CASE(2) LN_CASE(3) LN_CASE(4) default: return -1; }
#undef LN_CASE
  PICCL_OPS_CHECK_LAUNCH();
  colsum_parts_kernel<<<(C + 255) / 256, 256, 0, s>>>(pg, nblocks, C, (bf16*)dgamma, accumulate);
  colsum_parts_kernel<<<(C + 255) / 256, 256, 0, s>>>(pb, nblocks, C, (bf16*)dbeta, accumulate);
  PICCL_OPS_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
