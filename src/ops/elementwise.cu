// Fused element-wise model kernels: bias + GELU (forward / backward), bias
// gradient (column sums), softmax cross entropy with in-place gradient, and a
// flat AdamW step with fp32 master weights.
#include "ops_common.cuh"

namespace piccl_ops {

// g = gelu(h + bias); h_out = h + bias (kept for the backward pass); h may alias h_out
__global__ void __launch_bounds__(256) bias_gelu_fwd_kernel(const bf16* __restrict__ h, const bf16* __restrict__ bias, bf16* __restrict__ h_out,
                                                            bf16* __restrict__ g, size_t n8, int C8) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float v[8], b[8], o[8];
    unpack8(reinterpret_cast<const bf16x8*>(h)[i], v);
    if (bias) { unpack8(reinterpret_cast<const bf16x8*>(bias)[i % C8], b);
#pragma unroll
      for (int e = 0; e < 8; e++) v[e] += b[e]; }
    if (h_out) { bf16x8 p = pack8(v); reinterpret_cast<bf16x8*>(h_out)[i] = p; unpack8(p, v); }
#pragma unroll
    for (int e = 0; e < 8; e++) o[e] = gelu_f(v[e]);
    reinterpret_cast<bf16x8*>(g)[i] = pack8(o);
  }
}

// dh = dg * gelu'(h)    (h includes the bias); dh may alias dg
__global__ void __launch_bounds__(256) gelu_bwd_kernel(const bf16* __restrict__ dg, const bf16* __restrict__ h, bf16* __restrict__ dh, size_t n8) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float d[8], v[8], o[8];
    unpack8(reinterpret_cast<const bf16x8*>(dg)[i], d);
    unpack8(reinterpret_cast<const bf16x8*>(h)[i], v);
#pragma unroll
    for (int e = 0; e < 8; e++) o[e] = d[e] * gelu_grad_f(v[e]);
    reinterpret_cast<bf16x8*>(dh)[i] = pack8(o);
  }
}

// partial column sums: block (bx, by) sums rows [by*rpb, ...) of 8*32 = 256 columns starting at bx*256
__global__ void __launch_bounds__(256) colsum_kernel(const bf16* __restrict__ x, float* __restrict__ part, int rows, int C, int rows_per_block) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int c8 = blockIdx.x * 32 + lane;                 // index of the 8-column group
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
__global__ void colsum_finish_kernel(const float* __restrict__ part, int nparts, int C, bf16* __restrict__ out, int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (int p = 0; p < nparts; p++) s += part[(size_t)p * C + c];
  if (accumulate) s += __bfloat162float(out[c]);
  out[c] = __float2bfloat16_rn(s);
}

// One block per row: loss[row] = logsumexp(logits[:V]) - logits[target]; logits <- (softmax - onehot) * gscale
// (columns V..Vp-1 are padding: ignored in the sum, gradient zero).
__global__ void __launch_bounds__(512) ce_fwd_bwd_kernel(bf16* __restrict__ logits, const long long* __restrict__ targets, float* __restrict__ loss,
                                                         int V, int Vp, float gscale) {
  int row = blockIdx.x, tid = threadIdx.x;
  bf16* lp = logits + (size_t)row * Vp;
  const int n8 = Vp / 8;
  float m = -INFINITY, s = 0.f;
  for (int i = tid; i < n8; i += blockDim.x) {
    float v[8]; unpack8(reinterpret_cast<const bf16x8*>(lp)[i], v);
    float lm = m;
#pragma unroll
    for (int e = 0; e < 8; e++) if (i * 8 + e < V) lm = fmaxf(lm, v[e]);
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < 8; e++) if (i * 8 + e < V) acc += __expf(v[e] - lm);
    s = s * __expf(m - lm) + acc; m = lm;
  }
  __shared__ float shm[16], shs[16];
  // combine (m, s) pairs: first in the warp, then across warps
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    float mm = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * __expf(m - mm)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm)); m = mm;
  }
  int warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
  if (lane == 0) { shm[warp] = m; shs[warp] = s; }
  __syncthreads();
  float M = -INFINITY;
  for (int w = 0; w < nw; w++) M = fmaxf(M, shm[w]);
  float S = 0.f;
  for (int w = 0; w < nw; w++) if (shm[w] != -INFINITY) S += shs[w] * __expf(shm[w] - M);
  long long t = targets[row];
  float inv = 1.f / S;
  if (tid == 0) loss[row] = (t >= 0 && t < V) ? (logf(S) + M - __bfloat162float(lp[t])) : 0.f;
  __syncthreads();     // the target logit is read before anybody overwrites it
  const bool valid = t >= 0 && t < V;
  for (int i = tid; i < n8; i += blockDim.x) {
    float v[8], o[8]; unpack8(reinterpret_cast<const bf16x8*>(lp)[i], v);
#pragma unroll
    for (int e = 0; e < 8; e++) {
      int c = i * 8 + e;
      float p = (c < V && valid) ? __expf(v[e] - M) * inv : 0.f;
      if (c == t) p -= 1.f;
      o[e] = p * gscale;
    }
    reinterpret_cast<bf16x8*>(lp)[i] = pack8(o);
  }
}

// AdamW on flat buffers: bf16 gradient and parameter, fp32 master copy and moments.
__global__ void __launch_bounds__(256) adamw_kernel(bf16* __restrict__ p, float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                                    const bf16* __restrict__ g, size_t n8, float lr, float b1, float b2, float eps, float wd,
                                                    float bc1, float bc2, float gscale, const int* __restrict__ step_dev) {
  if (step_dev) {   // step number kept on the device (the launch can then be replayed from a CUDA graph)
    const float st = (float)*step_dev;
    bc1 = 1.f - powf(b1, st); bc2 = 1.f - powf(b2, st);
  }
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float gv[8]; unpack8(reinterpret_cast<const bf16x8*>(g)[i], gv);
    float4 w0 = reinterpret_cast<float4*>(master)[2 * i], w1 = reinterpret_cast<float4*>(master)[2 * i + 1];
    float4 m0 = reinterpret_cast<float4*>(m)[2 * i], m1 = reinterpret_cast<float4*>(m)[2 * i + 1];
    float4 v0 = reinterpret_cast<float4*>(v)[2 * i], v1 = reinterpret_cast<float4*>(v)[2 * i + 1];
    float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int e = 0; e < 8; e++) {
      float gr = gv[e] * gscale;
      mm[e] = b1 * mm[e] + (1.f - b1) * gr;
      vv[e] = b2 * vv[e] + (1.f - b2) * gr * gr;
      float upd = (mm[e] / bc1) / (sqrtf(vv[e] / bc2) + eps);
      w[e] = w[e] * (1.f - lr * wd) - lr * upd;
    }
    reinterpret_cast<float4*>(master)[2 * i] = make_float4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<float4*>(master)[2 * i + 1] = make_float4(w[4], w[5], w[6], w[7]);
    reinterpret_cast<float4*>(m)[2 * i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(m)[2 * i + 1] = make_float4(mm[4], mm[5], mm[6], mm[7]);
    reinterpret_cast<float4*>(v)[2 * i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    reinterpret_cast<float4*>(v)[2 * i + 1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
    reinterpret_cast<bf16x8*>(p)[i] = pack8(w);
  }
}

// out[r, :] = wte[idx[r], :] + wpe[r % S, :]
__global__ void __launch_bounds__(128) embed_fwd_kernel(const long long* __restrict__ idx, const bf16* __restrict__ wte, const bf16* __restrict__ wpe,
                                                        bf16* __restrict__ out, int rows, int S, int C8) {
  int row = blockIdx.x;
  long long t = idx[row];
  const bf16x8* a = reinterpret_cast<const bf16x8*>(wte) + (size_t)t * C8;
  const bf16x8* b = reinterpret_cast<const bf16x8*>(wpe) + (size_t)(row % S) * C8;
  for (int i = threadIdx.x; i < C8; i += blockDim.x) {
    float x[8], y[8]; unpack8(a[i], x); unpack8(b[i], y);
#pragma unroll
    for (int e = 0; e < 8; e++) x[e] += y[e];
    reinterpret_cast<bf16x8*>(out)[(size_t)row * C8 + i] = pack8(x);
  }
}

// dwpe[s, :] += sum over batch of dx[b*S + s, :]   (one block per position; deterministic)
__global__ void __launch_bounds__(128) wpe_bwd_kernel(const bf16* __restrict__ dx, bf16* __restrict__ dwpe, int B, int S, int C8, int accumulate) {
  int s = blockIdx.x;
  for (int i = threadIdx.x; i < C8; i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; e++) acc[e] = 0.f;
    for (int b = 0; b < B; b++) {
      float v[8]; unpack8(reinterpret_cast<const bf16x8*>(dx)[((size_t)b * S + s) * C8 + i], v);
#pragma unroll
      for (int e = 0; e < 8; e++) acc[e] += v[e];
    }
    if (accumulate) { float o[8]; unpack8(reinterpret_cast<const bf16x8*>(dwpe)[(size_t)s * C8 + i], o);
#pragma unroll
      for (int e = 0; e < 8; e++) acc[e] += o[e]; }
    reinterpret_cast<bf16x8*>(dwpe)[(size_t)s * C8 + i] = pack8(acc);
  }
}

// dwte[idx[r], :] += dx[r, :] in fp32 (atomics on an fp32 staging table), then folded into the bf16 gradient
__global__ void __launch_bounds__(128) wte_bwd_scatter_kernel(const long long* __restrict__ idx, const bf16* __restrict__ dx, float* __restrict__ stage, int C) {
  int row = blockIdx.x; long long t = idx[row];
  for (int c = threadIdx.x; c < C; c += blockDim.x) atomicAdd(&stage[(size_t)t * C + c], __bfloat162float(dx[(size_t)row * C + c]));
}
__global__ void __launch_bounds__(256) add_f32_into_bf16_kernel(const float* __restrict__ src, bf16* __restrict__ dst, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16_rn(__bfloat162float(dst[i]) + src[i]);
}

}  // namespace piccl_ops

using namespace piccl_ops;

static int grid_for(size_t n, int block) { size_t g = (n + block - 1) / block; return (int)(g > 148 * 16 ? 148 * 16 : (g ? g : 1)); }

extern "C" {

int piccl_ops_bias_gelu_fwd(const void* h, const void* bias, void* h_out, void* g, long long rows, int C, void* stream) {
  if (C % 8) return -1;
  size_t n8 = (size_t)rows * C / 8;
  bias_gelu_fwd_kernel<<<grid_for(n8, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)h, (const bf16*)bias, (bf16*)h_out, (bf16*)g, n8, C / 8);
  PICCL_OPS_CHECK_LAUNCH(); return 0;
}
int piccl_ops_gelu_bwd(const void* dg, const void* h, void* dh, long long n, void* stream) {
  if (n % 8) return -1;
  gelu_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)dg, (const bf16*)h, (bf16*)dh, (size_t)n / 8);
  PICCL_OPS_CHECK_LAUNCH(); return 0;
}
// workspace: ceil(rows / rows_per_block) * C floats
int piccl_ops_colsum(const void* x, void* out, float* workspace, int rows, int C, int rows_per_block, int accumulate, void* stream) {
  if (C % 8) return -1;
  int nparts = (rows + rows_per_block - 1) / rows_per_block;
  colsum_kernel<<<dim3((C + 255) / 256, nparts), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, workspace, rows, C, rows_per_block);
  colsum_finish_kernel<<<(C + 255) / 256, 256, 0, (cudaStream_t)stream>>>(workspace, nparts, C, (bf16*)out, accumulate);
  PICCL_OPS_CHECK_LAUNCH(); return 0;
}
int piccl_ops_ce_fwd_bwd(void* logits, const long long* targets, float* loss, int rows, int V, int Vp, float gscale, void* stream) {
  if (Vp % 8 || V > Vp) return -1;
  ce_fwd_bwd_kernel<<<rows, 512, 0, (cudaStream_t)stream>>>((bf16*)logits, targets, loss, V, Vp, gscale);
  PICCL_OPS_CHECK_LAUNCH(); return 0;
}
int piccl_ops_adamw(void* p, float* master, float* m, float* v, const void* g, long long n, float lr, float b1, float b2, float eps, float wd,
                    int step, float gscale, void* stream) {
  if (n % 8) return -1;
  float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  adamw_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>((bf16*)p, master, m, v, (const bf16*)g, (size_t)n / 8, lr, b1, b2, eps, wd, bc1, bc2, gscale, nullptr);
  PICCL_OPS_CHECK_LAUNCH(); return 0;
}
// Same update with the step number read from device memory (`step_dev`, an int the caller advances on the device).
int piccl_ops_adamw_devstep(void* p, float* master, float* m, float* v, const void* g, long long n, float lr, float b1, float b2, float eps, float wd,
                            const int* step_dev, float gscale, void* stream) {
  if (n % 8 || !step_dev) return -1;
  adamw_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>((bf16*)p, master, m, v, (const bf16*)g, (size_t)n / 8, lr, b1, b2, eps, wd, 1.f, 1.f, gscale, step_dev);
  PICCL_OPS_CHECK_LAUNCH(); return 0;
}
int piccl_ops_embed_fwd(const long long* idx, const void* wte, const void* wpe, void* out, int rows, int S, int C, void* stream) {
  if (C % 8) return -1;
  embed_fwd_kernel<<<rows, 128, 0, (cudaStream_t)stream>>>(idx, (const bf16*)wte, (const bf16*)wpe, (bf16*)out, rows, S, C / 8);
  PICCL_OPS_CHECK_LAUNCH(); return 0;
}
int piccl_ops_wpe_bwd(const void* dx, void* dwpe, int B, int S, int C, int accumulate, void* stream) {
  if (C % 8) return -1;
  wpe_bwd_kernel<<<S, 128, 0, (cudaStream_t)stream>>>((const bf16*)dx, (bf16*)dwpe, B, S, C / 8, accumulate);
  PICCL_OPS_CHECK_LAUNCH(); return 0;
}
// stage: fp32 [V, C], zeroed by the caller
int piccl_ops_wte_bwd(const long long* idx, const void* dx, float* stage, void* dwte, int rows, long long V, int C, void* stream) {
  wte_bwd_scatter_kernel<<<rows, 128, 0, (cudaStream_t)stream>>>(idx, (const bf16*)dx, stage, C);
  size_t n = (size_t)V * C;
  add_f32_into_bf16_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(stage, (bf16*)dwte, n);
  PICCL_OPS_CHECK_LAUNCH(); return 0;
}

}  // extern "C"
