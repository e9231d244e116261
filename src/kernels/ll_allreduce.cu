// Low-latency all-reduce for small messages and the exchange-type algorithms
// (RD / RM / PRD / PRM): every 16-byte line carries 8 bytes of payload and two
// copies of the call's epoch, written with one store, so a receiver that sees
// both flags has the data — no fence, no separate counter, no credit
// round trip.  A rank pushes its current value to all partners of the step,
// then polls the lines its partners pushed, reduces in rank order and moves on;
// every thread owns the same lines in all steps, so the kernel needs no barrier.
//
// Slot reuse is safe with two buffers (epoch parity) because each step is a
// symmetric exchange: a partner can only write epoch e+2 into a slot after it
// finished call e+1, which needed my data of call e+1, which I send after I
// finished reading call e.
// The reference runs these steps as ncclSend/ncclRecv groups plus a reduce
// kernel per step (src/coll/allreduce.c:282-614).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "ll_impl.cuh"

namespace piccl {

template <typename T, int OP>
__global__ void __launch_bounds__(kLLBlock) ll_allreduce_kernel(const LLArgs a) {
  __shared__ char* s_heap[kMaxRanks];
  ll_allreduce_body<T, OP>(a, blockIdx.x / a.n_cta, blockIdx.x % a.n_cta, s_heap);
}

#define LL_ROW(T) {ll_allreduce_kernel<T, 0>, ll_allreduce_kernel<T, 1>, ll_allreduce_kernel<T, 2>, ll_allreduce_kernel<T, 3>}
static LLKernelFn g_ll_table[DT_COUNT][4] = {LL_ROW(int8_t), LL_ROW(uint8_t), LL_ROW(int32_t), LL_ROW(uint32_t), LL_ROW(long long), LL_ROW(unsigned long long),
                                             LL_ROW(__half), LL_ROW(float), LL_ROW(double), LL_ROW(__nv_bfloat16)};

LLKernelFn ll_kernel_for(int dtype, int op) {
  if (dtype < 0 || dtype >= DT_COUNT || op < 0 || op > 3) return nullptr;
  return g_ll_table[dtype][op];
}
int ll_lines_per_cta() { return kLLBlock * kLLLinesPerThread; }

}  // namespace piccl
