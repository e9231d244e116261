// Lookup of the executor instantiation for a (dtype, op) pair.
#include "exec.cuh"

namespace piccl {
extern ExecKernelFn exec_table_I8[4], exec_table_U8[4], exec_table_I32[4], exec_table_U32[4], exec_table_I64[4], exec_table_U64[4],
    exec_table_F16[4], exec_table_F32[4], exec_table_F64[4], exec_table_BF16[4];

ExecKernelFn exec_kernel_for(int dtype, int op) {
  if (op < 0 || op > 3) return nullptr;
  switch (dtype) {
    case DT_I8: return exec_table_I8[op];
    case DT_U8: return exec_table_U8[op];
    case DT_I32: return exec_table_I32[op];
    case DT_U32: return exec_table_U32[op];
    case DT_I64: return exec_table_I64[op];
    case DT_U64: return exec_table_U64[op];
    case DT_F16: return exec_table_F16[op];
    case DT_F32: return exec_table_F32[op];
    case DT_F64: return exec_table_F64[op];
    case DT_BF16: return exec_table_BF16[op];
    default: return nullptr;
  }
}
extern ExecKernelFn exec_defer_table_I8[4], exec_defer_table_U8[4], exec_defer_table_I32[4], exec_defer_table_U32[4], exec_defer_table_I64[4], exec_defer_table_U64[4],
    exec_defer_table_F16[4], exec_defer_table_F32[4], exec_defer_table_F64[4], exec_defer_table_BF16[4];
// The variant that holds counter updates back until the CTA is about to block (exec_impl.cuh).
ExecKernelFn exec_defer_kernel_for(int dtype, int op) {
  if (op < 0 || op > 3) return nullptr;
  switch (dtype) {
    case DT_I8: return exec_defer_table_I8[op];
    case DT_U8: return exec_defer_table_U8[op];
    case DT_I32: return exec_defer_table_I32[op];
    case DT_U32: return exec_defer_table_U32[op];
    case DT_I64: return exec_defer_table_I64[op];
    case DT_U64: return exec_defer_table_U64[op];
    case DT_F16: return exec_defer_table_F16[op];
    case DT_F32: return exec_defer_table_F32[op];
    case DT_F64: return exec_defer_table_F64[op];
    case DT_BF16: return exec_defer_table_BF16[op];
    default: return nullptr;
  }
}
ExecKernelFn exec_defer_copy_kernel() { return exec_defer_table_U8[0]; }
extern ExecKernelFn exec_ll_table_I8[4], exec_ll_table_U8[4], exec_ll_table_I32[4], exec_ll_table_U32[4], exec_ll_table_I64[4], exec_ll_table_U64[4],
    exec_ll_table_F16[4], exec_ll_table_F32[4], exec_ll_table_F64[4], exec_ll_table_BF16[4];
ExecKernelFn exec_ll_kernel_for(int dtype, int op) {
  if (op < 0 || op > 3) return nullptr;
  switch (dtype) {
    case DT_I8: return exec_ll_table_I8[op];
    case DT_U8: return exec_ll_table_U8[op];
    case DT_I32: return exec_ll_table_I32[op];
    case DT_U32: return exec_ll_table_U32[op];
    case DT_I64: return exec_ll_table_I64[op];
    case DT_U64: return exec_ll_table_U64[op];
    case DT_F16: return exec_ll_table_F16[op];
    case DT_F32: return exec_ll_table_F32[op];
    case DT_F64: return exec_ll_table_F64[op];
    case DT_BF16: return exec_ll_table_BF16[op];
    default: return nullptr;
  }
}
ExecKernelFn exec_ll_copy_kernel() { return exec_ll_table_U8[0]; }
// Byte-wise instantiation used by the collectives that only move data.
ExecKernelFn exec_copy_kernel() { return exec_table_U8[0]; }
}  // namespace piccl
