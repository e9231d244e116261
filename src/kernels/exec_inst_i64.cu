// Executor instantiations for one element type (sum, prod, max, min).
#include "exec_ll.cuh"
PICCL_INSTANTIATE_EXEC(long long, I64)
