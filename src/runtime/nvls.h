// In-switch all-reduce: the multicast window of a communicator (runtime/nvls.cu).
#pragma once
#include <cuda_runtime.h>
#include <cstddef>

struct piccl_comm;

namespace piccl {

// Does this device support NVLink multicast objects (and did every driver entry point resolve)?
bool nvls_device_capable(int device);
// Builds the window together with all other ranks; on any failure the communicator simply has none.
// root_pid / root_id name the rendezvous socket (rank 0's process and heap address).
void nvls_setup(piccl_comm* c, int root_pid, unsigned long long root_id);
void nvls_destroy(piccl_comm* c);
bool nvls_ready(const piccl_comm* c);
bool nvls_dtype_supported(int dtype);      // kernels/nvls_allreduce.cu
// PICCL_OK: enqueued; PICCL_UNSUPPORTED: no window or data type not handled (sum / avg of fp32, fp16, bf16 only).
int nvls_allreduce(piccl_comm* c, const void* in, void* out, size_t count, int dtype, bool avg, cudaStream_t stream);

}  // namespace piccl
