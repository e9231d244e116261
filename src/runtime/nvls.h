// In-switch collectives: the multicast window of a communicator (runtime/nvls.cu).
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
// All ranks are virtual ranks of this process on this device: a plain window, the kernels emulate the switch.
void nvls_setup_emulated(piccl_comm* c);
void nvls_destroy(piccl_comm* c);
bool nvls_ready(const piccl_comm* c);
bool nvls_emulated(const piccl_comm* c);
// Can this call run in the switch (window present, type / operator / size handled)?  The same answer on every rank.  op: 0 sum, 2 max, 3 min.
bool nvls_eligible(const piccl_comm* c, int coll, int dtype, int op, size_t count);
// PICCL_OK: enqueued; PICCL_UNSUPPORTED: run it another way.  n: 1, or all virtual ranks of an emulated group.
int nvls_collective(piccl_comm** comms, int n, int coll, const void* const* in, void* const* out, size_t count, int dtype, int op, bool avg, int root,
                    cudaStream_t stream);

}  // namespace piccl
