// All-reduce through the NVSwitch: contributions are summed inside the switch
// (`multimem.ld_reduce`) and the sum is written to every GPU at once
// (`multimem.st`), so each GPU sends and receives the vector about once instead
// of 2(n-1)/n times.  The reference has no counterpart (its all-reduce is a
// sequence of ncclSend/ncclRecv groups and separate reduce kernels,
// src/coll/allreduce.c:97-614).
//
// Every rank owns a window of device memory that is bound, at the same offset,
// to one multicast object, and sees it at two addresses: `uc` (its own copy)
// and `mc` (all copies at once).  Layout of a window:
//   [ kNvlsFlagBytes: one 8-byte barrier counter per CTA index, 128 bytes apart ]
//   [ n_cta_max slots of chunk_bytes ]
// CTA b of every rank works on chunks b, b + n_cta, ... of the message, each in five phases:
//   1 copy the chunk from the send buffer to its slot of the own window (scaled for avg)
//   2 barrier of the CTAs with index b of all ranks (one multimem.red on the counter, poll the own copy)
//   3 ld_reduce the 1/n of the slot that this rank is responsible for, st the sums to all copies
//   4 barrier
//   5 copy the slot to the receive buffer
// Barrier counters only ever grow (n per barrier), over the life of the communicator.
// Every poll is bounded: on a time-out the CTA records a status, raises the abort flag and leaves.
#pragma once
#include <cstdint>
#include "../include/piccl.h"

namespace piccl {

constexpr int kNvlsFlagBytes = 65536;
constexpr int kNvlsMaxCta = 256;          // kNvlsFlagBytes / 128 would allow 512
constexpr int kNvlsBlock = 512;

struct NvlsArgs {
  char* uc; char* mc;                     // the window: own copy / all copies
  const void* in; void* out;
  long long bytes;                        // message size
  long long chunk_bytes;                  // bytes of the message per chunk, multiple of 16 * nranks, <= slot_bytes
  long long slot_bytes;                   // distance between two slots of the window
  int rank, nranks, n_cta, avg;
  float scale;
  unsigned long long timeout_ns;
  unsigned long long* bar_count;          // [kNvlsMaxCta] barriers passed so far per CTA index (device memory)
  int* abort_flag;
  piccl_status_t* status;
};

// dtype: DT_F16, DT_F32 or DT_BF16 (exec.cuh); sum only.  Returns cudaSuccess or the launch error.
int nvls_launch(const NvlsArgs& a, int dtype, void* stream);
bool nvls_dtype_supported(int dtype);

}  // namespace piccl
