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
// A pipelined variant (PICCL_NVLS_PIPE=1) splits the slot in two halves and overlaps the copy-in of the next chunk with
// the switch phase of the current one; see the kernel.
// Barrier counters only ever grow (n per barrier), over the life of the communicator.
// Every poll is bounded: on a time-out the CTA records a status, raises the abort flag and leaves.
#pragma once
#include <cstdint>
#include "../include/piccl.h"

namespace piccl {

constexpr int kNvlsFlagBytes = 131072;
constexpr int kNvlsMaxCta = 256;          // counters of the plain kernel: [0, 32 KiB)
constexpr int kNvlsPipeFlagOff = 32768;   // counters of the pipelined kernel: 4 per CTA index, [32 KiB, 96 KiB)
constexpr int kNvlsPipeMaxCta = 128;
constexpr int kNvlsBarCounts = kNvlsMaxCta + 2 * kNvlsPipeMaxCta;   // entries of NvlsArgs::bar_count
constexpr int kNvlsBlock = 512;

struct NvlsArgs {
  char* uc; char* mc;                     // the window: own copy / all copies
  const void* in; void* out;
  long long bytes;                        // message size
  long long chunk_bytes;                  // bytes of the message per chunk, multiple of 16 * nranks, <= slot_bytes
  long long slot_bytes;                   // distance between two slots of the window
  int rank, nranks, n_cta, avg;
  int pipelined;                          // 0: one chunk in flight per CTA; 1: two half slots, copy-in overlapped with the switch phase (n_cta <= kNvlsPipeMaxCta)
  float scale;
  unsigned long long timeout_ns;
  unsigned long long* bar_count;          // [kNvlsBarCounts] device memory: barriers passed per CTA index (plain kernel), then uses of each half slot (pipelined)
  int* abort_flag;
  piccl_status_t* status;
};

// dtype: DT_F16, DT_F32 or DT_BF16 (exec.cuh); sum only.  Returns cudaSuccess or the launch error.
int nvls_launch(const NvlsArgs& a, int dtype, void* stream);
bool nvls_dtype_supported(int dtype);

}  // namespace piccl
