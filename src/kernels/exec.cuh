// Device-side data structures of the fused collective executor and the
// layout of the per-rank symmetric heap.
//
//   heap = [ tail counters | head counters | scratch | FIFO slots ]
//
// tail[src][cta]  (in the receiver's heap, written by `src`): entries `src` has pushed
// head[dst][cta]  (in the sender's heap, written by `dst`):   entries `dst` has consumed
// slot(src, cta, i) (in the receiver's heap): payload of entry number e with e % nslot == i
//
// All counters only ever grow, over the whole life of the communicator, so a
// collective never has to reset anything and a captured CUDA graph can be
// replayed.  The reference has no counterpart: it moves data with
// ncclSend/ncclRecv groups and keeps three process-global scratch buffers
// (src/piccl.c:175-199).
#pragma once
#include <cstdint>
#include "../include/piccl.h"
#include "../include/piccl_sched.h"

namespace piccl {

constexpr int kFlagStride = 128;          // bytes between two counters
constexpr int kMaxVRanks = 8;             // virtual ranks one launch can carry (single-GPU emulation)
constexpr int kMaxBlock = 512;
constexpr int kLLFifoCta = 8, kLLFifoSlots = 8, kLLFifoSlotBytes = 8192;   // low-latency FIFO: CTAs, ring depth, bytes per slot (half of it payload)

struct RankCtx {
  int rank, nranks, max_cta, nslot;
  long long slot_bytes;
  long long tail_off, head_off, ll_off, scratch_off, fifo_off, heap_bytes;
  long long ll_slot_bytes;                // bytes of one low-latency slot (2 x the largest payload)
  long long scratch_bytes;
  long long llf_off, llf_head_off;                // low-latency FIFO of the executor: lines and head counters
  long long tp_flag_off, tp_data_off, tp_bytes;   // tensor-parallel workspace: epoch flags (1 MiB, zeroed) and payload
  char* heap[kMaxRanks];                  // every rank's heap as mapped in this process
  unsigned long long* sent;               // [nranks * max_cta] entries pushed per (peer, cta)
  unsigned long long* rcvd;               // [nranks * max_cta] entries consumed per (peer, cta)
  unsigned long long* sent_ll;            // [nranks * kLLFifoCta] the same for the low-latency FIFO
  unsigned long long* rcvd_ll;
  int* abort_flag;                        // device memory; non-zero: every wait gives up
  piccl_status_t* status;                 // pinned host memory, device address
};

struct LaunchRank {
  RankCtx* ctx;
  const Action* actions;
  int n_actions;
  int pad;
  const void* in;
  void* out;
};

struct KernelArgs {
  int n_vrank;
  int n_cta;
  int elem_size;
  int avg;                                // 1: scale original contributions by `scale`
  float scale;
  unsigned long long timeout_ns;
  LaunchRank r[kMaxVRanks];
};

// ---- low-latency all-reduce (ll_allreduce.cu)
constexpr int kLLMaxSteps = 6;
constexpr int kLLBlock = 256;
struct LLRank { RankCtx* ctx; const void* in; void* out; };
struct LLArgs {
  int n_vrank, n_cta, nsteps, avg;
  float scale;
  unsigned epoch;
  unsigned long long timeout_ns;
  long long count;
  uint8_t npeers[kLLMaxSteps];
  uint8_t peers[kMaxVRanks][kLLMaxSteps][kMaxActionPeers];     // ascending rank
  uint8_t self_pos[kMaxVRanks][kLLMaxSteps];                   // partners with a rank below mine
  LLRank r[kMaxVRanks];
};
typedef void (*LLKernelFn)(LLArgs);
// ---- low-latency all-gather / reduce-scatter: one exchange with every rank (ll_exchange.cu)
struct LLXArgs {
  int n_vrank, n_cta, avg;
  float scale;
  unsigned epoch;
  unsigned long long timeout_ns;
  long long count;                        // all-gather: BYTES per rank; reduce-scatter: elements per rank
  LLRank r[kMaxVRanks];
};
typedef void (*LLXKernelFn)(LLXArgs);
LLXKernelFn llx_allgather_kernel();
LLXKernelFn llx_reduce_scatter_kernel_for(int dtype, int op);
int llx_lines_per_cta();
LLKernelFn ll_kernel_for(int dtype, int op);
int ll_lines_per_cta();

// dtype index used by the launcher tables (order of ncclDataType_t)
enum DType : int { DT_I8 = 0, DT_U8 = 1, DT_I32 = 2, DT_U32 = 3, DT_I64 = 4, DT_U64 = 5, DT_F16 = 6, DT_F32 = 7, DT_F64 = 8, DT_BF16 = 9, DT_COUNT = 10 };
inline int dtype_size(int dt) {
  static const int s[DT_COUNT] = {1, 1, 4, 4, 8, 8, 2, 4, 8, 2};
  return (dt >= 0 && dt < DT_COUNT) ? s[dt] : 0;
}

typedef void (*ExecKernelFn)(KernelArgs);
// [dtype][op 0..3]; filled by the exec_inst_*.cu translation units.
ExecKernelFn exec_kernel_for(int dtype, int op);
ExecKernelFn exec_copy_kernel();
ExecKernelFn exec_defer_kernel_for(int dtype, int op);   // counter updates held back until the CTA is about to block (PICCL_EXEC_DEFER=1)
ExecKernelFn exec_defer_copy_kernel();
ExecKernelFn exec_ll_kernel_for(int dtype, int op);   // low-latency variant (exec_ll.cuh)
ExecKernelFn exec_ll_copy_kernel();

}  // namespace piccl
