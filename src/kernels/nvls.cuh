// Collectives through the NVSwitch: contributions are summed inside the switch
// (`multimem.ld_reduce`) and results are written to every GPU at once
// (`multimem.st`), so a GPU sends and receives each byte about once instead of
// (n-1) times.  All five collectives take this path for large messages.  The
// reference has no counterpart: its collectives are sequences of
// ncclSend/ncclRecv groups and separate reduce kernels (src/coll/*.c).
//
// Every rank owns a window of device memory that is bound, at the same offset,
// to one multicast object, and sees it at two addresses: `uc` (its own copy)
// and `mc` (all copies at once).  Layout of a window:
//   [ kNvlsFlagBytes: counters, three per (CTA index, part of its slot), 128 bytes apart ]
//   [ one slot of slot_bytes per CTA index, used as `depth` parts ]
// CTA b of every rank works on chunks b, b + n_cta, ... of the message; chunk j of a CTA goes
// through part j % depth of its slot, and the groups of warps of the CTA (fill, switch, out; the one
// that talks to the switch split further) work on different chunks at the same time.
// One use of a part has up to three stages, each closed by one counter that every rank
// raises (by n in total) on all copies with a single multimem.red:
//   FILLED    the chunk is in the part            (all-reduce, reduce-scatter, reduce: every rank copied its own
//             data into its own copy; all-gather: every rank stored its piece into every copy with
//             multimem.st; broadcast: the root stored the chunk into every copy)
//   REDUCED   all-reduce only: every rank has summed its 1/n of the chunk in the switch and stored the
//             sums into every copy
//   CONSUMED  nobody reads this use of the part any more (all-reduce, all-gather, broadcast: copied
//             out; reduce-scatter / reduce: the multimem.ld_reduce that wrote the result straight to the
//             receive buffer is done)
// Nobody writes into a part before CONSUMED of its previous use is complete, whichever
// collective that use belonged to, so calls of different collectives may follow each other freely.
// Counters only ever grow, over the life of the communicator; the number of uses so far is kept
// in device memory, so a captured graph can be replayed.  Every poll is bounded: on a time-out
// the CTA records a status, raises the abort flag and leaves.
//
// For tests on one GPU the same kernels run with the switch emulated: all ranks are virtual ranks
// of one cooperative launch, a load-reduce is a loop over the ranks' windows, a multicast store a
// loop of stores (template parameter EMU).
#pragma once
#include <cstdint>
#include "../include/piccl.h"
#include "exec.cuh"

namespace piccl {

constexpr int kNvlsMaxCta = 128;
constexpr int kNvlsMaxDepth = 8;          // parts per slot, at most
constexpr int kNvlsFlagBytes = 524288;    // 128 CTA indices x 8 parts x 3 counters x 128 bytes = 384 KiB, rounded up
constexpr int kNvlsBlock = 512;
constexpr int kNvlsUsedPerCta = 2 * kNvlsMaxDepth;   // uses so far per CTA index: fills of part 0..7, then reductions (all-reduce) of part 0..7
enum NvlsCounter : int { NVC_FILLED = 0, NVC_REDUCED = 1, NVC_CONSUMED = 2 };

struct NvlsRank {
  char* uc; char* mc;                     // the window: own copy / all copies (mc unused when the switch is emulated)
  const void* in; void* out;
  unsigned long long* used;               // [kNvlsMaxCta * kNvlsUsedPerCta] device memory of this rank
  int* abort_flag;
  piccl_status_t* status;
  int rank, pad;
  unsigned long long* prof;               // PICCL_NVLS_PROFILE=1: [kNvlsProfSlots] nanoseconds summed over CTAs and calls (null: off)
};
// profile slots: time of thread 0 inside each kind of phase, and chunks / CTAs counted
enum NvlsProf : int { NVP_FILL = 0, NVP_WAIT_FILLED = 1, NVP_SWITCH = 2, NVP_WAIT_REDUCED = 3, NVP_OUT = 4, NVP_WAIT_CONSUMED = 5, NVP_CHUNKS = 6, NVP_CTAS = 7, NVP_TOTAL = 8 };
constexpr int kNvlsProfSlots = 16;

struct NvlsArgs {
  int coll, nranks, n_cta, n_vrank;
  int avg, root;
  float scale;
  long long bytes;                        // all-reduce, broadcast, reduce: message bytes; all-gather, reduce-scatter: bytes of one rank's block
  long long chunk_bytes;                  // bytes of the message (or of each rank's block) per chunk; a multiple of 16, of 16 * nranks for all-reduce
  long long sub_stride;                   // all-gather, reduce-scatter: distance between two ranks' pieces inside a part (>= chunk_bytes, multiple of 16)
  long long slot_bytes;                   // distance between two slots; a part is slot_bytes / depth (multiple of 16)
  int depth;                              // parts per slot (2 .. kNvlsMaxDepth): chunks a CTA has in flight
  int n_sub;                              // groups the stage that issues the multimem instructions is split into (1 or 3)
  int strict_fences;                      // 1: a system-wide fence before every counter update (see nv_arrive)
  int use_bulk;                           // 1: aligned copies between user buffers and the window go through the bulk-copy engine (TMA)
  unsigned long long timeout_ns;
  NvlsRank r[kMaxVRanks];
};

// dtype: DT_F32 (sum), DT_F16 / DT_BF16 (sum, max, min); op as ncclRedOp_t (0 sum, 2 max, 3 min).
// Copy-only collectives (all-gather, broadcast) use any supported pair.  emulate: virtual ranks on one device, cooperative launch.
bool nvls_kernel_exists(int dtype, int op);
int nvls_launch(const NvlsArgs& a, int dtype, int op, bool emulate, void* stream);
int nvls_max_resident_ctas(bool emulate);   // co-resident CTAs of the kernel on the current device (for the cooperative launch)

}  // namespace piccl
