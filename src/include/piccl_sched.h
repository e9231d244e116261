// Schedule layer: every collective algorithm is compiled, per rank, into a
// short program of uniform "actions" that one fused device kernel executes.
//
// An action is   value = reduce(local src?, recv peers...)  ->  local dst?, send peers...
// Data between ranks only ever moves through per-connection FIFOs (one per
// directed rank pair and CTA), so a program is correct iff, for every
// connection, the k-th entry pushed by the sender is the k-th entry popped by
// the receiver.  The validator (validate.cc) checks exactly that, with bounded
// FIFO capacity, on real data.
//
// Reference parity: the schedules reproduce the send/recv patterns of
// src/coll/{allgather,allreduce,broadcast,reduce,reduce_scatter}.c of the
// reference (RING, K_RING, RD, RM, PRD, PRM), but reduction and block placement
// are folded into the transfers: there is no separate reduce or permutation
// pass (reference: src/kernels/reduce_kernel.cu, permutation_kernel.cu).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace piccl {

enum Coll : int { COLL_ALLGATHER = 0, COLL_ALLREDUCE = 1, COLL_BROADCAST = 2, COLL_REDUCE = 3, COLL_REDUCE_SCATTER = 4, COLL_COUNT = 5 };
// Same names as the reference's piccl_algo_t (src/include/piccl.h:13-21) plus AUTO and DIRECT.
// DIRECT has no counterpart in the reference: every rank talks to every other rank at once, which a
// switch with full bandwidth between all pairs allows.  All-reduce: each rank owns 1/n of the vector,
// one exchange delivers the contributions to the owners, a second one returns the sums (the ring's
// traffic, 2(n-1)/n of the vector per rank, in 2 steps instead of 2(n-1)).  All-gather and
// reduce-scatter: PRM with k = n.  Broadcast: the root scatters n slices, the ranks all-gather them.
// Reduce: the ranks reduce-scatter n slices, the root gathers them.  At most 8 ranks (one action
// addresses 7 peers); larger groups fall back to RING.
// NVLS (all-reduce only, no counterpart either) is not a step schedule: the switch sums the contributions
// (src/kernels/nvls.cuh).  The schedule layer treats it as RING, which is also what runs when a communicator
// has no multicast window.
enum Algo : int { ALGO_DEFAULT_NCCL = 0, ALGO_RING = 1, ALGO_K_RING = 2, ALGO_RD = 3, ALGO_RM = 4, ALGO_PRD = 5, ALGO_PRM = 6, ALGO_AUTO = 7, ALGO_DIRECT = 8, ALGO_NVLS = 9 };

enum Buf : uint8_t { BUF_NONE = 0, BUF_IN = 1, BUF_OUT = 2, BUF_SCRATCH = 3 };

constexpr int kMaxActionPeers = 7;   // k-1 for the largest supported radix (8)
constexpr int kMaxRanks = 64;

// Flags of an action.
constexpr uint8_t ACT_SCALE_SRC = 1;  // local source is an original contribution (pre-scaled for avg)

// One unit of work, executed by every CTA on its slice of [0,count).
// Fixed 48-byte layout shared with the device code.
struct Action {
  uint8_t src_buf = BUF_NONE;   // local operand (BUF_NONE: none)
  uint8_t dst_buf = BUF_NONE;   // local destination (BUF_NONE: none)
  uint8_t n_recv = 0;           // FIFO sources
  uint8_t n_send = 0;           // FIFO sinks
  uint8_t self_pos = 0;         // position of the local operand among the recv peers (rank order)
  uint8_t flags = 0;
  uint8_t step = 0;             // schedule step the action belongs to (informational)
  uint8_t pad = 0;
  uint8_t recv_peer[kMaxActionPeers + 1] = {0};
  uint8_t send_peer[kMaxActionPeers + 1] = {0};
  int64_t src_off = 0;          // element offsets into the local buffers
  int64_t dst_off = 0;
  int64_t count = 0;            // elements
};
static_assert(sizeof(Action) == 48, "Action layout is shared with device code");

struct Program {
  int rank = 0, nranks = 0;
  int nsteps = 0;
  int64_t scratch_elems = 0;      // local scratch the program needs (elements)
  std::vector<Action> actions;    // ordered; actions of one step are contiguous
};

struct CollArgs {
  Coll coll = COLL_ALLREDUCE;
  Algo algo = ALGO_RING;
  int k = -1;                // group size / radix as given by the user (may be invalid)
  int nranks = 1;
  int root = 0;
  int64_t count = 0;         // allreduce/bcast/reduce: total elements; allgather: per-rank send count;
                             // reduce_scatter: per-rank recv count
  int64_t block_stride = 0;  // distance between rank blocks in the n-block buffer (0: = count)
  int elem_size = 4;
  bool in_place = false;
};

// Why a (coll, algo, k, n) combination cannot be compiled as asked and which
// replacement was used instead.
struct Resolved {
  Algo algo;
  int k;                       // effective k
  std::vector<int> radices;    // per step radix for the recursive algorithms
  int core = 0;                // ranks taking part in the recursive core (< nranks: the rest are followers; allreduce only)
  std::string note;            // empty if the request was taken as is
};

// Normalises the request: k unset/invalid, group sizes that do not divide n,
// rank counts that are not a power of the radix (mixed radix), radices too large.
Resolved resolve(Coll coll, Algo algo, int k, int nranks);

// Compile the program of one rank.  Never fails for nranks >= 1 (falls back
// to RING shapes through resolve()).
Program compile(const CollArgs& a, int rank);

// Chunking used by allreduce: chunk c covers [displ(c), displ(c)+cnt(c)); chunk
// starts are multiples of 16 bytes; tail chunks may be short or empty.
void ar_chunks(int64_t count, int nranks, int elem_size, std::vector<int64_t>& displ, std::vector<int64_t>& cnt);

// Ordered list of blocks rank r holds before step s of a recursive allgather
// (held[0] = {r}); `permuted` selects farthest-partner-first (PRD/PRM).
std::vector<int> held_blocks(int r, int s, const std::vector<int>& radices, int nranks, bool permuted);
// Peers of rank r in step s (excluding r), in exchange order.
std::vector<int> step_peers(int r, int s, const std::vector<int>& radices, int nranks, bool permuted);

// perm[q] = digitwiseAdd_b(r, digitReverse_b(q, d)), d = log_b n — the placement
// table of the reference's computePermutationKernel
// (src/kernels/permutation_kernel.cu:166-207).  Returns false if n is not b^d.
bool permutation_index(int r, int n, int b, std::vector<int>& perm);

// ---- validation (CPU data-flow execution of all ranks' programs) ----
struct ValidateResult {
  bool ok = false;
  std::string error;
  int64_t fifo_entries = 0;       // transfers executed (segment granularity)
  int max_fifo_depth = 0;
  double max_abs_err = 0.0;
  int64_t bytes_sent_max_rank = 0;
};
// Executes the programs of all ranks on seeded data (fp32: uniform[-1,1),
// seed 0; int32 in [-1000,1000] when integer=true) with FIFOs of `fifo_cap`
// entries and segments of `seg_elems` elements, and compares with a serial
// reduction.  op: 0 sum, 1 prod, 2 max, 3 min.
// defer_publish models the executor variant that holds its counter updates back until it is about to block (exec_impl.cuh).
ValidateResult validate(const CollArgs& a, int op, bool integer, int fifo_cap, int64_t seg_elems, int n_cta, bool defer_publish = false);

// Symbolic check for sizes too large to materialise: coverage of every output
// element and FIFO order, no data.
ValidateResult validate_symbolic(const CollArgs& a, int fifo_cap, int n_cta, bool defer_publish = false);

// ---- dumps ----
// Transfers in the reference's schedule XML format
// (tools/loggp_sim/README.md:13-26): <collective ...><transfer id size src dst deps/>...
std::string dump_xml(const CollArgs& a);
std::string dump_json(const CollArgs& a, int rank);

const char* coll_name(Coll c);
const char* algo_name(Algo a);
Algo algo_from_string(const char* s);   // RING, K_RING, RD, RM, PRD, PRM, AUTO, DIRECT, NVLS; else DEFAULT_NCCL

}  // namespace piccl
