/* Public C interface of the B200-native PICCL library.
 *
 * The NCCL ABI itself (ncclAllReduce, ncclAllGather, ncclReduceScatter,
 * ncclReduce, ncclBroadcast, ncclCommInitRank, ncclCommDestroy, ...) is exported
 * by the same shared object for LD_PRELOAD use and is declared in <nccl.h>; the
 * reference exports the first seven of those (src/piccl.c:29-199).  Everything
 * below is additional: a direct API for programs that link or dlopen the
 * library (the Python package, the benchmarks), the schedule layer, statistics.
 *
 * dtype / op arguments use the numeric values of ncclDataType_t / ncclRedOp_t.
 * All collectives are stream ordered and return immediately.
 */
#ifndef PICCL_B200_H
#define PICCL_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- enums (values shared with the schedule layer) ---- */
enum { PICCL_ALLGATHER = 0, PICCL_ALLREDUCE = 1, PICCL_BROADCAST = 2, PICCL_REDUCE = 3, PICCL_REDUCE_SCATTER = 4 };
enum { PICCL_ALGO_DEFAULT = 0, PICCL_ALGO_RING = 1, PICCL_ALGO_K_RING = 2, PICCL_ALGO_RD = 3, PICCL_ALGO_RM = 4,
       PICCL_ALGO_PRD = 5, PICCL_ALGO_PRM = 6, PICCL_ALGO_AUTO = 7,
       PICCL_ALGO_DIRECT = 8 /* every rank exchanges with every other rank at once; at most 8 ranks */,
       PICCL_ALGO_NVLS = 9 /* through the NVSwitch: multimem load-reduce / multicast stores; without a multicast window the peer-to-peer choice of AUTO runs */ };
/* result codes: 0 ok; others mirror ncclResult_t */
enum { PICCL_OK = 0, PICCL_CUDA_ERROR = 1, PICCL_SYSTEM_ERROR = 2, PICCL_INTERNAL_ERROR = 3, PICCL_INVALID_ARGUMENT = 4,
       PICCL_INVALID_USAGE = 5, PICCL_REMOTE_ERROR = 6, PICCL_UNSUPPORTED = 100 };

/* ---- configuration ---- */
typedef struct {
  int max_cta;            /* FIFO channels (CTAs) per collective; 0: PICCL_MAX_CTA or 64 */
  int nslot;              /* FIFO depth per connection; 0: default 4 */
  long long slot_bytes;   /* bytes per FIFO slot; 0: PICCL_SLOT_KB or 512 KiB */
  long long scratch_bytes;/* local scratch for recursive reduce-scatter; 0: default 64 MiB */
  int block_size;         /* threads per CTA; 0: PICCL_BLOCK_SIZE or 512 */
  int timeout_ms;         /* bound of every device-side wait; 0: PICCL_TIMEOUT_MS or 10000 */
  long long tp_bytes;     /* workspace of the fused tensor-parallel kernels; 0: PICCL_TP_MB (default none) */
  int nvls_cta;           /* CTAs (slots of the multicast window) of the in-switch collectives; 0: PICCL_NVLS_CTA or 128.  Fewer CTAs leave
                             more SMs to kernels that run at the same time (48 suits gradient buckets overlapped with a backward pass) */
} piccl_config_t;

typedef struct piccl_comm piccl_comm_t;
/* Opaque blob a rank publishes so that its peers can map its heap. */
typedef struct { unsigned char bytes[128]; } piccl_handle_t;

/* Device-reported status of the last failed wait (all zero while healthy). */
typedef struct {
  int aborted;      /* 1 after a device-side wait ran out or piccl_comm_abort() */
  int code;         /* 1: wait for FIFO credit, 2: wait for FIFO data, 3: aborted by host/peer CTA,
                       5 / 6 / 7: in-switch collective, wait for a chunk to be filled / reduced / consumed by all ranks (segment = chunk);
                       8: in-switch collective, a bulk copy did not arrive */
  int rank, cta, action, peer, segment;
  unsigned long long want, have;   /* counter value waited for / last seen */
} piccl_status_t;

typedef struct {
  unsigned long long calls[5];      /* per collective */
  unsigned long long bytes[5];
  unsigned long long launches;      /* executor kernels launched */
  unsigned long long program_cache_hits, program_cache_misses;
  unsigned long long fallbacks;     /* calls the executor declined (reason logged with PICCL_LOG>=1) */
  unsigned long long timeouts;
  unsigned long long persistent_calls; /* calls served by the persistent launcher instead of a kernel launch */
  unsigned long long nvls_calls;       /* collectives run through the switch */
} piccl_stats_t;

/* ---- communicator life cycle ----
 * create (allocates and clears the symmetric heap on `device`) -> publish the
 * local handle to all ranks by any means -> connect with all ranks' handles. */
int piccl_comm_create(int rank, int nranks, int device, const piccl_config_t* cfg, piccl_comm_t** out);
int piccl_comm_local_handle(piccl_comm_t* c, piccl_handle_t* out);
int piccl_comm_connect(piccl_comm_t* c, const piccl_handle_t* all_handles);
int piccl_comm_destroy(piccl_comm_t* c);
int piccl_comm_abort(piccl_comm_t* c);                      /* makes running and future kernels return */
int piccl_comm_status(piccl_comm_t* c, piccl_status_t* out);/* never blocks */
int piccl_get_stats(piccl_comm_t* c, piccl_stats_t* out);
/* What AUTO resolves to for `nranks` ranks: PICCL_TUNE_FILE table first, then the built-in rule; *k gets the radix / group size. */
int piccl_select_algorithm(int nranks, int coll, unsigned long long bytes, int* k);
/* The same for a communicator that has (have_window != 0) or lacks an NVLink multicast window. */
int piccl_select_algorithm_ex(int nranks, int coll, unsigned long long bytes, int have_window, int* k);
/* The configuration in force as "key=value" pairs; returns the length needed, like snprintf. */
int piccl_env_describe(char* buf, int len);
/* Reads the PICCL_* environment again; call it on every rank at the same point between collectives. */
void piccl_env_reload(void);
int piccl_comm_rank(piccl_comm_t* c);
int piccl_comm_nranks(piccl_comm_t* c);
const char* piccl_last_error(void);                         /* thread-local text of the last failure */

/* ---- collectives ----  algo: PICCL_ALGO_*; k: group size / radix (<=0: default) */
int piccl_allreduce(piccl_comm_t* c, const void* send, void* recv, size_t count, int dtype, int op, int algo, int k, void* stream);
int piccl_allgather(piccl_comm_t* c, const void* send, void* recv, size_t sendcount, int dtype, int algo, int k, void* stream);
int piccl_reduce_scatter(piccl_comm_t* c, const void* send, void* recv, size_t recvcount, int dtype, int op, int algo, int k, void* stream);
int piccl_reduce(piccl_comm_t* c, const void* send, void* recv, size_t count, int dtype, int op, int root, int algo, int k, void* stream);
int piccl_broadcast(piccl_comm_t* c, const void* send, void* recv, size_t count, int dtype, int root, int algo, int k, void* stream);

/* Runs one collective over several communicators of THIS process that live on
 * the same device (virtual ranks) as a single cooperative kernel launch.  Used
 * to exercise the multi-rank protocol on one GPU. */
int piccl_group_collective(piccl_comm_t** comms, int ncomms, int coll, const void* const* send, void* const* recv,
                           size_t count, int dtype, int op, int root, int algo, int k, void* stream);

/* ---- fused tensor-parallel kernels (tcgen05 GEMM + peer-memory collective in one kernel) ----
 * All operands bf16, row-major, contiguous, 16-byte aligned.  The communicator needs tp_bytes >=
 * piccl_tp_workspace_bytes(...).  M % (128 * nranks) == 0, N % 256 == 0 (N_local % 128), K % 64 == 0.
 *
 * piccl_gemm_rs:  out[M/n, N] = rows [rank*M/n, (rank+1)*M/n) of  sum_r A_r[M, K_local] * B_r[N, K_local]^T
 * piccl_ag_gemm:  out[M, N_local] = concat_r(A_r[M/n, K]) * B[N_local, K]^T
 * The *_group variants run several communicators of this process (virtual ranks on one device) as a
 * single cooperative launch. */
long long piccl_tp_workspace_bytes(int which /*0 gemm_rs, 1 ag_gemm*/, int nranks, int M, int N, int K);
int piccl_gemm_rs(piccl_comm_t* c, const void* A, const void* B, void* out, int M, int N, int K_local, void* stream);
int piccl_ag_gemm(piccl_comm_t* c, const void* A_shard, const void* B, void* out, int M, int N_local, int K, void* stream);
int piccl_gemm_rs_group(piccl_comm_t** comms, int n, const void* const* A, const void* const* B, void* const* out, int M, int N, int K_local, void* stream);
int piccl_ag_gemm_group(piccl_comm_t** comms, int n, const void* const* A_shard, const void* const* B, void* const* out, int M, int N_local, int K, void* stream);
int piccl_tp_status(piccl_comm_t* c);   /* 0, or the role that gave up on a wait; synchronises */

/* Test hook: launches the executor with one action that waits for data nobody
 * sends.  The wait runs into its time limit, the kernel returns and the status
 * reports it; the communicator is unusable afterwards. */
int piccl_test_unmatched_wait(piccl_comm_t* c, int timeout_ms, void* stream);

/* ---- schedule layer (CPU only) ---- */
int piccl_algo_from_string(const char* s);
long long piccl_sched_xml(int coll, int algo, int k, int n, int root, long long count, int elem_size, char* buf, long long cap);
long long piccl_sched_json(int coll, int algo, int k, int n, int root, long long count, int elem_size, int rank, char* buf, long long cap);
int piccl_sched_resolve(int coll, int algo, int k, int n, int* out_algo, int* out_k, int* radices, int* n_radices, int* core, char* note, int note_cap);
int piccl_sched_validate(int coll, int algo, int k, int n, int root, long long count, long long stride, int elem_size, int in_place,
                         int op, int integer, int fifo_cap, long long seg_elems, int n_cta, int symbolic,
                         long long* fifo_entries, int* max_depth, double* max_err, long long* bytes_sent, char* err, int err_cap);
int piccl_permutation_index(int r, int n, int b, int* out);
int piccl_held_blocks(int r, int s, const int* radices, int n_radices, int n, int permuted, int* out);
int piccl_sched_counts(int coll, int algo, int k, int n, int root, long long count, int elem_size, int rank, int* n_actions, int* n_steps, long long* scratch_elems);

#ifdef __cplusplus
}
#endif
#endif
