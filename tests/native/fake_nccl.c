/* A stand-in for libnccl.so.2 for tests without a GPU: every entry point succeeds, touches no memory and counts its calls.
 * FAKE_NCCL_RANKS sets what ncclCommCount reports (default 1).  The counters are printed when the process ends.
 * Only the ABI matters here (pointer-sized handles, int enums), so no NCCL header is needed. */
#include <stdio.h>
#include <stdlib.h>
#include <stddef.h>

static unsigned long n_ar, n_ag, n_rs, n_rd, n_bc, n_init, n_destroy, n_group;
static int fake_comm;

static int ranks(void) { const char* v = getenv("FAKE_NCCL_RANKS"); return v ? atoi(v) : 1; }

int ncclAllReduce(const void* s, void* r, size_t c, int dt, int op, void* comm, void* st) { (void)s; (void)r; (void)c; (void)dt; (void)op; (void)comm; (void)st; n_ar++; return 0; }
int ncclAllGather(const void* s, void* r, size_t c, int dt, void* comm, void* st) { (void)s; (void)r; (void)c; (void)dt; (void)comm; (void)st; n_ag++; return 0; }
int ncclReduceScatter(const void* s, void* r, size_t c, int dt, int op, void* comm, void* st) { (void)s; (void)r; (void)c; (void)dt; (void)op; (void)comm; (void)st; n_rs++; return 0; }
int ncclReduce(const void* s, void* r, size_t c, int dt, int op, int root, void* comm, void* st) { (void)s; (void)r; (void)c; (void)dt; (void)op; (void)root; (void)comm; (void)st; n_rd++; return 0; }
int ncclBroadcast(const void* s, void* r, size_t c, int dt, int root, void* comm, void* st) { (void)s; (void)r; (void)c; (void)dt; (void)root; (void)comm; (void)st; n_bc++; return 0; }
int ncclBcast(void* b, size_t c, int dt, int root, void* comm, void* st) { (void)b; (void)c; (void)dt; (void)root; (void)comm; (void)st; n_bc++; return 0; }
int ncclCommInitRank(void** comm, int n, char id[128], int rank) { (void)n; (void)id; (void)rank; *comm = &fake_comm; n_init++; return 0; }
int ncclCommDestroy(void* comm) { (void)comm; n_destroy++; return 0; }
int ncclCommFinalize(void* comm) { (void)comm; return 0; }
int ncclCommSplit(void* comm, int color, int key, void** newcomm, void* config) { (void)comm; (void)color; (void)key; (void)config; *newcomm = &fake_comm; n_init++; return 0; }
int ncclCommAbort(void* comm) { (void)comm; return 0; }
int ncclCommGetAsyncError(void* comm, int* err) { (void)comm; *err = 0; return 0; }
int ncclCommCount(void* comm, int* n) { (void)comm; *n = ranks(); return 0; }
int ncclCommUserRank(void* comm, int* r) { (void)comm; *r = 0; return 0; }
int ncclCommCuDevice(void* comm, int* d) { (void)comm; *d = 0; return 0; }
int ncclGroupStart(void) { n_group++; return 0; }
int ncclGroupEnd(void) { return 0; }

__attribute__((destructor)) static void report(void) {
  printf("FAKE_NCCL allreduce=%lu allgather=%lu reduce_scatter=%lu reduce=%lu broadcast=%lu init=%lu destroy=%lu group=%lu\n", n_ar, n_ag, n_rs, n_rd, n_bc, n_init, n_destroy, n_group);
}
