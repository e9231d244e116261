/* A minimal "NCCL application" for tests without a GPU: one communicator, each collective twice (once inside a group),
 * then destroy.  NCCL_APP_ZERO_FIRST=1: the very first call is an all-gather of zero elements (what one rank of a job may
 * issue while the others send data).  NCCL_APP_SPLIT=1: the communicator is finalized, and a split hands out the same handle
 * again.  It links against whatever provides the NCCL symbols; with the preload library in front the calls go through the
 * interposer first.  Prints the result code of every call class. */
#include <stdio.h>
#include <stdlib.h>
#include <stddef.h>

int ncclAllReduce(const void*, void*, size_t, int, int, void*, void*);
int ncclAllGather(const void*, void*, size_t, int, void*, void*);
int ncclReduceScatter(const void*, void*, size_t, int, int, void*, void*);
int ncclReduce(const void*, void*, size_t, int, int, int, void*, void*);
int ncclBroadcast(const void*, void*, size_t, int, int, void*, void*);
int ncclCommInitRank(void**, int, char[128], int);
int ncclCommDestroy(void*);
int ncclCommFinalize(void*);
int ncclCommSplit(void*, int, int, void**, void*);
int ncclCommGetAsyncError(void*, int*);
int ncclGroupStart(void);
int ncclGroupEnd(void);

int main(void) {
  void* comm = NULL; char id[128] = {0}; static float a[1024], b[8192];
  int rc = ncclCommInitRank(&comm, 1, id, 0);
  printf("init=%d\n", rc);
  const int f32 = 7, sum = 0;
  int bad = 0;
  if (getenv("NCCL_APP_ZERO_FIRST")) bad |= ncclAllGather(a, b, 0, f32, comm, NULL);
  for (int round = 0; round < 2; round++) {
    if (round) ncclGroupStart();
    bad |= ncclAllReduce(a, a, 1024, f32, sum, comm, NULL);
    bad |= ncclAllGather(a, b, 1024, f32, comm, NULL);
    bad |= ncclReduceScatter(b, a, 1024, f32, sum, comm, NULL);
    bad |= ncclReduce(a, a, 1024, f32, sum, 0, comm, NULL);
    bad |= ncclBroadcast(a, a, 1024, f32, 0, comm, NULL);
    if (round) ncclGroupEnd();
  }
  if (getenv("NCCL_APP_SPLIT")) {
    void* again = NULL;
    bad |= ncclCommFinalize(comm);
    bad |= ncclCommSplit(comm, 0, 0, &again, NULL);
    bad |= ncclAllReduce(a, a, 1024, f32, sum, again, NULL);
    comm = again;
  }
  int err = -1;
  rc = ncclCommGetAsyncError(comm, &err);
  printf("collectives=%d async=%d/%d\n", bad, rc, err);
  printf("destroy=%d\n", ncclCommDestroy(comm));
  return bad;
}
