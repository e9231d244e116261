// Stand-alone driver of the descriptor hand-over (src/runtime/fdshare.cc) for the sanitizer builds:
//   fdshare_main RANK NRANKS NAME TIMEOUT_MS VOTE [FILE]
// Rank 0 opens FILE and hands the descriptor to the peers; every rank prints "rc all_ok first-bytes-of-the-file".
#include <cstdio>
#include <cstdlib>
#include <fcntl.h>
#include <unistd.h>

extern "C" int piccl_fdshare_selftest(int rank, int nranks, const char* name, int fd, int timeout_ms, int ok_in, int* fd_out, int* all_ok_out, char* err, int err_len);

int main(int argc, char** argv) {
  if (argc < 6) { fprintf(stderr, "usage: fdshare_main RANK NRANKS NAME TIMEOUT_MS VOTE [FILE]\n"); return 2; }
  const int rank = atoi(argv[1]), nranks = atoi(argv[2]), timeout_ms = atoi(argv[4]), vote = atoi(argv[5]);
  int fd = -1;
  if (rank == 0 && argc > 6) fd = open(argv[6], O_RDONLY);
  int out = -1, all_ok = 0; char err[256] = {0};
  const int rc = piccl_fdshare_selftest(rank, nranks, argv[3], fd, timeout_ms, vote, &out, &all_ok, err, sizeof err);
  char text[32] = {0};
  if (out >= 0) { ssize_t n = pread(out, text, sizeof text - 1, 0); if (n < 0) text[0] = 0; }
  printf("%d %d %s|%s\n", rc, all_ok, text, err);
  if (out >= 0 && out != fd) close(out);
  if (fd >= 0) close(fd);
  return 0;
}
