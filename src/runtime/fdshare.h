// Rendezvous of the ranks of one communicator that live on one host, over an
// abstract Unix-domain socket: rank 0 hands every peer one file descriptor
// (SCM_RIGHTS), then all ranks pass barriers that also carry a verdict, so that
// a set-up step that fails on one rank is abandoned by all of them.
//
// Used to share the handle of an NVLink multicast object (runtime/nvls.cu): a
// POSIX file descriptor cannot travel through the 128-byte handle exchange.
// No GPU is involved here; tests/test_shim_cpu.py drives it with ordinary files.
// The reference has no counterpart (it never maps peer memory).
#pragma once
#include <string>
#include <vector>

namespace piccl {

struct FdShare {
  int rank = 0, nranks = 1, timeout_ms = 10000;
  int listen_fd = -1;
  std::vector<int> socks;     // rank 0: socks[p] for peer p (socks[0] unused); other ranks: socks[0] = connection to rank 0
  std::string error;
};

// Every call returns false on failure or time-out and leaves a message in `error`.
// Rank 0: listens on `name`, accepts nranks-1 peers and sends each of them `fd`.
// Other ranks: connect (retrying while rank 0 is not listening yet) and receive the descriptor into *fd_out.
bool fdshare_open(FdShare& s, const std::string& name, int fd, int* fd_out);
// All ranks: blocks until everybody arrived; *all_ok is the conjunction of every rank's `ok`.
bool fdshare_barrier(FdShare& s, bool ok, bool* all_ok);
void fdshare_close(FdShare& s);

}  // namespace piccl
