#include "fdshare.h"
#include <algorithm>
#include <cerrno>
#include <cstddef>
#include <chrono>
#include <cstring>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <thread>
#include <unistd.h>

namespace piccl {

namespace {

typedef std::chrono::steady_clock Clock;
long long ms_left(Clock::time_point deadline) { return std::chrono::duration_cast<std::chrono::milliseconds>(deadline - Clock::now()).count(); }

// abstract namespace: no file to clean up, gone when the last descriptor closes
socklen_t make_addr(const std::string& name, sockaddr_un& a) {
  memset(&a, 0, sizeof a);
  a.sun_family = AF_UNIX;
  size_t n = std::min(name.size(), sizeof(a.sun_path) - 2);
  memcpy(a.sun_path + 1, name.data(), n);
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

bool wait_fd(int fd, short events, Clock::time_point deadline) {
  for (;;) {
    long long left = ms_left(deadline);
    if (left <= 0) return false;
    pollfd p{fd, events, 0};
    int r = poll(&p, 1, (int)std::min<long long>(left, 1000));
    if (r > 0) return (p.revents & (events | POLLHUP)) != 0;
    if (r < 0 && errno != EINTR) return false;
  }
}

bool send_all(int fd, const void* buf, size_t n, Clock::time_point deadline) {
  const char* p = (const char*)buf;
  while (n) {
    if (!wait_fd(fd, POLLOUT, deadline)) return false;
    ssize_t w = send(fd, p, n, MSG_NOSIGNAL);
    if (w < 0) { if (errno == EINTR || errno == EAGAIN) continue; return false; }
    p += w; n -= (size_t)w;
  }
  return true;
}

bool recv_all(int fd, void* buf, size_t n, Clock::time_point deadline) {
  char* p = (char*)buf;
  while (n) {
    if (!wait_fd(fd, POLLIN, deadline)) return false;
    ssize_t r = recv(fd, p, n, 0);
    if (r == 0) return false;                       // peer closed
    if (r < 0) { if (errno == EINTR || errno == EAGAIN) continue; return false; }
    p += r; n -= (size_t)r;
  }
  return true;
}

// one byte of payload carries the descriptor as ancillary data
bool send_fd(int sock, int fd, Clock::time_point deadline) {
  if (!wait_fd(sock, POLLOUT, deadline)) return false;
  char byte = 'F';
  iovec iov{&byte, 1};
  alignas(cmsghdr) char ctl[CMSG_SPACE(sizeof(int))];
  memset(ctl, 0, sizeof ctl);
  msghdr m{}; m.msg_iov = &iov; m.msg_iovlen = 1; m.msg_control = ctl; m.msg_controllen = sizeof ctl;
  cmsghdr* c = CMSG_FIRSTHDR(&m);
  c->cmsg_level = SOL_SOCKET; c->cmsg_type = SCM_RIGHTS; c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  for (;;) {
    ssize_t w = sendmsg(sock, &m, MSG_NOSIGNAL);
    if (w == 1) return true;
    if (w < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    return false;
  }
}

bool recv_fd(int sock, int* fd, Clock::time_point deadline) {
  if (!wait_fd(sock, POLLIN, deadline)) return false;
  char byte = 0;
  iovec iov{&byte, 1};
  alignas(cmsghdr) char ctl[CMSG_SPACE(sizeof(int))];
  memset(ctl, 0, sizeof ctl);
  msghdr m{}; m.msg_iov = &iov; m.msg_iovlen = 1; m.msg_control = ctl; m.msg_controllen = sizeof ctl;
  for (;;) {
    ssize_t r = recvmsg(sock, &m, MSG_CMSG_CLOEXEC);
    if (r < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    if (r != 1 || byte != 'F') return false;
    break;
  }
  for (cmsghdr* c = CMSG_FIRSTHDR(&m); c; c = CMSG_NXTHDR(&m, c))
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS && c->cmsg_len >= CMSG_LEN(sizeof(int))) { memcpy(fd, CMSG_DATA(c), sizeof(int)); return true; }
  return false;
}

bool fail(FdShare& s, const std::string& what) { s.error = what; return false; }

}  // namespace

bool fdshare_open(FdShare& s, const std::string& name, int fd, int* fd_out) {
  const auto deadline = Clock::now() + std::chrono::milliseconds(s.timeout_ms);
  sockaddr_un addr; socklen_t alen = make_addr(name, addr);
  if (s.nranks <= 1) { if (fd_out) *fd_out = -1; return true; }
  if (s.rank == 0) {
    s.socks.assign(s.nranks, -1);
    s.listen_fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (s.listen_fd < 0) return fail(s, std::string("socket: ") + strerror(errno));
    if (bind(s.listen_fd, (sockaddr*)&addr, alen) != 0) return fail(s, std::string("bind: ") + strerror(errno));
    if (listen(s.listen_fd, s.nranks) != 0) return fail(s, std::string("listen: ") + strerror(errno));
    for (int got = 0; got < s.nranks - 1;) {
      if (!wait_fd(s.listen_fd, POLLIN, deadline)) return fail(s, "timed out waiting for " + std::to_string(s.nranks - 1 - got) + " peer(s) to connect");
      int c = accept4(s.listen_fd, nullptr, nullptr, SOCK_CLOEXEC);
      if (c < 0) { if (errno == EINTR || errno == EAGAIN) continue; return fail(s, std::string("accept: ") + strerror(errno)); }
      int peer = -1;
      if (!recv_all(c, &peer, sizeof peer, deadline) || peer < 1 || peer >= s.nranks || s.socks[peer] != -1) { close(c); return fail(s, "a peer did not introduce itself with a valid rank"); }
      s.socks[peer] = c; got++;
    }
    for (int p = 1; p < s.nranks; p++)
      if (!send_fd(s.socks[p], fd, deadline)) return fail(s, "could not send the descriptor to rank " + std::to_string(p));
    if (fd_out) *fd_out = fd;
    return true;
  }
  s.socks.assign(1, -1);
  for (;;) {
    int c = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (c < 0) return fail(s, std::string("socket: ") + strerror(errno));
    if (connect(c, (sockaddr*)&addr, alen) == 0) { s.socks[0] = c; break; }
    int e = errno; close(c);
    if (e != ECONNREFUSED && e != ENOENT && e != EAGAIN && e != EINTR) return fail(s, std::string("connect: ") + strerror(e));
    if (ms_left(deadline) <= 0) return fail(s, "timed out waiting for rank 0 to listen");
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
  if (!send_all(s.socks[0], &s.rank, sizeof s.rank, deadline)) return fail(s, "could not reach rank 0");
  int got = -1;
  if (!recv_fd(s.socks[0], &got, deadline)) return fail(s, "no descriptor from rank 0");
  if (fd_out) *fd_out = got; else close(got);
  return true;
}

bool fdshare_barrier(FdShare& s, bool ok, bool* all_ok) {
  const auto deadline = Clock::now() + std::chrono::milliseconds(s.timeout_ms);
  if (all_ok) *all_ok = ok;
  if (s.nranks <= 1) return true;
  if (s.rank == 0) {
    char verdict = ok ? 1 : 0;
    for (int p = 1; p < s.nranks; p++) {
      char v = 0;
      if (!recv_all(s.socks[p], &v, 1, deadline)) { verdict = 0; s.error = "rank " + std::to_string(p) + " did not reach the barrier"; }
      else if (!v) verdict = 0;
    }
    // tell whoever still listens, also after a failure, so that nobody waits for its own time-out
    bool sent = true;
    const auto send_deadline = std::max(deadline, Clock::now() + std::chrono::milliseconds(1000));
    for (int p = 1; p < s.nranks; p++) sent &= send_all(s.socks[p], &verdict, 1, send_deadline);
    if (all_ok) *all_ok = verdict != 0;
    return sent && s.error.empty();
  }
  char v = ok ? 1 : 0, verdict = 0;
  if (!send_all(s.socks[0], &v, 1, deadline)) return fail(s, "could not reach rank 0");
  if (!recv_all(s.socks[0], &verdict, 1, deadline)) return fail(s, "no verdict from rank 0");
  if (all_ok) *all_ok = verdict != 0;
  return true;
}

void fdshare_close(FdShare& s) {
  for (int& c : s.socks) if (c >= 0) { close(c); c = -1; }
  if (s.listen_fd >= 0) { close(s.listen_fd); s.listen_fd = -1; }
}

}  // namespace piccl

// C entry point for the tests: the whole sequence with an ordinary descriptor.
// Returns 0 and the received descriptor in *fd_out; `ok_in` is this rank's vote in the
// barrier that follows, *all_ok_out the common verdict.  A negative result names the step that failed.
extern "C" int piccl_fdshare_selftest(int rank, int nranks, const char* name, int fd, int timeout_ms, int ok_in, int* fd_out, int* all_ok_out, char* err, int err_len) {
  piccl::FdShare s; s.rank = rank; s.nranks = nranks; s.timeout_ms = timeout_ms;
  int rc = 0; bool all_ok = false;
  if (!piccl::fdshare_open(s, name, fd, fd_out)) rc = -1;
  else if (!piccl::fdshare_barrier(s, ok_in != 0, &all_ok)) rc = -2;
  if (all_ok_out) *all_ok_out = all_ok ? 1 : 0;
  if (err && err_len > 0) { strncpy(err, s.error.c_str(), (size_t)err_len - 1); err[err_len - 1] = 0; }
  piccl::fdshare_close(s);
  return rc;
}
