// loggp_bench: PRTT (parametrised round trip time) measurements between two
// GPUs of one node, with the same primitives the collective executor uses
// (16-byte peer stores into the partner's memory, fence + release flag, acquire
// polling), timed on the device with %globaltimer.  Output is the raw table
// tools/loggp_param/get_loggp_param.py fits LogGP parameters from:
//
//   size n d PRTT(1,0,s) PRTT(n,0,s) PRTT(n,d,s) PRTT_server(n-1,d,s)      (seconds)
//
// PRTT(n,d,s): the client sends n messages of s bytes, waiting d between them; the server answers
// the last one with a message of s bytes; the client measures from its first send to the arrival of
// the answer.  PRTT_server: on the server, from the arrival of the first to the arrival of the last.
// The reference gets these numbers from its fork of the OSU micro-benchmarks over MPI
// (download_libs.sh:24-27), which is not available offline; its shipped profiles are A100 data.
//
//   loggp_bench [--dev0 0 --dev1 1] [--n 16] [--ctas 1] [--min 1] [--max 16777216] [--reps 20] > raw.csv
//
// Client and server kernels run on DIFFERENT GPUs; every wait has a limit (1 s) and sets an error flag.
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_)); exit(1); } } while (0)

struct Side {
  char* my_buf;                 // payload area in MY memory (the partner writes here)
  char* peer_buf;               // payload area in the PARTNER's memory
  unsigned long long* my_flag;  // [ctas] message counters in my memory
  unsigned long long* peer_flag;
  unsigned long long* result;   // [4] elapsed ns, error
};

__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ unsigned long long ld_acq(const unsigned long long* p) { unsigned long long v; asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ void st_rel(unsigned long long* p, unsigned long long v) { asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory"); }

__device__ bool wait_ge(const unsigned long long* f, unsigned long long want, unsigned long long* err) {
  unsigned long long t0 = gtime();
  for (unsigned it = 1;; it++) {
    if (ld_acq(f) >= want) return true;
    if ((it & 255u) == 0 && gtime() - t0 > 1000000000ull) { *err = 1; return false; }
  }
}

// every CTA moves its slice of the message, then publishes its own counter
__device__ void send_msg(const Side& s, long long bytes, unsigned long long seq, int cta, int nctas) {
  long long vecs = (bytes + 15) / 16, per = (vecs + nctas - 1) / nctas, lo = cta * per, hi = min(vecs, lo + per);
  uint4 v = make_uint4((unsigned)seq, 1, 2, 3);
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) reinterpret_cast<uint4*>(s.peer_buf)[i] = v;
  __syncthreads();
  if (threadIdx.x == 0) st_rel(s.peer_flag + cta * 16, seq);
}
__device__ bool recv_msg(const Side& s, unsigned long long seq, int cta, unsigned long long* err) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = wait_ge(s.my_flag + cta * 16, seq, err) ? 1 : 0;
  __syncthreads();
  return ok != 0;
}

// base: message counter value before this measurement (counters only grow)
__global__ void client_kernel(Side s, long long bytes, int n, unsigned long long delay_ns, unsigned long long base_out, unsigned long long base_in) {
  const int cta = blockIdx.x, nctas = gridDim.x;
  unsigned long long err = 0;
  unsigned long long t0 = gtime();
  for (int i = 0; i < n; i++) {
    send_msg(s, bytes, base_out + i + 1, cta, nctas);
    if (delay_ns && i + 1 < n) { unsigned long long w = gtime(); while (gtime() - w < delay_ns) {} }
  }
  bool ok = recv_msg(s, base_in + 1, cta, &err);
  unsigned long long t1 = gtime();
  if (threadIdx.x == 0 && cta == 0) { s.result[0] = t1 - t0; s.result[1] = ok ? 0 : 1; }
}
__global__ void server_kernel(Side s, long long bytes, int n, unsigned long long base_in, unsigned long long base_out) {
  const int cta = blockIdx.x, nctas = gridDim.x;
  unsigned long long err = 0, first = 0, last = 0;
  bool ok = true;
  for (int i = 0; i < n && ok; i++) {
    ok = recv_msg(s, base_in + i + 1, cta, &err);
    unsigned long long t = gtime();
    if (i == 0) first = t;
    last = t;
  }
  if (ok) send_msg(s, bytes, base_out + 1, cta, nctas);
  if (threadIdx.x == 0 && cta == 0) { s.result[0] = last - first; s.result[1] = ok ? 0 : 1; }
}

struct Ctx { int dev[2]; Side side[2]; cudaStream_t st[2]; unsigned long long sent[2]; unsigned long long* res_host[2]; };

static bool prtt(Ctx& c, long long bytes, int n, unsigned long long d_ns, int ctas, double* client_s, double* server_s) {
  // client = side 0, server = side 1
  CK(cudaSetDevice(c.dev[1]));
  server_kernel<<<ctas, 256, 0, c.st[1]>>>(c.side[1], bytes, n, c.sent[0], c.sent[1]);
  CK(cudaSetDevice(c.dev[0]));
  client_kernel<<<ctas, 256, 0, c.st[0]>>>(c.side[0], bytes, n, d_ns, c.sent[0], c.sent[1]);
  CK(cudaStreamSynchronize(c.st[0]));
  CK(cudaSetDevice(c.dev[1])); CK(cudaStreamSynchronize(c.st[1]));
  c.sent[0] += n; c.sent[1] += 1;
  unsigned long long r0[2], r1[2];
  CK(cudaSetDevice(c.dev[0])); CK(cudaMemcpy(r0, c.side[0].result, sizeof r0, cudaMemcpyDeviceToHost));
  CK(cudaSetDevice(c.dev[1])); CK(cudaMemcpy(r1, c.side[1].result, sizeof r1, cudaMemcpyDeviceToHost));
  if (r0[1] || r1[1]) return false;
  *client_s = r0[0] * 1e-9; *server_s = r1[0] * 1e-9;
  return true;
}

int main(int argc, char** argv) {
  int dev0 = 0, dev1 = 1, n = 16, ctas = 1, reps = 20; long long minb = 1, maxb = 16 << 20;
  for (int i = 1; i < argc; i++) {
    auto val = [&]() { if (i + 1 >= argc) { fprintf(stderr, "missing value\n"); exit(2); } return argv[++i]; };
    if (!strcmp(argv[i], "--dev0")) dev0 = atoi(val()); else if (!strcmp(argv[i], "--dev1")) dev1 = atoi(val());
    else if (!strcmp(argv[i], "--n")) n = atoi(val()); else if (!strcmp(argv[i], "--ctas")) ctas = atoi(val());
    else if (!strcmp(argv[i], "--min")) minb = atoll(val()); else if (!strcmp(argv[i], "--max")) maxb = atoll(val());
    else if (!strcmp(argv[i], "--reps")) reps = atoi(val()); else { fprintf(stderr, "unknown flag %s\n", argv[i]); return 2; }
  }
  int ndev = 0; CK(cudaGetDeviceCount(&ndev));
  if (ndev < 2 || dev0 == dev1 || dev0 >= ndev || dev1 >= ndev) { fprintf(stderr, "needs two different GPUs (the two kernels wait for each other)\n"); return 3; }
  int can01 = 0, can10 = 0; CK(cudaDeviceCanAccessPeer(&can01, dev0, dev1)); CK(cudaDeviceCanAccessPeer(&can10, dev1, dev0));
  if (!can01 || !can10) { fprintf(stderr, "no peer access between the two GPUs\n"); return 3; }
  if (ctas < 1) ctas = 1; if (ctas > 64) ctas = 64; if (n < 2) n = 2;
  Ctx c; c.dev[0] = dev0; c.dev[1] = dev1; c.sent[0] = c.sent[1] = 0;
  char* buf[2]; unsigned long long* flag[2]; unsigned long long* res[2];
  for (int s = 0; s < 2; s++) {
    CK(cudaSetDevice(c.dev[s])); CK(cudaDeviceEnablePeerAccess(c.dev[1 - s], 0));
    CK(cudaMalloc(&buf[s], maxb + 256)); CK(cudaMalloc(&flag[s], 64 * 16 * 8)); CK(cudaMalloc(&res[s], 64));
    CK(cudaMemset(flag[s], 0, 64 * 16 * 8)); CK(cudaMemset(res[s], 0, 64));
    CK(cudaStreamCreateWithFlags(&c.st[s], cudaStreamNonBlocking));
    CK(cudaDeviceSynchronize());
  }
  for (int s = 0; s < 2; s++) c.side[s] = Side{buf[s], buf[1 - s], flag[s], flag[1 - s], res[s]};
  printf("size n d PRTT(1,0,s) PRTT(n,0,s) PRTT(n,d,s) PRTT_server(n-1,d,s)\n");
  for (long long s = minb; s <= maxb; s *= 2) {
    auto med = [&](int nn, unsigned long long d, double* srv) {
      std::vector<double> cl, sv;
      for (int r = 0; r < reps + 3; r++) {
        double a, b; if (!prtt(c, s, nn, d, ctas, &a, &b)) { fprintf(stderr, "a wait ran out at size %lld\n", s); exit(4); }
        if (r >= 3) { cl.push_back(a); sv.push_back(b); }
      }
      std::sort(cl.begin(), cl.end()); std::sort(sv.begin(), sv.end());
      if (srv) *srv = sv[sv.size() / 2];
      return cl[cl.size() / 2];
    };
    double p1 = med(1, 0, nullptr);
    double pn0 = med(n, 0, nullptr);
    unsigned long long d_ns = (unsigned long long)(p1 * 1e9);           // d = PRTT(1,0,s), as in the PRTT method
    double srv = 0; double pnd = med(n, d_ns, &srv);
    printf("%lld %d %.9e %.9e %.9e %.9e %.9e\n", s, n, d_ns * 1e-9, p1, pn0, pnd, srv);
    fflush(stdout);
  }
  return 0;
}
