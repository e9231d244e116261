// coll_bench: OSU-style latency / bandwidth benchmark of the NCCL collectives,
// one forked process per GPU, no MPI.  It calls the plain NCCL ABI, so the
// library under test is chosen with LD_PRELOAD (this framework's piccl.so, the
// reference's piccl.so, or nothing = stock NCCL) and PICCL_<COLL>_ALGO / _K.
//
// The reference is benchmarked with its fork of the OSU micro-benchmarks under
// mpirun (README.md:40-44), neither of which is available offline; this harness
// follows the same protocol: warm-up, then `iters` back-to-back calls timed on
// the device with CUDA events, the MAXIMUM over ranks reported, 1000 iterations
// below 1 MB and 100 from 1 MB on, bus bandwidth with the nccl-tests factors.
//
//   coll_bench --gpus 8 --coll allreduce --dtype float --min 8 --max 1073741824 --check
//
// Sizes: --min/--max are bytes of the whole buffer for allreduce/broadcast/reduce and bytes
// per rank for allgather/reduce_scatter; powers of two in between (--step 4: every second one),
// or an explicit list with --sizes 8,4096,...
// --algos RING,K_RING:2,PRM:4,AUTO runs the size list once per entry inside the same processes: before each
// pass every rank sets PICCL_<COLL>_ALGO / _K and asks the preloaded library to read its environment again
// (piccl_env_reload, found with dlsym; without this framework's library preloaded the flag is refused).
// Rows are labelled <label>-<ALGO>-k<K>.
// Output: one CSV line per size on stdout (rank 0).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <signal.h>
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <utility>
#include <vector>

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { fprintf(stderr, "rank %d: %s: %s\n", g_rank, #x, cudaGetErrorString(e_)); _exit(10); } } while (0)
#define NK(x) do { ncclResult_t r_ = (x); if (r_ != ncclSuccess) { fprintf(stderr, "rank %d: %s: %s\n", g_rank, #x, ncclGetErrorString(r_)); _exit(11); } } while (0)

static int g_rank = -1;

struct Shared {
  ncclUniqueId id;
  std::atomic<int> id_ready;
  std::atomic<int> bar_count, bar_sense;
  double value[64];
  int flag[64];
};

static void host_barrier(Shared* sh, int n, int* local_sense) {
  *local_sense = !*local_sense;
  if (sh->bar_count.fetch_add(1) == n - 1) { sh->bar_count.store(0); sh->bar_sense.store(*local_sense); }
  else {
    // bounded: a rank that died must not leave the others spinning for ever
    long waited_us = 0; int spins = 0;
    while (sh->bar_sense.load() != *local_sense) {
      if (++spins > 1000) { usleep(50); waited_us += 50; }
      if (waited_us > 300L * 1000 * 1000) { fprintf(stderr, "rank %d: host barrier timed out\n", g_rank); _exit(12); }
    }
  }
}

enum CollKind { AR, AG, RS, RD, BC };
struct Opt {
  int gpus = 2; CollKind coll = AR; std::string coll_name = "allreduce"; ncclDataType_t dt = ncclFloat; std::string dt_name = "float";
  ncclRedOp_t op = ncclSum; std::string op_name = "sum"; size_t minb = 8, maxb = 1 << 26; int root = 0; bool check = false, in_place = false;
  int iters_small = 1000, iters_large = 100, warmup = 5, step = 2; size_t large = 1000000; std::string label = "";
  std::vector<size_t> sizes;                                  // --sizes: explicit list instead of min/max/step
  std::vector<std::pair<std::string, int>> algos;             // --algos: (algorithm, k) passes inside one process
};

static size_t dt_size(ncclDataType_t d) { switch (d) { case ncclFloat: return 4; case ncclInt32: return 4; case ncclBfloat16: return 2; case ncclHalf: return 2; case ncclDouble: return 8; default: return 1; } }

// deterministic per (rank, index) values: floats uniform in [-1,1), ints in [-1000,1000]
static inline unsigned hash32(unsigned a, unsigned b) { unsigned x = a * 2654435761u ^ (b + 0x9e3779b9u + (a << 6) + (a >> 2)); x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16; return x; }
static inline double gen_val(int rank, size_t i, bool integer) {
  unsigned h = hash32((unsigned)rank + 1, (unsigned)i);
  if (integer) return (double)((int)(h % 2001u) - 1000);
  return (double)(h >> 8) / 8388608.0 - 1.0;
}
static void fill_host(std::vector<unsigned char>& buf, ncclDataType_t dt, int rank, size_t count) {
  for (size_t i = 0; i < count; i++) {
    double v = gen_val(rank, i, dt == ncclInt32);
    switch (dt) {
      case ncclFloat: ((float*)buf.data())[i] = (float)v; break;
      case ncclInt32: ((int*)buf.data())[i] = (int)v; break;
      case ncclDouble: ((double*)buf.data())[i] = v; break;
      case ncclBfloat16: ((__nv_bfloat16*)buf.data())[i] = __float2bfloat16((float)v); break;
      case ncclHalf: ((__half*)buf.data())[i] = __float2half((float)v); break;
      default: buf[i] = (unsigned char)(int)v; break;
    }
  }
}
static double read_host(const unsigned char* buf, ncclDataType_t dt, size_t i) {
  switch (dt) {
    case ncclFloat: return ((const float*)buf)[i];
    case ncclInt32: return ((const int*)buf)[i];
    case ncclDouble: return ((const double*)buf)[i];
    case ncclBfloat16: return __bfloat162float(((const __nv_bfloat16*)buf)[i]);
    case ncclHalf: return __half2float(((const __half*)buf)[i]);
    default: return buf[i];
  }
}
static double quantize(double v, ncclDataType_t dt) {
  if (dt == ncclBfloat16) return __bfloat162float(__float2bfloat16((float)v));
  if (dt == ncclHalf) return __half2float(__float2half((float)v));
  if (dt == ncclFloat) return (float)v;
  return v;
}
static double reduce_ref(const Opt& o, int n, size_t i) {
  double acc = quantize(gen_val(0, i, o.dt == ncclInt32), o.dt);
  for (int r = 1; r < n; r++) {
    double v = quantize(gen_val(r, i, o.dt == ncclInt32), o.dt);
    switch (o.op) { case ncclSum: acc += v; break; case ncclProd: acc *= v; break; case ncclMax: acc = acc > v ? acc : v; break; default: acc = acc < v ? acc : v; }
  }
  return acc;
}

static int run_rank(const Opt& o, int rank, Shared* sh) {
  g_rank = rank;
  int n = o.gpus, sense = 0;
  CK(cudaSetDevice(rank));
  if (rank == 0) { NK(ncclGetUniqueId(&sh->id)); sh->id_ready.store(1); }
  else while (!sh->id_ready.load()) usleep(100);
  ncclComm_t comm;
  NK(ncclCommInitRank(&comm, n, sh->id, rank));
  cudaStream_t st; CK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
  size_t es = dt_size(o.dt);
  bool per_rank = (o.coll == AG || o.coll == RS);
  size_t maxb = o.maxb;
  if (!o.sizes.empty()) { maxb = 0; for (size_t b : o.sizes) maxb = b > maxb ? b : maxb; }
  size_t max_count = maxb / es; if (max_count == 0) max_count = 1;
  size_t big = per_rank ? max_count * n : max_count;
  char *sbuf, *rbuf;
  CK(cudaMalloc(&sbuf, big * es + 256)); CK(cudaMalloc(&rbuf, big * es + 256));
  CK(cudaMemset(sbuf, 0, big * es)); CK(cudaMemset(rbuf, 0, big * es));
  if (rank == 0) printf("# coll,label,dtype,op,ranks,bytes,iters,time_us,algbw_GBs,busbw_GBs,check\n");
  std::vector<size_t> sizes = o.sizes;
  if (sizes.empty()) for (size_t b = o.minb; b <= o.maxb; b *= o.step) sizes.push_back(b);
  typedef void (*ReloadFn)(void);
  ReloadFn reload = o.algos.empty() ? nullptr : (ReloadFn)dlsym(RTLD_DEFAULT, "piccl_env_reload");
  if (!o.algos.empty() && !reload) { fprintf(stderr, "rank %d: --algos needs this framework's library preloaded (piccl_env_reload not found)\n", rank); _exit(13); }
  const size_t passes = o.algos.empty() ? 1 : o.algos.size();
  for (size_t pass = 0; pass < passes; pass++) {
  std::string label = o.label;
  if (!o.algos.empty()) {
    std::string up = o.coll_name; for (auto& ch : up) ch = (char)toupper(ch);
    CK(cudaStreamSynchronize(st));
    host_barrier(sh, n, &sense);                              // nobody switches while a peer is still inside a collective of the last pass
    setenv(("PICCL_" + up + "_ALGO").c_str(), o.algos[pass].first.c_str(), 1);
    setenv(("PICCL_" + up + "_K").c_str(), std::to_string(o.algos[pass].second).c_str(), 1);
    reload();
    host_barrier(sh, n, &sense);
    label += (label.empty() ? "" : "-") + o.algos[pass].first + "-k" + std::to_string(o.algos[pass].second);
  }
  for (size_t bytes : sizes) {
    size_t count = bytes / es; if (count == 0) count = 1;
    size_t send_count = (o.coll == RS) ? count * n : count, recv_count = (o.coll == AG) ? count * n : count;
    const void* send = sbuf; void* recv = rbuf;
    if (o.in_place) { if (o.coll == AG) { recv = rbuf; send = rbuf + (size_t)rank * count * es; } else if (o.coll == RS) { send = sbuf; recv = sbuf + (size_t)rank * count * es; } else { send = rbuf; recv = rbuf; } }
    auto call = [&]() {
      switch (o.coll) {
        case AR: NK(ncclAllReduce(send, recv, count, o.dt, o.op, comm, st)); break;
        case AG: NK(ncclAllGather(send, recv, count, o.dt, comm, st)); break;
        case RS: NK(ncclReduceScatter(send, recv, count, o.dt, o.op, comm, st)); break;
        case RD: NK(ncclReduce(send, recv, count, o.dt, o.op, o.root, comm, st)); break;
        case BC: NK(ncclBroadcast(send, recv, count, o.dt, o.root, comm, st)); break;
      }
    };
    // ---- correctness on seeded data (sizes up to 64 MiB of send data: all elements; above: skipped)
    int check = -1;
    if (o.check && send_count * es <= ((size_t)64 << 20) && !o.in_place) {
      std::vector<unsigned char> h(send_count * es);
      fill_host(h, o.dt, rank, send_count);
      CK(cudaMemcpy(sbuf, h.data(), send_count * es, cudaMemcpyHostToDevice));
      CK(cudaMemset(rbuf, 0xff, recv_count * es));
      CK(cudaDeviceSynchronize());      // the fill runs on the legacy stream, the collective on a non-blocking one
      call(); CK(cudaStreamSynchronize(st));
      std::vector<unsigned char> out(recv_count * es);
      CK(cudaMemcpy(out.data(), rbuf, recv_count * es, cudaMemcpyDeviceToHost));
      check = 1;
      double tol = (o.dt == ncclBfloat16) ? 0.04 * n : (o.dt == ncclHalf) ? 0.004 * n : (o.dt == ncclFloat) ? 1e-5 * n : 0.0;
      size_t stride = recv_count > (1 << 22) ? 7 : 1;
      for (size_t i = 0; i < recv_count && check == 1; i += stride) {
        double want;
        switch (o.coll) {
          case AR: want = reduce_ref(o, n, i); break;
          case RD: if (rank != o.root) { i = recv_count; continue; } want = reduce_ref(o, n, i); break;
          case RS: want = reduce_ref(o, n, (size_t)rank * count + i); break;
          case AG: want = quantize(gen_val((int)(i / count), i % count, o.dt == ncclInt32), o.dt); break;
          default: want = quantize(gen_val(o.root, i, o.dt == ncclInt32), o.dt); break;
        }
        double got = read_host(out.data(), o.dt, i);
        if (!(std::fabs(got - want) <= tol + 1e-3 * tol * std::fabs(want))) { check = 0; fprintf(stderr, "rank %d: %s %zu B element %zu: got %g want %g\n", rank, o.coll_name.c_str(), bytes, i, got, want); }
      }
      sh->flag[rank] = check; host_barrier(sh, n, &sense);
      for (int r = 0; r < n; r++) if (sh->flag[r] == 0) check = 0;
      host_barrier(sh, n, &sense);
    }
    // ---- timing
    int iters = bytes < o.large ? o.iters_small : o.iters_large;
    for (int i = 0; i < o.warmup; i++) call();
    CK(cudaStreamSynchronize(st));
    host_barrier(sh, n, &sense);
    CK(cudaEventRecord(e0, st));
    for (int i = 0; i < iters; i++) call();
    CK(cudaEventRecord(e1, st));
    CK(cudaStreamSynchronize(st));
    float ms = 0; CK(cudaEventElapsedTime(&ms, e0, e1));
    sh->value[rank] = (double)ms * 1e3 / iters;
    host_barrier(sh, n, &sense);
    if (rank == 0) {
      double us = 0; for (int r = 0; r < n; r++) us = sh->value[r] > us ? sh->value[r] : us;
      double total = per_rank ? (double)count * es * n : (double)count * es;
      double algbw = total / us / 1e3;
      double factor = o.coll == AR ? 2.0 * (n - 1) / n : per_rank ? (double)(n - 1) / n : 1.0;
      printf("%s,%s,%s,%s,%d,%zu,%d,%.3f,%.3f,%.3f,%s\n", o.coll_name.c_str(), label.c_str(), o.dt_name.c_str(), o.op_name.c_str(), n, count * es, iters, us, algbw,
             algbw * factor, check < 0 ? "-" : check ? "ok" : "FAIL");
      fflush(stdout);
    }
    host_barrier(sh, n, &sense);
  }
  }
  CK(cudaStreamSynchronize(st));
  NK(ncclCommDestroy(comm));
  cudaFree(sbuf); cudaFree(rbuf);
  return 0;
}

int main(int argc, char** argv) {
  Opt o;
  for (int i = 1; i < argc; i++) {
    std::string f = argv[i];
    auto val = [&]() -> std::string { if (i + 1 >= argc) { fprintf(stderr, "missing value for %s\n", f.c_str()); exit(2); } return argv[++i]; };
    if (f == "--gpus") o.gpus = atoi(val().c_str());
    else if (f == "--coll") { o.coll_name = val(); o.coll = o.coll_name == "allreduce" ? AR : o.coll_name == "allgather" ? AG : o.coll_name == "reduce_scatter" ? RS : o.coll_name == "reduce" ? RD : BC; }
    else if (f == "--dtype") { o.dt_name = val(); o.dt = o.dt_name == "float" ? ncclFloat : o.dt_name == "int32" ? ncclInt32 : o.dt_name == "bf16" ? ncclBfloat16 : o.dt_name == "half" ? ncclHalf : o.dt_name == "double" ? ncclDouble : ncclUint8; }
    else if (f == "--op") { o.op_name = val(); o.op = o.op_name == "sum" ? ncclSum : o.op_name == "prod" ? ncclProd : o.op_name == "max" ? ncclMax : ncclMin; }
    else if (f == "--min") o.minb = strtoull(val().c_str(), nullptr, 10);
    else if (f == "--max") o.maxb = strtoull(val().c_str(), nullptr, 10);
    else if (f == "--root") o.root = atoi(val().c_str());
    else if (f == "--check") o.check = true;
    else if (f == "--in-place") o.in_place = true;
    else if (f == "--iters-small") o.iters_small = atoi(val().c_str());
    else if (f == "--iters-large") o.iters_large = atoi(val().c_str());
    else if (f == "--warmup") o.warmup = atoi(val().c_str());
    else if (f == "--label") o.label = val();
    else if (f == "--step") { o.step = atoi(val().c_str()); if (o.step < 2) o.step = 2; }
    else if (f == "--sizes") { std::string v = val(); size_t p = 0; while (p < v.size()) { size_t q = v.find(',', p); if (q == std::string::npos) q = v.size(); if (q > p) o.sizes.push_back(strtoull(v.substr(p, q - p).c_str(), nullptr, 10)); p = q + 1; } }
    else if (f == "--algos") { std::string v = val(); size_t p = 0; while (p < v.size()) { size_t q = v.find(',', p); if (q == std::string::npos) q = v.size(); std::string e = v.substr(p, q - p); size_t c = e.find(':'); if (!e.empty()) o.algos.push_back({e.substr(0, c), c == std::string::npos ? -1 : atoi(e.substr(c + 1).c_str())}); p = q + 1; } }
    else { fprintf(stderr, "unknown flag %s\n", f.c_str()); return 2; }
  }
  if (o.gpus < 1 || o.gpus > 64 || o.minb < 1 || o.maxb < o.minb) { fprintf(stderr, "bad arguments\n"); return 2; }
  Shared* sh = (Shared*)mmap(nullptr, sizeof(Shared), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
  if (sh == MAP_FAILED) { perror("mmap"); return 1; }
  memset((void*)sh, 0, sizeof(Shared));
  std::vector<pid_t> kids;
  for (int r = 0; r < o.gpus; r++) {
    pid_t p = fork();
    if (p < 0) { perror("fork"); return 1; }
    if (p == 0) { int rc = run_rank(o, r, sh); fflush(stdout); _exit(rc); }
    kids.push_back(p);
  }
  // wait for all ranks; if one fails, end the others (these exact children) instead of letting them wait
  int bad = 0; size_t left = kids.size();
  std::vector<bool> done(kids.size(), false);
  while (left) {
    for (size_t i = 0; i < kids.size(); i++) {
      if (done[i]) continue;
      int st = 0; pid_t r = waitpid(kids[i], &st, WNOHANG);
      if (r == kids[i]) {
        done[i] = true; left--;
        if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) {
          bad++;
          for (size_t j = 0; j < kids.size(); j++) if (!done[j]) kill(kids[j], SIGTERM);
        }
      }
    }
    usleep(2000);
  }
  return bad ? 1 : 0;
}
