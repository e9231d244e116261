// Per-call tracing (PICCL_TRACE=<file prefix>): one record per executor launch
// with host time and, resolved when the communicator is destroyed, the device
// time between two events; written as Chrome-trace JSON (<prefix>.<rank>.json).
// The reference only has one NVTX range around ncclAllGather (src/piccl.c:32,55,60).
#include <chrono>
#include <cstdio>
#include "comm.h"

namespace piccl {

static double now_us() {
  using namespace std::chrono;
  return duration_cast<duration<double, std::micro>>(steady_clock::now().time_since_epoch()).count();
}

TraceRec* trace_begin(piccl_comm* c, Coll coll, Algo algo, int k, long long bytes, int n_cta, cudaStream_t s) {
  if (env().trace_file.empty()) return nullptr;
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) { cudaGetLastError(); return nullptr; }
  if (c->trace.size() >= 100000) return nullptr;
  TraceRec r; r.coll = coll; r.algo = algo; r.k = k; r.n_cta = n_cta; r.bytes = bytes; r.host_us = now_us();
  if (cudaEventCreate(&r.start) != cudaSuccess || cudaEventCreate(&r.stop) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  cudaEventRecord(r.start, s);
  c->trace.push_back(r);
  return &c->trace.back();
}

void trace_end(piccl_comm*, TraceRec* r, cudaStream_t s) { if (r) cudaEventRecord(r->stop, s); }

void trace_dump(piccl_comm* c) {
  if (c->trace.empty()) return;
  char path[512]; snprintf(path, sizeof path, "%s.%d.json", env().trace_file.c_str(), c->rank);
  FILE* f = fopen(path, "w"); if (!f) return;
  fprintf(f, "{\"traceEvents\":[\n");
  bool first = true;
  for (auto& r : c->trace) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, r.start, r.stop) != cudaSuccess) { cudaGetLastError(); continue; }
    fprintf(f, "%s{\"name\":\"%s/%s\",\"ph\":\"X\",\"pid\":%d,\"tid\":0,\"ts\":%.3f,\"dur\":%.3f,\"args\":{\"bytes\":%lld,\"k\":%d,\"ctas\":%d}}", first ? "" : ",\n",
            coll_name((Coll)r.coll), algo_name((Algo)r.algo), c->rank, r.host_us, ms * 1000.0, r.bytes, r.k, r.n_cta);
    first = false;
  }
  fprintf(f, "\n]}\n"); fclose(f);
}

}  // namespace piccl
