// C entry points of the schedule layer (used by the Python tools and tests).
#include <cstring>
#include "coll_internal.h"
#include "../include/piccl.h"

using namespace piccl;

static CollArgs mk(int coll, int algo, int k, int n, int root, long long count, long long stride, int esz, int in_place) {
  CollArgs a; a.coll = (Coll)coll; a.algo = (Algo)algo; a.k = k; a.nranks = n; a.root = root; a.count = count;
  a.block_stride = stride; a.elem_size = esz; a.in_place = in_place != 0; return a;
}
static long long put(const std::string& s, char* buf, long long cap) {
  if (buf && cap > 0) { size_t m = std::min<size_t>(s.size(), (size_t)cap - 1); memcpy(buf, s.data(), m); buf[m] = 0; }
  return (long long)s.size() + 1;
}

extern "C" {

int piccl_algo_from_string(const char* s) { return (int)algo_from_string(s); }

long long piccl_sched_xml(int coll, int algo, int k, int n, int root, long long count, int esz, char* buf, long long cap) {
  return put(dump_xml(mk(coll, algo, k, n, root, count, 0, esz, 0)), buf, cap);
}
long long piccl_sched_json(int coll, int algo, int k, int n, int root, long long count, int esz, int rank, char* buf, long long cap) {
  return put(dump_json(mk(coll, algo, k, n, root, count, 0, esz, 0), rank), buf, cap);
}
int piccl_sched_resolve(int coll, int algo, int k, int n, int* out_algo, int* out_k, int* radices, int* n_radices, int* core, char* note, int note_cap) {
  Resolved r = resolve((Coll)coll, (Algo)algo, k, n);
  if (out_algo) *out_algo = r.algo;
  if (out_k) *out_k = r.k;
  if (core) *core = r.core;
  if (n_radices) { int m = (int)r.radices.size(); if (radices) for (int i = 0; i < m && i < *n_radices; i++) radices[i] = r.radices[i]; *n_radices = m; }
  put(r.note, note, note_cap);
  return 0;
}
int piccl_sched_validate(int coll, int algo, int k, int n, int root, long long count, long long stride, int esz, int in_place,
                         int op, int integer, int fifo_cap, long long seg_elems, int n_cta, int symbolic,
                         long long* fifo_entries, int* max_depth, double* max_err, long long* bytes_sent, char* err, int err_cap) {
  CollArgs a = mk(coll, algo, k, n, root, count, stride, esz, in_place);
  // `symbolic`: bit 0 = no data (coverage and FIFO order only), bit 1 = deferred publishing of the counters
  const bool defer = (symbolic & 2) != 0;
  ValidateResult v = (symbolic & 1) ? validate_symbolic(a, fifo_cap, n_cta, defer) : validate(a, op, integer != 0, fifo_cap, seg_elems, n_cta, defer);
  if (fifo_entries) *fifo_entries = v.fifo_entries;
  if (max_depth) *max_depth = v.max_fifo_depth;
  if (max_err) *max_err = v.max_abs_err;
  if (bytes_sent) *bytes_sent = v.bytes_sent_max_rank;
  put(v.error, err, err_cap);
  return v.ok ? 0 : 1;
}
int piccl_permutation_index(int r, int n, int b, int* out) {
  std::vector<int> p;
  if (!permutation_index(r, n, b, p)) return 1;
  for (int i = 0; i < n; i++) out[i] = p[i];
  return 0;
}
int piccl_held_blocks(int r, int s, const int* radices, int n_radices, int n, int permuted, int* out) {
  std::vector<int> rd(radices, radices + n_radices);
  auto h = held_blocks(r, s, rd, n, permuted != 0);
  for (size_t i = 0; i < h.size(); i++) out[i] = h[i];
  return (int)h.size();
}
int piccl_sched_counts(int coll, int algo, int k, int n, int root, long long count, int esz, int rank, int* n_actions, int* n_steps, long long* scratch_elems) {
  Program p = compile(mk(coll, algo, k, n, root, count, 0, esz, 0), rank);
  if (n_actions) *n_actions = (int)p.actions.size();
  if (n_steps) *n_steps = p.nsteps;
  if (scratch_elems) *scratch_elems = p.scratch_elems;
  return 0;
}

}  // extern "C"
