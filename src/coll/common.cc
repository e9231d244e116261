// Request normalisation, rank/block arithmetic and tree shapes shared by all
// schedule compilers.
#include <cstring>
#include "coll_internal.h"

namespace piccl {

const char* coll_name(Coll c) {
  static const char* n[] = {"allgather", "allreduce", "broadcast", "reduce", "reduce_scatter"};
  return (c >= 0 && c < COLL_COUNT) ? n[c] : "?";
}
const char* algo_name(Algo a) {
  static const char* n[] = {"DEFAULT", "RING", "K_RING", "RD", "RM", "PRD", "PRM", "AUTO", "DIRECT", "NVLS"};
  return (a >= 0 && a <= ALGO_NVLS) ? n[a] : "?";
}
// Accepted spellings are the reference's (src/piccl.c:262-283) plus AUTO;
// anything else selects the NCCL passthrough, as in the reference.
Algo algo_from_string(const char* s) {
  if (!s) return ALGO_DEFAULT_NCCL;
  if (!strcmp(s, "RING")) return ALGO_RING;
  if (!strcmp(s, "K_RING")) return ALGO_K_RING;
  if (!strcmp(s, "RD")) return ALGO_RD;
  if (!strcmp(s, "RM")) return ALGO_RM;
  if (!strcmp(s, "PRD")) return ALGO_PRD;
  if (!strcmp(s, "PRM")) return ALGO_PRM;
  if (!strcmp(s, "AUTO")) return ALGO_AUTO;
  if (!strcmp(s, "DIRECT")) return ALGO_DIRECT;
  if (!strcmp(s, "NVLS")) return ALGO_NVLS;
  return ALGO_DEFAULT_NCCL;
}

static int smallest_prime_factor(int n) {
  for (int f = 2; f * f <= n; f++) if (n % f == 0) return f;
  return n;
}

// n as a product of radices <= kmax where possible (larger prime factors are
// kept as their own step when they still fit one action).
static bool factorize(int n, int kmax, std::vector<int>& out) {
  out.clear();
  int rem = n;
  while (rem > 1) {
    int f = 0;
    for (int c = std::min(kmax, rem); c >= 2; c--) if (rem % c == 0) { f = c; break; }
    if (!f) f = smallest_prime_factor(rem);
    if (f - 1 > kMaxActionPeers) return false;
    out.push_back(f);
    rem /= f;
  }
  std::sort(out.begin(), out.end(), [](int a, int b) { return a > b; });
  return true;
}

static int ceil_log(int n, int k) { int p = 0; long v = 1; while (v < n) { v *= k; p++; } return p; }

Resolved resolve(Coll coll, Algo algo, int k, int n) {
  Resolved r; r.algo = algo; r.k = k; r.core = n;
  if (algo == ALGO_DEFAULT_NCCL || algo == ALGO_AUTO) { r.algo = ALGO_RING; r.k = 0; r.note = "no algorithm given: RING"; return r; }
  if (n <= 1) { r.algo = ALGO_RING; r.k = 0; return r; }
  if (n > kMaxRanks) { r.algo = ALGO_RING; r.k = 0; r.note = "more ranks than supported by one action table"; return r; }
  if (algo == ALGO_NVLS) { r.algo = ALGO_RING; r.k = 0; r.note = "NVLS is not a step schedule: RING"; return r; }
  if (algo == ALGO_RING) { r.k = 0; return r; }
  if (algo == ALGO_DIRECT) {
    if (n - 1 > kMaxActionPeers) { r.algo = ALGO_RING; r.k = 0; r.note = "DIRECT addresses at most 7 peers: RING"; return r; }
    r.k = n;
    if (coll == COLL_ALLGATHER || coll == COLL_REDUCE_SCATTER) { r.algo = ALGO_PRM; r.radices.assign(1, n); r.note = "DIRECT is PRM with k = n here"; }
    return r;
  }
  if (algo == ALGO_K_RING) {
    // The reference degrades to a plain ring when k does not divide n or k > n
    // (src/coll/allreduce.c:192-196); k unset (-1) is treated the same way.
    if (k < 1 || k > n || n % k != 0) { r.k = n; r.note = "k does not divide the rank count: one group (plain ring)"; }
    return r;
  }
  int kmax = (algo == ALGO_RD || algo == ALGO_PRD) ? 2 : k;
  if (kmax < 2) { kmax = 2; r.note = "radix unset or < 2: 2"; }
  if (kmax > kMaxActionPeers + 1) { kmax = kMaxActionPeers + 1; r.note = "radix limited to 8"; }
  if (kmax > n) { kmax = n; r.note = "radix limited to the rank count"; }
  r.k = kmax;
  if (coll == COLL_BROADCAST || coll == COLL_REDUCE) {
    // k-nomial trees work for every n; only the fan-out of one action is bounded.
    while (r.k > 2 && (r.k - 1) * ceil_log(n, r.k) > kMaxActionPeers) { r.k--; r.note = "radix lowered to bound the tree fan-out"; }
    if ((r.k - 1) * ceil_log(n, r.k) > kMaxActionPeers) { r.algo = ALGO_RING; r.k = 0; r.note = "tree fan-out too large: RING"; }
    return r;
  }
  if (factorize(n, kmax, r.radices)) {
    bool uniform = true; for (int f : r.radices) uniform &= (f == kmax);
    if (!uniform && r.note.empty()) r.note = "rank count is not a power of the radix: mixed radix";
    return r;
  }
  if (coll == COLL_ALLREDUCE) {
    // Largest power of the radix that fits; the other ranks hand their data
    // to a core rank first and get the result back at the end (the reference's
    // pre/post phases, src/coll/allreduce.c:308-345,377-441).
    int core = 1; while ((long)core * kmax <= n) core *= kmax;
    r.core = core; r.radices.clear();
    for (int c = core; c > 1; c /= kmax) r.radices.push_back(kmax);
    r.note = "rank count has a large prime factor: power-of-radix core plus followers";
    return r;
  }
  r.algo = ALGO_RING; r.k = 0; r.radices.clear();
  r.note = "rank count has a large prime factor: RING";
  return r;
}

void ar_chunks(int64_t count, int n, int esz, std::vector<int64_t>& displ, std::vector<int64_t>& cnt) {
  int64_t pack = esz >= 16 ? 1 : 16 / esz;
  int64_t per = (count + n - 1) / n;
  per = (per + pack - 1) / pack * pack;
  displ.assign(n, 0); cnt.assign(n, 0);
  for (int c = 0; c < n; c++) {
    int64_t d = std::min<int64_t>((int64_t)c * per, count);
    displ[c] = d; cnt[c] = std::min<int64_t>(per, count - d);
  }
}

std::vector<int> step_peers(int r, int s, const std::vector<int>& radices, int n, bool permuted) {
  std::vector<int> out;
  int f = radices[s];
  int64_t done = 1; for (int t = 0; t < s; t++) done *= radices[t];
  if (!permuted) {
    int R = (int)done, root = (r / (f * R)) * f * R, loc = r % R, myj = (r - root) / R;
    for (int j = 0; j < f; j++) if (j != myj) out.push_back(root + j * R + loc);
  } else {
    int size = n / (int)done, next = size / f, root = (r / size) * size, rel = r % size;
    for (int i = 1; i < f; i++) out.push_back(root + (rel + i * next) % size);
  }
  return out;
}

std::vector<int> held_blocks(int r, int s, const std::vector<int>& radices, int n, bool permuted) {
  if (s == 0) return {r};
  int t = s - 1, f = radices[t];
  int64_t done = 1; for (int u = 0; u < t; u++) done *= radices[u];
  std::vector<int> out;
  if (!permuted) {
    int R = (int)done, root = (r / (f * R)) * f * R, loc = r % R;
    for (int j = 0; j < f; j++) { auto h = held_blocks(root + j * R + loc, t, radices, n, permuted); out.insert(out.end(), h.begin(), h.end()); }
  } else {
    int size = n / (int)done, next = size / f, root = (r / size) * size, rel = r % size;
    for (int i = 0; i < f; i++) { auto h = held_blocks(root + (rel + i * next) % size, t, radices, n, permuted); out.insert(out.end(), h.begin(), h.end()); }
  }
  return out;
}

bool permutation_index(int r, int n, int b, std::vector<int>& perm) {
  if (b < 2) return false;
  int d = 0; long v = 1; while (v < n) { v *= b; d++; }
  if (v != n) return false;
  perm.assign(n, 0);
  for (int q = 0; q < n; q++) {
    // digit-reverse q over d digits, then add to r digit by digit without carry
    int rev = 0, x = q; for (int i = 0; i < d; i++) { rev = rev * b + x % b; x /= b; }
    int res = 0, mul = 1, a = r, c = rev;
    for (int i = 0; i < d; i++) { res += ((a % b + c % b) % b) * mul; mul *= b; a /= b; c /= b; }
    perm[q] = res;
  }
  return true;
}

RsChain rs_chain(int rank, int n, int k) {
  RsChain c;
  int g = n / k, grp = rank / k, gr = rank % k;
  int intra_right = grp * k + (gr + 1) % k, intra_left = grp * k + mod(gr - 1, k);
  int inter_right = ((grp + 1) % g) * k + (gr + 1) % k, inter_left = mod(grp - 1, g) * k + mod(gr - 1, k);
  int gs = mod(grp - 1, g) * k;
  int prev_from = -1;
  auto hop = [&](int chunk, int to, int from_of_next) { c.chunk.push_back(chunk); c.to.push_back(to); c.from.push_back(prev_from); prev_from = from_of_next; };
  for (int j = 0; j + 1 < k; j++) hop(gs + mod(gr - 1 - j, k), intra_right, intra_left);
  for (int t = 1; t < g; t++) {
    hop(gs + gr, inter_right, inter_left);
    gs = mod(gs - k, n);
    for (int j = 0; j + 1 < k; j++) hop(gs + mod(gr - 1 - j, k), intra_right, intra_left);
  }
  c.final_chunk = gs + gr;   // == rank
  c.final_from = prev_from;
  return c;
}

// ---- trees ----
static int virt(int r, int root, int n) { return mod(r - root, n); }
static int real(int v, int root, int n) { return (v + root) % n; }

Tree bcast_tree(Algo algo, int k, int n, int root, int rank) {
  Tree t; int v = virt(rank, root, n);
  if (n <= 1) return t;
  if (algo == ALGO_RING || (algo == ALGO_K_RING && (k <= 1 || k >= n))) {
    // chain root -> root+1 -> ... -> root-1 (reference src/coll/broadcast.c:24-32), pipelined by segments
    if (v > 0) t.parent = real(v - 1, root, n);
    if (v + 1 < n) t.children.push_back(real(v + 1, root, n));
    t.depth = v;
    return t;
  }
  if (algo == ALGO_K_RING) {
    // leaders = ranks congruent to the root modulo k, chained with stride k; each group is a chain
    // starting at its leader (reference src/coll/broadcast.c:59-89)
    int g = n / k, grp = rank / k, rel = rank % k, lrel = root % k;
    bool leader = rel == lrel;
    int succ = grp * k + (rel + 1) % k, pred = grp * k + mod(rel - 1, k);
    int hops_from_leader = mod(rel - lrel, k);
    int grp_dist = mod(grp - root / k, g);
    if (leader) {
      if (rank != root) t.parent = mod(rank - k, n);
      int nl = (rank + k) % n;
      if (nl != root) t.children.push_back(nl);
      if (k > 1) t.children.push_back(succ);
      t.depth = grp_dist;
    } else {
      t.parent = pred;
      if (succ % k != lrel) t.children.push_back(succ);
      t.depth = grp_dist + hops_from_leader;
    }
    return t;
  }
  bool farthest_first = (algo == ALGO_PRD || algo == ALGO_PRM);
  long span = 1; while (span < n) span *= k;
  if (farthest_first) {
    if (v != 0) { long d = 1; while (v % (d * k) == 0) d *= k; t.parent = real((int)(v - v % (d * k)), root, n); }
    int depth = 0; { int x = v; while (x) { if (x % k) depth++; x /= k; } } t.depth = depth;
    for (long dist = span / k; dist >= 1; dist /= k)
      if (v % (dist * k) == 0)
        for (int i = 1; i < k; i++) { long c = v + i * dist; if (c < n) t.children.push_back(real((int)c, root, n)); }
  } else {
    long R = 1; while (R * k <= v) R *= k;            // highest digit position of v
    if (v != 0) t.parent = real((int)(v % R), root, n);
    int depth = 0; { int x = v; while (x) { if (x % k) depth++; x /= k; } } t.depth = depth;
    long start = 1; while (start <= v) start *= k;   // first power of k above v
    for (long S = start; S < span; S *= k)
      for (int i = 1; i < k; i++) { long c = v + i * S; if (c < n) t.children.push_back(real((int)c, root, n)); }
  }
  return t;
}

Tree reduce_tree(Algo algo, int k, int n, int root, int rank) {
  if (algo == ALGO_RING || (algo == ALGO_K_RING && (k <= 1 || k >= n))) {
    // chain root+1 -> root+2 -> ... -> root (reference src/coll/reduce.c:20-43)
    Tree t; int v = virt(rank, root, n);
    if (n <= 1) return t;
    if (v != 0) t.parent = real((v + 1) % n, root, n);
    if (v == 0) t.children.push_back(real(n - 1, root, n));
    else if (v > 1) t.children.push_back(real(v - 1, root, n));
    t.depth = v == 0 ? n - 1 : v - 1;
    return t;
  }
  // every other shape is the broadcast tree with the arrows turned round
  return bcast_tree(algo, k, n, root, rank);
}

Program compile(const CollArgs& a, int rank) {
  Resolved rs = resolve(a.coll, a.algo, a.k, a.nranks);
  switch (a.coll) {
    case COLL_ALLGATHER: return compile_allgather(a, rs, rank);
    case COLL_ALLREDUCE: return compile_allreduce(a, rs, rank);
    case COLL_BROADCAST: return compile_broadcast(a, rs, rank);
    case COLL_REDUCE: return compile_reduce(a, rs, rank);
    case COLL_REDUCE_SCATTER: return compile_reduce_scatter(a, rs, rank);
    default: break;
  }
  return Program();
}

}  // namespace piccl
