// Schedule dumps: the transfer list of a compiled schedule in the schedule-XML
// format consumed by the LogGP simulator (reference format:
// tools/loggp_sim/README.md:13-26, parser tools/loggp_sim/parser.py:36-56), and
// a JSON view of one rank's action program.
#include <cstdio>
#include <deque>
#include <map>
#include <sstream>
#include "coll_internal.h"

namespace piccl {

namespace { struct Xfer { int id, src, dst, step; int64_t bytes; std::vector<int> deps; }; }

static std::string lower(const char* s) { std::string o(s); for (auto& c : o) c = (char)tolower(c); return o; }

std::string dump_xml(const CollArgs& a) {
  int n = a.nranks;
  Resolved rs = resolve(a.coll, a.algo, a.k, n);
  std::vector<Program> progs; for (int r = 0; r < n; r++) progs.push_back(compile(a, r));
  // pass 1: ids in (step, rank, action, peer) order; remember the push order per connection
  std::vector<Xfer> xf;
  std::map<std::pair<int, int>, std::deque<int>> conn;
  std::vector<std::vector<std::vector<int>>> out_ids(n);   // [rank][action] -> ids
  int maxstep = 0;
  for (int r = 0; r < n; r++) { out_ids[r].resize(progs[r].actions.size()); for (auto& ac : progs[r].actions) maxstep = std::max<int>(maxstep, ac.step); }
  for (int s = 0; s <= maxstep; s++)
    for (int r = 0; r < n; r++)
      for (size_t i = 0; i < progs[r].actions.size(); i++) {
        const Action& ac = progs[r].actions[i];
        if (ac.step != s) continue;
        for (int j = 0; j < ac.n_send; j++) {
          int id = (int)xf.size();
          xf.push_back(Xfer{id, r, ac.send_peer[j], s, ac.count * a.elem_size, {}});
          out_ids[r][i].push_back(id);
        }
      }
  // connection order is program order of the sender, not id order
  for (int r = 0; r < n; r++)
    for (size_t i = 0; i < progs[r].actions.size(); i++) {
      const Action& ac = progs[r].actions[i];
      for (int j = 0; j < ac.n_send; j++) conn[{r, ac.send_peer[j]}].push_back(out_ids[r][i][j]);
    }
  // pass 2: what each action receives, and from that the dependencies of what it sends
  for (int r = 0; r < n; r++) {
    std::vector<int> last_in;   // receives of the latest earlier step that had any
    int last_step = -1; std::vector<int> cur_step_in;
    for (size_t i = 0; i < progs[r].actions.size(); i++) {
      const Action& ac = progs[r].actions[i];
      if (ac.step != last_step) { if (!cur_step_in.empty()) last_in = cur_step_in; cur_step_in.clear(); last_step = ac.step; }
      std::vector<int> incoming;
      for (int j = 0; j < ac.n_recv; j++) { auto& q = conn[{ac.recv_peer[j], r}]; if (!q.empty()) { incoming.push_back(q.front()); q.pop_front(); } }
      for (int id : out_ids[r][i]) xf[id].deps = incoming.empty() ? last_in : incoming;
      cur_step_in.insert(cur_step_in.end(), incoming.begin(), incoming.end());
    }
  }
  std::ostringstream o;
  int64_t total = a.count * a.elem_size * ((a.coll == COLL_ALLGATHER || a.coll == COLL_REDUCE_SCATTER) ? n : 1);
  o << "<collective name=\"" << coll_name(a.coll) << "\" algorithm=\"" << lower(algo_name(rs.algo)) << "\"";
  if (rs.k > 0) o << " k=\"" << rs.k << "\"";
  o << " nodes=\"" << n << "\" buffer_size=\"" << total << "\">\n";
  int step = -1;
  for (auto& x : xf) {
    if (x.step != step) { step = x.step; o << "\n    # (round " << step << ")\n"; }
    o << "    <transfer id=\"" << x.id << "\" size=\"" << x.bytes << "\" src=\"" << x.src << "\" dst=\"" << x.dst << "\" deps=\"";
    if (x.deps.empty()) o << "-1";
    else for (size_t i = 0; i < x.deps.size(); i++) o << (i ? "," : "") << x.deps[i];
    o << "\"/>\n";
  }
  o << "</collective>\n";
  return o.str();
}

std::string dump_json(const CollArgs& a, int rank) {
  Program p = compile(a, rank);
  Resolved rs = resolve(a.coll, a.algo, a.k, a.nranks);
  static const char* bn[] = {"none", "in", "out", "scratch"};
  std::ostringstream o;
  o << "{\"collective\":\"" << coll_name(a.coll) << "\",\"algorithm\":\"" << algo_name(rs.algo) << "\",\"k\":" << rs.k
    << ",\"rank\":" << rank << ",\"nranks\":" << a.nranks << ",\"steps\":" << p.nsteps << ",\"scratch_elems\":" << p.scratch_elems
    << ",\"note\":\"" << rs.note << "\",\"actions\":[";
  for (size_t i = 0; i < p.actions.size(); i++) {
    const Action& ac = p.actions[i];
    o << (i ? "," : "") << "{\"step\":" << (int)ac.step << ",\"src\":\"" << bn[ac.src_buf] << "\",\"src_off\":" << ac.src_off
      << ",\"dst\":\"" << bn[ac.dst_buf] << "\",\"dst_off\":" << ac.dst_off << ",\"count\":" << ac.count << ",\"recv\":[";
    for (int j = 0; j < ac.n_recv; j++) o << (j ? "," : "") << (int)ac.recv_peer[j];
    o << "],\"send\":[";
    for (int j = 0; j < ac.n_send; j++) o << (j ? "," : "") << (int)ac.send_peer[j];
    o << "]}";
  }
  o << "]}";
  return o.str();
}

}  // namespace piccl
