// Hierarchical communicator stack.
//
// A level is produced by splitting the communicator under the cursor by a
// string key: ranks with equal keys form the level's *intra* group (ordered by
// their rank in the parent); the *inter* group links, for a cartesian level,
// the ranks that hold the same intra rank in every group, and for a tree level
// only the intra-rank-0 "roots" (every other rank gets a singleton).  A level
// is cartesian when all groups have the same size and cartesian communicators
// are enabled.  These are the semantics of the reference's split
// (lib/resources.cpp:187-350) and stack (lib/torch_mpi.cpp:38-135); here the
// key exchange is done by the caller on its control plane and groups are plain
// lists of world ranks, so a group-scoped GPU collective is the same kernel
// with a shorter peer table.
#include "common.h"
#include <algorithm>
#include <cstring>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

namespace tmpi {
namespace {

constexpr int kKeyLen = 1024;

struct Level {
  std::string key;
  std::vector<int> intra;  // world ranks, group-rank order
  std::vector<int> inter;
  std::vector<std::vector<int>> groups;  // every group of the split this rank took part in (world ranks, group-rank order)
  bool cartesian = true;
};

struct Stack {
  int world_rank = 0, world_size = 1;
  std::vector<Level> levels;
  int level = 0;
  bool inter = false;
  int span_begin = 0, span_end = 0;
};

Stack g;
std::mutex g_mu;

int index_of(const std::vector<int>& v, int x) {
  for (size_t i = 0; i < v.size(); ++i) if (v[i] == x) return (int)i;
  return -1;
}

const std::vector<int>& current_members_locked() {
  const Level& l = g.levels[g.level];
  if (g.level == 0) return l.intra;  // there is no global inter communicator
  return g.inter ? l.inter : l.intra;
}

}  // namespace
}  // namespace tmpi

using namespace tmpi;

extern "C" {

int tmpi_comm_reset(int world_rank, int world_size) {
  if (world_size < 1 || world_rank < 0 || world_rank >= world_size)
    return fail(TMPI_ERR_INVALID, "bad world rank/size %d/%d", world_rank, world_size);
  std::lock_guard<std::mutex> lk(g_mu);
  g = Stack();
  g.world_rank = world_rank; g.world_size = world_size;
  Level l0; l0.key = "global"; l0.cartesian = true;
  for (int i = 0; i < world_size; ++i) l0.intra.push_back(i);
  l0.inter.push_back(world_rank);
  g.levels.push_back(l0);
  return TMPI_OK;
}

int tmpi_comm_push(const char* keys, const int* parent_members, int parent_size, const char* my_key) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g.levels.empty()) return -fail(TMPI_ERR_STATE, "communicator stack not started");
  if (parent_size < 1) return -fail(TMPI_ERR_INVALID, "empty parent");
  int me = -1;
  for (int i = 0; i < parent_size; ++i) if (parent_members[i] == g.world_rank) me = i;
  if (me < 0) return -fail(TMPI_ERR_INVALID, "rank %d is not a member of the parent communicator", g.world_rank);

  std::vector<std::pair<std::string, int>> kr;
  for (int i = 0; i < parent_size; ++i) {
    const char* k = keys + (size_t)i * kKeyLen;
    kr.emplace_back(std::string(k, strnlen(k, kKeyLen)), i);
  }
  std::string mine(my_key ? my_key : "");
  if (kr[me].first != mine)
    return -fail(TMPI_ERR_INVALID, "key table row %d ('%s') differs from my key ('%s')", me, kr[me].first.c_str(), mine.c_str());
  std::sort(kr.begin(), kr.end());

  // groups in sorted-key order; members in parent-rank order
  std::vector<std::vector<int>> groups;
  std::vector<int> intra_rank_of(parent_size, 0);
  int my_group = -1;
  for (size_t i = 0; i < kr.size(); ++i) {
    if (i == 0 || kr[i].first != kr[i - 1].first) groups.emplace_back();
    intra_rank_of[kr[i].second] = (int)groups.back().size();
    groups.back().push_back(kr[i].second);
    if (kr[i].second == me) my_group = (int)groups.size() - 1;
  }
  bool same_size = true;
  for (auto& grp : groups) if (grp.size() != groups[0].size()) same_size = false;

  Level l;
  l.key = mine;
  l.cartesian = same_size && tunable("use_cartesian_communicator") != 0;
  for (int p : groups[my_group]) l.intra.push_back(parent_members[p]);
  for (auto& grp : groups) {
    l.groups.emplace_back();
    for (int p : grp) l.groups.back().push_back(parent_members[p]);
  }
  int my_intra = intra_rank_of[me];
  if (l.cartesian || my_intra == 0) {
    // every parent rank holding my intra rank, in parent-rank order
    for (int p = 0; p < parent_size; ++p)
      if (intra_rank_of[p] == my_intra) l.inter.push_back(parent_members[p]);
  } else {
    l.inter.push_back(g.world_rank);
  }
  g.levels.push_back(l);
  int idx = (int)g.levels.size() - 1;
  // a fresh level becomes the cursor, as the reference's start() descends into it
  g.level = idx; g.inter = false;
  return idx;
}

// The group of the split at `level` that holds `world_rank` (world ranks in group-rank order); the number of
// members, or 0 when that rank took no part in the split.
int tmpi_comm_group_of(int level, int world_rank, int* out, int cap) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (level < 0 || level >= (int)g.levels.size()) return -fail(TMPI_ERR_INVALID, "communicator level %d out of range", level);
  const Level& l = g.levels[level];
  if (level == 0) {
    int n = (int)l.intra.size();
    for (int i = 0; i < n && i < cap; ++i) out[i] = l.intra[i];
    return n;
  }
  for (auto& grp : l.groups)
    if (index_of(grp, world_rank) >= 0) {
      for (size_t i = 0; i < grp.size() && (int)i < cap; ++i) out[i] = grp[i];
      return (int)grp.size();
    }
  return 0;
}

int tmpi_comm_num_levels(void) { std::lock_guard<std::mutex> lk(g_mu); return (int)g.levels.size(); }

int tmpi_comm_set_typed(int level, int inter) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (level < 0 || level >= (int)g.levels.size())
    return fail(TMPI_ERR_INVALID, "communicator level %d outside [0, %d]", level, (int)g.levels.size() - 1);
  g.level = level; g.inter = inter != 0;
  return TMPI_OK;
}
int tmpi_comm_set(int level) { return tmpi_comm_set_typed(level, 0); }
int tmpi_comm_level(void) { std::lock_guard<std::mutex> lk(g_mu); return g.level; }
int tmpi_comm_is_inter(void) { std::lock_guard<std::mutex> lk(g_mu); return g.inter ? 1 : 0; }

int tmpi_comm_set_span(int begin, int end) {
  std::lock_guard<std::mutex> lk(g_mu);
  int maxl = (int)g.levels.size() - 1;
  if (begin < 0 || end > maxl || begin > end)
    return fail(TMPI_ERR_INVALID, "collective span [%d, %d] outside [0, %d]", begin, end, maxl);
  g.span_begin = begin; g.span_end = end;
  return TMPI_OK;
}
int tmpi_comm_get_span(int* b, int* e) {
  std::lock_guard<std::mutex> lk(g_mu);
  *b = g.span_begin; *e = g.span_end; return TMPI_OK;
}

int tmpi_comm_is_cartesian(int level) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (level < 0) level = g.level;
  if (level >= (int)g.levels.size()) return -fail(TMPI_ERR_INVALID, "no level %d", level);
  return g.levels[level].cartesian ? 1 : 0;
}

int tmpi_comm_members(int level, int inter, int* out, int cap) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (level < 0 || level >= (int)g.levels.size()) return -fail(TMPI_ERR_INVALID, "no level %d", level);
  auto& v = inter ? g.levels[level].inter : g.levels[level].intra;
  for (int i = 0; i < (int)v.size() && i < cap; ++i) out[i] = v[i];
  return (int)v.size();
}

int tmpi_comm_rank_in(int level, int inter) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (level < 0 || level >= (int)g.levels.size()) return -fail(TMPI_ERR_INVALID, "no level %d", level);
  return index_of(inter ? g.levels[level].inter : g.levels[level].intra, g.world_rank);
}

int tmpi_comm_key(int level, char* out, int cap) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (level < 0 || level >= (int)g.levels.size()) return -fail(TMPI_ERR_INVALID, "no level %d", level);
  snprintf(out, cap, "%s", g.levels[level].key.c_str());
  return TMPI_OK;
}

int tmpi_comm_current_members(int* out, int cap) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g.levels.empty()) return -fail(TMPI_ERR_STATE, "communicator stack not started");
  auto& v = current_members_locked();
  for (int i = 0; i < (int)v.size() && i < cap; ++i) out[i] = v[i];
  return (int)v.size();
}

int tmpi_comm_names(char* out, int cap) {
  std::lock_guard<std::mutex> lk(g_mu);
  std::ostringstream ss;
  ss << "current: " << g.level << " " << (g.inter ? "inter" : "intra") << "\n";
  for (int l = 0; l < (int)g.levels.size(); ++l) {
    auto& c = g.levels[l];
    ss << "l : " << l << " -> key(" << c.key << ") (" << c.inter.size() << " in intercomm, I am rank "
       << index_of(c.inter, g.world_rank) << ") ";
    if (l == g.level && g.inter) ss << "* ";
    ss << " (" << c.intra.size() << " in intracomm, I am rank " << index_of(c.intra, g.world_rank) << ") "
       << "cartesian: " << (c.cartesian ? "true" : "false");
    if (l == g.level) ss << " * ";
    ss << "\n";
  }
  std::string s = ss.str();
  snprintf(out, cap, "%s", s.c_str());
  return (int)s.size();
}

int tmpi_comm_has_inter_collective(int level) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (level <= 0 || level >= (int)g.levels.size()) return 0;
  return g.levels[level - 1].intra.size() != g.levels[level].intra.size() ? 1 : 0;
}
int tmpi_comm_has_intra_collective(int level) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (level < 0 || level >= (int)g.levels.size()) return 0;
  return g.levels[level].intra.size() > 1 ? 1 : 0;
}

int tmpi_comm_pop_to(int n) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (n < 1 || n > (int)g.levels.size()) return fail(TMPI_ERR_INVALID, "cannot keep %d levels", n);
  g.levels.resize(n);
  if (g.level >= n) { g.level = n - 1; g.inter = false; }
  if (g.span_end >= n) g.span_end = n - 1;
  if (g.span_begin > g.span_end) g.span_begin = g.span_end;
  return TMPI_OK;
}

// ---------------------------------------------------------------- ring plan
// Reduce phase, step s: chunk c is sent by ring index (c+s) mod size and
// received (and accumulated) by (c+s+1) mod size, so after size-1 steps ring
// index (c-1) mod size holds the complete chunk c.  Broadcast phase, step s:
// chunk c is sent by (c+s-1) mod size and received by (c+s) mod size.
// This is the schedule of lib/resources.cpp:588-678 / lib/detail/README.md:1-48.
static int pmod(int a, int n) { int r = a % n; return r < 0 ? r + n : r; }

int tmpi_ring_plan(int total_chunks, int size, int phase, int* out, int cap) {
  if (size < 1 || total_chunks < 1) return -fail(TMPI_ERR_INVALID, "bad ring plan request");
  int need = (size - 1) * total_chunks * 2;
  if (cap < need) return need;
  for (int s = 0; s < size - 1; ++s)
    for (int c = 0; c < total_chunks; ++c) {
      int snd = phase == 0 ? pmod(c + s, size) : pmod(c + s - 1, size);
      int rcv = phase == 0 ? pmod(c + s + 1, size) : pmod(c + s, size);
      out[(s * total_chunks + c) * 2 + 0] = snd;
      out[(s * total_chunks + c) * 2 + 1] = rcv;
    }
  return need;
}

// With one chunk per rank (total_chunks == size): which chunk does ring index i
// send / receive at step s?
int tmpi_ring_send_chunk(int i, int size, int s, int phase) {
  return phase == 0 ? pmod(i - s, size) : pmod(i - s + 1, size);
}
int tmpi_ring_recv_chunk(int i, int size, int s, int phase) {
  return phase == 0 ? pmod(i - s - 1, size) : pmod(i - s, size);
}

}  // extern "C"
