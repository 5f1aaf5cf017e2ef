// team.cc — see team.h.
#include "team.h"

namespace bshmem {

int TeamInfo::index_of(int pe) const {
  if (size <= 0 || stride <= 0) return -1;
  if (pe < pe_start) return -1;
  int d = pe - pe_start;
  if (d % stride != 0) return -1;
  int idx = d / stride;
  return idx < size ? idx : -1;
}

int Team::pe_in_world(int team_pe) const {
  if (!valid || team_pe < 0 || team_pe >= num_pes) return -1;
  return wrt_world.pe_at(team_pe);
}

int Team::pe_in_team(int world_pe) const {
  if (!valid) return -1;
  return wrt_world.index_of(world_pe);
}

int team_translate_pe(const Team& src, int src_pe, const Team& dst) {
  int w = src.pe_in_world(src_pe);
  if (w < 0) return -1;
  return dst.pe_in_team(w);
}

TeamTracker::TeamTracker(int world_size, int my_pe, int max_teams)
    : max_teams_(max_teams < 1 ? 1 : (max_teams > 64 ? 64 : max_teams)), teams_(max_teams_) {
  Team& w = teams_[0];
  w.valid = true;
  w.slot = 0;
  w.parent_slot = -1;
  w.world_size = world_size;
  w.my_pe_in_world = my_pe;
  w.wrt_world = TeamInfo{0, 1, world_size};
  w.wrt_parent = w.wrt_world;
  w.num_pes = world_size;
  w.my_pe = my_pe;
}

int TeamTracker::live_teams() const {
  std::lock_guard<std::mutex> g(mu_);
  int n = 0;
  for (auto& t : teams_) n += t.valid ? 1 : 0;
  return n;
}

const Team* TeamTracker::get(int slot) const {
  if (slot < 0 || slot >= max_teams_) return nullptr;
  return teams_[slot].valid ? &teams_[slot] : nullptr;
}

Team* TeamTracker::get_mut(int slot) {
  if (slot < 0 || slot >= max_teams_) return nullptr;
  return teams_[slot].valid ? &teams_[slot] : nullptr;
}

uint64_t TeamTracker::free_mask() const {
  std::lock_guard<std::mutex> g(mu_);
  uint64_t m = 0;
  for (int i = 1; i < max_teams_; ++i)
    if (!teams_[i].valid) m |= (1ull << i);
  return m;
}

int TeamTracker::pick_slot(uint64_t and_mask) {
  if (and_mask == 0) return -1;
  return __builtin_ctzll(and_mask);
}

int TeamTracker::plan_split(int parent_slot, int start, int stride, int size, Team* out,
                            bool* member) const {
  const Team* p = get(parent_slot);
  if (!p || !out || !member) return BSHMEM_ERR_INVALID;
  if (start < 0 || start >= p->num_pes || size < 1 || size > p->num_pes || stride < 1)
    return BSHMEM_ERR_INVALID;
  // The last member must still be a member of the parent.
  long last = (long)start + (long)stride * (size - 1);
  if (last >= p->num_pes) return BSHMEM_ERR_INVALID;

  Team t;
  t.valid = true;
  t.parent_slot = parent_slot;
  t.world_size = p->world_size;
  t.my_pe_in_world = p->my_pe_in_world;
  t.wrt_parent = TeamInfo{start, stride, size};
  t.wrt_world = TeamInfo{p->wrt_world.pe_at(start), stride * p->wrt_world.stride, size};
  t.num_pes = size;
  t.my_pe = t.wrt_world.index_of(t.my_pe_in_world);
  *member = t.my_pe >= 0;
  *out = t;
  return BSHMEM_OK;
}

int TeamTracker::commit(const Team& planned, int slot) {
  std::lock_guard<std::mutex> g(mu_);
  if (slot < 1 || slot >= max_teams_) return BSHMEM_ERR_LIMIT;
  if (teams_[slot].valid) return BSHMEM_ERR_STATE;
  teams_[slot] = planned;
  teams_[slot].slot = slot;
  teams_[slot].epoch = 0;
  return BSHMEM_OK;
}

int TeamTracker::destroy(int slot) {
  std::lock_guard<std::mutex> g(mu_);
  if (slot <= 0 || slot >= max_teams_) return BSHMEM_OK;  // world / invalid: no-op
  teams_[slot] = Team{};
  return BSHMEM_OK;
}

void TeamTracker::destroy_all() {
  std::lock_guard<std::mutex> g(mu_);
  for (int i = 1; i < max_teams_; ++i) teams_[i] = Team{};
}

}  // namespace bshmem
