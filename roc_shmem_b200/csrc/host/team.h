// team.h — PE-set arithmetic and the per-PE team table.
//
// A team is the strided PE set {start, start+stride, ...} of `size` members,
// described both relative to the world and relative to its parent.  Collectives
// on a team use the sync/scratch pool slice selected by the team's slot index,
// which all members agree on at creation time (bitmask intersection).
//
// Parity: library/src/team.hpp:38-157, team.cpp:47-107 (translation rules),
// team_tracker.hpp (max 40 teams incl. world, destroy_all), and the pool-slot
// agreement of gpu_ib/backend_ib.cpp:169-205.
#pragma once
#include <cstdint>
#include <mutex>
#include <vector>

#include "../include/bshmem_types.h"

namespace bshmem {

struct TeamInfo {
  int pe_start = 0;
  int stride = 1;
  int size = 0;
  // team-relative index -> PE in the frame this info is expressed in
  int pe_at(int idx) const { return pe_start + idx * stride; }
  // PE in the frame -> team-relative index, or -1 if not a member
  int index_of(int pe) const;
};

struct Team {
  bool valid = false;
  int slot = -1;            // pool slot == public handle
  int parent_slot = -1;
  int world_size = 0;
  int my_pe_in_world = -1;
  TeamInfo wrt_world;       // stride/start in world PE numbers
  TeamInfo wrt_parent;      // stride/start in parent-team PE numbers
  int num_pes = 0;
  int my_pe = -1;           // my index in this team
  uint64_t epoch = 0;       // collective sequence number (host backends)

  int pe_in_world(int team_pe) const;
  int pe_in_team(int world_pe) const;
};

// Translate `src_pe` of `src` into the numbering of `dst`; -1 when the PE is
// not a member of both.
int team_translate_pe(const Team& src, int src_pe, const Team& dst);

class TeamTracker {
 public:
  TeamTracker(int world_size, int my_pe, int max_teams = BSHMEM_MAX_TEAMS);

  int max_teams() const { return max_teams_; }
  int live_teams() const;
  const Team* get(int slot) const;
  Team* get_mut(int slot);

  // Bitmask of free slots (bit i set = slot i free) for the agreement step.
  uint64_t free_mask() const;
  // Lowest common free slot given the AND of all members' masks; -1 if none.
  static int pick_slot(uint64_t and_mask);

  // Validate split arguments against `parent`; returns BSHMEM_OK or
  // BSHMEM_ERR_INVALID.  On success fills `out` (without a slot) and sets
  // *member to whether this PE belongs to the new team.
  int plan_split(int parent_slot, int start, int stride, int size, Team* out, bool* member) const;
  // Install a planned team into `slot`.
  int commit(const Team& planned, int slot);
  int destroy(int slot);   // world / invalid are no-ops
  void destroy_all();      // finalize: everything but world

 private:
  int max_teams_;
  std::vector<Team> teams_;
  mutable std::mutex mu_;
};

}  // namespace bshmem
