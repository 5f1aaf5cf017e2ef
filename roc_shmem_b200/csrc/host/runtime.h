// runtime.h — the per-PE runtime object behind a bshmem_handle_t.
//
// Owns the symmetric-heap allocator, the team table, the host contexts and the
// statistics, and forwards data movement to a Backend.  Pointer arguments of
// the public API are local symmetric addresses; the runtime converts them to
// heap offsets (and range-checks them) before calling the backend.
//
// Parity: library/src/roc_shmem.cpp (host shim), context.hpp / context_host.cpp
// (Context: option bits, per-context stats, zero-size early-out).
#pragma once
#include <memory>
#include <mutex>
#include <thread>
#include <string>
#include <vector>

#include "../include/bshmem.h"
#include "allocator.h"
#include "backend.h"
#include "team.h"

namespace bshmem {

struct HostContext {
  bool live = false;
  long options = 0;
  std::thread::id owner;  // creating thread: a BSHMEM_CTX_PRIVATE context is for that thread alone (checked in debug mode)
  int team_slot = 0;      // PEs passed with this ctx are relative to this team
  HostStats stats;
};

}  // namespace bshmem

struct bshmem_runtime {
  bshmem_config_t cfg;
  std::unique_ptr<bshmem::Backend> backend;
  std::unique_ptr<bshmem::Pow2BuddyAllocator> heap;
  std::unique_ptr<bshmem::TeamTracker> teams;
  std::vector<std::unique_ptr<bshmem::HostContext>> ctxs;
  bshmem::HostStats global_stats;
  std::mutex mu;
  std::string last_error;
  bool finalized = false;

  bshmem_runtime(std::unique_ptr<bshmem::Backend> be, const bshmem_config_t& c);

  // address helpers -------------------------------------------------------
  bool to_offset(const void* p, uint64_t n, uint64_t* off) const;
  int fail(int code, const std::string& msg);
  bshmem::HostContext* ctx(int idx);
  // Resolve a ctx-relative PE to a world PE (-1 if out of range).
  int resolve_pe(int ctx_idx, int pe);
  int group_of_team(int slot, bshmem::CollGroup* g);
  int group_of_active_set(int start, int log_stride, int size, const long* psync, bshmem::CollGroup* g);
};

namespace bshmem {
// Wrap a backend into a runtime handle (used by every backend's init entry).
bshmem_runtime* make_runtime(std::unique_ptr<Backend> be, const bshmem_config_t* cfg);
}
