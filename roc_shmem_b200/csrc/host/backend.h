// backend.h — the transport interface the runtime drives, plus statistics.
//
// A Backend moves bytes between heaps addressed as (pe, offset).  The CPU
// backend implements it with memcpy/std::atomic over a shared mapping; the
// NVLink backend with copies and kernels on the peer-mapped CUDA VMM heap; the
// reverse-offload proxy executes ring descriptors through the same interface.
//
// Parity: library/src/backend_bc.hpp:63-304 (Backend owns heap, teams,
// contexts, stats) and backend_type.hpp (dispatch).  The reference picks the
// backend with #ifdef at compile time; here it is a run-time virtual call on
// the host (device code never goes through it).
#pragma once
#include <atomic>
#include <cstdint>
#include <string>

#include "../include/bshmem_types.h"
#include "team.h"

namespace bshmem {

// Host-side API call counters (library/src/stats.hpp:82-115 has 31 of them).
enum HostStat {
  ST_PUT = 0, ST_PUT_NBI, ST_GET, ST_GET_NBI, ST_PUT_SIGNAL, ST_P, ST_G,
  ST_AMO_FADD, ST_AMO_FINC, ST_AMO_FETCH, ST_AMO_FCSWAP, ST_AMO_ADD, ST_AMO_INC, ST_AMO_CSWAP,
  ST_AMO_SET, ST_AMO_SWAP, ST_AMO_FAND, ST_AMO_FOR, ST_AMO_FXOR, ST_AMO_AND, ST_AMO_OR, ST_AMO_XOR,
  ST_FENCE, ST_QUIET, ST_WAIT_UNTIL, ST_TEST, ST_BARRIER_ALL, ST_SYNC_ALL, ST_TEAM_SYNC,
  ST_BROADCAST, ST_TO_ALL, ST_REDUCE_SCATTER, ST_FCOLLECT, ST_ALLTOALL,
  ST_MALLOC, ST_FREE, ST_CTX_CREATE, ST_CTX_DESTROY, ST_TEAM_SPLIT, ST_TEAM_DESTROY,
  ST_BYTES_PUT, ST_BYTES_GET, ST_TIMEOUTS,
  ST_COUNT
};
const char* host_stat_name(int idx);

class HostStats {
 public:
  void enable(bool on) { on_ = on; }
  void inc(int idx, uint64_t by = 1) {
    if (on_) c_[idx].fetch_add(by, std::memory_order_relaxed);
  }
  uint64_t get(int idx) const { return c_[idx].load(std::memory_order_relaxed); }
  void reset() { for (auto& c : c_) c.store(0, std::memory_order_relaxed); }
  void accumulate(const HostStats& o) { for (int i = 0; i < ST_COUNT; ++i) c_[i] += o.get(i); }
 private:
  bool on_ = true;
  std::atomic<uint64_t> c_[ST_COUNT] = {};
};

// A collective's PE set and the sync resource it uses.
struct CollGroup {
  TeamInfo set;          // members in world PE numbers
  int my_idx = -1;       // my index in the set
  int slot = -1;         // team pool slot, or -1 for an active set
  uint64_t psync_off = 0;  // active set: offset of the user's pSync array
  int size() const { return set.size; }
};

class Backend {
 public:
  virtual ~Backend() {}
  virtual const char* name() const = 0;
  virtual int my_pe() const = 0;
  virtual int n_pes() const = 0;
  virtual uint64_t heap_bytes() const = 0;
  virtual uint64_t reserved_bytes() const = 0;     // internal region at heap start
  virtual char* local_base() const = 0;            // this PE's heap in this address space
  virtual char* peer_base(int pe) const = 0;       // PE's heap as mapped here (may be null)
  virtual bool host_dereferenceable() const = 0;

  // RMA; `local` may be any pointer valid for the backend's copy engine.
  virtual int put(int pe, uint64_t dst_off, const void* local, uint64_t n, bool nbi) = 0;
  virtual int get(int pe, void* local, uint64_t src_off, uint64_t n, bool nbi) = 0;
  virtual int put_signal(int pe, uint64_t dst_off, const void* local, uint64_t n, uint64_t sig_off,
                         uint64_t sig_val, int sig_op, bool nbi) = 0;
  virtual int amo(int pe, uint64_t off, int dtype, int op, uint64_t value, uint64_t cond,
                  uint64_t* fetched) = 0;
  virtual int fence() = 0;
  virtual int quiet() = 0;
  // Host contexts as ordering domains (one MPI window each in the reference, library/src/host/host.cpp:85-131): a
  // backend may keep resources per context — the NVLink backend a CUDA stream and pinned result slots, so that
  // quiet() on a context completes that context's operations only.  ctx_select names the context the calling
  // thread's next RMA / atomic / fence / quiet belongs to (thread-local; the runtime resets it to the default
  // context after each call); backends without per-context state ignore all three.
  virtual int ctx_open(int idx, long options) { (void)idx; (void)options; return BSHMEM_OK; }
  virtual void ctx_close(int idx) { (void)idx; }
  virtual void ctx_select(int idx) { (void)idx; }
  // cmp on local symmetric memory; blocks at most timeout_us.
  virtual int wait_until(uint64_t off, int dtype, int cmp, uint64_t value, uint64_t timeout_us) = 0;
  virtual int test(uint64_t off, int dtype, int cmp, uint64_t value, int* result) = 0;

  virtual int sync(const CollGroup& g) = 0;
  virtual int broadcast(const CollGroup& g, uint64_t dst_off, uint64_t src_off, uint64_t nbytes, int root) = 0;
  virtual int reduce(const CollGroup& g, int dtype, int op, uint64_t dst_off, uint64_t src_off, uint64_t nelems) = 0;
  virtual int reduce_root(const CollGroup& g, int dtype, int op, uint64_t dst_off, uint64_t src_off, uint64_t nelems, int root) = 0;
  virtual int reduce_scatter(const CollGroup& g, int dtype, int op, uint64_t dst_off, uint64_t src_off,
                             uint64_t nelems_per_pe) = 0;
  virtual int fcollect(const CollGroup& g, uint64_t dst_off, uint64_t src_off, uint64_t nbytes) = 0;
  virtual int alltoall(const CollGroup& g, uint64_t dst_off, uint64_t src_off, uint64_t nbytes) = 0;
  // Small host-side allgather among the members (team slot agreement).
  virtual int exchange_u64(const CollGroup& g, uint64_t mine, uint64_t* all) = 0;
  virtual int global_exit(int status) = 0;
  virtual int zero_local(uint64_t off, uint64_t n) = 0;   // memset 0 on the local heap
  // A team slot was released locally: clear its sync state so a later team can reuse it.
  virtual void reset_slot(int slot) { (void)slot; }
  virtual void set_timeout_us(uint64_t t) = 0;
  virtual bshmem_error_record_t last_record(bool clear) = 0;
  virtual std::string last_error() const = 0;
};

}  // namespace bshmem
