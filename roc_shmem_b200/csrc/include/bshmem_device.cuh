// bshmem_device.cuh — header-only device API (sm_100a): the calls a user kernel
// makes to move data between PEs over NVLink.
//
// Every PE's symmetric heap is mapped into every other PE's address space (CUDA
// VMM / IPC), so a remote access is a plain load, store or atomic on
// `heap_base[pe] + offset`; there is no NIC queue to post to and no completion
// queue to poll.  put/get exist at thread, warp (32 lanes) and block scope; the
// collectives in bshmem_coll.cuh are block collectives that can also be striped
// over many CTAs.
//
// API-shape parity: device functions of library/include/roc_shmem.hpp:474-832
// and the roc_shmemx_*_{wave,wg} extensions :2029-2566; semantics from
// library/src/ipc_policy.hpp:41-147 (IPC loads/stores/atomics),
// context_tmpl_device.hpp:199-246 (wait_until/test), fence_policy.hpp:45-63
// (CTX_NOSTORE skips the publishing fence).  Additions: putmem_signal, bounded
// waits that return a status instead of spinning for ever, all 15 AMOs natively.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#ifdef __cplusplus
#include <type_traits>
#endif

#include "bshmem_types.h"

// ---- layout of the runtime-internal region at the start of every heap ----------
#define BSHMEM_INTERNAL_BYTES (72ull << 20)
/* Staging for one-exchange collectives of the world team (host-launched; fcollect, alltoall, reduce-scatter and the
 * first half of mid-size allreduces): 40 MiB .. 72 MiB, [2 parities][16 MiB]; sender k's block starts at k * (bytes
 * per sender).  The parity is the low bit of a call sequence number that the host supplies (same on every PE).     */
#define BSHMEM_OFF_STAGE (40ull << 20)
#define BSHMEM_STAGE_BYTES (16ull << 20)
/* Multicast barrier of the world team: per channel, a counter every PE adds to with one multimem.red (replicated in
 * every heap) and a local epoch word.                                                                            */
#define BSHMEM_OFF_MCBAR (960ull << 10)
#define BSHMEM_MCBAR_BYTES (2ull * BSHMEM_MAX_COLL_CTAS * 8)
/* Low-latency allreduce slots for host-launched, multi-block calls (epoch supplied by the host): 4 MiB .. 36 MiB,
 * [2 parities][sender PE][512 KiB of payload as 8-byte words].                                                    */
#define BSHMEM_OFF_LLB (4ull << 20)
#define BSHMEM_LLB_PAYLOAD_BYTES (512ull << 10)
#define BSHMEM_LLB_SLOT_BYTES (2 * BSHMEM_LLB_PAYLOAD_BYTES)
#define BSHMEM_LLB_BYTES (2ull * BSHMEM_MAX_PES * BSHMEM_LLB_SLOT_BYTES)
/* The same for every other team (single block, at most 1 KiB): 36 MiB .. 38.6 MiB, [team slot][64-byte header with the
 * team's epoch word, then 2 parities][sender index][2 KiB]; zeroed when a team slot is (re)assigned.                 */
#define BSHMEM_OFF_LLT (36ull << 20)
#define BSHMEM_LLT_PAYLOAD_BYTES 1024ull
#define BSHMEM_LLT_SLOT_BYTES (2 * BSHMEM_LLT_PAYLOAD_BYTES)
#define BSHMEM_LLT_TEAM_BYTES (64 + 2ull * BSHMEM_MAX_PES * BSHMEM_LLT_SLOT_BYTES)
#define BSHMEM_OFF_FLAGS 0ull                                   /* [team][cta][pe] u64, written by peers   */
#define BSHMEM_FLAGS_BYTES ((uint64_t)BSHMEM_MAX_TEAMS * BSHMEM_MAX_COLL_CTAS * BSHMEM_MAX_PES * 8)
#define BSHMEM_OFF_EPOCHS (BSHMEM_OFF_FLAGS + BSHMEM_FLAGS_BYTES) /* [team][cta] u64, local only           */
#define BSHMEM_EPOCHS_BYTES ((uint64_t)BSHMEM_MAX_TEAMS * BSHMEM_MAX_COLL_CTAS * 8)
#define BSHMEM_OFF_XCHG (BSHMEM_OFF_EPOCHS + BSHMEM_EPOCHS_BYTES)  /* [team][pe] u64 host-side exchange      */
#define BSHMEM_XCHG_BYTES ((uint64_t)BSHMEM_MAX_TEAMS * BSHMEM_MAX_PES * 8)
#define BSHMEM_OFF_SCRATCH (BSHMEM_OFF_XCHG + BSHMEM_XCHG_BYTES)   /* 64 KiB bounce area (host p/g/AMO)      */
#define BSHMEM_SCRATCH_BYTES (64ull << 10)
/* Low-latency allreduce slots at 1 MiB: a local epoch word, then [2 parities][sender PE][payload words of 8 bytes =
 * 4 bytes of data + the 32-bit epoch], written by peers with single 8-byte stores (data and flag arrive together).   */
#define BSHMEM_OFF_LL (1ull << 20)
#define BSHMEM_LL_PAYLOAD_BYTES 4096ull
#define BSHMEM_LL_SLOT_BYTES (2 * BSHMEM_LL_PAYLOAD_BYTES)
#define BSHMEM_LL_BYTES (64 + 2ull * BSHMEM_MAX_PES * BSHMEM_LL_SLOT_BYTES)
#define BSHMEM_OFF_SLAB (2ull << 20)                              /* device-callable slab allocator region   */
#define BSHMEM_SLAB_BYTES (2ull << 20)

typedef struct {
  int pe_start, stride, size, my_idx;
  int slot;        /* team pool slot; -1 = legacy active set synchronising through psync */
  int reserved;
  long* psync;     /* active set only: the caller's symmetric pSync array (>= 2 longs)  */
} bshmem_team_dev_t;

typedef struct {
  int32_t my_pe, n_pes;
  uint64_t heap_bytes;
  char* heap_base[BSHMEM_MAX_PES];     /* every PE's heap as mapped in this process            */
  char* mc_base;                       /* NVLink multicast mapping of the heaps, or null       */
  bshmem_error_record_t* err;          /* device-visible pinned host record                     */
  unsigned long long timeout_ns;       /* bound of every device-side wait                       */
  unsigned long long* stats;           /* device counters (BSHMEM_DSTAT_*), or null              */
  void* proxy;                         /* reverse-offload ring descriptor, or null               */
  uint32_t debug;
  uint32_t reserved;
} bshmem_dev_state_t;

enum {
  BSHMEM_DSTAT_PUT = 0, BSHMEM_DSTAT_GET, BSHMEM_DSTAT_PUT_SIGNAL, BSHMEM_DSTAT_P, BSHMEM_DSTAT_G, BSHMEM_DSTAT_AMO,
  BSHMEM_DSTAT_FENCE, BSHMEM_DSTAT_QUIET, BSHMEM_DSTAT_WAIT, BSHMEM_DSTAT_WAIT_NS, BSHMEM_DSTAT_BARRIER,
  BSHMEM_DSTAT_BARRIER_NS, BSHMEM_DSTAT_COLL, BSHMEM_DSTAT_BYTES_PUT, BSHMEM_DSTAT_BYTES_GET, BSHMEM_DSTAT_TIMEOUTS,
  BSHMEM_DSTAT_PROXY_OPS, BSHMEM_DSTAT_COUNT
};

/* Optional event ring behind the counters (same allocation, so the state struct does not grow):
 *   stats[BSHMEM_DSTAT_COUNT]      capacity in events, 0 = tracing off
 *   stats[BSHMEM_DSTAT_COUNT + 1]  events recorded so far (the ring keeps the last `capacity`)
 *   then 4 words per event: %globaltimer ns, op | pe << 8 | block << 32, bytes, sequence number */
#define BSHMEM_TRACE_MAX_EVENTS 16384
#define BSHMEM_TRACE_WORDS (2 + 4 * BSHMEM_TRACE_MAX_EVENTS)
enum {
  BSHMEM_TRACE_PUT = 1, BSHMEM_TRACE_GET, BSHMEM_TRACE_PUT_SIGNAL, BSHMEM_TRACE_AMO, BSHMEM_TRACE_WAIT, BSHMEM_TRACE_BARRIER,
  BSHMEM_TRACE_COLL, BSHMEM_TRACE_TIMEOUT
};

#ifdef __CUDACC__
namespace bshmem {
namespace dev {

enum Scope { THREAD = 0, WARP = 1, BLOCK = 2 };
using State = bshmem_dev_state_t;
using Team = bshmem_team_dev_t;

// ---- small helpers ------------------------------------------------------------------
__device__ __forceinline__ unsigned long long timer() {   // nanoseconds, same clock on every SM
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ int my_pe(const State& s) { return s.my_pe; }
__device__ __forceinline__ int n_pes(const State& s) { return s.n_pes; }
__device__ __forceinline__ void stat(const State& s, int idx, unsigned long long by = 1) {
  if (s.stats) atomicAdd(&s.stats[idx], by);
}
// One timeline event (who, what, how much, when); a no-op unless the host switched tracing on.
__device__ __forceinline__ void trace(const State& s, int op, int pe, unsigned long long bytes) {
  if (!s.stats) return;
  const unsigned long long cap = *reinterpret_cast<volatile unsigned long long*>(&s.stats[BSHMEM_DSTAT_COUNT]);
  if (!cap) return;
  const unsigned long long i = atomicAdd(&s.stats[BSHMEM_DSTAT_COUNT + 1], 1ull);
  unsigned long long* e = s.stats + BSHMEM_DSTAT_COUNT + 2 + 4 * (i % cap);
  e[0] = timer();
  e[1] = (unsigned long long)(op & 0xFF) | ((unsigned long long)(pe & 0xFFFFFF) << 8) | ((unsigned long long)blockIdx.x << 32);
  e[2] = bytes;
  e[3] = i;
}
__device__ __forceinline__ int team_pe(const Team& t, int idx) { return t.pe_start + idx * t.stride; }
// world PE -> index in team, -1 if not a member
__device__ __forceinline__ int team_index(const Team& t, int pe) {
  int d = pe - t.pe_start;
  if (d < 0 || d % t.stride) return -1;
  d /= t.stride;
  return d < t.size ? d : -1;
}
__device__ __forceinline__ int team_translate_pe(const Team& src, int src_pe, const Team& dst) {
  if (src_pe < 0 || src_pe >= src.size) return -1;
  return team_index(dst, team_pe(src, src_pe));
}
__device__ __forceinline__ Team team_world(const State& s) { return Team{0, 1, s.n_pes, s.my_pe, 0, 0, nullptr}; }

// Local symmetric address -> the same object on `pe` (always mapped on one NVSwitch node).
template <typename T>
__device__ __forceinline__ T* ptr(const State& s, const T* local, int pe) {
  uint64_t off = reinterpret_cast<const char*>(local) - s.heap_base[s.my_pe];
  return reinterpret_cast<T*>(s.heap_base[pe] + off);
}
__device__ __forceinline__ bool in_heap(const State& s, const void* p, size_t n) {
  uint64_t off = reinterpret_cast<const char*>(p) - s.heap_base[s.my_pe];
  return off <= s.heap_bytes && n <= s.heap_bytes - off;
}

__device__ __forceinline__ void record_error(const State& s, uint32_t code, int pe, uint32_t where, uint64_t addr,
                                             uint64_t expected, uint64_t seen) {
  if (!s.err) return;
  if (atomicAdd(&s.err->count, 1u) == 0) {   // first error wins; later ones only count
    s.err->pe = pe; s.err->where = where; s.err->addr = addr; s.err->expected = expected; s.err->seen = seen;
    __threadfence_system();
    s.err->code = code;
  }
  stat(s, BSHMEM_DSTAT_TIMEOUTS);
  trace(s, BSHMEM_TRACE_TIMEOUT, pe, where);
}

// Debug-build argument check: records BSHMEM_ERR_RANGE and tells the caller to skip the access.
__device__ __forceinline__ bool check_target(const State& s, const void* sym, size_t n, int pe) {
  if (!s.debug) return true;
  if (pe < 0 || pe >= s.n_pes || !in_heap(s, sym, n)) {
    record_error(s, BSHMEM_ERR_RANGE, pe, BSHMEM_WHERE_BOUNDS, (uint64_t)sym, n, 0);
    return false;
  }
  return true;
}

// ---- ordering ---------------------------------------------------------------------------
// fence: puts issued before it are delivered to each PE before puts issued after it.
// quiet: every outstanding put/get/atomic of this thread is complete and visible.
// With a load/store transport both are a system-scope fence.
__device__ __forceinline__ void fence(const State& s) { asm volatile("fence.acq_rel.sys;" ::: "memory"); stat(s, BSHMEM_DSTAT_FENCE); }
__device__ __forceinline__ void fence_pe(const State& s, int) { fence(s); }
__device__ __forceinline__ void quiet(const State& s) { asm volatile("fence.acq_rel.sys;" ::: "memory"); stat(s, BSHMEM_DSTAT_QUIET); }
__device__ __forceinline__ void threadfence_system() { __threadfence_system(); }

// ---- the copy engine: 16-byte vectors when both sides allow it ---------------------------
template <Scope S> __device__ __forceinline__ int scope_rank() {
  if (S == THREAD) return 0;
  if (S == WARP) return threadIdx.x & 31;
  return threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
}
template <Scope S> __device__ __forceinline__ int scope_size() {
  if (S == THREAD) return 1;
  if (S == WARP) return 32;
  return blockDim.x * blockDim.y * blockDim.z;
}
template <Scope S> __device__ __forceinline__ void scope_sync() {
  if (S == WARP) __syncwarp();
  if (S == BLOCK) __syncthreads();
}

template <Scope S>
__device__ __forceinline__ void copy_bytes(char* __restrict__ dst, const char* __restrict__ src, size_t n) {
  const int r = scope_rank<S>(), w = scope_size<S>();
  if (n == 0) return;
  // Same misalignment on both sides: byte head, 16-byte body, byte tail.
  if ((((uintptr_t)dst ^ (uintptr_t)src) & 15) == 0) {
    size_t head = (16 - ((uintptr_t)dst & 15)) & 15;
    if (head > n) head = n;
    for (size_t i = r; i < head; i += w) dst[i] = src[i];
    size_t body = (n - head) >> 4;
    const uint4* s4 = reinterpret_cast<const uint4*>(src + head);
    uint4* d4 = reinterpret_cast<uint4*>(dst + head);
    size_t i = r;
    // eight, then four independent 16-byte accesses in flight per thread
    for (; i + 7 * (size_t)w < body; i += 8 * (size_t)w) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = s4[i + u * (size_t)w];
#pragma unroll
      for (int u = 0; u < 8; ++u) d4[i + u * (size_t)w] = v[u];
    }
    for (; i + 3 * (size_t)w < body; i += 4 * (size_t)w) {
      uint4 a = s4[i], b = s4[i + w], c = s4[i + 2 * (size_t)w], d = s4[i + 3 * (size_t)w];
      d4[i] = a; d4[i + w] = b; d4[i + 2 * (size_t)w] = c; d4[i + 3 * (size_t)w] = d;
    }
    for (; i < body; i += w) d4[i] = s4[i];
    size_t done = head + (body << 4);
    for (size_t k = done + r; k < n; k += w) dst[k] = src[k];
  } else if ((((uintptr_t)dst | (uintptr_t)src | n) & 3) == 0) {
    const uint32_t* s1 = reinterpret_cast<const uint32_t*>(src);
    uint32_t* d1 = reinterpret_cast<uint32_t*>(dst);
    for (size_t i = r; i < (n >> 2); i += w) d1[i] = s1[i];
  } else {
    for (size_t i = r; i < n; i += w) dst[i] = src[i];
  }
}

// ---- large-message copy engine: bulk async copies staged through shared memory --------------------------
// One thread drives a ring of kStages chunks: cp.async.bulk global -> shared (completion on an mbarrier), then
// cp.async.bulk shared -> global (bulk-group completion).  Either side may be a peer's memory; nothing here is a
// multicast copy.  No registers carry payload, so one CTA keeps (kStages - 1) * kChunk bytes of loads in flight.
// Needs 16-byte aligned src, dst and n, `smem` of kStages * kChunk bytes (16-byte aligned) plus kStages mbarriers.
// Block scope: every thread calls; returns BSHMEM_OK or BSHMEM_ERR_TIMEOUT (a bounded mbarrier wait ran out).
template <int kStages, int kChunk>
__device__ __forceinline__ int bulk_copy_block(const State& s, char* dst, const char* src, size_t n, char* smem, uint64_t* bars) {
  __shared__ int bulk_status;
  if (threadIdx.x == 0) {
    bulk_status = BSHMEM_OK;
    for (int i = 0; i < kStages; ++i)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&bars[i])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const size_t nchunks = (n + kChunk - 1) / kChunk;
    auto issue_load = [&](size_t k) {
      const int st = (int)(k % kStages);
      const uint32_t bytes = (uint32_t)((k + 1) * (size_t)kChunk <= n ? kChunk : n - k * (size_t)kChunk);
      const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&bars[st]);
      const uint32_t sm = (uint32_t)__cvta_generic_to_shared(smem + (size_t)st * kChunk);
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(sm), "l"(src + k * (size_t)kChunk), "r"(bytes), "r"(bar) : "memory");
    };
    for (size_t k = 0; k < nchunks && k < (size_t)(kStages - 1); ++k) issue_load(k);
    const unsigned long long t0 = timer();
    for (size_t i = 0; i < nchunks; ++i) {
      const int st = (int)(i % kStages);
      const uint32_t parity = (uint32_t)((i / kStages) & 1);
      const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&bars[st]);
      uint32_t ok = 0, it = 0;
      while (true) {
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) break;
        if ((++it & 63) == 0 && timer() - t0 > s.timeout_ns) {
          record_error(s, BSHMEM_ERR_TIMEOUT, -1, BSHMEM_WHERE_MBARRIER, (uint64_t)(src + i * (size_t)kChunk), i, 0);
          bulk_status = BSHMEM_ERR_TIMEOUT;
          break;
        }
      }
      if (!ok) break;
      const uint32_t bytes = (uint32_t)((i + 1) * (size_t)kChunk <= n ? kChunk : n - i * (size_t)kChunk);
      const uint32_t sm = (uint32_t)__cvta_generic_to_shared(smem + (size_t)st * kChunk);
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + i * (size_t)kChunk), "r"(sm), "r"(bytes) : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      // chunk i + kStages - 1 goes into the stage chunk i - 1 was stored from: that store must have read its data
      const size_t nxt = i + kStages - 1;
      if (nxt < nchunks) {
        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        issue_load(nxt);
      }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");      // every store has been written
  }
  __syncthreads();
  const int rc = bulk_status;
  __syncthreads();
  return rc;
}

// ---- RMA ------------------------------------------------------------------------------------
// put: returns when `src` is reusable; delivery is guaranteed after fence()/quiet()/a barrier.
// _nbi forms are identical on this transport (stores are issued before the call returns).
template <Scope S = THREAD>
__device__ __forceinline__ void putmem(const State& s, void* dest, const void* src, size_t n, int pe, long ctx_options = 0) {
  if (n == 0 || !check_target(s, dest, n, pe)) return;
  copy_bytes<S>(reinterpret_cast<char*>(ptr(s, reinterpret_cast<char*>(dest), pe)), reinterpret_cast<const char*>(src), n);
  if (!(ctx_options & BSHMEM_CTX_NOSTORE)) __threadfence();
  if (scope_rank<S>() == 0) { stat(s, BSHMEM_DSTAT_PUT); stat(s, BSHMEM_DSTAT_BYTES_PUT, n); trace(s, BSHMEM_TRACE_PUT, pe, n); }
  scope_sync<S>();
}
template <Scope S = THREAD>
__device__ __forceinline__ void putmem_nbi(const State& s, void* dest, const void* src, size_t n, int pe) {
  if (n == 0 || !check_target(s, dest, n, pe)) return;
  copy_bytes<S>(reinterpret_cast<char*>(ptr(s, reinterpret_cast<char*>(dest), pe)), reinterpret_cast<const char*>(src), n);
  if (scope_rank<S>() == 0) { stat(s, BSHMEM_DSTAT_PUT); stat(s, BSHMEM_DSTAT_BYTES_PUT, n); trace(s, BSHMEM_TRACE_PUT, pe, n); }
}
template <Scope S = THREAD>
__device__ __forceinline__ void getmem(const State& s, void* dest, const void* src, size_t n, int pe) {
  if (n == 0 || !check_target(s, src, n, pe)) return;
  copy_bytes<S>(reinterpret_cast<char*>(dest), reinterpret_cast<const char*>(ptr(s, reinterpret_cast<const char*>(src), pe)), n);
  if (scope_rank<S>() == 0) { stat(s, BSHMEM_DSTAT_GET); stat(s, BSHMEM_DSTAT_BYTES_GET, n); trace(s, BSHMEM_TRACE_GET, pe, n); }
  scope_sync<S>();
}
template <Scope S = THREAD>
__device__ __forceinline__ void getmem_nbi(const State& s, void* dest, const void* src, size_t n, int pe) {
  getmem<S>(s, dest, src, n, pe);   // loads have returned when the call returns
}
template <typename T, Scope S = THREAD>
__device__ __forceinline__ void put(const State& s, T* dest, const T* src, size_t nelems, int pe) { putmem<S>(s, dest, src, nelems * sizeof(T), pe); }
template <typename T, Scope S = THREAD>
__device__ __forceinline__ void get(const State& s, T* dest, const T* src, size_t nelems, int pe) { getmem<S>(s, dest, src, nelems * sizeof(T), pe); }
template <typename T>
__device__ __forceinline__ void p(const State& s, T* dest, T value, int pe) {
  if (!check_target(s, dest, sizeof(T), pe)) return;
  *ptr(s, dest, pe) = value;
  stat(s, BSHMEM_DSTAT_P);
}
template <typename T>
__device__ __forceinline__ T g(const State& s, const T* src, int pe) {
  if (!check_target(s, src, sizeof(T), pe)) return T();
  stat(s, BSHMEM_DSTAT_G);
  return *reinterpret_cast<const volatile T*>(ptr(s, src, pe));
}

// put-with-signal (OpenSHMEM 1.5): the payload is visible to whoever observes the signal update.
template <Scope S = THREAD>
__device__ __forceinline__ void putmem_signal(const State& s, void* dest, const void* src, size_t n, uint64_t* sig_addr,
                                              uint64_t signal, int sig_op, int pe) {
  if (!check_target(s, sig_addr, 8, pe)) return;
  if (n) copy_bytes<S>(reinterpret_cast<char*>(ptr(s, reinterpret_cast<char*>(dest), pe)), reinterpret_cast<const char*>(src), n);
  scope_sync<S>();   // every participant's stores are ordered before the leader's release
  if (scope_rank<S>() == 0) {
    uint64_t* rs = ptr(s, sig_addr, pe);
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    if (sig_op == BSHMEM_SIGNAL_ADD) asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(rs), "l"(signal) : "memory");
    else asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(rs), "l"(signal) : "memory");
    stat(s, BSHMEM_DSTAT_PUT_SIGNAL);
    trace(s, BSHMEM_TRACE_PUT_SIGNAL, pe, n);
    stat(s, BSHMEM_DSTAT_BYTES_PUT, n);
  }
}
__device__ __forceinline__ uint64_t signal_fetch(const State&, const uint64_t* sig_addr) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(sig_addr) : "memory");
  return v;
}

// ---- atomics (system scope, on the peer mapping) ---------------------------------------------
template <typename T> struct AmoWord;   // maps T to the CUDA atomic word type
template <> struct AmoWord<int> { using type = int; };
template <> struct AmoWord<unsigned int> { using type = unsigned int; };
template <> struct AmoWord<long> { using type = unsigned long long; };
template <> struct AmoWord<unsigned long> { using type = unsigned long long; };
template <> struct AmoWord<long long> { using type = unsigned long long; };
template <> struct AmoWord<unsigned long long> { using type = unsigned long long; };
template <> struct AmoWord<float> { using type = unsigned int; };
template <> struct AmoWord<double> { using type = unsigned long long; };

template <typename T> __device__ __forceinline__ typename AmoWord<T>::type amo_bits(T v) {
  typename AmoWord<T>::type w;
  memcpy(&w, &v, sizeof(T));
  return w;
}
template <typename T> __device__ __forceinline__ T amo_unbits(typename AmoWord<T>::type w) {
  T v;
  memcpy(&v, &w, sizeof(T));
  return v;
}

template <typename T>
__device__ __forceinline__ T atomic_fetch_add(const State& s, T* dest, T value, int pe) {
  using W = typename AmoWord<T>::type;
  if (!check_target(s, dest, sizeof(T), pe)) return T();
  stat(s, BSHMEM_DSTAT_AMO);
  W* r = reinterpret_cast<W*>(ptr(s, dest, pe));
  if constexpr (sizeof(T) == sizeof(W) && !(std::is_same<T, float>::value || std::is_same<T, double>::value))
    return amo_unbits<T>(atomicAdd_system(r, amo_bits(value)));
  else if constexpr (std::is_same<T, float>::value)
    return atomicAdd_system(reinterpret_cast<float*>(r), value);
  else
    return atomicAdd_system(reinterpret_cast<double*>(r), value);
}
template <typename T> __device__ __forceinline__ void atomic_add(const State& s, T* dest, T value, int pe) { (void)atomic_fetch_add(s, dest, value, pe); }
template <typename T> __device__ __forceinline__ T atomic_fetch_inc(const State& s, T* dest, int pe) { return atomic_fetch_add(s, dest, (T)1, pe); }
template <typename T> __device__ __forceinline__ void atomic_inc(const State& s, T* dest, int pe) { (void)atomic_fetch_add(s, dest, (T)1, pe); }
template <typename T>
__device__ __forceinline__ T atomic_fetch(const State& s, const T* src, int pe) {
  using W = typename AmoWord<T>::type;
  if (!check_target(s, src, sizeof(T), pe)) return T();
  stat(s, BSHMEM_DSTAT_AMO);
  W* r = reinterpret_cast<W*>(ptr(s, const_cast<T*>(src), pe));
  return amo_unbits<T>(atomicOr_system(r, (W)0));
}
template <typename T>
__device__ __forceinline__ T atomic_compare_swap(const State& s, T* dest, T cond, T value, int pe) {
  using W = typename AmoWord<T>::type;
  if (!check_target(s, dest, sizeof(T), pe)) return T();
  stat(s, BSHMEM_DSTAT_AMO);
  return amo_unbits<T>(atomicCAS_system(reinterpret_cast<W*>(ptr(s, dest, pe)), amo_bits(cond), amo_bits(value)));
}
template <typename T>
__device__ __forceinline__ T atomic_swap(const State& s, T* dest, T value, int pe) {
  using W = typename AmoWord<T>::type;
  if (!check_target(s, dest, sizeof(T), pe)) return T();
  stat(s, BSHMEM_DSTAT_AMO);
  return amo_unbits<T>(atomicExch_system(reinterpret_cast<W*>(ptr(s, dest, pe)), amo_bits(value)));
}
template <typename T> __device__ __forceinline__ void atomic_set(const State& s, T* dest, T value, int pe) { (void)atomic_swap(s, dest, value, pe); }
#define BSHMEM_DEV_BITWISE(NAME, FN)                                                                    \
  template <typename T> __device__ __forceinline__ T atomic_fetch_##NAME(const State& s, T* dest, T value, int pe) { \
    using W = typename AmoWord<T>::type;                                                                \
    if (!check_target(s, dest, sizeof(T), pe)) return T();                                              \
    stat(s, BSHMEM_DSTAT_AMO);                                                                          \
    return amo_unbits<T>(FN(reinterpret_cast<W*>(ptr(s, dest, pe)), amo_bits(value)));                  \
  }                                                                                                     \
  template <typename T> __device__ __forceinline__ void atomic_##NAME(const State& s, T* dest, T value, int pe) { \
    (void)atomic_fetch_##NAME(s, dest, value, pe);                                                      \
  }
BSHMEM_DEV_BITWISE(and, atomicAnd_system)
BSHMEM_DEV_BITWISE(or, atomicOr_system)
BSHMEM_DEV_BITWISE(xor, atomicXor_system)
#undef BSHMEM_DEV_BITWISE

// ---- point-to-point synchronisation -------------------------------------------------------------
template <typename T> __device__ __forceinline__ bool cmp_holds(int cmp, T a, T b) {
  switch (cmp) {
    case BSHMEM_CMP_EQ: return a == b;
    case BSHMEM_CMP_NE: return a != b;
    case BSHMEM_CMP_GT: return a > b;
    case BSHMEM_CMP_GE: return a >= b;
    case BSHMEM_CMP_LT: return a < b;
    default: return a <= b;
  }
}
template <typename T> __device__ __forceinline__ T load_acquire_sys(const T* p) {
  T v;
  if constexpr (sizeof(T) == 8) { uint64_t w; asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory"); memcpy(&v, &w, 8); }
  else if constexpr (sizeof(T) == 4) { uint32_t w; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(w) : "l"(p) : "memory"); memcpy(&v, &w, 4); }
  else if constexpr (sizeof(T) == 2) { uint16_t w; asm volatile("ld.acquire.sys.global.u16 %0, [%1];" : "=h"(w) : "l"(p) : "memory"); memcpy(&v, &w, 2); }
  else { uint32_t w; asm volatile("ld.acquire.sys.global.u8 %0, [%1];" : "=r"(w) : "l"(p) : "memory"); uint8_t b = (uint8_t)w; memcpy(&v, &b, 1); }
  return v;
}
template <typename T>
__device__ __forceinline__ int test(const State&, const T* ivar, int cmp, T value) {
  return cmp_holds(cmp, load_acquire_sys(ivar), value) ? 1 : 0;
}
// Spins on local symmetric memory until `*ivar cmp value`, at most state.timeout_ns.
// Returns BSHMEM_OK or BSHMEM_ERR_TIMEOUT (and fills the error record).
template <typename T>
__device__ __forceinline__ int wait_until(const State& s, const T* ivar, int cmp, T value, uint32_t where = BSHMEM_WHERE_WAIT_UNTIL, int pe = -1) {
  T seen = load_acquire_sys(ivar);
  if (cmp_holds(cmp, seen, value)) return BSHMEM_OK;
  unsigned long long t0 = timer();
  unsigned it = 0;
  while (true) {
    seen = load_acquire_sys(ivar);
    if (cmp_holds(cmp, seen, value)) break;
    if ((++it & 31) == 0) {
      if (timer() - t0 > s.timeout_ns) {
        uint64_t e = 0, g = 0;
        memcpy(&e, &value, sizeof(T));
        memcpy(&g, &seen, sizeof(T));
        record_error(s, BSHMEM_ERR_TIMEOUT, pe, where, (uint64_t)ivar, e, g);
        return BSHMEM_ERR_TIMEOUT;
      }
      __nanosleep(64);
    }
  }
  if (s.stats) { stat(s, BSHMEM_DSTAT_WAIT); stat(s, BSHMEM_DSTAT_WAIT_NS, timer() - t0); trace(s, BSHMEM_TRACE_WAIT, s.my_pe, timer() - t0); }
  return BSHMEM_OK;
}

// ---- contexts ---------------------------------------------------------------------------------------
// A device context is the option bits plus the team its PE numbers are relative to.  It lives wherever
// the caller keeps it (typically __shared__, as with roc_shmem_wg_ctx_create); nothing is pooled.
struct Ctx {
  long options;
  Team team;
};
__device__ __forceinline__ int wg_init() { return BSHMEM_THREAD_MULTIPLE; }
// Any requested level is granted as THREAD_MULTIPLE (every device call is safe from every thread).
__device__ __forceinline__ int wg_init_thread(int /*requested*/, int* provided) {
  if (provided) *provided = BSHMEM_THREAD_MULTIPLE;
  return BSHMEM_OK;
}
__device__ __forceinline__ void wg_finalize() {}
__device__ __forceinline__ int query_thread() { return BSHMEM_THREAD_MULTIPLE; }
// Called by every thread of the block; the handle is valid after the call returns.
__device__ __forceinline__ int wg_ctx_create(const State& s, long options, Ctx* ctx) {
  if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) { ctx->options = options; ctx->team = team_world(s); }
  __syncthreads();
  return BSHMEM_OK;
}
__device__ __forceinline__ int wg_team_create_ctx(const State&, const Team& team, long options, Ctx* ctx) {
  if (team.my_idx < 0) return BSHMEM_ERR_INVALID;
  if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) { ctx->options = options; ctx->team = team; }
  __syncthreads();
  return BSHMEM_OK;
}
__device__ __forceinline__ void wg_ctx_destroy(Ctx*) {}
// ---- context forms of every operation ------------------------------------------------------------------
// PE arguments are relative to the context's team (world numbering for a context made by wg_ctx_create), for
// RMA, atomics, put-with-signal and fence(pe) alike; BSHMEM_CTX_NOSTORE skips the fence that publishes the
// caller's earlier plain stores after a blocking put.  Parity: library/include/roc_shmem.hpp:559-725 (ctx RMA,
// fence, quiet, p/g), :1548-1953 (ctx AMOs), library/src/roc_shmem_gpu.cpp:240-247 (translate_pe), :298-661.
__device__ __forceinline__ int ctx_pe(const Ctx& c, int pe) { return team_pe(c.team, pe); }
__device__ __forceinline__ int ctx_my_pe(const Ctx& c) { return c.team.my_idx; }
__device__ __forceinline__ int ctx_n_pes(const Ctx& c) { return c.team.size; }
__device__ __forceinline__ void ctx_fence(const State& s, const Ctx&) { fence(s); }
__device__ __forceinline__ void ctx_fence(const State& s, const Ctx& c, int pe) { fence_pe(s, ctx_pe(c, pe)); }
__device__ __forceinline__ void ctx_quiet(const State& s, const Ctx&) { quiet(s); }
__device__ __forceinline__ void ctx_threadfence_system(const State&, const Ctx&) { threadfence_system(); }
template <typename T> __device__ __forceinline__ T* ctx_ptr(const State& s, const Ctx& c, const T* local, int pe) { return ptr(s, local, ctx_pe(c, pe)); }

template <Scope S = THREAD>
__device__ __forceinline__ void ctx_putmem(const State& s, const Ctx& c, void* dest, const void* src, size_t n, int pe) {
  putmem<S>(s, dest, src, n, ctx_pe(c, pe), c.options);
}
template <Scope S = THREAD>
__device__ __forceinline__ void ctx_putmem_nbi(const State& s, const Ctx& c, void* dest, const void* src, size_t n, int pe) {
  putmem_nbi<S>(s, dest, src, n, ctx_pe(c, pe));
}
template <Scope S = THREAD>
__device__ __forceinline__ void ctx_getmem(const State& s, const Ctx& c, void* dest, const void* src, size_t n, int pe) {
  getmem<S>(s, dest, src, n, ctx_pe(c, pe));
}
template <Scope S = THREAD>
__device__ __forceinline__ void ctx_getmem_nbi(const State& s, const Ctx& c, void* dest, const void* src, size_t n, int pe) {
  getmem_nbi<S>(s, dest, src, n, ctx_pe(c, pe));
}
template <typename T, Scope S = THREAD>
__device__ __forceinline__ void ctx_put(const State& s, const Ctx& c, T* dest, const T* src, size_t nelems, int pe) {
  putmem<S>(s, dest, src, nelems * sizeof(T), ctx_pe(c, pe), c.options);
}
template <typename T, Scope S = THREAD>
__device__ __forceinline__ void ctx_put_nbi(const State& s, const Ctx& c, T* dest, const T* src, size_t nelems, int pe) {
  putmem_nbi<S>(s, dest, src, nelems * sizeof(T), ctx_pe(c, pe));
}
template <typename T, Scope S = THREAD>
__device__ __forceinline__ void ctx_get(const State& s, const Ctx& c, T* dest, const T* src, size_t nelems, int pe) {
  getmem<S>(s, dest, src, nelems * sizeof(T), ctx_pe(c, pe));
}
template <typename T, Scope S = THREAD>
__device__ __forceinline__ void ctx_get_nbi(const State& s, const Ctx& c, T* dest, const T* src, size_t nelems, int pe) {
  getmem_nbi<S>(s, dest, src, nelems * sizeof(T), ctx_pe(c, pe));
}
template <typename T> __device__ __forceinline__ void ctx_p(const State& s, const Ctx& c, T* dest, T value, int pe) { p(s, dest, value, ctx_pe(c, pe)); }
template <typename T> __device__ __forceinline__ T ctx_g(const State& s, const Ctx& c, const T* src, int pe) { return g(s, src, ctx_pe(c, pe)); }
template <Scope S = THREAD>
__device__ __forceinline__ void ctx_putmem_signal(const State& s, const Ctx& c, void* dest, const void* src, size_t n,
                                                  uint64_t* sig_addr, uint64_t signal, int sig_op, int pe) {
  putmem_signal<S>(s, dest, src, n, sig_addr, signal, sig_op, ctx_pe(c, pe));
}
// the 15 atomics, one line per signature class
#define BSHMEM_DEV_CTX_AMO_VALUE(RET, NAME)                                                                           \
  template <typename T> __device__ __forceinline__ RET ctx_##NAME(const State& s, const Ctx& c, T* dest, T value, int pe) { \
    return NAME(s, dest, value, ctx_pe(c, pe));                                                                         \
  }
#define BSHMEM_DEV_CTX_AMO_NOVALUE(RET, NAME)                                                                         \
  template <typename T> __device__ __forceinline__ RET ctx_##NAME(const State& s, const Ctx& c, T* dest, int pe) {      \
    return NAME(s, dest, ctx_pe(c, pe));                                                                                \
  }
BSHMEM_DEV_CTX_AMO_VALUE(T, atomic_fetch_add)
BSHMEM_DEV_CTX_AMO_VALUE(void, atomic_add)
BSHMEM_DEV_CTX_AMO_VALUE(T, atomic_swap)
BSHMEM_DEV_CTX_AMO_VALUE(void, atomic_set)
BSHMEM_DEV_CTX_AMO_VALUE(T, atomic_fetch_and)
BSHMEM_DEV_CTX_AMO_VALUE(void, atomic_and)
BSHMEM_DEV_CTX_AMO_VALUE(T, atomic_fetch_or)
BSHMEM_DEV_CTX_AMO_VALUE(void, atomic_or)
BSHMEM_DEV_CTX_AMO_VALUE(T, atomic_fetch_xor)
BSHMEM_DEV_CTX_AMO_VALUE(void, atomic_xor)
BSHMEM_DEV_CTX_AMO_NOVALUE(T, atomic_fetch_inc)
BSHMEM_DEV_CTX_AMO_NOVALUE(void, atomic_inc)
#undef BSHMEM_DEV_CTX_AMO_VALUE
#undef BSHMEM_DEV_CTX_AMO_NOVALUE
template <typename T> __device__ __forceinline__ T ctx_atomic_fetch(const State& s, const Ctx& c, const T* src, int pe) {
  return atomic_fetch(s, src, ctx_pe(c, pe));
}
template <typename T> __device__ __forceinline__ T ctx_atomic_compare_swap(const State& s, const Ctx& c, T* dest, T cond, T value, int pe) {
  return atomic_compare_swap(s, dest, cond, value, ctx_pe(c, pe));
}

}  // namespace dev
}  // namespace bshmem
#endif  // __CUDACC__
