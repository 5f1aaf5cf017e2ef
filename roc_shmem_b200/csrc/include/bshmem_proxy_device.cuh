// bshmem_proxy_device.cuh — device side of reverse offload: a kernel hands an operation
// to the PE's CPU service thread by writing a 128-byte descriptor into the pinned host ring.
//
// Slot reservation is warp-aggregated: the lowest active lane takes one ticket range for
// all active lanes of the warp with a single atomic on the device-resident ticket counter,
// every lane then owns ticket base + (its rank among the active lanes).  A lane waits —
// bounded — for the consumer to have moved past ticket - capacity, fills its slot with
// plain stores to mapped host memory, fences, and publishes ticket + 1 in the slot's `valid`
// word.  Blocking operations poll the slot's completion word, again bounded, and read the
// fetched value / status from the result word.
//
// Parity: library/src/reverse_offload/context_ro_device.cpp:407-517 (next_write_slot:
// wave-aggregated reservation under a spin lock; build_queue_element: fill, threadfence,
// valid flag, optional s_sleep wait on a per-thread status byte).  Here the ticket makes the
// lock unnecessary and completion is per slot, so any number of blocks can share one ring.
#pragma once
#include "bshmem_device.cuh"
#include "bshmem_proxy.h"

#ifdef __CUDACC__
namespace bshmem {
namespace proxy {

using dev::State;

__device__ __forceinline__ uint64_t ld_sys_u64(const volatile uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Submit one command.  `cmd` holds the command fields (op, pe, offsets, ...); ticket/valid are
// filled here.  Returns BSHMEM_OK, BSHMEM_ERR_TIMEOUT, BSHMEM_ERR_STATE (no proxy attached) or,
// for blocking non-fetching commands, the status the host reported.
__device__ __forceinline__ int submit(const State& s, bshmem_proxy_desc_t cmd, uint64_t* result = nullptr) {
  const bshmem_proxy_ring_t* ring = static_cast<const bshmem_proxy_ring_t*>(s.proxy);
  if (!ring) return BSHMEM_ERR_STATE;
  // ---- warp-aggregated ticket ----
  const unsigned active = __activemask();
  const int lane = threadIdx.x & 31;
  const int leader = __ffs(active) - 1;
  const int rank = __popc(active & ((1u << lane) - 1));
  // ---- back-pressure: tickets for the whole warp are only taken while the ring has room for them (the consumer
  // has moved past last ticket - capacity), so a warp that gives up has reserved nothing and leaves no hole ----
  const unsigned long long want = (unsigned long long)__popc(active);
  unsigned long long base = ~0ull;
  unsigned long long t0 = dev::timer();
  unsigned it = 0;
  if (lane == leader) {
    while (true) {
      const unsigned long long w = *reinterpret_cast<volatile unsigned long long*>(ring->write_index);
      if (w + want - ld_sys_u64(ring->read_index) <= ring->capacity) {
        if (atomicCAS(ring->write_index, w, w + want) == w) { base = w; break; }
        continue;
      }
      if ((++it & 15) == 0) {
        if (dev::timer() - t0 > ring->timeout_ns) {
          dev::record_error(s, BSHMEM_ERR_TIMEOUT, cmd.pe, BSHMEM_WHERE_PROXY_SLOT, w, w + want - ring->capacity, ld_sys_u64(ring->read_index));
          break;
        }
        __nanosleep(200);
      }
    }
  }
  base = __shfl_sync(active, base, leader);
  if (base == ~0ull) return BSHMEM_ERR_TIMEOUT;
  const uint64_t ticket = base + rank;
  const uint64_t mask = ring->capacity - 1;
  // ---- fill and publish ----
  bshmem_proxy_desc_t* slot = &ring->slots[ticket & mask];
  cmd.block_id = blockIdx.x;
  cmd.ticket = ticket;
  const uint64_t* src = reinterpret_cast<const uint64_t*>(&cmd);
  volatile uint64_t* dst = reinterpret_cast<volatile uint64_t*>(slot);
#pragma unroll
  for (int i = 0; i < 10; ++i) dst[i] = src[i];     // command fields + ticket (80 bytes)
  __threadfence_system();
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(&slot->valid), "l"(ticket + 1) : "memory");
  dev::stat(s, BSHMEM_DSTAT_PROXY_OPS);
  if (!(cmd.flags & BSHMEM_PROXY_FLAG_BLOCKING)) return BSHMEM_OK;
  // ---- bounded wait for the host ----
  t0 = dev::timer();
  it = 0;
  while (ld_sys_u64(&ring->completion[ticket & mask]) < ticket + 1) {   // >=: the slot may already serve a later ticket
    if ((++it & 15) == 0) {
      if (dev::timer() - t0 > ring->timeout_ns) {
        dev::record_error(s, BSHMEM_ERR_TIMEOUT, cmd.pe, BSHMEM_WHERE_PROXY_DONE, ticket, ticket + 1, ld_sys_u64(&ring->completion[ticket & mask]));
        return BSHMEM_ERR_TIMEOUT;
      }
      __nanosleep(500);
    }
  }
  uint64_t res = ring->result[ticket & mask];
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(&ring->consumed[ticket & mask]), "l"(ticket + 1) : "memory");
  const bool fetches = cmd.op == BSHMEM_PROXY_G || cmd.op == BSHMEM_PROXY_AMO;
  if (fetches) {
    if (result) *result = res;
    return BSHMEM_OK;
  }
  return (int)res;
}

__device__ __forceinline__ bshmem_proxy_desc_t make_cmd(uint32_t op, int pe) {
  bshmem_proxy_desc_t d;
  memset(&d, 0, sizeof(d));
  d.op = op;
  d.pe = pe;
  return d;
}
__device__ __forceinline__ uint64_t heap_off(const State& s, const void* sym) {
  return reinterpret_cast<const char*>(sym) - s.heap_base[s.my_pe];
}

// The OpenSHMEM-style calls, proxy flavour (every op is one descriptor).
__device__ __forceinline__ int p64(const State& s, uint64_t* dest, uint64_t value, int pe) {
  bshmem_proxy_desc_t d = make_cmd(BSHMEM_PROXY_P, pe);
  d.dtype = BSHMEM_UINT64;
  d.sym_off = heap_off(s, dest);
  d.value = value;
  return submit(s, d);
}
__device__ __forceinline__ uint64_t g64(const State& s, const uint64_t* src, int pe, int* status = nullptr) {
  bshmem_proxy_desc_t d = make_cmd(BSHMEM_PROXY_G, pe);
  d.dtype = BSHMEM_UINT64;
  d.sym_off = heap_off(s, src);
  d.flags = BSHMEM_PROXY_FLAG_BLOCKING;
  uint64_t r = 0;
  int rc = submit(s, d, &r);
  if (status) *status = rc;
  return r;
}
// All 15 atomic flavours go through one command (the reference's RO_NET_AMO_FOP).
__device__ __forceinline__ uint64_t amo64(const State& s, int amo_op, uint64_t* dest, uint64_t value, uint64_t cond, int pe,
                                          int* status = nullptr) {
  bshmem_proxy_desc_t d = make_cmd(BSHMEM_PROXY_AMO, pe);
  d.dtype = BSHMEM_UINT64;
  d.sub_op = amo_op;
  d.sym_off = heap_off(s, dest);
  d.value = value;
  d.cond = cond;
  d.flags = BSHMEM_PROXY_FLAG_BLOCKING;
  uint64_t r = 0;
  int rc = submit(s, d, &r);
  if (status) *status = rc;
  return r;
}
// ---- element type codes for the typed forms ------------------------------------------------------------
template <typename T> struct DtypeOf;
template <> struct DtypeOf<int> { static constexpr int value = BSHMEM_INT32; };
template <> struct DtypeOf<unsigned int> { static constexpr int value = BSHMEM_UINT32; };
template <> struct DtypeOf<long> { static constexpr int value = BSHMEM_INT64; };
template <> struct DtypeOf<unsigned long> { static constexpr int value = BSHMEM_UINT64; };
template <> struct DtypeOf<long long> { static constexpr int value = BSHMEM_INT64; };
template <> struct DtypeOf<unsigned long long> { static constexpr int value = BSHMEM_UINT64; };
template <> struct DtypeOf<float> { static constexpr int value = BSHMEM_FLOAT; };
template <> struct DtypeOf<double> { static constexpr int value = BSHMEM_DOUBLE; };
template <typename T> __device__ __forceinline__ uint64_t to_bits(T v) { uint64_t w = 0; memcpy(&w, &v, sizeof(T)); return w; }
template <typename T> __device__ __forceinline__ T from_bits(uint64_t w) { T v; memcpy(&v, &w, sizeof(T)); return v; }

// ---- scoped RMA: the scope's first thread submits one descriptor for the whole scope -----------------------
// (library/src/reverse_offload/context_ro_device.cpp:63-354: putmem / getmem x {thread, wg, wave} x {blocking, nbi}).
// The status comes back to the submitting thread; the other threads of the scope get BSHMEM_OK.
template <dev::Scope S = dev::THREAD>
__device__ __forceinline__ int putmem(const State& s, void* dest, const void* src, size_t n, int pe, bool nbi = false) {
  int rc = BSHMEM_OK;
  dev::scope_sync<S>();                    // every participant's writes to `src` precede the submission
  if (dev::scope_rank<S>() == 0) {
    bshmem_proxy_desc_t d = make_cmd(nbi ? BSHMEM_PROXY_PUT_NBI : BSHMEM_PROXY_PUT, pe);
    d.sym_off = heap_off(s, dest);
    d.local = reinterpret_cast<uint64_t>(src);
    d.nbytes = n;
    d.flags = nbi ? 0 : BSHMEM_PROXY_FLAG_BLOCKING;
    __threadfence_system();
    rc = submit(s, d);
  }
  dev::scope_sync<S>();
  return rc;
}
template <dev::Scope S = dev::THREAD>
__device__ __forceinline__ int putmem_nbi(const State& s, void* dest, const void* src, size_t n, int pe) { return putmem<S>(s, dest, src, n, pe, true); }
template <dev::Scope S = dev::THREAD>
__device__ __forceinline__ int getmem(const State& s, void* dest, const void* src, size_t n, int pe, bool nbi = false) {
  int rc = BSHMEM_OK;
  if (dev::scope_rank<S>() == 0) {
    bshmem_proxy_desc_t d = make_cmd(nbi ? BSHMEM_PROXY_GET_NBI : BSHMEM_PROXY_GET, pe);
    d.sym_off = heap_off(s, src);
    d.local = reinterpret_cast<uint64_t>(dest);
    d.nbytes = n;
    d.flags = nbi ? 0 : BSHMEM_PROXY_FLAG_BLOCKING;
    rc = submit(s, d);
  }
  dev::scope_sync<S>();
  return rc;
}
template <dev::Scope S = dev::THREAD>
__device__ __forceinline__ int getmem_nbi(const State& s, void* dest, const void* src, size_t n, int pe) { return getmem<S>(s, dest, src, n, pe, true); }
template <typename T, dev::Scope S = dev::THREAD>
__device__ __forceinline__ int put(const State& s, T* dest, const T* src, size_t nelems, int pe) { return putmem<S>(s, dest, src, nelems * sizeof(T), pe); }
template <typename T, dev::Scope S = dev::THREAD>
__device__ __forceinline__ int get(const State& s, T* dest, const T* src, size_t nelems, int pe) { return getmem<S>(s, dest, src, nelems * sizeof(T), pe); }
template <dev::Scope S = dev::THREAD>
__device__ __forceinline__ int putmem_signal(const State& s, void* dest, const void* src, size_t n, uint64_t* sig_addr, uint64_t signal,
                                             int sig_op, int pe) {
  int rc = BSHMEM_OK;
  dev::scope_sync<S>();
  if (dev::scope_rank<S>() == 0) {
    bshmem_proxy_desc_t d = make_cmd(BSHMEM_PROXY_PUT_SIGNAL, pe);
    d.sym_off = heap_off(s, dest);
    d.local = reinterpret_cast<uint64_t>(src);
    d.nbytes = n;
    d.value = signal;
    d.cond = heap_off(s, sig_addr);
    d.sub_op = sig_op;
    d.flags = BSHMEM_PROXY_FLAG_BLOCKING;
    __threadfence_system();
    rc = submit(s, d);
  }
  dev::scope_sync<S>();
  return rc;
}

// ---- typed p / g / atomics for 4- and 8-byte types (context_ro_tmpl_device.hpp:206-301: 13 typed AMOs, p, g) ----
template <typename T> __device__ __forceinline__ int p(const State& s, T* dest, T value, int pe) {
  static_assert(sizeof(T) == 4 || sizeof(T) == 8, "proxy p: 4- and 8-byte types");
  bshmem_proxy_desc_t d = make_cmd(BSHMEM_PROXY_P, pe);
  d.dtype = DtypeOf<T>::value;
  d.sym_off = heap_off(s, dest);
  d.value = to_bits(value);
  return submit(s, d);
}
template <typename T> __device__ __forceinline__ T g(const State& s, const T* src, int pe, int* status = nullptr) {
  static_assert(sizeof(T) == 4 || sizeof(T) == 8, "proxy g: 4- and 8-byte types");
  bshmem_proxy_desc_t d = make_cmd(BSHMEM_PROXY_G, pe);
  d.dtype = DtypeOf<T>::value;
  d.sym_off = heap_off(s, src);
  d.flags = BSHMEM_PROXY_FLAG_BLOCKING;
  uint64_t r = 0;
  int rc = submit(s, d, &r);
  if (status) *status = rc;
  return from_bits<T>(r);
}
template <typename T> __device__ __forceinline__ T amo(const State& s, int amo_op, T* dest, T value, T cond, int pe, int* status = nullptr) {
  static_assert(sizeof(T) == 4 || sizeof(T) == 8, "proxy atomics: 4- and 8-byte types");
  bshmem_proxy_desc_t d = make_cmd(BSHMEM_PROXY_AMO, pe);
  d.dtype = DtypeOf<T>::value;
  d.sub_op = amo_op;
  d.sym_off = heap_off(s, dest);
  d.value = to_bits(value);
  d.cond = to_bits(cond);
  d.flags = BSHMEM_PROXY_FLAG_BLOCKING;
  uint64_t r = 0;
  int rc = submit(s, d, &r);
  if (status) *status = rc;
  return from_bits<T>(r);
}
template <typename T> __device__ __forceinline__ T atomic_fetch_add(const State& s, T* d, T v, int pe) { return amo<T>(s, BSHMEM_AMO_FETCH_ADD, d, v, T(), pe); }
template <typename T> __device__ __forceinline__ void atomic_add(const State& s, T* d, T v, int pe) { (void)amo<T>(s, BSHMEM_AMO_ADD, d, v, T(), pe); }
template <typename T> __device__ __forceinline__ T atomic_fetch_inc(const State& s, T* d, int pe) { return amo<T>(s, BSHMEM_AMO_FETCH_INC, d, T(), T(), pe); }
template <typename T> __device__ __forceinline__ void atomic_inc(const State& s, T* d, int pe) { (void)amo<T>(s, BSHMEM_AMO_INC, d, T(), T(), pe); }
template <typename T> __device__ __forceinline__ T atomic_fetch(const State& s, const T* d, int pe) { return amo<T>(s, BSHMEM_AMO_FETCH, const_cast<T*>(d), T(), T(), pe); }
template <typename T> __device__ __forceinline__ T atomic_compare_swap(const State& s, T* d, T cond, T v, int pe) { return amo<T>(s, BSHMEM_AMO_FETCH_CSWAP, d, v, cond, pe); }
template <typename T> __device__ __forceinline__ T atomic_swap(const State& s, T* d, T v, int pe) { return amo<T>(s, BSHMEM_AMO_SWAP, d, v, T(), pe); }
template <typename T> __device__ __forceinline__ void atomic_set(const State& s, T* d, T v, int pe) { (void)amo<T>(s, BSHMEM_AMO_SET, d, v, T(), pe); }
template <typename T> __device__ __forceinline__ T atomic_fetch_and(const State& s, T* d, T v, int pe) { return amo<T>(s, BSHMEM_AMO_FETCH_AND, d, v, T(), pe); }
template <typename T> __device__ __forceinline__ void atomic_and(const State& s, T* d, T v, int pe) { (void)amo<T>(s, BSHMEM_AMO_AND, d, v, T(), pe); }
template <typename T> __device__ __forceinline__ T atomic_fetch_or(const State& s, T* d, T v, int pe) { return amo<T>(s, BSHMEM_AMO_FETCH_OR, d, v, T(), pe); }
template <typename T> __device__ __forceinline__ void atomic_or(const State& s, T* d, T v, int pe) { (void)amo<T>(s, BSHMEM_AMO_OR, d, v, T(), pe); }
template <typename T> __device__ __forceinline__ T atomic_fetch_xor(const State& s, T* d, T v, int pe) { return amo<T>(s, BSHMEM_AMO_FETCH_XOR, d, v, T(), pe); }
template <typename T> __device__ __forceinline__ void atomic_xor(const State& s, T* d, T v, int pe) { (void)amo<T>(s, BSHMEM_AMO_XOR, d, v, T(), pe); }

// ---- ordering ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int simple(const State& s, uint32_t op, int team = 0) {
  bshmem_proxy_desc_t d = make_cmd(op, 0);
  d.team = team;
  d.flags = BSHMEM_PROXY_FLAG_BLOCKING;
  return submit(s, d);
}
__device__ __forceinline__ int quiet(const State& s) { return simple(s, BSHMEM_PROXY_QUIET); }
__device__ __forceinline__ int fence(const State& s) { return simple(s, BSHMEM_PROXY_FENCE); }
__device__ __forceinline__ int fence_pe(const State& s, int) { return simple(s, BSHMEM_PROXY_FENCE); }

// ---- work-group collectives: every thread of the block calls, thread 0 submits one descriptor, all get its status
// (context_ro_device.cpp barrier_all / sync_all / sync(team); context_ro_tmpl_device.hpp:112-375 to_all, broadcast,
// alltoall, fcollect).  `team` is the team's slot on this PE; dest and source are symmetric.
__device__ __forceinline__ int wg_submit(const State& s, bshmem_proxy_desc_t d) {
  __shared__ int wg_rc;
  __syncthreads();                         // the block's earlier stores precede the submission
  if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
    d.flags |= BSHMEM_PROXY_FLAG_BLOCKING;
    __threadfence_system();
    wg_rc = submit(s, d);
  }
  __syncthreads();
  const int rc = wg_rc;
  __syncthreads();
  return rc;
}
__device__ __forceinline__ int barrier_all(const State& s) { return simple(s, BSHMEM_PROXY_BARRIER_ALL); }     // single thread
__device__ __forceinline__ int wg_barrier_all(const State& s) { return wg_submit(s, make_cmd(BSHMEM_PROXY_BARRIER_ALL, 0)); }
__device__ __forceinline__ int wg_sync_all(const State& s) { return wg_submit(s, make_cmd(BSHMEM_PROXY_SYNC_ALL, 0)); }
__device__ __forceinline__ int wg_team_sync(const State& s, int team) {
  bshmem_proxy_desc_t d = make_cmd(BSHMEM_PROXY_TEAM_SYNC, 0);
  d.team = team;
  return wg_submit(s, d);
}
__device__ __forceinline__ bshmem_proxy_desc_t coll_cmd(const State& s, uint32_t op, int team, void* dest, const void* source, uint64_t count) {
  bshmem_proxy_desc_t d = make_cmd(op, 0);
  d.team = team;
  d.sym_off = heap_off(s, dest);
  d.local = heap_off(s, source);
  d.flags = BSHMEM_PROXY_FLAG_SRC_IS_OFFSET;
  d.nbytes = count;
  return d;
}
template <typename T> __device__ __forceinline__ int wg_to_all(const State& s, int team, int op, T* dest, const T* source, size_t n) {
  bshmem_proxy_desc_t d = coll_cmd(s, BSHMEM_PROXY_TO_ALL, team, dest, source, n);
  d.dtype = DtypeOf<T>::value;
  d.sub_op = op;
  return wg_submit(s, d);
}
template <typename T> __device__ __forceinline__ int wg_broadcast(const State& s, int team, T* dest, const T* source, size_t n, int root) {
  bshmem_proxy_desc_t d = coll_cmd(s, BSHMEM_PROXY_BROADCAST, team, dest, source, n * sizeof(T));
  d.root = root;
  return wg_submit(s, d);
}
template <typename T> __device__ __forceinline__ int wg_alltoall(const State& s, int team, T* dest, const T* source, size_t n) {
  return wg_submit(s, coll_cmd(s, BSHMEM_PROXY_ALLTOALL, team, dest, source, n * sizeof(T)));
}
template <typename T> __device__ __forceinline__ int wg_fcollect(const State& s, int team, T* dest, const T* source, size_t n) {
  return wg_submit(s, coll_cmd(s, BSHMEM_PROXY_FCOLLECT, team, dest, source, n * sizeof(T)));
}

// ---- context forms: PEs relative to the context's team, collectives on the context's team ---------------------
// (the descriptor carries world PE numbers; the translation happens here, on the device)
template <dev::Scope S = dev::THREAD>
__device__ __forceinline__ int ctx_putmem(const State& s, const dev::Ctx& c, void* dest, const void* src, size_t n, int pe) { return putmem<S>(s, dest, src, n, dev::ctx_pe(c, pe)); }
template <dev::Scope S = dev::THREAD>
__device__ __forceinline__ int ctx_putmem_nbi(const State& s, const dev::Ctx& c, void* dest, const void* src, size_t n, int pe) { return putmem<S>(s, dest, src, n, dev::ctx_pe(c, pe), true); }
template <dev::Scope S = dev::THREAD>
__device__ __forceinline__ int ctx_getmem(const State& s, const dev::Ctx& c, void* dest, const void* src, size_t n, int pe) { return getmem<S>(s, dest, src, n, dev::ctx_pe(c, pe)); }
template <dev::Scope S = dev::THREAD>
__device__ __forceinline__ int ctx_getmem_nbi(const State& s, const dev::Ctx& c, void* dest, const void* src, size_t n, int pe) { return getmem<S>(s, dest, src, n, dev::ctx_pe(c, pe), true); }
template <dev::Scope S = dev::THREAD>
__device__ __forceinline__ int ctx_putmem_signal(const State& s, const dev::Ctx& c, void* dest, const void* src, size_t n, uint64_t* sig,
                                                 uint64_t v, int op, int pe) { return putmem_signal<S>(s, dest, src, n, sig, v, op, dev::ctx_pe(c, pe)); }
template <typename T> __device__ __forceinline__ int ctx_p(const State& s, const dev::Ctx& c, T* dest, T value, int pe) { return p<T>(s, dest, value, dev::ctx_pe(c, pe)); }
template <typename T> __device__ __forceinline__ T ctx_g(const State& s, const dev::Ctx& c, const T* src, int pe) { return g<T>(s, src, dev::ctx_pe(c, pe)); }
template <typename T> __device__ __forceinline__ T ctx_amo(const State& s, const dev::Ctx& c, int amo_op, T* dest, T value, T cond, int pe) {
  return amo<T>(s, amo_op, dest, value, cond, dev::ctx_pe(c, pe));
}
#define BSHMEM_PROXY_CTX_AMO_VALUE(RET, NAME)                                                                           \
  template <typename T> __device__ __forceinline__ RET ctx_##NAME(const State& s, const dev::Ctx& c, T* dest, T value, int pe) { \
    return NAME<T>(s, dest, value, dev::ctx_pe(c, pe));                                                                     \
  }
#define BSHMEM_PROXY_CTX_AMO_NOVALUE(RET, NAME)                                                                         \
  template <typename T> __device__ __forceinline__ RET ctx_##NAME(const State& s, const dev::Ctx& c, T* dest, int pe) {   \
    return NAME<T>(s, dest, dev::ctx_pe(c, pe));                                                                            \
  }
BSHMEM_PROXY_CTX_AMO_VALUE(T, atomic_fetch_add)
BSHMEM_PROXY_CTX_AMO_VALUE(void, atomic_add)
BSHMEM_PROXY_CTX_AMO_VALUE(T, atomic_swap)
BSHMEM_PROXY_CTX_AMO_VALUE(void, atomic_set)
BSHMEM_PROXY_CTX_AMO_VALUE(T, atomic_fetch_and)
BSHMEM_PROXY_CTX_AMO_VALUE(void, atomic_and)
BSHMEM_PROXY_CTX_AMO_VALUE(T, atomic_fetch_or)
BSHMEM_PROXY_CTX_AMO_VALUE(void, atomic_or)
BSHMEM_PROXY_CTX_AMO_VALUE(T, atomic_fetch_xor)
BSHMEM_PROXY_CTX_AMO_VALUE(void, atomic_xor)
BSHMEM_PROXY_CTX_AMO_NOVALUE(T, atomic_fetch_inc)
BSHMEM_PROXY_CTX_AMO_NOVALUE(void, atomic_inc)
#undef BSHMEM_PROXY_CTX_AMO_VALUE
#undef BSHMEM_PROXY_CTX_AMO_NOVALUE
template <typename T> __device__ __forceinline__ T ctx_atomic_fetch(const State& s, const dev::Ctx& c, const T* src, int pe) {
  return atomic_fetch<T>(s, src, dev::ctx_pe(c, pe));
}
template <typename T> __device__ __forceinline__ T ctx_atomic_compare_swap(const State& s, const dev::Ctx& c, T* dest, T cond, T value, int pe) {
  return atomic_compare_swap<T>(s, dest, cond, value, dev::ctx_pe(c, pe));
}
__device__ __forceinline__ int ctx_wg_barrier_all(const State& s, const dev::Ctx&) { return wg_barrier_all(s); }
__device__ __forceinline__ int ctx_wg_sync_all(const State& s, const dev::Ctx&) { return wg_sync_all(s); }
__device__ __forceinline__ int ctx_quiet(const State& s, const dev::Ctx&) { return quiet(s); }
__device__ __forceinline__ int ctx_fence(const State& s, const dev::Ctx&) { return fence(s); }
__device__ __forceinline__ int ctx_wg_team_sync(const State& s, const dev::Ctx& c) { return wg_team_sync(s, c.team.slot); }
template <typename T> __device__ __forceinline__ int ctx_wg_to_all(const State& s, const dev::Ctx& c, int op, T* dest, const T* src, size_t n) {
  return wg_to_all<T>(s, c.team.slot, op, dest, src, n);
}
template <typename T> __device__ __forceinline__ int ctx_wg_broadcast(const State& s, const dev::Ctx& c, T* dest, const T* src, size_t n, int root) {
  return wg_broadcast<T>(s, c.team.slot, dest, src, n, root);
}
template <typename T> __device__ __forceinline__ int ctx_wg_alltoall(const State& s, const dev::Ctx& c, T* dest, const T* src, size_t n) {
  return wg_alltoall<T>(s, c.team.slot, dest, src, n);
}
template <typename T> __device__ __forceinline__ int ctx_wg_fcollect(const State& s, const dev::Ctx& c, T* dest, const T* src, size_t n) {
  return wg_fcollect<T>(s, c.team.slot, dest, src, n);
}

}  // namespace proxy
}  // namespace bshmem
#endif
