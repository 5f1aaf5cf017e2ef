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
  unsigned long long base = 0;
  if (lane == leader) base = atomicAdd(ring->write_index, (unsigned long long)__popc(active));
  base = __shfl_sync(active, base, leader);
  const uint64_t ticket = base + rank;
  const uint64_t mask = ring->capacity - 1;
  // ---- back-pressure: wait until the consumer has freed this slot ----
  unsigned long long t0 = dev::timer();
  unsigned it = 0;
  while (ticket - ld_sys_u64(ring->read_index) >= ring->capacity) {
    if ((++it & 15) == 0) {
      if (dev::timer() - t0 > ring->timeout_ns) {
        dev::record_error(s, BSHMEM_ERR_TIMEOUT, cmd.pe, BSHMEM_WHERE_PROXY_SLOT, ticket, ticket - ring->capacity + 1, ld_sys_u64(ring->read_index));
        return BSHMEM_ERR_TIMEOUT;
      }
      __nanosleep(200);
    }
  }
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
__device__ __forceinline__ int putmem(const State& s, void* dest, const void* src, size_t n, int pe, bool nbi = false) {
  bshmem_proxy_desc_t d = make_cmd(nbi ? BSHMEM_PROXY_PUT_NBI : BSHMEM_PROXY_PUT, pe);
  d.sym_off = heap_off(s, dest);
  d.local = reinterpret_cast<uint64_t>(src);
  d.nbytes = n;
  d.flags = nbi ? 0 : BSHMEM_PROXY_FLAG_BLOCKING;
  return submit(s, d);
}
__device__ __forceinline__ int getmem(const State& s, void* dest, const void* src, size_t n, int pe) {
  bshmem_proxy_desc_t d = make_cmd(BSHMEM_PROXY_GET, pe);
  d.sym_off = heap_off(s, src);
  d.local = reinterpret_cast<uint64_t>(dest);
  d.nbytes = n;
  d.flags = BSHMEM_PROXY_FLAG_BLOCKING;
  return submit(s, d);
}
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
__device__ __forceinline__ int quiet(const State& s) {
  bshmem_proxy_desc_t d = make_cmd(BSHMEM_PROXY_QUIET, 0);
  d.flags = BSHMEM_PROXY_FLAG_BLOCKING;
  return submit(s, d);
}
__device__ __forceinline__ int fence(const State& s) {
  bshmem_proxy_desc_t d = make_cmd(BSHMEM_PROXY_FENCE, 0);
  d.flags = BSHMEM_PROXY_FLAG_BLOCKING;
  return submit(s, d);
}
__device__ __forceinline__ int barrier_all(const State& s) {
  bshmem_proxy_desc_t d = make_cmd(BSHMEM_PROXY_BARRIER_ALL, 0);
  d.flags = BSHMEM_PROXY_FLAG_BLOCKING;
  return submit(s, d);
}

}  // namespace proxy
}  // namespace bshmem
#endif
