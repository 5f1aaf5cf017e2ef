// proxy.cc — reverse-offload service thread, host producer and the executor that
// runs commands through the runtime's backend.  See proxy.h / bshmem_proxy.h.
#include "proxy.h"

#include <sched.h>
#include <time.h>

#include <cstdlib>
#include <cstring>
#include <vector>

#include "runtime.h"

namespace bshmem {

namespace {
inline uint64_t now_ns() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + ts.tv_nsec;
}
inline void backoff(unsigned spins) {
  if (spins < 256) {
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
  } else if (spins < 4096) {
    sched_yield();
  } else {
    timespec ts{0, 20000};
    nanosleep(&ts, nullptr);
  }
}
}  // namespace

int RuntimeExecutor::execute(const bshmem_proxy_desc_t& d, uint64_t* result) {
  bshmem_handle_t h = h_;
  char* base = static_cast<char*>(bshmem_heap_base(h));
  void* sym = base + d.sym_off;
  void* local = (d.flags & BSHMEM_PROXY_FLAG_SRC_IS_OFFSET) ? static_cast<void*>(base + d.local)
                                                            : reinterpret_cast<void*>(d.local);
  switch (d.op) {
    case BSHMEM_PROXY_NOP: return BSHMEM_OK;
    case BSHMEM_PROXY_PUT: return bshmem_ctx_putmem(h, 0, sym, local, d.nbytes, d.pe);
    case BSHMEM_PROXY_PUT_NBI: return bshmem_ctx_putmem_nbi(h, 0, sym, local, d.nbytes, d.pe);
    case BSHMEM_PROXY_GET: return bshmem_ctx_getmem(h, 0, local, sym, d.nbytes, d.pe);
    case BSHMEM_PROXY_GET_NBI: return bshmem_ctx_getmem_nbi(h, 0, local, sym, d.nbytes, d.pe);
    case BSHMEM_PROXY_P: {
      uint64_t v = d.value;
      return bshmem_ctx_putmem_nbi(h, 0, sym, &v, bshmem_dtype_size(d.dtype), d.pe);
    }
    case BSHMEM_PROXY_G: {
      uint64_t v = 0;
      int rc = bshmem_ctx_getmem(h, 0, &v, sym, bshmem_dtype_size(d.dtype), d.pe);
      if (result) *result = v;
      return rc;
    }
    case BSHMEM_PROXY_AMO: return bshmem_ctx_amo(h, 0, d.dtype, d.sub_op, sym, d.value, d.cond, d.pe, result);
    case BSHMEM_PROXY_PUT_SIGNAL:
      return bshmem_ctx_putmem_signal(h, 0, sym, local, d.nbytes, reinterpret_cast<uint64_t*>(base + d.cond), d.value,
                                      d.sub_op, d.pe);
    case BSHMEM_PROXY_FENCE: return bshmem_ctx_fence(h, 0);
    case BSHMEM_PROXY_QUIET: return bshmem_ctx_quiet(h, 0);
    case BSHMEM_PROXY_BARRIER_ALL: return bshmem_barrier_all(h);
    case BSHMEM_PROXY_SYNC_ALL: return bshmem_sync_all(h);
    case BSHMEM_PROXY_TEAM_SYNC: return bshmem_team_sync(h, d.team);
    case BSHMEM_PROXY_TO_ALL: return bshmem_team_reduce(h, d.team, d.dtype, d.sub_op, sym, local, d.nbytes);
    case BSHMEM_PROXY_BROADCAST: return bshmem_team_broadcast(h, d.team, sym, local, d.nbytes, d.root);
    case BSHMEM_PROXY_ALLTOALL: return bshmem_team_alltoall(h, d.team, sym, local, d.nbytes);
    case BSHMEM_PROXY_FCOLLECT: return bshmem_team_fcollect(h, d.team, sym, local, d.nbytes);
    case BSHMEM_PROXY_FINALIZE: return BSHMEM_OK;
    default: return BSHMEM_ERR_INVALID;
  }
}

uint64_t proxy_ring_bytes(uint64_t capacity) {
  // slots | completion | result | consumed | read_index (own cache line)
  return capacity * sizeof(bshmem_proxy_desc_t) + capacity * 8 * 3 + 128;
}

bshmem_proxy* proxy_start(void* block, uint64_t capacity, unsigned long long* write_index, unsigned long long timeout_ns,
                          std::unique_ptr<ProxyExecutor> exec) {
  static_assert(sizeof(bshmem_proxy_desc_t) == 128, "descriptor must be 128 bytes");
  if (!block || capacity < 2 || (capacity & (capacity - 1))) return nullptr;
  bshmem_proxy* px = new bshmem_proxy();
  char* p = static_cast<char*>(block);
  px->ring.capacity = capacity;
  px->ring.slots = reinterpret_cast<bshmem_proxy_desc_t*>(p);
  p += capacity * sizeof(bshmem_proxy_desc_t);
  px->ring.completion = reinterpret_cast<volatile uint64_t*>(p);
  p += capacity * 8;
  px->ring.result = reinterpret_cast<volatile uint64_t*>(p);
  p += capacity * 8;
  px->ring.consumed = reinterpret_cast<volatile uint64_t*>(p);
  p += capacity * 8;
  px->ring.read_index = reinterpret_cast<volatile uint64_t*>(p);
  px->ring.write_index = write_index ? write_index : reinterpret_cast<unsigned long long*>(&px->host_write_index);
  px->ring.timeout_ns = timeout_ns;
  px->exec = std::move(exec);
  px->worker = std::thread([px] { px->run(); });
  return px;
}

}  // namespace bshmem

using namespace bshmem;

void bshmem_proxy::run() {
  exec->thread_init();
  uint64_t read = 0;
  const uint64_t mask = ring.capacity - 1;
  unsigned idle = 0;
  std::vector<uint8_t> lap_blocking(ring.capacity, 0);
  while (!stop.load(std::memory_order_acquire)) {
    if (paused.load(std::memory_order_acquire)) {
      timespec ts{0, 50000};
      nanosleep(&ts, nullptr);
      continue;
    }
    bshmem_proxy_desc_t* slot = &ring.slots[read & mask];
    uint64_t v = __atomic_load_n(&slot->valid, __ATOMIC_ACQUIRE);
    if (v != read + 1) {
      counters[PX_IDLE_POLLS].fetch_add(1, std::memory_order_relaxed);
      backoff(idle++);
      continue;
    }
    idle = 0;
    bshmem_proxy_desc_t cmd;
    memcpy(&cmd, slot, sizeof(cmd));
    // The blocking producer that owned this slot one lap ago must have read its result before it is overwritten
    // (bounded: a producer whose own wait ran out never acknowledges).
    if (read >= ring.capacity && lap_blocking[read & mask]) {
      const uint64_t want = read - ring.capacity + 1;
      const uint64_t deadline = now_ns() + ring.timeout_ns;
      for (unsigned spins = 0; __atomic_load_n(&ring.consumed[read & mask], __ATOMIC_ACQUIRE) < want; ++spins) {
        if ((spins & 255) == 255 && now_ns() > deadline) break;
        backoff(spins);
      }
    }
    lap_blocking[read & mask] = (cmd.flags & BSHMEM_PROXY_FLAG_BLOCKING) != 0;
    int to_drop = drop.load(std::memory_order_acquire);
    if (to_drop > 0 && drop.compare_exchange_strong(to_drop, to_drop - 1)) {
      // injected fault: the command vanishes (neither executed nor completed)
      counters[PX_DROPPED].fetch_add(1, std::memory_order_relaxed);
    } else {
      uint64_t res = 0;
      int rc = exec->execute(cmd, &res);
      if (rc != BSHMEM_OK) counters[PX_ERRORS].fetch_add(1, std::memory_order_relaxed);
      switch (cmd.op) {
        case BSHMEM_PROXY_AMO: counters[PX_AMO].fetch_add(1, std::memory_order_relaxed); break;
        case BSHMEM_PROXY_FENCE: case BSHMEM_PROXY_QUIET: counters[PX_ORDER].fetch_add(1, std::memory_order_relaxed); break;
        case BSHMEM_PROXY_BARRIER_ALL: case BSHMEM_PROXY_SYNC_ALL: case BSHMEM_PROXY_TEAM_SYNC: case BSHMEM_PROXY_TO_ALL:
        case BSHMEM_PROXY_BROADCAST: case BSHMEM_PROXY_ALLTOALL: case BSHMEM_PROXY_FCOLLECT:
          counters[PX_COLL].fetch_add(1, std::memory_order_relaxed); break;
        default: counters[PX_RMA].fetch_add(1, std::memory_order_relaxed); break;
      }
      // result word: the fetched value for G / AMO, otherwise the status of the operation
      bool fetches = cmd.op == BSHMEM_PROXY_G || cmd.op == BSHMEM_PROXY_AMO;
      ring.result[read & mask] = (fetches && rc == BSHMEM_OK) ? res : (uint64_t)rc;
      __atomic_store_n(&ring.completion[read & mask], read + 1, __ATOMIC_RELEASE);
      counters[PX_PROCESSED].fetch_add(1, std::memory_order_relaxed);
    }
    ++read;
    __atomic_store_n(ring.read_index, read, __ATOMIC_RELEASE);
    if (cmd.op == BSHMEM_PROXY_FINALIZE) break;
  }
}

extern "C" {

int bshmem_proxy_create_host(bshmem_handle_t h, uint64_t capacity, uint64_t timeout_us, bshmem_proxy_t** out) {
  if (!h || !out || capacity < 2 || (capacity & (capacity - 1))) return BSHMEM_ERR_INVALID;
  uint64_t bytes = proxy_ring_bytes(capacity);
  void* block = nullptr;
  if (posix_memalign(&block, 128, bytes) != 0) return BSHMEM_ERR_NOMEM;
  memset(block, 0, bytes);
  bshmem_proxy* px = proxy_start(block, capacity, nullptr, timeout_us * 1000ull,
                                 std::unique_ptr<ProxyExecutor>(new RuntimeExecutor(h)));
  if (!px) { free(block); return BSHMEM_ERR_INVALID; }
  px->ring_mem = block;
  px->free_ring = [](bshmem_proxy* p) { free(p->ring_mem); };
  *out = px;
  return BSHMEM_OK;
}

int bshmem_proxy_host_submit(bshmem_proxy_t* px, const bshmem_proxy_desc_t* cmd, uint64_t* result) {
  if (!px || !cmd) return BSHMEM_ERR_INVALID;
  bshmem_proxy_ring_t& r = px->ring;
  const uint64_t mask = r.capacity - 1;
  uint64_t deadline = now_ns() + r.timeout_ns;
  // A ticket is only taken while the ring has room for it (the consumer moved past ticket - capacity): a producer
  // that gives up on a full ring has reserved nothing, so the consumer never waits for a slot nobody will fill.
  uint64_t ticket;
  for (unsigned spins = 0;; ++spins) {
    ticket = __atomic_load_n(r.write_index, __ATOMIC_ACQUIRE);
    if (ticket - __atomic_load_n(r.read_index, __ATOMIC_ACQUIRE) < r.capacity) {
      unsigned long long expect = ticket;
      if (__atomic_compare_exchange_n(r.write_index, &expect, ticket + 1, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE)) break;
      continue;
    }
    if ((spins & 255) == 255 && now_ns() > deadline) return BSHMEM_ERR_TIMEOUT;
    backoff(spins);
  }
  bshmem_proxy_desc_t* slot = &r.slots[ticket & mask];
  memcpy(slot, cmd, offsetof(bshmem_proxy_desc_t, ticket));
  slot->ticket = ticket;
  __atomic_store_n(&slot->valid, ticket + 1, __ATOMIC_RELEASE);
  if (!(cmd->flags & BSHMEM_PROXY_FLAG_BLOCKING)) return BSHMEM_OK;
  for (unsigned spins = 0; __atomic_load_n(&r.completion[ticket & mask], __ATOMIC_ACQUIRE) < ticket + 1; ++spins) {
    if ((spins & 255) == 255 && now_ns() > deadline) return BSHMEM_ERR_TIMEOUT;
    backoff(spins);
  }
  uint64_t res = r.result[ticket & mask];
  __atomic_store_n(&r.consumed[ticket & mask], ticket + 1, __ATOMIC_RELEASE);   // the slot's result may be overwritten now
  bool fetches = cmd->op == BSHMEM_PROXY_G || cmd->op == BSHMEM_PROXY_AMO;
  if (fetches) {
    if (result) *result = res;
    return BSHMEM_OK;
  }
  return (int)res;
}

int bshmem_proxy_pause(bshmem_proxy_t* px, int paused) {
  if (!px) return BSHMEM_ERR_INVALID;
  px->paused.store(paused != 0, std::memory_order_release);
  return BSHMEM_OK;
}

int bshmem_proxy_drop_next(bshmem_proxy_t* px, int n) {
  if (!px || n < 0) return BSHMEM_ERR_INVALID;
  px->drop.store(n, std::memory_order_release);
  return BSHMEM_OK;
}

int bshmem_proxy_get_counters(bshmem_proxy_t* px, uint64_t out[8]) {
  if (!px || !out) return BSHMEM_ERR_INVALID;
  for (int i = 0; i < PX_COUNT; ++i) out[i] = px->counters[i].load(std::memory_order_relaxed);
  return BSHMEM_OK;
}

int bshmem_proxy_get_ring(bshmem_proxy_t* px, bshmem_proxy_ring_t* out) {
  if (!px || !out) return BSHMEM_ERR_INVALID;
  *out = px->ring;
  return BSHMEM_OK;
}

int bshmem_proxy_set_timeout_us(bshmem_proxy_t* px, uint64_t timeout_us) {
  if (!px || timeout_us == 0) return BSHMEM_ERR_INVALID;
  px->ring.timeout_ns = timeout_us * 1000ull;
  return BSHMEM_OK;
}

int bshmem_proxy_stop(bshmem_proxy_t* px) {
  if (!px) return BSHMEM_ERR_INVALID;
  px->stop.store(true, std::memory_order_release);
  px->paused.store(false, std::memory_order_release);
  if (px->worker.joinable()) px->worker.join();
  if (px->free_ring) px->free_ring(px);
  delete px;
  return BSHMEM_OK;
}

}  // extern "C"
