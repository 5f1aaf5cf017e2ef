// cpu_backend.cc — PEs as threads or processes over one shared mapping.
//
// Layout of the mapping:  [control block, 1 MiB][heap PE0][heap PE1]...
// RMA is memcpy on the peer's heap, atomics are __atomic builtins, barriers are
// all-to-all epoch flags in each PE's control area (the same scheme the NVLink
// kernels use), and collectives read the peers' sources in place between two
// barriers.  Every wait is bounded and also watches the job-wide abort flag and
// the per-PE "dead" marks, so a test can inject failures from the host.
//
// This backend is the oracle the GPU paths are compared with, and the fake the
// reference's test-suite lacks (it can only test on real multi-process jobs,
// clients/functional_tests/tester.cpp:494-564).  Semantics follow
// library/src/host/host.cpp and host_templates.hpp (host RMA / AMO / to_all).
#include <fcntl.h>
#include <sched.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "backend.h"
#include "runtime.h"

namespace bshmem {
namespace {

constexpr uint64_t kMagic = 0x62736d656d435055ull;   // "bsmemCPU"
constexpr uint64_t kControlBytes = 1ull << 20;

struct alignas(64) PeArea {
  std::atomic<uint64_t> flags[BSHMEM_MAX_TEAMS][BSHMEM_MAX_PES];
  uint64_t xchg[BSHMEM_MAX_TEAMS][BSHMEM_MAX_PES];
  std::atomic<uint32_t> dead;
  std::atomic<uint32_t> attached;
};

struct Control {
  uint64_t magic;
  uint64_t n_pes;
  uint64_t heap_bytes;     // per PE, page rounded
  std::atomic<uint32_t> aborted;
  std::atomic<int32_t> abort_status;
  PeArea pe[BSHMEM_MAX_PES];
};
static_assert(sizeof(Control) <= kControlBytes, "control block too large");

struct CpuWorld {
  std::string name;
  bool owner = false;
  size_t map_bytes = 0;
  char* map = nullptr;
  Control* ctl() const { return reinterpret_cast<Control*>(map); }
  char* heap(int pe) const { return map + kControlBytes + (uint64_t)pe * ctl()->heap_bytes; }
};

inline uint64_t now_us() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000ull + ts.tv_nsec / 1000;
}

inline void relax(unsigned spins) {
  if (spins < 64) {
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
  } else if (spins < 4096) {
    sched_yield();
  } else {
    timespec ts{0, 50000};
    nanosleep(&ts, nullptr);
  }
}

// ---- bf16 / fp16 <-> float -------------------------------------------------
inline float bf16_to_f(uint16_t v) { uint32_t u = (uint32_t)v << 16; float f; memcpy(&f, &u, 4); return f; }
inline uint16_t f_to_bf16(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);   // quiet NaN
  u += 0x7fffu + ((u >> 16) & 1);   // round to nearest even
  return (uint16_t)(u >> 16);
}
inline float fp16_to_f(uint16_t v) { _Float16 h; memcpy(&h, &v, 2); return (float)h; }
inline uint16_t f_to_fp16(float f) { _Float16 h = (_Float16)f; uint16_t v; memcpy(&v, &h, 2); return v; }

template <typename T> inline T apply_op(int op, T a, T b) {
  switch (op) {
    case BSHMEM_SUM: return (T)(a + b);
    case BSHMEM_MIN: return b < a ? b : a;
    case BSHMEM_MAX: return b > a ? b : a;
    case BSHMEM_PROD: return (T)(a * b);
    default: return a;
  }
}
template <typename T> inline T apply_bitop(int op, T a, T b) {
  switch (op) {
    case BSHMEM_AND: return (T)(a & b);
    case BSHMEM_OR: return (T)(a | b);
    case BSHMEM_XOR: return (T)(a ^ b);
    default: return apply_op<T>(op, a, b);
  }
}

// out[i] = reduce over srcs[k][i] in set order (k = 0..n-1): deterministic.
template <typename T, bool kInt>
void reduce_typed(int op, T* out, const std::vector<const char*>& srcs, uint64_t nelems) {
  const T* s0 = reinterpret_cast<const T*>(srcs[0]);
  for (uint64_t i = 0; i < nelems; ++i) {
    T acc = s0[i];
    for (size_t k = 1; k < srcs.size(); ++k) {
      T v = reinterpret_cast<const T*>(srcs[k])[i];
      if constexpr (kInt) acc = apply_bitop<T>(op, acc, v); else acc = apply_op<T>(op, acc, v);
    }
    out[i] = acc;
  }
}

// 16-bit floats accumulate in fp32 and round once, like the device kernels.
template <float (*LOAD)(uint16_t), uint16_t (*STORE)(float)>
void reduce_half(int op, uint16_t* out, const std::vector<const char*>& srcs, uint64_t nelems) {
  for (uint64_t i = 0; i < nelems; ++i) {
    float acc = LOAD(reinterpret_cast<const uint16_t*>(srcs[0])[i]);
    for (size_t k = 1; k < srcs.size(); ++k) acc = apply_op<float>(op, acc, LOAD(reinterpret_cast<const uint16_t*>(srcs[k])[i]));
    out[i] = STORE(acc);
  }
}

void reduce_any(int dtype, int op, void* out, const std::vector<const char*>& srcs, uint64_t n) {
  switch (dtype) {
    case BSHMEM_INT8: reduce_typed<int8_t, true>(op, (int8_t*)out, srcs, n); break;
    case BSHMEM_UINT8: reduce_typed<uint8_t, true>(op, (uint8_t*)out, srcs, n); break;
    case BSHMEM_INT16: reduce_typed<int16_t, true>(op, (int16_t*)out, srcs, n); break;
    case BSHMEM_UINT16: reduce_typed<uint16_t, true>(op, (uint16_t*)out, srcs, n); break;
    case BSHMEM_INT32: reduce_typed<int32_t, true>(op, (int32_t*)out, srcs, n); break;
    case BSHMEM_UINT32: reduce_typed<uint32_t, true>(op, (uint32_t*)out, srcs, n); break;
    case BSHMEM_INT64: reduce_typed<int64_t, true>(op, (int64_t*)out, srcs, n); break;
    case BSHMEM_UINT64: reduce_typed<uint64_t, true>(op, (uint64_t*)out, srcs, n); break;
    case BSHMEM_FLOAT: reduce_typed<float, false>(op, (float*)out, srcs, n); break;
    case BSHMEM_DOUBLE: reduce_typed<double, false>(op, (double*)out, srcs, n); break;
    case BSHMEM_BF16: reduce_half<bf16_to_f, f_to_bf16>(op, (uint16_t*)out, srcs, n); break;
    case BSHMEM_FP16: reduce_half<fp16_to_f, f_to_fp16>(op, (uint16_t*)out, srcs, n); break;
  }
}

template <typename T> bool compare(int cmp, T a, T b) {
  switch (cmp) {
    case BSHMEM_CMP_EQ: return a == b;
    case BSHMEM_CMP_NE: return a != b;
    case BSHMEM_CMP_GT: return a > b;
    case BSHMEM_CMP_GE: return a >= b;
    case BSHMEM_CMP_LT: return a < b;
    case BSHMEM_CMP_LE: return a <= b;
  }
  return false;
}

template <typename T> T from_bits(uint64_t v) { T t; memcpy(&t, &v, sizeof(T)); return t; }

bool compare_any(const char* p, int dtype, int cmp, uint64_t value) {
  switch (dtype) {
    case BSHMEM_INT8: return compare<int8_t>(cmp, __atomic_load_n((const int8_t*)p, __ATOMIC_ACQUIRE), from_bits<int8_t>(value));
    case BSHMEM_UINT8: return compare<uint8_t>(cmp, __atomic_load_n((const uint8_t*)p, __ATOMIC_ACQUIRE), from_bits<uint8_t>(value));
    case BSHMEM_INT16: return compare<int16_t>(cmp, __atomic_load_n((const int16_t*)p, __ATOMIC_ACQUIRE), from_bits<int16_t>(value));
    case BSHMEM_UINT16: return compare<uint16_t>(cmp, __atomic_load_n((const uint16_t*)p, __ATOMIC_ACQUIRE), from_bits<uint16_t>(value));
    case BSHMEM_INT32: return compare<int32_t>(cmp, __atomic_load_n((const int32_t*)p, __ATOMIC_ACQUIRE), from_bits<int32_t>(value));
    case BSHMEM_UINT32: return compare<uint32_t>(cmp, __atomic_load_n((const uint32_t*)p, __ATOMIC_ACQUIRE), from_bits<uint32_t>(value));
    case BSHMEM_INT64: return compare<int64_t>(cmp, __atomic_load_n((const int64_t*)p, __ATOMIC_ACQUIRE), from_bits<int64_t>(value));
    case BSHMEM_UINT64: return compare<uint64_t>(cmp, __atomic_load_n((const uint64_t*)p, __ATOMIC_ACQUIRE), value);
    case BSHMEM_FLOAT: { uint32_t u = __atomic_load_n((const uint32_t*)p, __ATOMIC_ACQUIRE); return compare<float>(cmp, from_bits<float>(u), from_bits<float>(value)); }
    case BSHMEM_DOUBLE: { uint64_t u = __atomic_load_n((const uint64_t*)p, __ATOMIC_ACQUIRE); return compare<double>(cmp, from_bits<double>(u), from_bits<double>(value)); }
    case BSHMEM_BF16: { uint16_t u = __atomic_load_n((const uint16_t*)p, __ATOMIC_ACQUIRE); return compare<float>(cmp, bf16_to_f(u), bf16_to_f((uint16_t)value)); }
    case BSHMEM_FP16: { uint16_t u = __atomic_load_n((const uint16_t*)p, __ATOMIC_ACQUIRE); return compare<float>(cmp, fp16_to_f(u), fp16_to_f((uint16_t)value)); }
  }
  return false;
}

// Atomic op on an integer word of type U; float/double add goes through CAS.
template <typename U>
uint64_t amo_word(U* p, int dtype, int op, uint64_t value, uint64_t cond) {
  U v = (U)value, c = (U)cond, old = 0;
  bool fp = (dtype == BSHMEM_FLOAT || dtype == BSHMEM_DOUBLE);
  auto fadd = [&](U add) -> U {   // returns the previous value
    if (!fp) return __atomic_fetch_add(p, add, __ATOMIC_ACQ_REL);
    U cur = __atomic_load_n(p, __ATOMIC_RELAXED);
    while (true) {
      U next;
      if (sizeof(U) == 4) { float a = from_bits<float>(cur), b = from_bits<float>(add); float r = a + b; uint32_t rb; memcpy(&rb, &r, 4); next = (U)rb; }
      else { double a = from_bits<double>(cur), b = from_bits<double>(add); double r = a + b; uint64_t rb; memcpy(&rb, &r, 8); next = (U)rb; }
      if (__atomic_compare_exchange_n(p, &cur, next, false, __ATOMIC_ACQ_REL, __ATOMIC_RELAXED)) return cur;
    }
  };
  U one;
  if (dtype == BSHMEM_FLOAT) { float f = 1.0f; uint32_t b; memcpy(&b, &f, 4); one = (U)b; }
  else if (dtype == BSHMEM_DOUBLE) { double d = 1.0; uint64_t b; memcpy(&b, &d, 8); one = (U)b; }
  else one = 1;
  switch (op) {
    case BSHMEM_AMO_FETCH_ADD: case BSHMEM_AMO_ADD: old = fadd(v); break;
    case BSHMEM_AMO_FETCH_INC: case BSHMEM_AMO_INC: old = fadd(one); break;
    case BSHMEM_AMO_FETCH: old = __atomic_load_n(p, __ATOMIC_ACQUIRE); break;
    case BSHMEM_AMO_FETCH_CSWAP: case BSHMEM_AMO_CSWAP:
      old = c;
      __atomic_compare_exchange_n(p, &old, v, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE);
      break;
    case BSHMEM_AMO_SET: __atomic_store_n(p, v, __ATOMIC_RELEASE); break;
    case BSHMEM_AMO_SWAP: old = __atomic_exchange_n(p, v, __ATOMIC_ACQ_REL); break;
    case BSHMEM_AMO_FETCH_AND: case BSHMEM_AMO_AND: old = __atomic_fetch_and(p, v, __ATOMIC_ACQ_REL); break;
    case BSHMEM_AMO_FETCH_OR: case BSHMEM_AMO_OR: old = __atomic_fetch_or(p, v, __ATOMIC_ACQ_REL); break;
    case BSHMEM_AMO_FETCH_XOR: case BSHMEM_AMO_XOR: old = __atomic_fetch_xor(p, v, __ATOMIC_ACQ_REL); break;
  }
  return (uint64_t)old;
}

class CpuBackend final : public Backend {
 public:
  CpuBackend(CpuWorld* w, int pe) : w_(w), pe_(pe) {
    memset(epoch_, 0, sizeof(epoch_));
    w_->ctl()->pe[pe_].attached.store(1);
  }
  ~CpuBackend() override { w_->ctl()->pe[pe_].attached.store(0); }

  const char* name() const override { return "cpu"; }
  int my_pe() const override { return pe_; }
  int n_pes() const override { return (int)w_->ctl()->n_pes; }
  uint64_t heap_bytes() const override { return w_->ctl()->heap_bytes; }
  uint64_t reserved_bytes() const override { return 0; }
  char* local_base() const override { return w_->heap(pe_); }
  char* peer_base(int pe) const override { return w_->heap(pe); }
  bool host_dereferenceable() const override { return true; }
  void set_timeout_us(uint64_t t) override { timeout_us_ = t; }
  std::string last_error() const override { return err_; }
  bshmem_error_record_t last_record(bool clear) override {
    bshmem_error_record_t r = rec_;
    if (clear) memset(&rec_, 0, sizeof(rec_));
    return r;
  }

  int put(int pe, uint64_t dst_off, const void* local, uint64_t n, bool) override {
    memcpy(w_->heap(pe) + dst_off, local, n);
    return BSHMEM_OK;
  }
  int get(int pe, void* local, uint64_t src_off, uint64_t n, bool) override {
    memcpy(local, w_->heap(pe) + src_off, n);
    return BSHMEM_OK;
  }
  int put_signal(int pe, uint64_t dst_off, const void* local, uint64_t n, uint64_t sig_off, uint64_t sig_val,
                 int sig_op, bool) override {
    if (n) memcpy(w_->heap(pe) + dst_off, local, n);
    uint64_t* s = reinterpret_cast<uint64_t*>(w_->heap(pe) + sig_off);
    // release: the payload is visible before the signal update
    if (sig_op == BSHMEM_SIGNAL_ADD) __atomic_fetch_add(s, sig_val, __ATOMIC_RELEASE);
    else __atomic_store_n(s, sig_val, __ATOMIC_RELEASE);
    return BSHMEM_OK;
  }
  int amo(int pe, uint64_t off, int dtype, int op, uint64_t value, uint64_t cond, uint64_t* fetched) override {
    char* p = w_->heap(pe) + off;
    uint64_t old = bshmem_dtype_size(dtype) == 4 ? amo_word<uint32_t>((uint32_t*)p, dtype, op, value, cond)
                                                : amo_word<uint64_t>((uint64_t*)p, dtype, op, value, cond);
    if (fetched) *fetched = old;
    return BSHMEM_OK;
  }
  int fence() override { __atomic_thread_fence(__ATOMIC_SEQ_CST); return BSHMEM_OK; }
  int quiet() override { __atomic_thread_fence(__ATOMIC_SEQ_CST); return BSHMEM_OK; }

  int wait_until(uint64_t off, int dtype, int cmp, uint64_t value, uint64_t timeout_us) override {
    const char* p = local_base() + off;
    uint64_t deadline = now_us() + timeout_us;
    for (unsigned spins = 0;; ++spins) {
      if (compare_any(p, dtype, cmp, value)) return BSHMEM_OK;
      int rc = check_job(deadline, spins, -1);
      if (rc != BSHMEM_OK) {
        uint64_t seen = 0;
        memcpy(&seen, p, bshmem_dtype_size(dtype));
        record(rc, -1, BSHMEM_WHERE_WAIT_UNTIL, off, value, seen);
        return rc;
      }
      relax(spins);
    }
  }
  int test(uint64_t off, int dtype, int cmp, uint64_t value, int* result) override {
    *result = compare_any(local_base() + off, dtype, cmp, value) ? 1 : 0;
    return BSHMEM_OK;
  }

  int sync(const CollGroup& g) override {
    // a job that was aborted by global_exit does not run further collectives
    if (w_->ctl()->aborted.load(std::memory_order_acquire)) {
      record(BSHMEM_ERR_ABORTED, -1, BSHMEM_WHERE_BARRIER, 0, 0, 0);
      return BSHMEM_ERR_ABORTED;
    }
    return g.slot >= 0 ? sync_slot(g) : sync_psync(g);
  }

  int broadcast(const CollGroup& g, uint64_t dst_off, uint64_t src_off, uint64_t nbytes, int root) override {
    int rc = sync(g);   // the root's source is ready
    if (rc != BSHMEM_OK) return rc;
    if (g.my_idx != root && nbytes) memcpy(local_base() + dst_off, w_->heap(g.set.pe_at(root)) + src_off, nbytes);
    return sync(g);     // the root may reuse its source
  }

  int reduce(const CollGroup& g, int dtype, int op, uint64_t dst_off, uint64_t src_off, uint64_t nelems) override {
    int rc = sync(g);
    if (rc != BSHMEM_OK) return rc;
    uint64_t bytes = nelems * bshmem_dtype_size(dtype);
    std::vector<char> tmp(bytes);   // dest may alias source, and peers still read our source
    if (nelems) reduce_any(dtype, op, tmp.data(), sources(g, src_off), nelems);
    rc = sync(g);       // everyone has read every source
    if (rc != BSHMEM_OK) return rc;
    if (bytes) memcpy(local_base() + dst_off, tmp.data(), bytes);
    return BSHMEM_OK;
  }

  int reduce_root(const CollGroup& g, int dtype, int op, uint64_t dst_off, uint64_t src_off, uint64_t nelems, int root) override {
    int rc = sync(g);
    if (rc != BSHMEM_OK) return rc;
    uint64_t bytes = nelems * bshmem_dtype_size(dtype);
    std::vector<char> tmp(g.my_idx == root ? bytes : 0);   // dest may alias source
    if (g.my_idx == root && nelems) reduce_any(dtype, op, tmp.data(), sources(g, src_off), nelems);
    rc = sync(g);       // the root has read every source
    if (rc != BSHMEM_OK) return rc;
    if (g.my_idx == root && bytes) memcpy(local_base() + dst_off, tmp.data(), bytes);
    return BSHMEM_OK;
  }

  int reduce_scatter(const CollGroup& g, int dtype, int op, uint64_t dst_off, uint64_t src_off, uint64_t per_pe) override {
    int rc = sync(g);
    if (rc != BSHMEM_OK) return rc;
    uint64_t bytes = per_pe * bshmem_dtype_size(dtype);
    std::vector<char> tmp(bytes);
    if (per_pe) reduce_any(dtype, op, tmp.data(), sources(g, src_off + (uint64_t)g.my_idx * bytes), per_pe);
    rc = sync(g);
    if (rc != BSHMEM_OK) return rc;
    if (bytes) memcpy(local_base() + dst_off, tmp.data(), bytes);
    return BSHMEM_OK;
  }

  int fcollect(const CollGroup& g, uint64_t dst_off, uint64_t src_off, uint64_t nbytes) override {
    int rc = sync(g);
    if (rc != BSHMEM_OK) return rc;
    for (int i = 0; i < g.size() && nbytes; ++i)
      memcpy(local_base() + dst_off + (uint64_t)i * nbytes, w_->heap(g.set.pe_at(i)) + src_off, nbytes);
    return sync(g);
  }

  int alltoall(const CollGroup& g, uint64_t dst_off, uint64_t src_off, uint64_t nbytes) override {
    int rc = sync(g);
    if (rc != BSHMEM_OK) return rc;
    // Block my_idx of PE i's source lands in block i of my dest.
    for (int i = 0; i < g.size() && nbytes; ++i)
      memcpy(local_base() + dst_off + (uint64_t)i * nbytes,
             w_->heap(g.set.pe_at(i)) + src_off + (uint64_t)g.my_idx * nbytes, nbytes);
    return sync(g);
  }

  int exchange_u64(const CollGroup& g, uint64_t mine, uint64_t* all) override {
    if (g.slot < 0) return BSHMEM_ERR_UNSUPPORTED;
    for (int i = 0; i < g.size(); ++i) w_->ctl()->pe[g.set.pe_at(i)].xchg[g.slot][g.my_idx] = mine;
    int rc = sync_slot(g);
    if (rc != BSHMEM_OK) return rc;
    for (int i = 0; i < g.size(); ++i) all[i] = w_->ctl()->pe[pe_].xchg[g.slot][i];
    return sync_slot(g);
  }

  int global_exit(int status) override {
    w_->ctl()->abort_status.store(status);
    w_->ctl()->aborted.store(1, std::memory_order_release);
    return BSHMEM_OK;
  }

  int zero_local(uint64_t off, uint64_t n) override { memset(local_base() + off, 0, n); return BSHMEM_OK; }

  void reset_slot(int slot) override {
    if (slot <= 0 || slot >= BSHMEM_MAX_TEAMS) return;
    for (auto& f : w_->ctl()->pe[pe_].flags[slot]) f.store(0, std::memory_order_relaxed);
    epoch_[slot] = 0;
  }

 private:
  std::vector<const char*> sources(const CollGroup& g, uint64_t src_off) const {
    std::vector<const char*> s(g.size());
    for (int i = 0; i < g.size(); ++i) s[i] = w_->heap(g.set.pe_at(i)) + src_off;
    return s;
  }

  void record(int code, int pe, uint32_t where, uint64_t addr, uint64_t expected, uint64_t seen) {
    rec_.code = code; rec_.pe = pe; rec_.where = where; rec_.count++;
    rec_.addr = addr; rec_.expected = expected; rec_.seen = seen;
    err_ = std::string(bshmem_status_string(code)) + " (site " + std::to_string(where) + ", pe " + std::to_string(pe) + ")";
  }

  // Checked every few spins of any wait: abort flag, dead peers, deadline.
  int check_job(uint64_t deadline, unsigned spins, int waiting_for_pe) {
    if ((spins & 63) != 63) return BSHMEM_OK;
    Control* c = w_->ctl();
    if (c->aborted.load(std::memory_order_acquire)) return BSHMEM_ERR_ABORTED;
    if (waiting_for_pe >= 0 && c->pe[waiting_for_pe].dead.load(std::memory_order_acquire)) return BSHMEM_ERR_PEER_DEAD;
    if (now_us() > deadline) return BSHMEM_ERR_TIMEOUT;
    return BSHMEM_OK;
  }

  // All-to-all epoch barrier on a team slot: publish my epoch in every
  // member's flag row, then wait until every member's flag in my row caught up.
  int sync_slot(const CollGroup& g) {
    uint64_t e = ++epoch_[g.slot];
    Control* c = w_->ctl();
    for (int i = 0; i < g.size(); ++i)
      c->pe[g.set.pe_at(i)].flags[g.slot][g.my_idx].store(e, std::memory_order_release);
    uint64_t deadline = now_us() + timeout_us_;
    for (int i = 0; i < g.size(); ++i) {
      auto& f = c->pe[pe_].flags[g.slot][i];
      for (unsigned spins = 0;; ++spins) {
        uint64_t seen = f.load(std::memory_order_acquire);
        if (seen >= e) break;
        int rc = check_job(deadline, spins, g.set.pe_at(i));
        if (rc != BSHMEM_OK) { record(rc, g.set.pe_at(i), BSHMEM_WHERE_BARRIER, (uint64_t)g.slot, e, seen); return rc; }
        relax(spins);
      }
    }
    return BSHMEM_OK;
  }

  // Active-set barrier on the user's pSync: members count in on the first
  // member's pSync[0]; it resets the counter, then releases everyone through
  // pSync[1], which each member resets itself.  Both words end at SYNC_VALUE.
  int sync_psync(const CollGroup& g) {
    int root = g.set.pe_at(0);
    long* root_count = reinterpret_cast<long*>(w_->heap(root) + g.psync_off);
    long* my_release = reinterpret_cast<long*>(local_base() + g.psync_off) + 1;
    uint64_t deadline = now_us() + timeout_us_;
    __atomic_fetch_add(root_count, 1L, __ATOMIC_ACQ_REL);
    if (g.my_idx == 0) {
      for (unsigned spins = 0;; ++spins) {
        long seen = __atomic_load_n(root_count, __ATOMIC_ACQUIRE);
        if (seen == (long)g.size()) break;
        int rc = check_job(deadline, spins, -1);
        if (rc != BSHMEM_OK) { record(rc, -1, BSHMEM_WHERE_BARRIER, g.psync_off, g.size(), (uint64_t)seen); return rc; }
        relax(spins);
      }
      __atomic_store_n(root_count, (long)BSHMEM_SYNC_VALUE, __ATOMIC_RELEASE);
      for (int i = 1; i < g.size(); ++i) {
        long* rel = reinterpret_cast<long*>(w_->heap(g.set.pe_at(i)) + g.psync_off) + 1;
        __atomic_store_n(rel, 1L, __ATOMIC_RELEASE);
      }
    } else {
      for (unsigned spins = 0;; ++spins) {
        long seen = __atomic_load_n(my_release, __ATOMIC_ACQUIRE);
        if (seen == 1) break;
        int rc = check_job(deadline, spins, root);
        if (rc != BSHMEM_OK) { record(rc, root, BSHMEM_WHERE_BARRIER, g.psync_off + 8, 1, (uint64_t)seen); return rc; }
        relax(spins);
      }
      __atomic_store_n(my_release, (long)BSHMEM_SYNC_VALUE, __ATOMIC_RELEASE);
    }
    return BSHMEM_OK;
  }

  CpuWorld* w_;
  int pe_;
  uint64_t timeout_us_ = 30ull * 1000 * 1000;
  uint64_t epoch_[BSHMEM_MAX_TEAMS];
  bshmem_error_record_t rec_{};
  std::string err_;
};

}  // namespace
}  // namespace bshmem

using namespace bshmem;

extern "C" {

int bshmem_cpu_world_create(const char* name, int n_pes, uint64_t heap_bytes, void** world) {
  if (!world || n_pes < 1 || n_pes > BSHMEM_MAX_PES || heap_bytes == 0) return BSHMEM_ERR_INVALID;
  uint64_t hb = (heap_bytes + 4095) / 4096 * 4096;
  size_t total = kControlBytes + hb * (uint64_t)n_pes;
  void* m = MAP_FAILED;
  if (name && name[0]) {
    int fd = shm_open(name, O_CREAT | O_RDWR | O_EXCL, 0600);
    if (fd < 0) { shm_unlink(name); fd = shm_open(name, O_CREAT | O_RDWR | O_EXCL, 0600); }
    if (fd < 0) return BSHMEM_ERR_STATE;
    if (ftruncate(fd, (off_t)total) != 0) { close(fd); shm_unlink(name); return BSHMEM_ERR_NOMEM; }
    m = mmap(nullptr, total, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
  } else {
    m = mmap(nullptr, total, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
  }
  if (m == MAP_FAILED) { if (name && name[0]) shm_unlink(name); return BSHMEM_ERR_NOMEM; }
  CpuWorld* w = new CpuWorld();
  w->name = name ? name : "";
  w->owner = true;
  w->map_bytes = total;
  w->map = static_cast<char*>(m);
  Control* c = new (m) Control();   // fresh pages are zero; this just runs the atomics' constructors
  c->n_pes = n_pes;
  c->heap_bytes = hb;
  std::atomic_thread_fence(std::memory_order_release);
  c->magic = kMagic;
  *world = w;
  return BSHMEM_OK;
}

int bshmem_cpu_world_open(const char* name, void** world) {
  if (!world || !name || !name[0]) return BSHMEM_ERR_INVALID;
  int fd = shm_open(name, O_RDWR, 0600);
  if (fd < 0) return BSHMEM_ERR_STATE;
  struct stat st;
  if (fstat(fd, &st) != 0 || (size_t)st.st_size < kControlBytes) { close(fd); return BSHMEM_ERR_STATE; }
  void* m = mmap(nullptr, (size_t)st.st_size, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (m == MAP_FAILED) return BSHMEM_ERR_NOMEM;
  Control* c = static_cast<Control*>(m);
  if (c->magic != kMagic) { munmap(m, (size_t)st.st_size); return BSHMEM_ERR_STATE; }
  CpuWorld* w = new CpuWorld();
  w->name = name;
  w->owner = false;
  w->map_bytes = (size_t)st.st_size;
  w->map = static_cast<char*>(m);
  *world = w;
  return BSHMEM_OK;
}

int bshmem_cpu_world_destroy(void* world) {
  CpuWorld* w = static_cast<CpuWorld*>(world);
  if (!w) return BSHMEM_ERR_INVALID;
  munmap(w->map, w->map_bytes);
  if (w->owner && !w->name.empty()) shm_unlink(w->name.c_str());
  delete w;
  return BSHMEM_OK;
}

int bshmem_cpu_world_mark_dead(void* world, int pe) {
  CpuWorld* w = static_cast<CpuWorld*>(world);
  if (!w || pe < 0 || pe >= (int)w->ctl()->n_pes) return BSHMEM_ERR_INVALID;
  w->ctl()->pe[pe].dead.store(1, std::memory_order_release);
  return BSHMEM_OK;
}

int bshmem_cpu_init(void* world, int pe, const bshmem_config_t* cfg, bshmem_handle_t* out) {
  CpuWorld* w = static_cast<CpuWorld*>(world);
  if (!w || !out || pe < 0 || pe >= (int)w->ctl()->n_pes) return BSHMEM_ERR_INVALID;
  *out = make_runtime(std::unique_ptr<Backend>(new CpuBackend(w, pe)), cfg);
  return BSHMEM_OK;
}

}  // extern "C"
