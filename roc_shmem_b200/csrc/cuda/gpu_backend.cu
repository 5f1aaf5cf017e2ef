// gpu_backend.cu — the NVLink transport behind the host API, and the kernels the
// host launches on behalf of a PE.
//
// Host-initiated RMA is a copy on the peer mapping; host atomics, waits and
// signals are one-thread kernels using the device API; host collectives launch
// the device collectives striped over several CTAs.  Everything is ordered on one
// CUDA stream per PE (settable, so a PyTorch caller can pass its current stream);
// in blocking mode each call also synchronises the stream and reports device-side
// timeouts, in stream mode calls only enqueue work.
//
// Parity: this replaces the reference's host path over MPI windows
// (library/src/host/host.cpp:160-235, host_templates.hpp) and the GPU-IB backend
// wiring (gpu_ib/backend_ib.cpp:70-111); there is no NIC, so no queue pairs,
// segments or doorbells exist here.
#include <vector>
#include <cuda_runtime.h>

#include <cstring>
#include <memory>
#include <string>

#include "../host/backend.h"
#include "../host/runtime.h"
#include "../include/bshmem_coll.cuh"
#include "../include/bshmem_gpu.h"
#include "coll_kernels.h"
#include "gpu_heap.h"

using namespace bshmem;
using dev::State;
using DTeam = bshmem::dev::Team;
using collk::CollArgs;

namespace {

// ---------------------------------------------------------------------------------
// kernels
// ---------------------------------------------------------------------------------
template <typename W>
__device__ uint64_t amo_exec(W* p, int dtype, int op, uint64_t value, uint64_t cond) {
  W v = (W)value, c = (W)cond, old = 0;
  switch (op) {
    case BSHMEM_AMO_FETCH_ADD: case BSHMEM_AMO_ADD: case BSHMEM_AMO_FETCH_INC: case BSHMEM_AMO_INC: {
      bool inc = (op == BSHMEM_AMO_FETCH_INC || op == BSHMEM_AMO_INC);
      if (dtype == BSHMEM_FLOAT) {
        float f = inc ? 1.0f : __uint_as_float((unsigned)v);
        old = (W)__float_as_uint(atomicAdd_system(reinterpret_cast<float*>(p), f));
      } else if (dtype == BSHMEM_DOUBLE) {
        double d = inc ? 1.0 : __longlong_as_double((long long)v);
        old = (W)__double_as_longlong(atomicAdd_system(reinterpret_cast<double*>(p), d));
      } else {
        old = atomicAdd_system(p, inc ? (W)1 : v);
      }
      break;
    }
    case BSHMEM_AMO_FETCH: old = atomicOr_system(p, (W)0); break;
    case BSHMEM_AMO_FETCH_CSWAP: case BSHMEM_AMO_CSWAP: old = atomicCAS_system(p, c, v); break;
    case BSHMEM_AMO_SET: case BSHMEM_AMO_SWAP: old = atomicExch_system(p, v); break;
    case BSHMEM_AMO_FETCH_AND: case BSHMEM_AMO_AND: old = atomicAnd_system(p, v); break;
    case BSHMEM_AMO_FETCH_OR: case BSHMEM_AMO_OR: old = atomicOr_system(p, v); break;
    case BSHMEM_AMO_FETCH_XOR: case BSHMEM_AMO_XOR: old = atomicXor_system(p, v); break;
  }
  return (uint64_t)old;
}

__global__ void k_amo(State s, int pe, uint64_t off, int dtype, int op, uint64_t value, uint64_t cond, uint64_t* out) {
  char* p = s.heap_base[pe] + off;
  uint64_t r = (bshmem_dtype_size(dtype) == 4) ? amo_exec<unsigned int>((unsigned int*)p, dtype, op, value, cond)
                                               : amo_exec<unsigned long long>((unsigned long long*)p, dtype, op, value, cond);
  if (out) *out = r;
}

template <typename T> __device__ T bits_as(uint64_t v) { T t; memcpy(&t, &v, sizeof(T)); return t; }

__device__ int wait_dispatch(const State& s, const char* p, int dtype, int cmp, uint64_t value) {
  switch (dtype) {
    case BSHMEM_INT8: return dev::wait_until<int8_t>(s, (const int8_t*)p, cmp, bits_as<int8_t>(value));
    case BSHMEM_UINT8: return dev::wait_until<uint8_t>(s, (const uint8_t*)p, cmp, bits_as<uint8_t>(value));
    case BSHMEM_INT16: return dev::wait_until<int16_t>(s, (const int16_t*)p, cmp, bits_as<int16_t>(value));
    case BSHMEM_UINT16: return dev::wait_until<uint16_t>(s, (const uint16_t*)p, cmp, bits_as<uint16_t>(value));
    case BSHMEM_INT32: return dev::wait_until<int32_t>(s, (const int32_t*)p, cmp, bits_as<int32_t>(value));
    case BSHMEM_UINT32: return dev::wait_until<uint32_t>(s, (const uint32_t*)p, cmp, bits_as<uint32_t>(value));
    case BSHMEM_INT64: return dev::wait_until<int64_t>(s, (const int64_t*)p, cmp, bits_as<int64_t>(value));
    case BSHMEM_UINT64: return dev::wait_until<uint64_t>(s, (const uint64_t*)p, cmp, value);
    case BSHMEM_FLOAT: return dev::wait_until<float>(s, (const float*)p, cmp, bits_as<float>(value));
    case BSHMEM_DOUBLE: return dev::wait_until<double>(s, (const double*)p, cmp, bits_as<double>(value));
    default: return BSHMEM_ERR_UNSUPPORTED;
  }
}

__global__ void k_wait_until(State s, uint64_t off, int dtype, int cmp, uint64_t value, int* status) {
  *status = wait_dispatch(s, s.heap_base[s.my_pe] + off, dtype, cmp, value);
}

// Runs after the payload copy on the same stream: publish, then update the signal word.
__global__ void k_signal(State s, int pe, uint64_t sig_off, uint64_t value, int sig_op) {
  uint64_t* sig = reinterpret_cast<uint64_t*>(s.heap_base[pe] + sig_off);
  asm volatile("fence.acq_rel.sys;" ::: "memory");
  if (sig_op == BSHMEM_SIGNAL_ADD) asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(sig), "l"(value) : "memory");
  else asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(sig), "l"(value) : "memory");
}

// Large messages: each CTA moves its share with bulk async copies through a shared-memory ring (no payload in
// registers; see dev::bulk_copy_block).  `src` / `dst` are already translated to the peer mapping.
constexpr int kBulkStages = 4, kBulkChunk = 32768;
__global__ void __launch_bounds__(128) k_rma_bulk(State s, char* dst, const char* src, uint64_t n, int* status) {
  extern __shared__ __align__(128) char bulk_smem[];
  __shared__ __align__(8) uint64_t bars[kBulkStages];
  uint64_t per = ((n + gridDim.x - 1) / gridDim.x + 127) & ~127ull;
  uint64_t b = per * blockIdx.x, e = b + per < n ? b + per : n;
  if (b >= n) return;
  int rc = dev::bulk_copy_block<kBulkStages, kBulkChunk>(s, dst + b, src + b, e - b, bulk_smem, bars);
  if (rc != BSHMEM_OK && threadIdx.x == 0) atomicCAS(status, 0, rc);
}

// Device-initiated put / get of a large message striped over the grid.  The grid walks the message in 256 KiB pieces,
// piece i to CTA i mod grid: at any time the CTAs touch one window of grid x 256 KiB instead of one 2 MiB page each,
// which matters once the message is much larger than what the address-translation caches cover (132 CTAs on
// 256 MiB lost 8 % with one contiguous share per CTA).
constexpr uint64_t kRmaPiece = 256u << 10;
__global__ void __launch_bounds__(512) k_rma(State s, int pe, uint64_t sym_off, char* local, uint64_t n, int is_put, int scope) {
  char* sym = s.heap_base[s.my_pe] + sym_off;
  // a message of up to grid x 256 KiB is still split evenly: every CTA gets one contiguous share
  uint64_t piece = ((n + gridDim.x - 1) / gridDim.x + 15) & ~15ull;
  if (piece > kRmaPiece) piece = kRmaPiece;
  for (uint64_t b = (uint64_t)blockIdx.x * piece; b < n; b += (uint64_t)gridDim.x * piece) {
    const uint64_t e = b + piece < n ? b + piece : n;
    if (scope == dev::BLOCK) {
      if (is_put) dev::putmem_nbi<dev::BLOCK>(s, sym + b, local + b, e - b, pe);
      else dev::getmem<dev::BLOCK>(s, local + b, sym + b, e - b, pe);
    } else if (scope == dev::WARP) {
      // each warp takes a contiguous share of the piece
      int nw = blockDim.x >> 5, w = threadIdx.x >> 5;
      uint64_t wper = (((e - b) + nw - 1) / nw + 15) & ~15ull;
      uint64_t wb = b + wper * w, we = wb + wper < e ? wb + wper : e;
      if (wb < e) {
        if (is_put) dev::putmem_nbi<dev::WARP>(s, sym + wb, local + wb, we - wb, pe);
        else dev::getmem<dev::WARP>(s, local + wb, sym + wb, we - wb, pe);
      }
    } else {
      int nt = blockDim.x, t = threadIdx.x;
      uint64_t tper = (((e - b) + nt - 1) / nt + 15) & ~15ull;
      uint64_t tb = b + tper * t, te = tb + tper < e ? tb + tper : e;
      if (tb < e) {
        if (is_put) dev::putmem_nbi<dev::THREAD>(s, sym + tb, local + tb, te - tb, pe);
        else dev::getmem<dev::THREAD>(s, local + tb, sym + tb, te - tb, pe);
      }
    }
  }
}

// ---------------------------------------------------------------------------------
// Backend
// ---------------------------------------------------------------------------------
#define RT_TRY(call) do { cudaError_t _e = (call); if (_e != cudaSuccess) return cuda_fail(#call, _e); } while (0)

constexpr int kResultSlots = 64;
struct Pinned {
  bshmem_error_record_t err;       // lane 0's copy is the device-visible error record of the PE
  uint64_t amo_result[kResultSlots];
  int status[kResultSlots];
};

// What a host context owns on this backend: its ordering domain (a stream) and the pinned words its blocking calls
// read results from.  Lane 0 is the default context; its stream is the settable PE stream.  Result words are handed
// out round-robin per call, so threads that share a context do not read each other's answers.
struct Lane {
  cudaStream_t stream = nullptr;
  Pinned* pinned = nullptr;
  int* dstatus = nullptr;          // device status word of collectives launched on this lane
  std::atomic<unsigned> next{0};
  bool open = false;
};

// Selection of the calling thread (see Backend::ctx_select) and an optional binding of the thread to one lane for
// everything it issues, collectives included (the reverse-offload service thread runs on a lane of its own).
thread_local int tl_selected_ctx = 0;
thread_local const void* tl_bound_backend = nullptr;
thread_local int tl_bound_ctx = -1;
thread_local std::string tl_err;

class GpuBackend final : public Backend {
 public:
  GpuBackend(gpu::Heap* heap, bool own_heap) : heap_(heap), own_heap_(own_heap) {}

  int setup(const bshmem_config_t& cfg, int coll_ctas) {
    RT_TRY(cudaSetDevice(heap_->device));
    RT_TRY(cudaStreamCreateWithFlags(&own_stream_, cudaStreamNonBlocking));
    stream_ = own_stream_;
    RT_TRY(cudaHostAlloc(&pinned_, sizeof(Pinned), cudaHostAllocMapped));
    memset(pinned_, 0, sizeof(Pinned));
    lanes_[0].pinned = pinned_;
    lanes_[0].open = true;
    // counters followed by the (initially disabled) event ring
    RT_TRY(cudaMalloc(&dstats_, sizeof(unsigned long long) * (BSHMEM_DSTAT_COUNT + BSHMEM_TRACE_WORDS)));
    RT_TRY(cudaMemset(dstats_, 0, sizeof(unsigned long long) * (BSHMEM_DSTAT_COUNT + BSHMEM_TRACE_WORDS)));
    RT_TRY(cudaMalloc(&dstatus_, sizeof(int)));
    RT_TRY(cudaMemset(dstatus_, 0, sizeof(int)));
    lanes_[0].dstatus = dstatus_;
    memset(&state_, 0, sizeof(state_));
    state_.my_pe = heap_->my_pe;
    state_.n_pes = heap_->n_pes;
    state_.heap_bytes = heap_->heap_bytes;
    for (int p = 0; p < heap_->n_pes; ++p) state_.heap_base[p] = heap_->base[p];
    state_.mc_base = heap_->mc_base;
    state_.err = &pinned_->err;
    state_.timeout_ns = cfg.timeout_us * 1000ull;
    state_.stats = cfg.profile ? dstats_ : nullptr;
    state_.debug = cfg.debug;
    coll_ctas_ = coll_ctas < 1 ? 1 : (coll_ctas > BSHMEM_MAX_COLL_CTAS ? BSHMEM_MAX_COLL_CTAS : coll_ctas);
    int sms = 0;
    RT_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, heap_->device));
    if (coll_ctas_ > sms) coll_ctas_ = sms;
    return BSHMEM_OK;
  }

  ~GpuBackend() override {
    cudaSetDevice(heap_->device);
    cudaDeviceSynchronize();
    for (int i = 1; i < BSHMEM_MAX_CTXS; ++i) ctx_close(i);
    if (own_stream_) cudaStreamDestroy(own_stream_);
    if (dstats_) cudaFree(dstats_);
    if (dstatus_) cudaFree(dstatus_);
    if (pinned_) cudaFreeHost(pinned_);
    if (own_heap_) gpu::heap_destroy(heap_);
  }

  const char* name() const override { return "nvlink"; }
  int my_pe() const override { return heap_->my_pe; }
  int n_pes() const override { return heap_->n_pes; }
  uint64_t heap_bytes() const override { return heap_->heap_bytes; }
  uint64_t reserved_bytes() const override { return BSHMEM_INTERNAL_BYTES; }
  char* local_base() const override { return heap_->base[heap_->my_pe]; }
  char* peer_base(int pe) const override { return heap_->mapped[pe] ? heap_->base[pe] : nullptr; }
  bool host_dereferenceable() const override { return false; }
  void set_timeout_us(uint64_t t) override { state_.timeout_ns = t * 1000ull; }
  std::string last_error() const override { return tl_err; }

  // ---- host contexts -----------------------------------------------------------------
  int ctx_open(int idx, long) override {
    if (idx <= 0 || idx >= BSHMEM_MAX_CTXS) return BSHMEM_ERR_INVALID;
    Lane& L = lanes_[idx];
    if (L.open) return BSHMEM_OK;
    RT_TRY(cudaSetDevice(heap_->device));
    RT_TRY(cudaStreamCreateWithFlags(&L.stream, cudaStreamNonBlocking));
    RT_TRY(cudaHostAlloc(&L.pinned, sizeof(Pinned), cudaHostAllocMapped));
    memset(L.pinned, 0, sizeof(Pinned));
    RT_TRY(cudaMalloc(&L.dstatus, sizeof(int)));
    RT_TRY(cudaMemset(L.dstatus, 0, sizeof(int)));
    L.open = true;
    return BSHMEM_OK;
  }
  void ctx_close(int idx) override {
    if (idx <= 0 || idx >= BSHMEM_MAX_CTXS || !lanes_[idx].open) return;
    Lane& L = lanes_[idx];
    L.open = false;
    if (L.stream) { cudaStreamSynchronize(L.stream); cudaStreamDestroy(L.stream); L.stream = nullptr; }
    if (L.pinned) { cudaFreeHost(L.pinned); L.pinned = nullptr; }
    if (L.dstatus) { cudaFree(L.dstatus); L.dstatus = nullptr; }
  }
  void ctx_select(int idx) override { tl_selected_ctx = idx; }
  // Everything the calling thread issues from now on (collectives too) runs on context idx's lane; -1 unbinds.
  int bind_thread(int idx) {
    if (idx >= 0 && (idx >= BSHMEM_MAX_CTXS || !lanes_[idx].open)) return BSHMEM_ERR_INVALID;
    tl_bound_backend = idx >= 0 ? this : nullptr;
    tl_bound_ctx = idx;
    return BSHMEM_OK;
  }
  bool thread_is_bound() const { return tl_bound_backend == this && tl_bound_ctx >= 0; }
  Lane& lane() {
    int i = thread_is_bound() ? tl_bound_ctx : tl_selected_ctx;
    if (i < 0 || i >= BSHMEM_MAX_CTXS || !lanes_[i].open) i = 0;
    return lanes_[i];
  }
  // Collectives belong to no context: they run on the PE stream unless the thread is bound to a lane.
  Lane& coll_lane() { return thread_is_bound() ? lanes_[tl_bound_ctx] : lanes_[0]; }
  cudaStream_t stream_of(const Lane& L) const { return &L == &lanes_[0] ? stream_ : L.stream; }

  bshmem_error_record_t last_record(bool clear) override {
    bshmem_error_record_t r = pinned_->err;
    if (clear) memset(&pinned_->err, 0, sizeof(pinned_->err));
    return r;
  }

  // ---- knobs used by the C entry points below ---------------------------------
  // (cudaStream_t)-1 selects the runtime's own stream; any other handle (0 = the legacy default stream) is used as given.
  void set_stream(cudaStream_t s) { stream_ = (s == reinterpret_cast<cudaStream_t>(-1)) ? own_stream_ : s; }
  cudaStream_t stream() const { return stream_; }
  void set_blocking(bool b) { blocking_ = b; }
  void set_coll_ctas(int n) { if (n >= 1 && n <= BSHMEM_MAX_COLL_CTAS) coll_ctas_ = n; }
  void set_nvls(bool on) { use_nvls_ = on && heap_->mc_base != nullptr; }
  const State& state() const { return state_; }
  gpu::Heap* heap() const { return heap_; }
  unsigned long long* dstats() const { return dstats_; }
  void refresh_mc() { state_.mc_base = heap_->mc_base; }

  // a thread bound to a lane (the reverse-offload service thread) always completes what it issues: the device
  // producer that waits for its answer cannot synchronise a host stream
  bool blocking_now() const { return blocking_ || thread_is_bound(); }
  int finish(const char* what, cudaStream_t st) {
    if (!blocking_now()) return BSHMEM_OK;
    RT_TRY(cudaStreamSynchronize(st));
    return check_device_error(what);
  }

  int check_device_error(const char* what) {
    if (pinned_->err.code != 0) {
      int code = (int)pinned_->err.code;
      tl_err = std::string(what) + ": device-side " + bshmem_status_string(code) + " at site " +
             std::to_string(pinned_->err.where) + " waiting for pe " + std::to_string(pinned_->err.pe);
      return code;
    }
    return BSHMEM_OK;
  }

  // ---- RMA ------------------------------------------------------------------------
  int put(int pe, uint64_t dst_off, const void* local, uint64_t n, bool nbi) override {
    const cudaStream_t st = stream_of(lane());
    RT_TRY(cudaMemcpyAsync(heap_->base[pe] + dst_off, local, n, cudaMemcpyDefault, st));
    if (nbi) return BSHMEM_OK;
    return finish("put", st);
  }
  int get(int pe, void* local, uint64_t src_off, uint64_t n, bool nbi) override {
    const cudaStream_t st = stream_of(lane());
    RT_TRY(cudaMemcpyAsync(local, heap_->base[pe] + src_off, n, cudaMemcpyDefault, st));
    if (nbi) return BSHMEM_OK;
    return finish("get", st);
  }
  int put_signal(int pe, uint64_t dst_off, const void* local, uint64_t n, uint64_t sig_off, uint64_t sig_val, int sig_op,
                 bool nbi) override {
    const cudaStream_t st = stream_of(lane());
    if (n) RT_TRY(cudaMemcpyAsync(heap_->base[pe] + dst_off, local, n, cudaMemcpyDefault, st));
    k_signal<<<1, 1, 0, st>>>(state_, pe, sig_off, sig_val, sig_op);
    RT_TRY(cudaGetLastError());
    if (nbi) return BSHMEM_OK;
    return finish("put_signal", st);
  }
  int amo(int pe, uint64_t off, int dtype, int op, uint64_t value, uint64_t cond, uint64_t* fetched) override {
    Lane& L = lane();
    const cudaStream_t st = stream_of(L);
    uint64_t* slot = &L.pinned->amo_result[L.next.fetch_add(1, std::memory_order_relaxed) % kResultSlots];
    k_amo<<<1, 1, 0, st>>>(state_, pe, off, dtype, op, value, cond, slot);
    RT_TRY(cudaGetLastError());
    bool fetching = op <= BSHMEM_AMO_FETCH_CSWAP || op == BSHMEM_AMO_SWAP || (op >= BSHMEM_AMO_FETCH_AND && op <= BSHMEM_AMO_FETCH_XOR);
    if (fetching || blocking_now()) {
      RT_TRY(cudaStreamSynchronize(st));
      if (fetched) *fetched = *slot;
    }
    return BSHMEM_OK;
  }
  int fence() override { return BSHMEM_OK; }   // operations of one stream reach each PE in order
  int quiet() override {
    // Stream mode: operations of the PE's stream complete in order, and whatever the caller
    // enqueues next on that stream runs after them, so there is nothing to wait for on the
    // host; bshmem_gpu_synchronize() is the explicit host-side wait.
    if (!blocking_now()) return BSHMEM_OK;
    RT_TRY(cudaStreamSynchronize(stream_of(lane())));     // this context's operations only
    return check_device_error("quiet");
  }
  int wait_until(uint64_t off, int dtype, int cmp, uint64_t value, uint64_t timeout_us) override {
    State s = state_;
    s.timeout_ns = timeout_us * 1000ull;
    Lane& L = lane();
    const cudaStream_t st = stream_of(L);
    int* slot = &L.pinned->status[L.next.fetch_add(1, std::memory_order_relaxed) % kResultSlots];
    *slot = 0;
    k_wait_until<<<1, 1, 0, st>>>(s, off, dtype, cmp, value, slot);
    RT_TRY(cudaGetLastError());
    if (!blocking_now()) return BSHMEM_OK;
    RT_TRY(cudaStreamSynchronize(st));
    int rc = *slot;
    if (rc != BSHMEM_OK) tl_err = "wait_until: device-side timeout";
    return rc;
  }
  int test(uint64_t off, int dtype, int cmp, uint64_t value, int* result) override {
    State s = state_;
    s.timeout_ns = 0;   // a wait that gives up at once is a test
    s.err = nullptr;
    s.stats = nullptr;
    Lane& L = lane();
    const cudaStream_t st = stream_of(L);
    int* slot = &L.pinned->status[L.next.fetch_add(1, std::memory_order_relaxed) % kResultSlots];
    *slot = 0;
    k_wait_until<<<1, 1, 0, st>>>(s, off, dtype, cmp, value, slot);
    RT_TRY(cudaGetLastError());
    RT_TRY(cudaStreamSynchronize(st));
    *result = *slot == BSHMEM_OK ? 1 : 0;
    return BSHMEM_OK;
  }

  // ---- collectives ---------------------------------------------------------------------
  DTeam team_of(const CollGroup& g) const {
    DTeam t;
    t.pe_start = g.set.pe_start; t.stride = g.set.stride; t.size = g.set.size; t.my_idx = g.my_idx;
    t.slot = g.slot; t.reserved = 0; t.psync = nullptr;
    return t;
  }

  int launch(const CollGroup& g, CollArgs a, uint64_t bytes, const char* what) {
    if (heap_->mode == gpu::HEAP_LOCAL_GROUP) {
      // PEs of a local group share one GPU: a per-PE launch that waits for the others must not
      // exist.  Host syncs are no-ops (the caller owns ordering); data collectives go through
      // bshmem_gpu_group_collective, which runs all PEs in one cooperative launch.
      if (a.kind == BSHMEM_COLL_SYNC || a.kind == BSHMEM_COLL_BARRIER) return BSHMEM_OK;
      tl_err = std::string(what) + ": use the group collective entry for a local group";
      return BSHMEM_ERR_UNSUPPORTED;
    }
    a.psync_off = g.psync_off;
    // in-switch reductions pay off from four PEs on (with two, pulling the one peer's data is faster)
    a.use_nvls = (use_nvls_ && (heap_->n_pes > 2 || a.kind == BSHMEM_COLL_FCOLLECT)) ? 1 : 0;
    int ctas = 1;
    if (g.slot >= 0 && bytes > (32u << 10)) {   // one CTA per 32 KiB: remote latency, not bandwidth, bounds a CTA
      ctas = (int)((bytes + (32u << 10) - 1) / (32u << 10));
      if (ctas > coll_ctas_) ctas = coll_ctas_;
    }
    Lane& L = coll_lane();
    const cudaStream_t st = stream_of(L);
    const bool main_lane = &L == &lanes_[0];   // the slot / staging fast paths count calls per PE, so only the PE stream takes them
    a.ll_epoch = 0;
    const uint64_t unit = bshmem_dtype_size(a.dtype) > 4 ? bshmem_dtype_size(a.dtype) : 4;
    if (main_lane && a.kind == BSHMEM_COLL_REDUCE && g.slot == 0 && g.set.size == heap_->n_pes &&
        bytes > BSHMEM_LL_PAYLOAD_BYTES && bytes <= BSHMEM_LLB_PAYLOAD_BYTES && bytes % unit == 0 &&
        ((a.dst_off | a.src_off) & (unit - 1)) == 0) {
      // mid-size allreduce on the world team: one exchange through the per-sender slots.  The conditions are exactly
      // those under which the kernel takes that path, and every PE makes the same sequence of such calls, so this
      // counter is the same everywhere and its parity alternates between consecutive uses of the slots.
      a.ll_epoch = ++ll_epoch_;
      ctas = (int)((bytes + (4u << 10) - 1) / (4u << 10));      // 4 KiB of payload per block: four words per thread, polled one after the other
      if (ctas > coll_ctas_) ctas = coll_ctas_;
    }
    // One exchange through the staging region instead of sync + work + barrier: world team, what a PE receives fits a
    // staging half, 16-byte granular.  Every PE evaluates the same conditions on the same arguments, so the call
    // number (and with it the staging half) is the same everywhere.
    a.stage_seq = 0;
    a.stage_oneshot = 0;
    if (main_lane && g.slot == 0 && g.set.size == heap_->n_pes && heap_->n_pes > 1 && a.ll_epoch == 0 && bytes >= 16 &&
        bytes + 4096 <= BSHMEM_STAGE_BYTES && ((a.dst_off | a.src_off) & 15) == 0) {
      const uint64_t es = bshmem_dtype_size(a.dtype);
      bool fits = false;
      switch (a.kind) {
        case BSHMEM_COLL_FCOLLECT: case BSHMEM_COLL_ALLTOALL: fits = a.n % 16 == 0; break;
        case BSHMEM_COLL_REDUCE_SCATTER: fits = (a.n * es) % 16 == 0; break;
        // the multicast reduction needs no staging; below the one-shot limit the pull form is a single pass
        case BSHMEM_COLL_REDUCE: fits = !(a.use_nvls && a.op == BSHMEM_SUM && (a.dtype == BSHMEM_FLOAT || a.dtype == BSHMEM_BF16)) &&
                                        bytes > BSHMEM_LLB_PAYLOAD_BYTES; break;
        default: break;
      }
      if (fits) {
        a.stage_seq = ++stage_seq_;
        if (a.kind == BSHMEM_COLL_REDUCE) {
          // one exchange moves (P-1) vectors per PE, two exchanges 2 (P-1)/P: the single exchange wins while the
          // extra (P-1)(P-2)/P vectors cost less than a flag exchange (about 8 us, i.e. about 5 MiB on the links)
          const uint64_t P = (uint64_t)heap_->n_pes;
          const uint64_t slot = (BSHMEM_STAGE_BYTES / P) & ~(uint64_t)15;
          if (bytes <= slot && bytes * (P - 1) * (P - 2) / P <= (5ull << 20)) a.stage_oneshot = 1;
        }
        // every channel runs its own flag exchange and the kernel ends with the slowest one, so a staged call wants
        // few, fat channels; a block pushes its share to P-1 peers at about 50 GB/s, so the share shrinks with P:
        // 64 KiB with two PEs, 32 KiB with four, 16 KiB with eight and more
        uint64_t gran = (128ull << 10) / (uint64_t)heap_->n_pes;
        if (gran < (16u << 10)) gran = 16u << 10;
        ctas = (int)((bytes + gran - 1) / gran);
        if (ctas > coll_ctas_) ctas = coll_ctas_;
        if (ctas < 1) ctas = 1;
      }
    }
    RT_TRY(collk::launch(state_, team_of(g), a, ctas, L.dstatus, st));
    if (!blocking_now()) return BSHMEM_OK;
    int rc = 0;
    RT_TRY(cudaMemcpyAsync(&rc, L.dstatus, sizeof(int), cudaMemcpyDeviceToHost, st));
    RT_TRY(cudaStreamSynchronize(st));
    if (rc != 0) {
      cudaMemsetAsync(L.dstatus, 0, sizeof(int), st);
      check_device_error(what);
      if (tl_err.empty()) tl_err = std::string(what) + " failed on the device";
      return rc;
    }
    return BSHMEM_OK;
  }

  int sync(const CollGroup& g) override {
    CollArgs a{}; a.kind = BSHMEM_COLL_SYNC;
    return launch(g, a, 0, "sync");
  }
  int broadcast(const CollGroup& g, uint64_t d, uint64_t s, uint64_t nbytes, int root) override {
    CollArgs a{}; a.kind = BSHMEM_COLL_BROADCAST; a.dst_off = d; a.src_off = s; a.n = nbytes; a.root = root;
    return launch(g, a, nbytes, "broadcast");
  }
  int reduce(const CollGroup& g, int dtype, int op, uint64_t d, uint64_t s, uint64_t nelems) override {
    CollArgs a{}; a.kind = BSHMEM_COLL_REDUCE; a.dtype = dtype; a.op = op; a.dst_off = d; a.src_off = s; a.n = nelems;
    return launch(g, a, nelems * bshmem_dtype_size(dtype), "to_all");
  }
  int reduce_root(const CollGroup& g, int dtype, int op, uint64_t d, uint64_t s, uint64_t nelems, int root) override {
    CollArgs a{}; a.kind = BSHMEM_COLL_REDUCE_ROOT; a.dtype = dtype; a.op = op; a.dst_off = d; a.src_off = s; a.n = nelems; a.root = root;
    return launch(g, a, nelems * bshmem_dtype_size(dtype), "reduce");
  }
  int reduce_scatter(const CollGroup& g, int dtype, int op, uint64_t d, uint64_t s, uint64_t per_pe) override {
    CollArgs a{}; a.kind = BSHMEM_COLL_REDUCE_SCATTER; a.dtype = dtype; a.op = op; a.dst_off = d; a.src_off = s; a.n = per_pe;
    return launch(g, a, per_pe * bshmem_dtype_size(dtype) * g.size(), "reduce_scatter");
  }
  int fcollect(const CollGroup& g, uint64_t d, uint64_t s, uint64_t nbytes) override {
    CollArgs a{}; a.kind = BSHMEM_COLL_FCOLLECT; a.dst_off = d; a.src_off = s; a.n = nbytes;
    return launch(g, a, nbytes * g.size(), "fcollect");
  }
  int alltoall(const CollGroup& g, uint64_t d, uint64_t s, uint64_t nbytes) override {
    CollArgs a{}; a.kind = BSHMEM_COLL_ALLTOALL; a.dst_off = d; a.src_off = s; a.n = nbytes;
    return launch(g, a, nbytes * g.size(), "alltoall");
  }
  int exchange_u64(const CollGroup& g, uint64_t mine, uint64_t* all) override {
    if (g.slot < 0) return BSHMEM_ERR_UNSUPPORTED;
    CollArgs a{}; a.kind = BSHMEM_COLL_EXCHANGE; a.n = mine;
    bool was = blocking_;
    blocking_ = true;
    int rc = launch(g, a, 0, "exchange");
    blocking_ = was;
    if (rc != BSHMEM_OK) return rc;
    RT_TRY(cudaMemcpy(all, local_base() + BSHMEM_OFF_XCHG + (uint64_t)g.slot * BSHMEM_MAX_PES * 8, 8 * g.size(),
                      cudaMemcpyDeviceToHost));
    // a second sync keeps a fast member's next exchange from overwriting rows still being read
    CollArgs b{}; b.kind = BSHMEM_COLL_SYNC;
    blocking_ = true;
    rc = launch(g, b, 0, "exchange");
    blocking_ = was;
    return rc;
  }
  int global_exit(int) override { return BSHMEM_OK; }   // the Python layer raises the job-wide flag in the store
  int zero_local(uint64_t off, uint64_t n) override {
    RT_TRY(cudaMemsetAsync(local_base() + off, 0, n, stream_));
    RT_TRY(cudaStreamSynchronize(stream_));
    return BSHMEM_OK;
  }
  void reset_slot(int slot) override {
    if (slot <= 0 || slot >= BSHMEM_MAX_TEAMS) return;
    cudaStreamSynchronize(stream_);
    cudaMemset(local_base() + BSHMEM_OFF_FLAGS + (uint64_t)slot * BSHMEM_MAX_COLL_CTAS * BSHMEM_MAX_PES * 8, 0,
               (uint64_t)BSHMEM_MAX_COLL_CTAS * BSHMEM_MAX_PES * 8);
    cudaMemset(local_base() + BSHMEM_OFF_EPOCHS + (uint64_t)slot * BSHMEM_MAX_COLL_CTAS * 8, 0, BSHMEM_MAX_COLL_CTAS * 8);
    // the slot's low-latency allreduce block: epoch word and per-sender slots start from zero for the new team
    cudaMemset(local_base() + BSHMEM_OFF_LLT + (uint64_t)slot * BSHMEM_LLT_TEAM_BYTES, 0, BSHMEM_LLT_TEAM_BYTES);
  }

  int cuda_fail(const char* what, cudaError_t e) {
    tl_err = std::string(what) + ": " + cudaGetErrorString(e);
    return BSHMEM_ERR_CUDA;
  }

  int* dstatus() const { return dstatus_; }

 private:
  gpu::Heap* heap_;
  bool own_heap_;
  State state_{};
  cudaStream_t own_stream_ = nullptr, stream_ = nullptr;
  Pinned* pinned_ = nullptr;
  unsigned long long* dstats_ = nullptr;
  int* dstatus_ = nullptr;
  bool blocking_ = true;
  bool use_nvls_ = false;
  int coll_ctas_ = 32;
  Lane lanes_[BSHMEM_MAX_CTXS];
  unsigned long long ll_epoch_ = 0;     // epochs of host-launched low-latency allreduces
  unsigned long long stage_seq_ = 0;    // call numbers of staged one-exchange collectives
};

GpuBackend* gpu_of(bshmem_handle_t h) {
  if (!h || h->finalized || !h->backend) return nullptr;
  return dynamic_cast<GpuBackend*>(h->backend.get());
}

thread_local std::string g_err;

}  // namespace

// ---------------------------------------------------------------------------------
// C entry points (bshmem_gpu.h)
// ---------------------------------------------------------------------------------
extern "C" {

const char* bshmem_gpu_last_error(void) {
  if (!g_err.empty()) return g_err.c_str();
  return gpu::heap_error().c_str();
}

int bshmem_gpu_heap_create(int my_pe, int n_pes, uint64_t heap_bytes, int device, int mode, void** heap) {
  gpu::Heap* h = nullptr;
  int rc = gpu::heap_create(my_pe, n_pes, heap_bytes, device, mode, &h);
  if (rc == BSHMEM_OK) *heap = h;
  return rc;
}
int bshmem_gpu_heap_create_local_group(int n_pes, uint64_t heap_bytes, int device, void** heaps) {
  return gpu::heap_create_local_group(n_pes, heap_bytes, device, reinterpret_cast<gpu::Heap**>(heaps));
}
int bshmem_gpu_heap_export_fd(void* heap, int* fd) { return gpu::heap_export_fd(static_cast<gpu::Heap*>(heap), fd); }
int bshmem_gpu_heap_import_fd(void* heap, int pe, int fd) { return gpu::heap_import_fd(static_cast<gpu::Heap*>(heap), pe, fd); }
int bshmem_gpu_heap_export_ipc(void* heap, void* handle64) { return gpu::heap_export_ipc(static_cast<gpu::Heap*>(heap), handle64); }
int bshmem_gpu_heap_import_ipc(void* heap, int pe, const void* handle64) { return gpu::heap_import_ipc(static_cast<gpu::Heap*>(heap), pe, handle64); }
int bshmem_gpu_multicast_supported(int device) { return gpu::heap_multicast_supported(device); }
int bshmem_gpu_multicast_create(void* heap, int* fd) { return gpu::heap_multicast_create(static_cast<gpu::Heap*>(heap), fd); }
int bshmem_gpu_multicast_import(void* heap, int fd) { return gpu::heap_multicast_import(static_cast<gpu::Heap*>(heap), fd); }
int bshmem_gpu_multicast_add_device(void* heap) { return gpu::heap_multicast_add_device(static_cast<gpu::Heap*>(heap)); }
int bshmem_gpu_multicast_bind(void* heap) { return gpu::heap_multicast_bind(static_cast<gpu::Heap*>(heap)); }
int bshmem_gpu_heap_destroy(void* heap) { return gpu::heap_destroy(static_cast<gpu::Heap*>(heap)); }
uint64_t bshmem_gpu_heap_bytes(void* heap) { return static_cast<gpu::Heap*>(heap)->heap_bytes; }

int bshmem_gpu_init(void* heap, const bshmem_config_t* cfg, int coll_ctas, int own_heap, bshmem_handle_t* out) {
  if (!heap || !out) return BSHMEM_ERR_INVALID;
  bshmem_config_t c;
  if (cfg) c = *cfg; else bshmem_config_default(&c);
  if (c.timeout_us == 0) c.timeout_us = 30ull * 1000 * 1000;
  auto* be = new GpuBackend(static_cast<gpu::Heap*>(heap), own_heap != 0);
  int rc = be->setup(c, coll_ctas);
  // Load every kernel of this library now.  With lazy module loading the first launch of a kernel
  // can need a device-wide quiet point; if that first launch came from the proxy thread while a user
  // kernel is spinning on the proxy's answer, neither would ever finish.
  {
    cudaFuncAttributes fa;
    cudaFuncGetAttributes(&fa, k_amo);
    cudaFuncGetAttributes(&fa, k_wait_until);
    cudaFuncGetAttributes(&fa, k_signal);
    cudaFuncGetAttributes(&fa, k_rma);
    cudaFuncGetAttributes(&fa, k_rma_bulk);
    collk::preload();
  }
  if (rc != BSHMEM_OK) { g_err = be->last_error(); delete be; return rc; }
  *out = make_runtime(std::unique_ptr<Backend>(be), &c);
  return BSHMEM_OK;
}

int bshmem_gpu_set_stream(bshmem_handle_t h, void* stream) {
  GpuBackend* g = gpu_of(h);
  if (!g) return BSHMEM_ERR_STATE;
  g->set_stream(static_cast<cudaStream_t>(stream));
  return BSHMEM_OK;
}
// Binds the calling thread to host context `ctx` of this PE: everything the thread issues from now on, collectives
// included, runs on that context's stream and completes before the call returns; ctx < 0 unbinds.  The
// reverse-offload service thread uses this so that its work never queues behind the kernel that waits for it.
int bshmem_gpu_bind_thread_ctx(bshmem_handle_t h, int ctx) {
  GpuBackend* g = gpu_of(h);
  if (!g) return BSHMEM_ERR_STATE;
  return g->bind_thread(ctx);
}
int bshmem_gpu_get_device(bshmem_handle_t h, int* device) {
  GpuBackend* g = gpu_of(h);
  if (!g || !device) return BSHMEM_ERR_STATE;
  *device = g->heap()->device;
  return BSHMEM_OK;
}
int bshmem_gpu_get_stream(bshmem_handle_t h, void** stream) {
  GpuBackend* g = gpu_of(h);
  if (!g || !stream) return BSHMEM_ERR_STATE;
  *stream = g->stream();
  return BSHMEM_OK;
}
// Waits for everything enqueued on the PE's stream and reports device-side timeouts.
int bshmem_gpu_synchronize(bshmem_handle_t h) {
  GpuBackend* g = gpu_of(h);
  if (!g) return BSHMEM_ERR_STATE;
  if (cudaStreamSynchronize(g->stream()) != cudaSuccess) return BSHMEM_ERR_CUDA;
  return g->check_device_error("synchronize");
}
int bshmem_gpu_set_blocking(bshmem_handle_t h, int blocking) {
  GpuBackend* g = gpu_of(h);
  if (!g) return BSHMEM_ERR_STATE;
  g->set_blocking(blocking != 0);
  return BSHMEM_OK;
}
int bshmem_gpu_set_coll_ctas(bshmem_handle_t h, int n) {
  GpuBackend* g = gpu_of(h);
  if (!g) return BSHMEM_ERR_STATE;
  g->set_coll_ctas(n);
  return BSHMEM_OK;
}
int bshmem_gpu_set_nvls(bshmem_handle_t h, int on) {
  GpuBackend* g = gpu_of(h);
  if (!g) return BSHMEM_ERR_STATE;
  g->refresh_mc();
  g->set_nvls(on != 0);
  return BSHMEM_OK;
}
// Copies the device-side state (peer base table etc.) for a user kernel's argument list.
int bshmem_gpu_get_state(bshmem_handle_t h, bshmem_dev_state_t* out) {
  GpuBackend* g = gpu_of(h);
  if (!g || !out) return BSHMEM_ERR_STATE;
  *out = g->state();
  return BSHMEM_OK;
}
int bshmem_gpu_check_error(bshmem_handle_t h) {
  GpuBackend* g = gpu_of(h);
  if (!g) return BSHMEM_ERR_STATE;
  return g->check_device_error("check");
}
int bshmem_gpu_get_device_stats(bshmem_handle_t h, uint64_t* out, int n) {
  GpuBackend* g = gpu_of(h);
  if (!g) return BSHMEM_ERR_STATE;
  unsigned long long tmp[BSHMEM_DSTAT_COUNT];
  if (cudaMemcpy(tmp, g->dstats(), sizeof(tmp), cudaMemcpyDeviceToHost) != cudaSuccess) return BSHMEM_ERR_CUDA;
  for (int i = 0; i < n && i < BSHMEM_DSTAT_COUNT; ++i) out[i] = tmp[i];
  return BSHMEM_OK;
}
// Device timeline: keep the last `capacity` events (0 switches tracing off; at most BSHMEM_TRACE_MAX_EVENTS).
// Synchronises the runtime's stream, so call it between kernels.
int bshmem_gpu_trace_enable(bshmem_handle_t h, int capacity) {
  GpuBackend* g = gpu_of(h);
  if (!g || !g->dstats()) return BSHMEM_ERR_STATE;
  if (capacity < 0 || capacity > BSHMEM_TRACE_MAX_EVENTS) return BSHMEM_ERR_INVALID;
  if (cudaStreamSynchronize(g->stream()) != cudaSuccess) return BSHMEM_ERR_CUDA;
  unsigned long long head[2] = {(unsigned long long)capacity, 0ull};
  return cudaMemcpy(g->dstats() + BSHMEM_DSTAT_COUNT, head, sizeof(head), cudaMemcpyHostToDevice) == cudaSuccess ? BSHMEM_OK
                                                                                                                  : BSHMEM_ERR_CUDA;
}
// Copies the recorded events, oldest first, into out[4 * max_events] (time ns, op | pe << 8 | block << 32, bytes,
// sequence number); *n_out = events copied, *total = events recorded since tracing was enabled.
int bshmem_gpu_trace_read(bshmem_handle_t h, uint64_t* out, int max_events, int* n_out, uint64_t* total) {
  GpuBackend* g = gpu_of(h);
  if (!g || !g->dstats() || !out || !n_out) return BSHMEM_ERR_STATE;
  if (cudaStreamSynchronize(g->stream()) != cudaSuccess) return BSHMEM_ERR_CUDA;
  std::vector<unsigned long long> buf(BSHMEM_TRACE_WORDS);
  if (cudaMemcpy(buf.data(), g->dstats() + BSHMEM_DSTAT_COUNT, sizeof(unsigned long long) * BSHMEM_TRACE_WORDS,
                 cudaMemcpyDeviceToHost) != cudaSuccess)
    return BSHMEM_ERR_CUDA;
  const unsigned long long cap = buf[0], count = buf[1];
  if (total) *total = count;
  unsigned long long have = cap ? (count < cap ? count : cap) : 0;
  if (have > (unsigned long long)max_events) have = max_events;
  for (unsigned long long k = 0; k < have; ++k) {
    const unsigned long long seq = count - have + k;
    const unsigned long long* e = &buf[2 + 4 * (seq % cap)];
    for (int w = 0; w < 4; ++w) out[4 * k + w] = e[w];
  }
  *n_out = (int)have;
  return BSHMEM_OK;
}
int bshmem_gpu_reset_device_stats(bshmem_handle_t h) {
  GpuBackend* g = gpu_of(h);
  if (!g) return BSHMEM_ERR_STATE;
  return cudaMemset(g->dstats(), 0, sizeof(unsigned long long) * BSHMEM_DSTAT_COUNT) == cudaSuccess ? BSHMEM_OK : BSHMEM_ERR_CUDA;
}

// Device-initiated put/get of `n` bytes between `local` (any device pointer) and the symmetric
// address `sym` on `pe`, striped over `ctas` CTAs of `threads` threads at the given scope
// (0 thread, 1 warp, 2 block).  This is the path the point-to-point bandwidth sweep times.
int bshmem_gpu_rma_kernel(bshmem_handle_t h, void* sym, void* local, uint64_t n, int pe, int is_put, int scope,
                          int ctas, int threads) {
  GpuBackend* g = gpu_of(h);
  if (!g) return BSHMEM_ERR_STATE;
  uint64_t off;
  if (!h->to_offset(sym, n, &off) || pe < 0 || pe >= g->n_pes()) return BSHMEM_ERR_RANGE;
  if (ctas < 1) ctas = 1;
  if (threads < 32) threads = 32;
  if (threads > 512) threads = 512;     // the kernel's launch bound: eight 16-byte accesses in flight per thread need the registers
  // scope 3 = bulk async copies through shared memory
  const bool aligned = ((reinterpret_cast<uintptr_t>(local) | off | n) & 15) == 0;
  if (scope == 3 && !aligned) return BSHMEM_ERR_INVALID;
  if (scope == 3) {
    static bool attr_set[64] = {};
    const int d = g->heap()->device;
    if (d >= 0 && d < 64 && !attr_set[d]) {
      cudaFuncSetAttribute(k_rma_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkStages * kBulkChunk);
      attr_set[d] = true;
    }
    char* remote = g->heap()->base[pe] + off;
    char* loc = static_cast<char*>(local);
    k_rma_bulk<<<ctas, 128, kBulkStages * kBulkChunk, g->stream()>>>(g->state(), is_put ? remote : loc, is_put ? loc : remote, n,
                                                                     g->dstatus());
  } else {
    k_rma<<<ctas, threads, 0, g->stream()>>>(g->state(), pe, off, static_cast<char*>(local), n, is_put, scope);
  }
  cudaError_t ce = cudaGetLastError();
  if (ce != cudaSuccess) {
    g_err = std::string("rma kernel launch: ") + cudaGetErrorString(ce);
    return BSHMEM_ERR_CUDA;
  }
  return BSHMEM_OK;
}

// One collective for a whole local group in a single cooperative launch (single-GPU emulation).
// handles[n]: the group's runtimes; team_slot: the team to run on (every member passes the same
// offsets, as with any symmetric call).
int bshmem_gpu_group_collective(bshmem_handle_t* handles, int n, int team_slot, int kind, int dtype, int op, int root,
                                uint64_t dst_off, uint64_t src_off, uint64_t count, int ctas) {
  if (!handles || n < 1 || n > BSHMEM_MAX_PES) return BSHMEM_ERR_INVALID;
  State hs[BSHMEM_MAX_PES];
  DTeam ht[BSHMEM_MAX_PES];
  GpuBackend* g0 = gpu_of(handles[0]);
  if (!g0) return BSHMEM_ERR_STATE;
  for (int i = 0; i < n; ++i) {
    GpuBackend* g = gpu_of(handles[i]);
    if (!g) return BSHMEM_ERR_STATE;
    hs[i] = g->state();
    CollGroup cg;
    if (handles[i]->group_of_team(team_slot, &cg) == BSHMEM_OK) ht[i] = g->team_of(cg);
    else { memset(&ht[i], 0, sizeof(DTeam)); ht[i].my_idx = -1; }
  }
  if (ctas > BSHMEM_MAX_COLL_CTAS) ctas = BSHMEM_MAX_COLL_CTAS;     // one flag row per channel exists, no more
  for (int i = 0; i < n; ++i) {
    if (ht[i].my_idx < 0) continue;
    uint64_t sb = 0, db = 0;
    collk::extent(kind, dtype, count, ht[i].size, &sb, &db);
    if (src_off > hs[i].heap_bytes || sb > hs[i].heap_bytes - src_off || dst_off > hs[i].heap_bytes || db > hs[i].heap_bytes - dst_off)
      return BSHMEM_ERR_RANGE;
  }
  State* ds = nullptr;
  DTeam* dt = nullptr;
  if (cudaMalloc(&ds, sizeof(State) * n) != cudaSuccess || cudaMalloc(&dt, sizeof(DTeam) * n) != cudaSuccess) return BSHMEM_ERR_CUDA;
  cudaMemcpy(ds, hs, sizeof(State) * n, cudaMemcpyHostToDevice);
  cudaMemcpy(dt, ht, sizeof(DTeam) * n, cudaMemcpyHostToDevice);
  CollArgs a{};
  a.kind = kind; a.dtype = dtype; a.op = op; a.root = root; a.dst_off = dst_off; a.src_off = src_off; a.n = count;
  int* status = g0->dstatus();
  if (ctas < 1) ctas = 1;
  cudaError_t e = collk::launch_group(ds, dt, a, ctas, n, status, g0->stream());
  int rc = BSHMEM_OK;
  if (e != cudaSuccess) { g_err = std::string("cooperative launch: ") + cudaGetErrorString(e); rc = BSHMEM_ERR_CUDA; }
  else if (cudaStreamSynchronize(g0->stream()) != cudaSuccess) rc = BSHMEM_ERR_CUDA;
  else {
    int st = 0;
    cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost);
    if (st) { cudaMemset(status, 0, sizeof(int)); rc = st; }
  }
  cudaFree(ds);
  cudaFree(dt);
  return rc;
}


// DTeam split for a local group, done for all PEs at once on the calling thread (the slot
// agreement of bshmem_team_split_strided needs a host exchange between PEs, which a
// single-threaded group cannot run).
int bshmem_gpu_group_team_split(bshmem_handle_t* handles, int n, int parent_slot, int start, int stride, int size,
                                int* out_slots) {
  if (!handles || !out_slots || n < 1 || n > BSHMEM_MAX_PES) return BSHMEM_ERR_INVALID;
  bshmem::Team plans[BSHMEM_MAX_PES];
  bool member[BSHMEM_MAX_PES];
  uint64_t mask = ~0ull;
  for (int i = 0; i < n; ++i) {
    out_slots[i] = -1;
    member[i] = false;
    if (!handles[i]->teams->get(parent_slot) || handles[i]->teams->get(parent_slot)->my_pe < 0) continue;
    int rc = handles[i]->teams->plan_split(parent_slot, start, stride, size, &plans[i], &member[i]);
    if (rc != BSHMEM_OK) return rc;
    if (member[i]) mask &= handles[i]->teams->free_mask();
  }
  int slot = TeamTracker::pick_slot(mask);
  if (slot < 0) return BSHMEM_ERR_LIMIT;
  for (int i = 0; i < n; ++i) {
    if (!member[i]) continue;
    int rc = handles[i]->teams->commit(plans[i], slot);
    if (rc != BSHMEM_OK) return rc;
    out_slots[i] = slot;
  }
  return BSHMEM_OK;
}

}  // extern "C"
