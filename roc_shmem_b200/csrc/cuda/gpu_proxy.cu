// gpu_proxy.cu — reverse-offload mode on the GPU backend: the command ring lives in pinned,
// device-mapped host memory, the ticket counter in device memory, and the service thread
// executes descriptors through the PE's runtime on a host context of its own (its own CUDA
// stream, so host work for the proxy never queues behind the kernel that is waiting for it).
//
// Parity: library/src/reverse_offload/backend_ro.cpp:47-109 (ROBackend wiring: queues in
// host-coherent memory, worker thread) and context_ro_device.cpp (device-side enqueue, here
// in bshmem_proxy_device.cuh).  The functional kernel below is the analogue of running the
// device test matrix with the RO build.
#include <cuda_runtime.h>

#include <cstring>
#include <string>

#include "../host/proxy.h"
#include "../host/runtime.h"
#include "../include/bshmem_gpu.h"
#include "../include/bshmem_proxy_device.cuh"

using namespace bshmem;
using dev::State;

namespace {

// Executes descriptors through the PE's own runtime, on a host context of its own: the service thread binds itself
// to that context, so everything it issues (RMA, atomics and team collectives alike) runs on the context's stream,
// never behind the kernel on the PE stream that is waiting for the answer, and teams created on the PE are known.
class GpuExecutor final : public ProxyExecutor {
 public:
  GpuExecutor(bshmem_handle_t h, int device) : inner_(h), h_(h), device_(device) {}
  ~GpuExecutor() override {
    if (ctx_ > 0) bshmem_ctx_destroy(h_, ctx_);
  }
  void thread_init() override {
    cudaSetDevice(device_);
    if (bshmem_ctx_create(h_, BSHMEM_CTX_ZERO, &ctx_) == BSHMEM_OK) bshmem_gpu_bind_thread_ctx(h_, ctx_);
  }
  int execute(const bshmem_proxy_desc_t& d, uint64_t* result) override { return inner_.execute(d, result); }
 private:
  RuntimeExecutor inner_;
  bshmem_handle_t h_;
  int device_;
  bshmem_ctx_t ctx_ = BSHMEM_CTX_INVALID;
};

thread_local std::string g_err;

// One block: lane-divergent commands from several warps (exercises the aggregated ticket),
// then thread 0 checks put / get / p / g / atomics / quiet / barrier through the ring.
__global__ void k_proxy_selftest(State s, uint64_t* sym, uint64_t* scratch_dev, int peer, int* results) {
  // every thread of the block adds its index to sym[1] on `peer` through the proxy
  int st = BSHMEM_OK;
  proxy::amo64(s, BSHMEM_AMO_ADD, sym + 1, (uint64_t)threadIdx.x + 1, 0, peer, &st);
  __syncthreads();
  if (threadIdx.x != 0) return;
  int r = 0;
  const uint64_t n = blockDim.x;
  results[r++] = st == BSHMEM_OK ? 1 : 1000 + st;   // raw status when it is not OK
  results[r++] = proxy::g64(s, sym + 1, peer) == n * (n + 1) / 2;
  results[r++] = proxy::p64(s, sym, 4242ull, peer) == BSHMEM_OK;
  results[r++] = proxy::quiet(s) == BSHMEM_OK;
  results[r++] = proxy::g64(s, sym, peer) == 4242ull;
  results[r++] = proxy::amo64(s, BSHMEM_AMO_FETCH_ADD, sym, 8ull, 0, peer) == 4242ull;
  results[r++] = proxy::amo64(s, BSHMEM_AMO_FETCH_CSWAP, sym, 1ull, 4250ull, peer) == 4250ull;
  results[r++] = proxy::amo64(s, BSHMEM_AMO_SWAP, sym, 77ull, 0, peer) == 1ull;
  // put / get of a small device buffer
  for (int i = 0; i < 16; ++i) scratch_dev[i] = 1000 + i;
  __threadfence_system();
  results[r++] = proxy::putmem(s, sym + 8, scratch_dev, 16 * 8, peer) == BSHMEM_OK;
  results[r++] = proxy::getmem(s, scratch_dev + 16, sym + 8, 16 * 8, peer) == BSHMEM_OK;
  bool same = true;
  for (int i = 0; i < 16; ++i) same &= (reinterpret_cast<volatile uint64_t*>(scratch_dev)[16 + i] == 1000ull + i);
  results[r++] = same;
  results[r++] = proxy::fence(s) == BSHMEM_OK;
  results[r++] = -1;
}

// A blocking command whose completion never comes (the host dropped or paused): must return TIMEOUT.
__global__ void k_proxy_expect_timeout(State s, uint64_t* sym, int peer, int* status) {
  int st = BSHMEM_OK;
  proxy::amo64(s, BSHMEM_AMO_FETCH_ADD, sym, 1ull, 0, peer, &st);
  *status = st;
}

}  // namespace

struct GpuProxyHandle {
  bshmem_proxy* px;
  bshmem_proxy_ring_t* ring_dev;      // device copy of the ring descriptor (what state.proxy points to)
  unsigned long long* write_index;    // device ticket counter
  void* pinned;
};

extern "C" {

const char* bshmem_gpu_proxy_last_error(void) { return g_err.c_str(); }

// heap: the PE's GPU heap object; main: the PE's runtime handle (its stream stays untouched).
// Returns the device pointer to put into bshmem_dev_state_t::proxy via *ring_dev_out.
int bshmem_gpu_proxy_create(void* heap, bshmem_handle_t main, uint64_t capacity, uint64_t timeout_us, int device,
                            void** handle_out, void** ring_dev_out, bshmem_proxy_t** px_out) {
  if (!heap || !main || !handle_out || capacity < 2 || (capacity & (capacity - 1))) return BSHMEM_ERR_INVALID;
  if (cudaSetDevice(device) != cudaSuccess) { g_err = "cudaSetDevice failed"; return BSHMEM_ERR_CUDA; }
  uint64_t bytes = proxy_ring_bytes(capacity);
  void* pinned = nullptr;
  if (cudaHostAlloc(&pinned, bytes, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
    g_err = "cudaHostAlloc(ring) failed";
    return BSHMEM_ERR_CUDA;
  }
  memset(pinned, 0, bytes);
  unsigned long long* widx = nullptr;
  bshmem_proxy_ring_t* ring_dev = nullptr;
  if (cudaMalloc(&widx, sizeof(unsigned long long)) != cudaSuccess || cudaMemset(widx, 0, sizeof(unsigned long long)) != cudaSuccess ||
      cudaMalloc(&ring_dev, sizeof(bshmem_proxy_ring_t)) != cudaSuccess) {
    g_err = "cudaMalloc(ring descriptor) failed";
    return BSHMEM_ERR_CUDA;
  }
  bshmem_proxy* px = proxy_start(pinned, capacity, widx, timeout_us * 1000ull,
                                 std::unique_ptr<ProxyExecutor>(new GpuExecutor(main, device)));
  if (!px) { g_err = "proxy_start failed"; return BSHMEM_ERR_INVALID; }
  // with unified addressing the pinned host pointers are valid on the device as they are
  bshmem_proxy_ring_t ring = px->ring;
  if (cudaMemcpy(ring_dev, &ring, sizeof(ring), cudaMemcpyHostToDevice) != cudaSuccess) { g_err = "ring copy failed"; return BSHMEM_ERR_CUDA; }
  GpuProxyHandle* gh = new GpuProxyHandle{px, ring_dev, widx, pinned};
  *handle_out = gh;
  if (ring_dev_out) *ring_dev_out = ring_dev;
  if (px_out) *px_out = px;
  return BSHMEM_OK;
}

int bshmem_gpu_proxy_set_timeout_us(void* handle, uint64_t timeout_us) {
  GpuProxyHandle* gh = static_cast<GpuProxyHandle*>(handle);
  if (!gh || timeout_us == 0) return BSHMEM_ERR_INVALID;
  gh->px->ring.timeout_ns = timeout_us * 1000ull;
  bshmem_proxy_ring_t ring = gh->px->ring;
  return cudaMemcpy(gh->ring_dev, &ring, sizeof(ring), cudaMemcpyHostToDevice) == cudaSuccess ? BSHMEM_OK : BSHMEM_ERR_CUDA;
}

int bshmem_gpu_proxy_destroy(void* handle) {
  GpuProxyHandle* gh = static_cast<GpuProxyHandle*>(handle);
  if (!gh) return BSHMEM_OK;
  cudaDeviceSynchronize();
  bshmem_proxy_stop(gh->px);        // joins the thread; the executor finalizes the worker runtime
  cudaFree(gh->ring_dev);
  cudaFree(gh->write_index);
  cudaFreeHost(gh->pinned);
  delete gh;
  return BSHMEM_OK;
}

// Functional kernel: `threads` threads issue proxy commands against `peer`; results[i] = 1/0, -1 terminates.
int bshmem_gpu_proxy_selftest(bshmem_handle_t h, void* ring_dev, void* sym, void* scratch_dev, int peer, int threads, int* results_dev) {
  State st;
  int rc = bshmem_gpu_get_state(h, &st);
  if (rc != BSHMEM_OK) return rc;
  st.proxy = ring_dev;
  void* sv = nullptr;
  bshmem_gpu_get_stream(h, &sv);
  cudaStream_t stream = static_cast<cudaStream_t>(sv);
  k_proxy_selftest<<<1, threads, 0, stream>>>(st, static_cast<uint64_t*>(sym), static_cast<uint64_t*>(scratch_dev), peer, results_dev);
  if (cudaGetLastError() != cudaSuccess) return BSHMEM_ERR_CUDA;
  return cudaStreamSynchronize(stream) == cudaSuccess ? BSHMEM_OK : BSHMEM_ERR_CUDA;
}

int bshmem_gpu_proxy_expect_timeout(bshmem_handle_t h, void* ring_dev, void* sym, int peer, int* status_dev) {
  State st;
  int rc = bshmem_gpu_get_state(h, &st);
  if (rc != BSHMEM_OK) return rc;
  st.proxy = ring_dev;
  void* sv = nullptr;
  bshmem_gpu_get_stream(h, &sv);
  cudaStream_t stream = static_cast<cudaStream_t>(sv);
  k_proxy_expect_timeout<<<1, 1, 0, stream>>>(st, static_cast<uint64_t*>(sym), peer, status_dev);
  if (cudaGetLastError() != cudaSuccess) return BSHMEM_ERR_CUDA;
  return cudaStreamSynchronize(stream) == cudaSuccess ? BSHMEM_OK : BSHMEM_ERR_CUDA;
}

}  // extern "C"
