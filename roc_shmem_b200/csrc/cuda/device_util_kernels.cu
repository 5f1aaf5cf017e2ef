// device_util_kernels.cu — test kernels for bshmem_device_util.cuh, mirroring the reference's
// device unit tests: mutex tests launch N blocks x M threads that bump a counter under the lock
// (clients/unit_tests/abql_block_mutex_gtest.hpp:44-118, spin_ebo_block_mutex_gtest), slab heap
// allocations from many blocks (slab_heap_gtest), notifier, index strategies (index_strategy_gtest),
// wave bit tricks / share strategy (bitwise_gtest), and the coalescer's merge rule.
#include <cuda_runtime.h>

#include "../include/bshmem_device_util.cuh"
#include "../include/bshmem_types.h"

using namespace bshmem;

namespace {

struct UtilScratch {
  util::SpinEBOBlockMutex spin;
  util::ABQLBlockMutex abql;
  util::SlabHeap slab;
  unsigned long long counter_plain;     // incremented non-atomically under a lock
  unsigned long long share_counter;
  int status;
};

__global__ void k_util_init(UtilScratch* s, char* slab_base, unsigned long long slab_bytes) {
  s->spin.locked = 0; s->spin.owner = 0; s->spin.depth = 0;
  s->abql.init();
  s->slab.init(slab_base, slab_bytes);
  s->counter_plain = 0;
  s->share_counter = 0;
  s->status = 0;
}

// which: 0 = spin/EBO (taken twice: re-entrant), 1 = ABQL
__global__ void k_mutex_counter(UtilScratch* s, int which, int iters, unsigned long long timeout_ns) {
  for (int i = 0; i < iters; ++i) {
    if (which == 0) {
      int rc = s->spin.lock(timeout_ns);
      if (rc == BSHMEM_OK) rc = s->spin.lock(timeout_ns);          // re-entrance by the same block
      if (rc != BSHMEM_OK) { if (threadIdx.x == 0) atomicCAS(&s->status, 0, rc); return; }
      if (threadIdx.x == 0) { volatile unsigned long long* c = &s->counter_plain; *c = *c + 1; }
      s->spin.unlock();
      s->spin.unlock();
    } else {
      unsigned long long tk = s->abql.lock(timeout_ns);
      if (tk == ~0ull) { if (threadIdx.x == 0) atomicCAS(&s->status, 0, BSHMEM_ERR_TIMEOUT); return; }
      if (threadIdx.x == 0) { volatile unsigned long long* c = &s->counter_plain; *c = *c + 1; }
      s->abql.unlock(tk);
    }
  }
}

// every block allocates `allocs` chunks of (blockIdx+1)*64 bytes and writes its id into them
__global__ void k_slab_alloc(UtilScratch* s, int allocs, unsigned long long* offsets, unsigned long long timeout_ns) {
  for (int a = 0; a < allocs; ++a) {
    size_t size = (size_t)(blockIdx.x + 1) * 64;
    char* p = s->slab.malloc_block(size, timeout_ns);
    // every thread of the block must have received the same pointer
    unsigned long long mine = reinterpret_cast<unsigned long long>(p);
    unsigned long long lead = util::Notifier<unsigned long long>::broadcast(mine);
    if (mine != lead) atomicCAS(&s->status, 0, 100);
    if (p) {
      for (size_t i = threadIdx.x; i < size; i += blockDim.x) p[i] = (char)(blockIdx.x + 1);
      if (threadIdx.x == 0) offsets[blockIdx.x * allocs + a] = p - s->slab.base;
    } else if (threadIdx.x == 0) {
      offsets[blockIdx.x * allocs + a] = ~0ull;
    }
  }
}

// visits[i] += 1 for every element the strategy hands to this thread
__global__ void k_index_strategy(int strategy, unsigned int* visits, size_t n) {
  util::Array<unsigned int> arr{visits, n};
  arr.for_each(strategy, [](unsigned int& v, size_t) { atomicAdd(&v, 1u); });
}

// odd lanes drop out; the remaining lanes draw tickets from one counter with a single atomic per warp
__global__ void k_share(UtilScratch* s, unsigned long long* tickets) {
  size_t gt = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  tickets[gt] = ~0ull;
  if (threadIdx.x & 1) return;
  tickets[gt] = util::share_fetch_incr(&s->share_counter);
}

// lane l describes message (pe, base + off[l], dbase + off[l], size): out_send / out_size per lane
__global__ void k_coalesce(const int* pes, const long long* offs, int size, int* out_send, long long* out_size) {
  int lane = threadIdx.x;
  if (offs[lane] < 0) { out_send[lane] = -1; return; }          // lane does not take part
  size_t n = size;
  const char* src = reinterpret_cast<const char*>(0x10000000ull) + offs[lane];
  const char* dst = reinterpret_cast<const char*>(0x20000000ull) + offs[lane];
  bool send = util::warp_coalesce(pes[lane], src, dst, &n);
  out_send[lane] = send ? 1 : 0;
  out_size[lane] = send ? (long long)n : 0;
}

}  // namespace

extern "C" {

int bshmem_util_scratch_bytes(void) { return (int)sizeof(UtilScratch); }

int bshmem_util_init(void* scratch, void* slab_base, unsigned long long slab_bytes) {
  k_util_init<<<1, 1>>>(static_cast<UtilScratch*>(scratch), static_cast<char*>(slab_base), slab_bytes);
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : 7;
}

int bshmem_util_mutex_test(void* scratch, int which, int blocks, int threads, int iters, int timeout_ms, unsigned long long* counter_out,
                           int* status_out) {
  UtilScratch* s = static_cast<UtilScratch*>(scratch);
  k_mutex_counter<<<blocks, threads>>>(s, which, iters, (unsigned long long)timeout_ms * 1000000ull);
  if (cudaDeviceSynchronize() != cudaSuccess) return 7;
  UtilScratch h;
  if (cudaMemcpy(&h, s, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return 7;
  *counter_out = h.counter_plain;
  *status_out = h.status;
  return 0;
}

int bshmem_util_slab_test(void* scratch, int blocks, int threads, int allocs, unsigned long long* offsets_dev, int timeout_ms, int* status_out) {
  UtilScratch* s = static_cast<UtilScratch*>(scratch);
  k_slab_alloc<<<blocks, threads>>>(s, allocs, offsets_dev, (unsigned long long)timeout_ms * 1000000ull);
  if (cudaDeviceSynchronize() != cudaSuccess) return 7;
  UtilScratch h;
  if (cudaMemcpy(&h, s, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return 7;
  *status_out = h.status;
  return 0;
}

int bshmem_util_index_test(int strategy, int blocks, int threads, unsigned int* visits_dev, unsigned long long n) {
  k_index_strategy<<<blocks, threads>>>(strategy, visits_dev, n);
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : 7;
}

int bshmem_util_share_test(void* scratch, int blocks, int threads, unsigned long long* tickets_dev) {
  k_share<<<blocks, threads>>>(static_cast<UtilScratch*>(scratch), tickets_dev);
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : 7;
}

int bshmem_util_coalesce_test(const int* pes_dev, const long long* offs_dev, int size, int* send_dev, long long* size_dev) {
  k_coalesce<<<1, 32>>>(pes_dev, offs_dev, size, send_dev, size_dev);
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : 7;
}

}  // extern "C"
