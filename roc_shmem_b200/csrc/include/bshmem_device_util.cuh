// bshmem_device_util.cuh — small device-side building blocks: block mutexes, a block
// notifier, a device-callable slab (bump) allocator, a warp coalescer for contiguous
// messages, and the iteration / sharing strategies of the test containers.
//
// Parity:
//   SpinEBOBlockMutex   library/src/sync/spin_ebo_block_mutex.cpp:34-100 (per-block re-entrant lock,
//                       exponential back-off)
//   ABQLBlockMutex      library/src/sync/abql_block_mutex.hpp:43-109 (array-based queue lock, 32 turn
//                       slots padded to 256 bytes)
//   Notifier            library/src/memory/notifier.hpp:46-68 (thread 0 publishes a value to its block)
//   SlabHeap            library/src/memory/slab_heap.cpp:45-92 (block takes the lock, thread 0 bumps)
//   WarpCoalescer       library/src/wf_coal_policy.cpp:57-172 (merge contiguous lane messages) — for
//                       32-lane warps; with a load/store transport it only saves address arithmetic,
//                       so the put/get paths do not call it by default
//   IndexStrategy       library/src/containers/index_strategy.hpp:518-527 (7 iteration schemes)
//   ShareStrategy       library/src/containers/share_strategy.hpp:70-83 (warp-aggregated fetch_incr)
// Unlike the reference every spin is bounded and reports BSHMEM_ERR_TIMEOUT.
#pragma once
#include "bshmem_device.cuh"

#ifdef __CUDACC__
namespace bshmem {
namespace util {

__device__ __forceinline__ bool is_block_leader() { return threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0; }
__device__ __forceinline__ int flat_block_id() { return blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z); }

// ---- spin lock with exponential back-off, owned by a thread block, re-entrant ---------------
struct SpinEBOBlockMutex {
  int locked;       // 0 free, 1 held
  int owner;        // flat block id + 1 of the holder
  int depth;        // re-entrance count
  // Block-collective.  Returns BSHMEM_OK or BSHMEM_ERR_TIMEOUT (same value in all threads).
  __device__ int lock(unsigned long long timeout_ns) {
    __shared__ int st;
    if (is_block_leader()) {
      st = BSHMEM_OK;
      const int me = flat_block_id() + 1;
      if (*reinterpret_cast<volatile int*>(&owner) == me) {
        ++depth;
      } else {
        unsigned ns = 32;
        unsigned long long t0 = dev::timer();
        while (atomicCAS(&locked, 0, 1) != 0) {
          __nanosleep(ns);
          if (ns < 8192) ns <<= 1;                       // exponential back-off
          if (dev::timer() - t0 > timeout_ns) { st = BSHMEM_ERR_TIMEOUT; break; }
        }
        if (st == BSHMEM_OK) { __threadfence(); owner = me; depth = 1; }
      }
    }
    __syncthreads();
    int r = st;
    __syncthreads();
    return r;
  }
  __device__ void unlock() {
    __syncthreads();
    if (is_block_leader() && --depth == 0) {
      owner = 0;
      __threadfence();
      atomicExch(&locked, 0);
    }
    __syncthreads();
  }
};

// ---- array-based queue lock: FIFO, each waiter spins on its own padded slot --------------------
struct ABQLBlockMutex {
  static constexpr int kSlots = 32;
  struct alignas(256) Turn { unsigned long long grant; };
  Turn turns[kSlots];                 // turns[t % 32].grant == t  ⇔  ticket t may enter
  alignas(256) unsigned long long next_ticket;
  // Host or one device thread before first use.
  __host__ __device__ void init() {
    for (int i = 0; i < kSlots; ++i) turns[i].grant = ~0ull;
    turns[0].grant = 0;
    next_ticket = 0;
  }
  // Block-collective: returns the ticket to hand to unlock(), or ~0 on timeout.
  __device__ unsigned long long lock(unsigned long long timeout_ns) {
    __shared__ unsigned long long tk;
    if (is_block_leader()) {
      unsigned long long t = atomicAdd(&next_ticket, 1ull);
      volatile unsigned long long* slot = &turns[t % kSlots].grant;
      unsigned long long t0 = dev::timer();
      tk = t;
      while (*slot != t) {
        __nanosleep(64);
        if (dev::timer() - t0 > timeout_ns) { tk = ~0ull; break; }
      }
      __threadfence();
    }
    __syncthreads();
    unsigned long long r = tk;
    __syncthreads();
    return r;
  }
  __device__ void unlock(unsigned long long ticket) {
    __syncthreads();
    if (is_block_leader()) {
      __threadfence();
      turns[ticket % kSlots].grant = ~0ull;
      *reinterpret_cast<volatile unsigned long long*>(&turns[(ticket + 1) % kSlots].grant) = ticket + 1;
    }
    __syncthreads();
  }
};

// ---- notifier: the block leader publishes one value to every thread of its block ------------------
template <typename T>
struct Notifier {
  __device__ static T broadcast(T leader_value) {
    __shared__ T slot;
    if (is_block_leader()) slot = leader_value;
    __syncthreads();
    T v = slot;
    __syncthreads();
    return v;
  }
};

// ---- slab heap: bump allocation callable by whole blocks ---------------------------------------------
struct SlabHeap {
  char* base;
  unsigned long long bytes;
  unsigned long long used;
  ABQLBlockMutex mutex;
  __host__ __device__ void init(char* b, unsigned long long n) { base = b; bytes = n; used = 0; mutex.init(); }
  // Block-collective; every thread gets the same pointer (nullptr when exhausted or on lock timeout).
  __device__ char* malloc_block(size_t size, unsigned long long timeout_ns, size_t align = 128) {
    unsigned long long tk = mutex.lock(timeout_ns);
    char* p = nullptr;
    if (tk != ~0ull) {
      if (is_block_leader()) {
        unsigned long long start = (used + align - 1) / align * align;
        if (size && start + size <= bytes) { p = base + start; used = start + size; }
      }
      mutex.unlock(tk);
    }
    return Notifier<char*>::broadcast(p);
  }
};

// ---- warp coalescer: contiguous messages of neighbouring lanes become one -----------------------------
// Each active lane describes a message (pe, src, dst, size).  A lane whose message directly continues
// the message of the previous active lane (same pe, same size, src and dst contiguous) is folded into
// the first lane of its run.  Returns true if this lane still has to send; *size is the merged length.
__device__ __forceinline__ bool warp_coalesce(int pe, const void* src, const void* dst, size_t* size) {
  const unsigned active = __activemask();
  const int lane = threadIdx.x & 31;
  const unsigned long long s = reinterpret_cast<unsigned long long>(src), d = reinterpret_cast<unsigned long long>(dst);
  const unsigned long long n = *size;
  // neighbour = previous lane (only meaningful if it is active)
  int ppe = __shfl_up_sync(active, pe, 1);
  unsigned long long ps = __shfl_up_sync(active, s, 1), pd = __shfl_up_sync(active, d, 1), pn = __shfl_up_sync(active, n, 1);
  bool prev_active = lane > 0 && (active & (1u << (lane - 1)));
  bool continues = prev_active && ppe == pe && pn == n && ps + pn == s && pd + pn == d;
  unsigned heads = __ballot_sync(active, !continues);          // lanes that start a run
  if (continues) return false;
  // run length = distance to the next head (or to the end of the contiguous active lanes)
  unsigned later_heads = heads & ~((2u << lane) - 1);
  int next_head = later_heads ? __ffs(later_heads) - 1 : 32;
  unsigned run_mask = (next_head == 32 ? ~0u : ((1u << next_head) - 1)) & ~((1u << lane) - 1);
  int run = __popc(active & run_mask);
  *size = n * run;
  return true;
}

// ---- iteration schemes over [0, n) -------------------------------------------------------------------------
enum IndexStrategy {
  IDX_THREAD_SEQUENTIAL = 0,   // every thread visits all elements
  IDX_BLOCK_STRIDED = 1,       // threads of a block share the range, stride blockDim
  IDX_BLOCK_CHUNKED = 2,       // threads of a block take contiguous chunks
  IDX_WARP_STRIDED = 3,        // lanes of a warp share the range, stride 32
  IDX_GRID_STRIDED = 4,        // all threads of the grid, stride gridDim*blockDim
  IDX_GRID_CHUNKED = 5,        // all threads of the grid, contiguous chunks
  IDX_LEADER_ONLY = 6          // only the block leader iterates
};
struct IndexRange { size_t begin, end, step; };
__device__ __forceinline__ IndexRange index_range(int strategy, size_t n) {
  const size_t tib = threadIdx.x, bs = blockDim.x;
  const size_t gt = blockIdx.x * bs + tib, gs = (size_t)gridDim.x * bs;
  switch (strategy) {
    case IDX_THREAD_SEQUENTIAL: return {0, n, 1};
    case IDX_BLOCK_STRIDED: return {tib, n, bs};
    case IDX_BLOCK_CHUNKED: { size_t per = (n + bs - 1) / bs, b = per * tib; return {b < n ? b : n, b + per < n ? b + per : n, 1}; }
    case IDX_WARP_STRIDED: return {tib & 31, n, 32};
    case IDX_GRID_STRIDED: return {gt, n, gs};
    case IDX_GRID_CHUNKED: { size_t per = (n + gs - 1) / gs, b = per * gt; return {b < n ? b : n, b + per < n ? b + per : n, 1}; }
    default: return {0, is_block_leader() ? n : 0, 1};
  }
}

// Array / Matrix views used by the container tests.
template <typename T> struct Array {
  T* data; size_t n;
  template <typename F> __device__ void for_each(int strategy, F f) {
    IndexRange r = index_range(strategy, n);
    for (size_t i = r.begin; i < r.end; i += r.step) f(data[i], i);
  }
};
template <typename T> struct Matrix {
  T* data; size_t rows, cols;
  __device__ T& at(size_t r, size_t c) { return data[r * cols + c]; }
};

// Warp-aggregated fetch-and-increment: one atomic per warp, each active lane gets a distinct value.
__device__ __forceinline__ unsigned long long share_fetch_incr(unsigned long long* counter) {
  const unsigned active = __activemask();
  const int lane = threadIdx.x & 31, leader = __ffs(active) - 1;
  unsigned long long base = 0;
  if (lane == leader) base = atomicAdd(counter, (unsigned long long)__popc(active));
  base = __shfl_sync(active, base, leader);
  return base + __popc(active & ((1u << lane) - 1));
}

}  // namespace util
}  // namespace bshmem
#endif
