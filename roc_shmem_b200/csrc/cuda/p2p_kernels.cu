// p2p_kernels.cu — device-initiated point-to-point micro-benchmarks and functional
// test kernels built on the public device API (bshmem_device.cuh).
//
// They mirror the reference's functional testers: ping-pong latency with p +
// wait_until (clients/functional_tests/ping_pong_tester.cpp:32-63), put_nbi message
// rate in windows of 64 + quiet (primitive_mr_tester.cpp:32-58), atomic latency
// (amo_standard_tester.cpp:119-165) and the per-thread "swarm" get
// (swarm_tester.cpp) — plus put-with-signal, which the reference lacks.  Times are
// taken on the device with %globaltimer and returned in nanoseconds.
#include <cuda_runtime.h>

#include "../host/runtime.h"
#include "../include/bshmem_coll.cuh"
#include "../include/bshmem_gpu.h"

using namespace bshmem;
using dev::State;

namespace {

struct BenchOut {
  unsigned long long ns;
  int status;
  int pad;
};

// Both PEs run this with one thread; the initiator sends i, the responder echoes it.
__global__ void k_pingpong(State s, uint64_t* flag, int peer, int iters, int initiator, BenchOut* out) {
  unsigned long long t0 = dev::timer();
  int rc = BSHMEM_OK;
  for (int i = 1; i <= iters && rc == BSHMEM_OK; ++i) {
    if (initiator) {
      dev::p<uint64_t>(s, flag, (uint64_t)i, peer);
      rc = dev::wait_until<uint64_t>(s, flag, BSHMEM_CMP_EQ, (uint64_t)i);
    } else {
      rc = dev::wait_until<uint64_t>(s, flag, BSHMEM_CMP_EQ, (uint64_t)i);
      dev::p<uint64_t>(s, flag, (uint64_t)i, peer);
    }
  }
  out->ns = dev::timer() - t0;
  out->status = rc;
}

// One block per PE: payload + signal there, payload + signal back.
__global__ void k_put_signal_pingpong(State s, char* data, uint64_t* sig, size_t nbytes, int peer, int iters, int initiator,
                                      BenchOut* out) {
  __shared__ int rc_sh;
  if (threadIdx.x == 0) rc_sh = BSHMEM_OK;
  __syncthreads();
  unsigned long long t0 = dev::timer();
  for (int i = 1; i <= iters; ++i) {
    if (initiator) dev::putmem_signal<dev::BLOCK>(s, data, data, nbytes, sig, (uint64_t)i, BSHMEM_SIGNAL_SET, peer);
    if (threadIdx.x == 0) {
      int rc = dev::wait_until<uint64_t>(s, sig, BSHMEM_CMP_GE, (uint64_t)i);
      if (rc != BSHMEM_OK) rc_sh = rc;
    }
    __syncthreads();
    if (rc_sh != BSHMEM_OK) break;
    if (!initiator) dev::putmem_signal<dev::BLOCK>(s, data, data, nbytes, sig, (uint64_t)i, BSHMEM_SIGNAL_SET, peer);
  }
  __syncthreads();
  if (threadIdx.x == 0) { out->ns = dev::timer() - t0; out->status = rc_sh; }
}

__global__ void k_amo_latency(State s, unsigned long long* target, int peer, int iters, int op, BenchOut* out) {
  unsigned long long t0 = dev::timer();
  unsigned long long acc = 0;
  for (int i = 0; i < iters; ++i) {
    switch (op) {
      case BSHMEM_AMO_FETCH_ADD: acc += dev::atomic_fetch_add<unsigned long long>(s, target, 1ull, peer); break;
      case BSHMEM_AMO_FETCH_CSWAP: acc += dev::atomic_compare_swap<unsigned long long>(s, target, acc, acc + 1, peer); break;
      case BSHMEM_AMO_SWAP: acc += dev::atomic_swap<unsigned long long>(s, target, (unsigned long long)i, peer); break;
      case BSHMEM_AMO_FETCH: acc += dev::atomic_fetch<unsigned long long>(s, target, peer); break;
      default: dev::atomic_add<unsigned long long>(s, target, 1ull, peer); break;
    }
  }
  dev::quiet(s);
  out->ns = dev::timer() - t0;
  out->status = (int)(acc & 0);
}

// Every thread issues windows of 64 non-blocking puts of `size` bytes, then quiet.
__global__ void k_put_msgrate(State s, char* dest, const char* src, size_t size, int peer, int windows, BenchOut* out) {
  size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  char* d = dest + tid * size * 64;
  const char* sp = src + tid * size * 64;
  unsigned long long t0 = dev::timer();
  for (int w = 0; w < windows; ++w) {
#pragma unroll 4
    for (int i = 0; i < 64; ++i) dev::putmem_nbi<dev::THREAD>(s, d + i * size, sp + i * size, size, peer);
    dev::quiet(s);
  }
  unsigned long long dt = dev::timer() - t0;
  if (tid == 0) { out->ns = dt; out->status = BSHMEM_OK; }
}

// Every thread of the grid issues `iters` fetch-adds on one of `words` target words of the peer (thread t uses word
// t % words): the rate of independent 8-byte atomics over NVLink as the number of issuing CTAs grows.
__global__ void k_amo_rate(State s, unsigned long long* target, int words, int peer, int iters, BenchOut* out) {
  size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  unsigned long long* t = target + tid % (size_t)words;
  unsigned long long t0 = dev::timer(), acc = 0;
  for (int i = 0; i < iters; ++i) acc += dev::atomic_fetch_add<unsigned long long>(s, t, 1ull, peer);
  unsigned long long dt = dev::timer() - t0;
  if (tid == 0) { out->ns = dt; out->status = (int)(acc & 0); }
}

// One-way putmem_signal stream: every CTA puts its share of `nbytes` and adds 1 to the signal word, `iters` times;
// the target PE is not involved (its signal word just counts), so this measures put-with-signal bandwidth.
__global__ void __launch_bounds__(1024) k_put_signal_stream(State s, char* data, const char* src, uint64_t* sig, size_t nbytes, int peer,
                                                           int iters) {
  size_t per = ((nbytes + gridDim.x - 1) / gridDim.x + 15) & ~(size_t)15;
  size_t b = per * blockIdx.x, e = b + per < nbytes ? b + per : nbytes;
  if (b >= nbytes) return;
  for (int i = 0; i < iters; ++i)
    dev::putmem_signal<dev::BLOCK>(s, data + b, src + b, e - b, sig, 1ull, BSHMEM_SIGNAL_ADD, peer);
}

// "swarm": every thread of the grid does its own get (THREAD_MULTIPLE use of the API).
__global__ void k_swarm_get(State s, char* local, const char* sym, size_t size, int peer) {
  size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  dev::getmem<dev::THREAD>(s, local + tid * size, sym + tid * size, size, peer);
}

// Functional sweep of the typed device API on one PE pair: writes a result code per check.
__global__ void k_api_selftest(State s, int* sym_i, unsigned long long* sym_u, float* sym_f, int peer, int* results) {
  int r = 0;
  if (threadIdx.x == 0) {
    // p / g
    dev::p<int>(s, sym_i, 1234, peer);
    dev::quiet(s);
    results[r++] = dev::g<int>(s, sym_i, peer) == 1234;
    // standard AMOs
    dev::atomic_set<unsigned long long>(s, sym_u, 10ull, peer);
    results[r++] = dev::atomic_fetch_add<unsigned long long>(s, sym_u, 5ull, peer) == 10ull;
    results[r++] = dev::atomic_fetch_inc<unsigned long long>(s, sym_u, peer) == 15ull;
    results[r++] = dev::atomic_fetch<unsigned long long>(s, sym_u, peer) == 16ull;
    results[r++] = dev::atomic_compare_swap<unsigned long long>(s, sym_u, 16ull, 100ull, peer) == 16ull;
    results[r++] = dev::atomic_compare_swap<unsigned long long>(s, sym_u, 16ull, 7ull, peer) == 100ull;   // no swap
    results[r++] = dev::atomic_swap<unsigned long long>(s, sym_u, 0xF0ull, peer) == 100ull;
    dev::atomic_add<unsigned long long>(s, sym_u, 0ull, peer);
    dev::atomic_inc<unsigned long long>(s, sym_u + 1, peer);
    // bitwise
    results[r++] = dev::atomic_fetch_and<unsigned long long>(s, sym_u, 0x3Cull, peer) == 0xF0ull;
    results[r++] = dev::atomic_fetch_or<unsigned long long>(s, sym_u, 0x03ull, peer) == 0x30ull;
    results[r++] = dev::atomic_fetch_xor<unsigned long long>(s, sym_u, 0xFFull, peer) == 0x33ull;
    dev::atomic_and<unsigned long long>(s, sym_u, 0xF0ull, peer);
    dev::atomic_or<unsigned long long>(s, sym_u, 0x01ull, peer);
    dev::atomic_xor<unsigned long long>(s, sym_u, 0x10ull, peer);
    results[r++] = dev::atomic_fetch<unsigned long long>(s, sym_u, peer) == 0xD1ull;
    // float extended AMOs
    dev::atomic_set<float>(s, sym_f, 1.5f, peer);
    results[r++] = dev::atomic_swap<float>(s, sym_f, 2.5f, peer) == 1.5f;
    results[r++] = dev::atomic_fetch<float>(s, sym_f, peer) == 2.5f;
    results[r++] = dev::atomic_fetch_add<float>(s, sym_f, 1.0f, peer) == 2.5f;
    // ptr() and test()
    int* remote = dev::ptr(s, sym_i, peer);
    results[r++] = remote != nullptr && *reinterpret_cast<volatile int*>(remote) == 1234;
    results[r++] = dev::test<int>(s, dev::ptr(s, sym_i, peer), BSHMEM_CMP_EQ, 1234) == 1;
    results[r++] = dev::test<int>(s, dev::ptr(s, sym_i, peer), BSHMEM_CMP_LT, 1000) == 0;
    results[r++] = -1;   // terminator
  }
}

// Block-scope work-group collectives called roc_shmem-style from a user kernel (one block per PE).
__global__ void k_wg_collectives(State s, float* dst, float* src, int n, int* status) {
  __shared__ dev::Ctx ctx;
  dev::wg_init();
  dev::wg_ctx_create(s, BSHMEM_CTX_WG_PRIVATE, &ctx);
  dev::Team world = dev::team_world(s);
  int rc = coll::wg_barrier_all(s);
  if (rc == BSHMEM_OK) rc = coll::wg_to_all<float>(s, world, BSHMEM_SUM, dst, src, n);
  if (rc == BSHMEM_OK) rc = coll::wg_sync_all(s);
  dev::wg_ctx_destroy(&ctx);
  dev::wg_finalize();
  if (threadIdx.x == 0) *status = rc;
}

BenchOut* pinned_out() {
  static thread_local BenchOut* p = nullptr;
  if (!p) cudaHostAlloc(&p, sizeof(BenchOut), cudaHostAllocMapped);
  return p;
}

int get_state(bshmem_handle_t h, State* st, cudaStream_t* stream) {
  int rc = bshmem_gpu_get_state(h, st);
  if (rc != BSHMEM_OK) return rc;
  void* s = nullptr;
  bshmem_gpu_get_stream(h, &s);
  *stream = static_cast<cudaStream_t>(s);
  return BSHMEM_OK;
}

int finish(cudaStream_t stream, BenchOut* o, uint64_t* ns) {
  if (cudaGetLastError() != cudaSuccess) return BSHMEM_ERR_CUDA;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return BSHMEM_ERR_CUDA;
  if (ns) *ns = o->ns;
  return o->status;
}

}  // namespace

extern "C" {

int bshmem_gpu_bench_pingpong(bshmem_handle_t h, void* flag_sym, int peer, int iters, int initiator, uint64_t* ns) {
  State st; cudaStream_t stream;
  int rc = get_state(h, &st, &stream);
  if (rc != BSHMEM_OK) return rc;
  BenchOut* o = pinned_out();
  o->ns = 0; o->status = 0;
  k_pingpong<<<1, 1, 0, stream>>>(st, static_cast<uint64_t*>(flag_sym), peer, iters, initiator, o);
  return finish(stream, o, ns);
}

int bshmem_gpu_bench_put_signal(bshmem_handle_t h, void* data_sym, void* sig_sym, uint64_t nbytes, int peer, int iters,
                                int initiator, int threads, uint64_t* ns) {
  State st; cudaStream_t stream;
  int rc = get_state(h, &st, &stream);
  if (rc != BSHMEM_OK) return rc;
  BenchOut* o = pinned_out();
  o->ns = 0; o->status = 0;
  k_put_signal_pingpong<<<1, threads, 0, stream>>>(st, static_cast<char*>(data_sym), static_cast<uint64_t*>(sig_sym), nbytes, peer,
                                                   iters, initiator, o);
  return finish(stream, o, ns);
}

int bshmem_gpu_bench_amo(bshmem_handle_t h, void* target_sym, int peer, int iters, int op, uint64_t* ns) {
  State st; cudaStream_t stream;
  int rc = get_state(h, &st, &stream);
  if (rc != BSHMEM_OK) return rc;
  BenchOut* o = pinned_out();
  o->ns = 0; o->status = 0;
  k_amo_latency<<<1, 1, 0, stream>>>(st, static_cast<unsigned long long*>(target_sym), peer, iters, op, o);
  return finish(stream, o, ns);
}

int bshmem_gpu_bench_msgrate(bshmem_handle_t h, void* dest_sym, const void* src, uint64_t size, int peer, int windows, int ctas,
                             int threads, uint64_t* ns) {
  State st; cudaStream_t stream;
  int rc = get_state(h, &st, &stream);
  if (rc != BSHMEM_OK) return rc;
  BenchOut* o = pinned_out();
  o->ns = 0; o->status = 0;
  k_put_msgrate<<<ctas, threads, 0, stream>>>(st, static_cast<char*>(dest_sym), static_cast<const char*>(src), size, peer, windows, o);
  return finish(stream, o, ns);
}

int bshmem_gpu_bench_amo_rate(bshmem_handle_t h, void* target_sym, int words, int peer, int iters, int ctas, int threads, uint64_t* ns) {
  State st; cudaStream_t stream;
  int rc = get_state(h, &st, &stream);
  if (rc != BSHMEM_OK) return rc;
  if (words < 1 || ctas < 1 || threads < 1 || threads > 1024) return BSHMEM_ERR_INVALID;
  BenchOut* o = pinned_out();
  o->ns = 0; o->status = 0;
  k_amo_rate<<<ctas, threads, 0, stream>>>(st, static_cast<unsigned long long*>(target_sym), words, peer, iters, o);
  return finish(stream, o, ns);
}

// Enqueues the one-way put-with-signal stream (time it with CUDA events around the call).
int bshmem_gpu_put_signal_stream(bshmem_handle_t h, void* data_sym, const void* src, void* sig_sym, uint64_t nbytes, int peer,
                                 int iters, int ctas, int threads) {
  State st; cudaStream_t stream;
  int rc = get_state(h, &st, &stream);
  if (rc != BSHMEM_OK) return rc;
  if (ctas < 1 || threads < 32 || threads > 1024) return BSHMEM_ERR_INVALID;
  k_put_signal_stream<<<ctas, threads, 0, stream>>>(st, static_cast<char*>(data_sym), static_cast<const char*>(src),
                                                    static_cast<uint64_t*>(sig_sym), nbytes, peer, iters);
  return cudaGetLastError() == cudaSuccess ? BSHMEM_OK : BSHMEM_ERR_CUDA;
}

int bshmem_gpu_swarm_get(bshmem_handle_t h, void* local, const void* sym, uint64_t size, int peer, int ctas, int threads) {
  State st; cudaStream_t stream;
  int rc = get_state(h, &st, &stream);
  if (rc != BSHMEM_OK) return rc;
  k_swarm_get<<<ctas, threads, 0, stream>>>(st, static_cast<char*>(local), static_cast<const char*>(sym), size, peer);
  if (cudaGetLastError() != cudaSuccess) return BSHMEM_ERR_CUDA;
  return cudaStreamSynchronize(stream) == cudaSuccess ? BSHMEM_OK : BSHMEM_ERR_CUDA;
}

// Runs the typed device API checks against `peer`; results[i] is 1/0 per check, -1 terminates.
int bshmem_gpu_api_selftest(bshmem_handle_t h, void* sym_i, void* sym_u, void* sym_f, int peer, int* results_dev) {
  State st; cudaStream_t stream;
  int rc = get_state(h, &st, &stream);
  if (rc != BSHMEM_OK) return rc;
  k_api_selftest<<<1, 32, 0, stream>>>(st, static_cast<int*>(sym_i), static_cast<unsigned long long*>(sym_u),
                                       static_cast<float*>(sym_f), peer, results_dev);
  if (cudaGetLastError() != cudaSuccess) return BSHMEM_ERR_CUDA;
  return cudaStreamSynchronize(stream) == cudaSuccess ? BSHMEM_OK : BSHMEM_ERR_CUDA;
}

// One block per PE calling the work-group collectives from inside a user kernel.
int bshmem_gpu_wg_collectives(bshmem_handle_t h, void* dst_sym, void* src_sym, int n, int* status_out) {
  State st; cudaStream_t stream;
  int rc = get_state(h, &st, &stream);
  if (rc != BSHMEM_OK) return rc;
  BenchOut* o = pinned_out();
  o->status = -1;
  k_wg_collectives<<<1, 256, 0, stream>>>(st, static_cast<float*>(dst_sym), static_cast<float*>(src_sym), n, &o->status);
  if (cudaGetLastError() != cudaSuccess) return BSHMEM_ERR_CUDA;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return BSHMEM_ERR_CUDA;
  if (status_out) *status_out = o->status;
  return BSHMEM_OK;
}

}  // extern "C"
