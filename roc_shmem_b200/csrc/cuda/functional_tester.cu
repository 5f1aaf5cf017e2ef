// functional_tester.cu — the kernels of the functional test driver: one timed, self-verifying kernel per family of
// device operations, selected by a test-type number and run over a sweep of message sizes by
// roc_shmem_b200/bench/functional.py.
//
// Every kernel follows the same protocol: each work-group (CTA) owns a slice of the buffers, runs `skip` untimed and
// `loops` timed iterations of the operation through a context (the world's, or a team's with team-relative PE
// numbers), completes them with quiet, and stores its elapsed %globaltimer nanoseconds in timers[wg].  The host
// brackets the launch with CUDA events; latency and message rate come from the device timers, bandwidth from the
// events.  A bounded wait that gives up stores the error code in *status and the kernel returns.
//
// Parity: the reference's single test binary and its test types (clients/functional_tests/tester.hpp:34-87,
// tester.cpp:494-616; primitive_tester.cpp, primitive_mr_tester.cpp, amo_standard_tester.cpp, ping_pong_tester.cpp,
// swarm_tester.cpp, random_access_tester.cpp, barrier_all_tester.cpp, sync_tester.cpp, reduction/broadcast/alltoall/
// fcollect testers, shmem_ptr_tester.cpp).  The type numbers are the ones its command line takes with -a.
#include <cuda_runtime.h>

#include "../host/runtime.h"
#include "../include/bshmem_coll.cuh"
#include "../include/bshmem_gpu.h"
#include "functional_tester.h"

using namespace bshmem;
using dev::State;
using DTeam = bshmem::dev::Team;
using ft::FtArgs;
using ft::ft_fail;

namespace {

enum FtType {
  FT_GET = 0, FT_GET_NBI = 1, FT_PUT = 2, FT_PUT_NBI = 3, FT_GET_SWARM = 4, FT_REDUCTION = 5,
  FT_AMO_FADD = 6, FT_AMO_FINC = 7, FT_AMO_FETCH = 8, FT_AMO_FCSWAP = 9, FT_AMO_ADD = 10, FT_AMO_INC = 11, FT_AMO_CSWAP = 12,
  FT_INIT = 13, FT_PING_PONG = 14, FT_RANDOM_ACCESS = 16, FT_BARRIER_ALL = 17, FT_SYNC_ALL = 18, FT_SYNC = 19,
  FT_BROADCAST = 20, FT_COLLECT = 21, FT_FCOLLECT = 22, FT_ALLTOALL = 23, FT_ALLTOALLS = 24, FT_SHMEM_PTR = 25, FT_P = 26, FT_G = 27,
  FT_WG_GET = 28, FT_WG_GET_NBI = 29, FT_WG_PUT = 30, FT_WG_PUT_NBI = 31,
  FT_WAVE_GET = 32, FT_WAVE_GET_NBI = 33, FT_WAVE_PUT = 34, FT_WAVE_PUT_NBI = 35,
  FT_TEAM_BROADCAST = 36, FT_TEAM_REDUCTION = 37,
  FT_TEAM_CTX_GET = 38, FT_TEAM_CTX_GET_NBI = 39, FT_TEAM_CTX_PUT = 40, FT_TEAM_CTX_PUT_NBI = 41, FT_TEAM_CTX_INFRA = 42,
  FT_PUT_NBI_MR = 43, FT_AMO_SET = 44, FT_AMO_SWAP = 45, FT_AMO_FAND = 46, FT_AMO_FOR = 47, FT_AMO_FXOR = 48,
  FT_AMO_AND = 49, FT_AMO_OR = 50, FT_AMO_XOR = 51,
  FT_PUT_SIGNAL = 52,          // OpenSHMEM 1.5 put-with-signal (no counterpart in the reference)
  FT_COUNT = 53
};

// ---- put / get at thread, warp and block scope, blocking and nbi (types 0-3, 28-35, 38-41) ----------------------
template <dev::Scope S, bool kPut, bool kNbi>
__global__ void k_ft_rma(State s, DTeam team, FtArgs a) {
  __shared__ dev::Ctx ctx;
  dev::wg_init();
  if (dev::wg_team_create_ctx(s, team, a.ctx_options, &ctx) != BSHMEM_OK) { if (threadIdx.x == 0) ft_fail(a, BSHMEM_ERR_INVALID); return; }
  const bool active = S == dev::BLOCK || (S == dev::WARP && threadIdx.x < 32) || (S == dev::THREAD && threadIdx.x == 0);
  char* remote = a.sym_a + (size_t)blockIdx.x * a.size;
  char* mine = a.local + (size_t)blockIdx.x * a.size;
  unsigned long long t0 = 0;
  for (int i = 0; i < a.skip + a.loops; ++i) {
    if (i == a.skip) { if (S == dev::BLOCK) __syncthreads(); t0 = dev::timer(); }
    if (active) {
      if (kPut) {
        if (kNbi) dev::ctx_putmem_nbi<S>(s, ctx, remote, mine, a.size, a.peer);
        else dev::ctx_putmem<S>(s, ctx, remote, mine, a.size, a.peer);
      } else {
        if (kNbi) dev::ctx_getmem_nbi<S>(s, ctx, mine, remote, a.size, a.peer);
        else dev::ctx_getmem<S>(s, ctx, mine, remote, a.size, a.peer);
      }
    }
  }
  if (active) dev::ctx_quiet(s, ctx);
  if (S == dev::BLOCK) __syncthreads();
  if (threadIdx.x == 0) a.timers[blockIdx.x] = dev::timer() - t0;
  dev::wg_ctx_destroy(&ctx);
  dev::wg_finalize();
}

// ---- p / g (types 26, 27): thread 0 of each work-group moves one element of 1, 2, 4 or 8 bytes --------------------
template <typename T>
__device__ __forceinline__ void ft_pg_loop(const State& s, const dev::Ctx& ctx, const FtArgs& a, bool is_p, unsigned long long* t0) {
  T* remote = reinterpret_cast<T*>(a.sym_a + (size_t)blockIdx.x * 8);
  T* mine = reinterpret_cast<T*>(a.local + (size_t)blockIdx.x * 8);
  T acc = 0;
  for (int i = 0; i < a.skip + a.loops; ++i) {
    if (i == a.skip) *t0 = dev::timer();
    if (is_p) dev::ctx_p<T>(s, ctx, remote, (T)0x5A, a.peer);
    else acc = (T)(acc + dev::ctx_g<T>(s, ctx, remote, a.peer));
  }
  if (!is_p) *mine = dev::ctx_g<T>(s, ctx, remote, a.peer) + (T)(acc - acc);
}
__global__ void k_ft_pg(State s, DTeam team, FtArgs a) {
  __shared__ dev::Ctx ctx;
  dev::wg_team_create_ctx(s, team, a.ctx_options, &ctx);
  if (threadIdx.x != 0) return;
  unsigned long long t0 = 0;
  const bool is_p = a.type == FT_P;
  switch (a.size) {
    case 1: ft_pg_loop<unsigned char>(s, ctx, a, is_p, &t0); break;
    case 2: ft_pg_loop<unsigned short>(s, ctx, a, is_p, &t0); break;
    case 4: ft_pg_loop<unsigned int>(s, ctx, a, is_p, &t0); break;
    default: ft_pg_loop<unsigned long long>(s, ctx, a, is_p, &t0); break;
  }
  dev::ctx_quiet(s, ctx);
  a.timers[blockIdx.x] = dev::timer() - t0;
}

// ---- atomics (types 6-12, 44-51): every thread of every work-group issues; word 0 is shared, compare-swap chains
//      run on a word per thread so that each has a closed-form result ----------------------------------------------------
__global__ void k_ft_amo(State s, DTeam team, FtArgs a) {
  __shared__ dev::Ctx ctx;
  dev::wg_team_create_ctx(s, team, a.ctx_options, &ctx);
  using U = unsigned long long;
  U* shared_word = a.words;
  U* own_word = a.words + 64 + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  U sink = 0;
  unsigned long long t0 = 0;
  const int pe = a.peer;
  for (int i = 0; i < a.skip + a.loops; ++i) {
    if (i == a.skip) { __syncthreads(); t0 = dev::timer(); }
    switch (a.type) {
      case FT_AMO_FADD: sink += dev::ctx_atomic_fetch_add<U>(s, ctx, shared_word, 2ull, pe); break;
      case FT_AMO_FINC: sink += dev::ctx_atomic_fetch_inc<U>(s, ctx, shared_word, pe); break;
      case FT_AMO_FETCH: sink += dev::ctx_atomic_fetch<U>(s, ctx, shared_word, pe); break;
      case FT_AMO_FCSWAP: sink += dev::ctx_atomic_compare_swap<U>(s, ctx, own_word, (U)i, (U)i + 1, pe); break;
      case FT_AMO_ADD: dev::ctx_atomic_add<U>(s, ctx, shared_word, 2ull, pe); break;
      case FT_AMO_INC: dev::ctx_atomic_inc<U>(s, ctx, shared_word, pe); break;
      case FT_AMO_CSWAP: (void)dev::ctx_atomic_compare_swap<U>(s, ctx, own_word, (U)i, (U)i + 1, pe); break;
      case FT_AMO_SET: dev::ctx_atomic_set<U>(s, ctx, shared_word, 44ull, pe); break;
      case FT_AMO_SWAP: sink += dev::ctx_atomic_swap<U>(s, ctx, shared_word, 45ull, pe); break;
      case FT_AMO_FAND: sink += dev::ctx_atomic_fetch_and<U>(s, ctx, shared_word, 0x0Full, pe); break;
      case FT_AMO_FOR: sink += dev::ctx_atomic_fetch_or<U>(s, ctx, shared_word, 0xF0ull, pe); break;
      case FT_AMO_FXOR: sink += dev::ctx_atomic_fetch_xor<U>(s, ctx, shared_word, 1ull, pe); break;
      case FT_AMO_AND: dev::ctx_atomic_and<U>(s, ctx, shared_word, 0x0Full, pe); break;
      case FT_AMO_OR: dev::ctx_atomic_or<U>(s, ctx, shared_word, 0xF0ull, pe); break;
      default: dev::ctx_atomic_xor<U>(s, ctx, shared_word, 1ull, pe); break;
    }
  }
  dev::ctx_quiet(s, ctx);
  __syncthreads();
  if (threadIdx.x == 0) a.timers[blockIdx.x] = dev::timer() - t0;
  if (sink == 0x7fffffffffffffffull) a.local[0] = 1;   // keeps the fetched values alive
}

// ---- ping-pong (type 14): p + wait_until on a flag per work-group; both PEs launch --------------------------------
__global__ void k_ft_pingpong(State s, DTeam team, FtArgs a) {
  __shared__ dev::Ctx ctx;
  dev::wg_team_create_ctx(s, team, a.ctx_options, &ctx);
  if (threadIdx.x != 0) return;
  unsigned long long* flag = a.words + blockIdx.x;
  unsigned long long t0 = 0;
  int rc = BSHMEM_OK;
  for (int i = 1; i <= a.skip + a.loops && rc == BSHMEM_OK; ++i) {
    if (i == a.skip + 1) t0 = dev::timer();
    if (a.initiator) {
      dev::ctx_p<unsigned long long>(s, ctx, flag, (unsigned long long)i, a.peer);
      rc = dev::wait_until<unsigned long long>(s, flag, BSHMEM_CMP_EQ, (unsigned long long)i);
    } else {
      rc = dev::wait_until<unsigned long long>(s, flag, BSHMEM_CMP_EQ, (unsigned long long)i);
      dev::ctx_p<unsigned long long>(s, ctx, flag, (unsigned long long)i, a.peer);
    }
  }
  a.timers[blockIdx.x] = dev::timer() - t0;
  ft_fail(a, rc);
}

// ---- put-with-signal stream (type 52): the initiator's work-groups send `loops` messages that each add 1 to the
//      work-group's signal word; the target's work-groups wait for the full count --------------------------------------
__global__ void k_ft_put_signal(State s, DTeam team, FtArgs a) {
  __shared__ dev::Ctx ctx;
  dev::wg_team_create_ctx(s, team, a.ctx_options, &ctx);
  unsigned long long* sig = a.words + blockIdx.x;
  char* remote = a.sym_a + (size_t)blockIdx.x * a.size;
  char* mine = a.local + (size_t)blockIdx.x * a.size;
  unsigned long long t0 = 0;
  if (a.initiator) {
    for (int i = 0; i < a.skip + a.loops; ++i) {
      if (i == a.skip) { __syncthreads(); t0 = dev::timer(); }
      dev::ctx_putmem_signal<dev::BLOCK>(s, ctx, remote, mine, a.size, reinterpret_cast<uint64_t*>(sig), 1ull, BSHMEM_SIGNAL_ADD, a.peer);
    }
    if (threadIdx.x == 0) dev::ctx_quiet(s, ctx);
  } else if (threadIdx.x == 0) {
    t0 = dev::timer();
    ft_fail(a, dev::wait_until<unsigned long long>(s, sig, BSHMEM_CMP_GE, (unsigned long long)(a.skip + a.loops)));
  }
  __syncthreads();
  if (threadIdx.x == 0) a.timers[blockIdx.x] = dev::timer() - t0;
}

// ---- put_nbi message rate (type 43): windows of 64 non-blocking puts closed by one quiet --------------------------
__global__ void k_ft_put_mr(State s, DTeam team, FtArgs a) {
  __shared__ dev::Ctx ctx;
  dev::wg_team_create_ctx(s, team, a.ctx_options, &ctx);
  if (threadIdx.x != 0) return;
  char* remote = a.sym_a + (size_t)blockIdx.x * a.size;
  char* mine = a.local + (size_t)blockIdx.x * a.size;
  unsigned long long t0 = 0;
  for (int i = 0; i < a.skip + a.loops; ++i) {
    if (i == a.skip) t0 = dev::timer();
    for (int j = 0; j < 64; ++j) dev::ctx_putmem_nbi(s, ctx, remote, mine, a.size, a.peer);
    dev::ctx_quiet(s, ctx);
  }
  a.timers[blockIdx.x] = dev::timer() - t0;
}

// ---- swarm get (type 4): every thread of every work-group gets its own slice --------------------------------------
__global__ void k_ft_swarm(State s, DTeam team, FtArgs a) {
  __shared__ dev::Ctx ctx;
  dev::wg_team_create_ctx(s, team, a.ctx_options, &ctx);
  const size_t slice = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * a.size;
  unsigned long long t0 = 0;
  for (int i = 0; i < a.skip + a.loops; ++i) {
    if (i == a.skip) { __syncthreads(); t0 = dev::timer(); }
    dev::ctx_getmem(s, ctx, a.local + slice, a.sym_a + slice, a.size, a.peer);
  }
  dev::ctx_quiet(s, ctx);
  __syncthreads();
  if (threadIdx.x == 0) a.timers[blockIdx.x] = dev::timer() - t0;
}

// ---- random access (type 16): every thread puts `size` bytes into pseudo-random bins of the peer's buffer; the
//      content of a bin depends only on the bin, so any interleaving leaves the same bytes ----------------------------
__device__ __forceinline__ unsigned ft_lcg(unsigned x) { return x * 1664525u + 1013904223u; }
__global__ void k_ft_random(State s, DTeam team, FtArgs a, unsigned n_bins) {
  __shared__ dev::Ctx ctx;
  dev::wg_team_create_ctx(s, team, a.ctx_options, &ctx);
  unsigned x = ft_lcg(blockIdx.x * blockDim.x + threadIdx.x + 12345u);
  unsigned long long t0 = 0;
  for (int i = 0; i < a.skip + a.loops; ++i) {
    if (i == a.skip) { __syncthreads(); t0 = dev::timer(); }
    x = ft_lcg(x);
    const unsigned bin = (x >> 8) % n_bins;
    dev::ctx_putmem_nbi(s, ctx, a.sym_a + (size_t)bin * a.size, a.local + (size_t)bin * a.size, a.size, a.peer);
  }
  dev::ctx_quiet(s, ctx);
  __syncthreads();
  if (threadIdx.x == 0) a.timers[blockIdx.x] = dev::timer() - t0;
}

// ---- barrier_all / sync_all / team sync (types 17-19): one channel per work-group ---------------------------------
__global__ void k_ft_sync(State s, DTeam team, FtArgs a) {
  unsigned long long t0 = 0;
  int rc = BSHMEM_OK;
  const DTeam world = dev::team_world(s);
  for (int i = 0; i < a.skip + a.loops && rc == BSHMEM_OK; ++i) {
    if (i == a.skip) t0 = dev::timer();
    if (a.type == FT_BARRIER_ALL) rc = coll::team_barrier(s, world, blockIdx.x);
    else if (a.type == FT_SYNC_ALL) rc = coll::team_sync(s, world, blockIdx.x);
    else rc = coll::team_sync(s, team, blockIdx.x);
  }
  if (threadIdx.x == 0) { a.timers[blockIdx.x] = dev::timer() - t0; ft_fail(a, rc); }
}

// ---- shmem_ptr (type 25) and init (type 13) ------------------------------------------------------------------------
__global__ void k_ft_ptr(State s, DTeam team, FtArgs a) {
  __shared__ dev::Ctx ctx;
  int provided = -1;
  dev::wg_init_thread(BSHMEM_THREAD_MULTIPLE, &provided);
  dev::wg_team_create_ctx(s, team, a.ctx_options, &ctx);
  if (threadIdx.x == 0) {
    const unsigned long long t0 = dev::timer();
    int ok = provided == BSHMEM_THREAD_MULTIPLE && dev::query_thread() == BSHMEM_THREAD_MULTIPLE;
    if (a.type == FT_SHMEM_PTR) {
      unsigned long long* w = a.words + blockIdx.x;
      unsigned long long* rp = dev::ctx_ptr(s, ctx, w, a.peer);
      unsigned long long* lp = dev::ctx_ptr(s, ctx, w, dev::ctx_my_pe(ctx));
      ok = ok && rp != nullptr && lp == w;
      if (rp) { *rp = 0xC0FFEEull + blockIdx.x; dev::ctx_quiet(s, ctx); ok = ok && dev::ctx_g<unsigned long long>(s, ctx, w, a.peer) == 0xC0FFEEull + blockIdx.x; }
    }
    a.timers[blockIdx.x] = dev::timer() - t0;
    if (!ok) ft_fail(a, BSHMEM_ERR_INVALID);
  }
  dev::wg_ctx_destroy(&ctx);
  dev::wg_finalize();
}

template <dev::Scope S>
void launch_rma(bool put, bool nbi, int wgs, int wg_size, cudaStream_t st, const State& s, const DTeam& t, const FtArgs& a) {
  if (put) {
    if (nbi) k_ft_rma<S, true, true><<<wgs, wg_size, 0, st>>>(s, t, a);
    else k_ft_rma<S, true, false><<<wgs, wg_size, 0, st>>>(s, t, a);
  } else {
    if (nbi) k_ft_rma<S, false, true><<<wgs, wg_size, 0, st>>>(s, t, a);
    else k_ft_rma<S, false, false><<<wgs, wg_size, 0, st>>>(s, t, a);
  }
}

}  // namespace

extern "C" {

// Launches the kernel of test `type` once on the PE's stream and waits for it.
//   team_slot    team of the context (0 = world); `peer` is relative to it
//   sym_a/sym_b  symmetric buffers; local_dev: private device buffer; words: symmetric 8-byte words
//   timers_dev   [wgs] elapsed nanoseconds of the timed iterations per work-group; status_dev: first error code
//   n_bins       random access only: bins of `size` bytes in sym_a / local_dev
//   kernel_ms    CUDA-event time of the launch
// The caller sizes the buffers for the type (roc_shmem_b200/bench/functional.py holds the table).
int bshmem_gpu_functional_run(bshmem_handle_t h, int type, int team_slot, int peer, int wgs, int wg_size, int loops, int skip,
                              uint64_t size, void* sym_a, void* sym_b, void* local_dev, void* words, void* timers_dev, int* status_dev,
                              long ctx_options, int initiator, unsigned n_bins, float* kernel_ms) {
  State st;
  int rc = bshmem_gpu_get_state(h, &st);
  if (rc != BSHMEM_OK) return rc;
  if (type < 0 || type >= FT_COUNT || type == 15 || wgs < 1 || wg_size < 1 || wg_size > 1024 || loops < 1 || skip < 0)
    return BSHMEM_ERR_INVALID;
  DTeam t;
  t.my_idx = bshmem_team_my_pe(h, team_slot);
  t.size = bshmem_team_n_pes(h, team_slot);
  if (t.my_idx < 0 || t.size < 1 || peer < 0 || peer >= t.size) return BSHMEM_ERR_INVALID;
  t.slot = team_slot; t.reserved = 0; t.psync = nullptr;
  t.pe_start = bshmem_team_translate_pe(h, team_slot, 0, BSHMEM_TEAM_WORLD);
  t.stride = t.size > 1 ? bshmem_team_translate_pe(h, team_slot, 1, BSHMEM_TEAM_WORLD) - t.pe_start : 1;
  void* sv = nullptr;
  bshmem_gpu_get_stream(h, &sv);
  cudaStream_t stream = static_cast<cudaStream_t>(sv);
  FtArgs a;
  a.type = type; a.loops = loops; a.skip = skip; a.peer = peer; a.size = size;
  a.sym_a = static_cast<char*>(sym_a); a.sym_b = static_cast<char*>(sym_b); a.local = static_cast<char*>(local_dev);
  a.words = static_cast<unsigned long long*>(words); a.timers = static_cast<unsigned long long*>(timers_dev);
  a.status = status_dev; a.ctx_options = ctx_options; a.initiator = initiator;
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return BSHMEM_ERR_CUDA;
  cudaEventRecord(e0, stream);
  switch (type) {
    case FT_GET: case FT_TEAM_CTX_GET: launch_rma<dev::THREAD>(false, false, wgs, wg_size, stream, st, t, a); break;
    case FT_GET_NBI: case FT_TEAM_CTX_GET_NBI: launch_rma<dev::THREAD>(false, true, wgs, wg_size, stream, st, t, a); break;
    case FT_PUT: case FT_TEAM_CTX_PUT: launch_rma<dev::THREAD>(true, false, wgs, wg_size, stream, st, t, a); break;
    case FT_PUT_NBI: case FT_TEAM_CTX_PUT_NBI: launch_rma<dev::THREAD>(true, true, wgs, wg_size, stream, st, t, a); break;
    case FT_WG_GET: launch_rma<dev::BLOCK>(false, false, wgs, wg_size, stream, st, t, a); break;
    case FT_WG_GET_NBI: launch_rma<dev::BLOCK>(false, true, wgs, wg_size, stream, st, t, a); break;
    case FT_WG_PUT: launch_rma<dev::BLOCK>(true, false, wgs, wg_size, stream, st, t, a); break;
    case FT_WG_PUT_NBI: launch_rma<dev::BLOCK>(true, true, wgs, wg_size, stream, st, t, a); break;
    case FT_WAVE_GET: launch_rma<dev::WARP>(false, false, wgs, wg_size, stream, st, t, a); break;
    case FT_WAVE_GET_NBI: launch_rma<dev::WARP>(false, true, wgs, wg_size, stream, st, t, a); break;
    case FT_WAVE_PUT: launch_rma<dev::WARP>(true, false, wgs, wg_size, stream, st, t, a); break;
    case FT_WAVE_PUT_NBI: launch_rma<dev::WARP>(true, true, wgs, wg_size, stream, st, t, a); break;
    case FT_P: case FT_G: k_ft_pg<<<wgs, wg_size, 0, stream>>>(st, t, a); break;
    case FT_PING_PONG: k_ft_pingpong<<<wgs, wg_size, 0, stream>>>(st, t, a); break;
    case FT_PUT_SIGNAL: k_ft_put_signal<<<wgs, wg_size, 0, stream>>>(st, t, a); break;
    case FT_PUT_NBI_MR: k_ft_put_mr<<<wgs, wg_size, 0, stream>>>(st, t, a); break;
    case FT_GET_SWARM: k_ft_swarm<<<wgs, wg_size, 0, stream>>>(st, t, a); break;
    case FT_RANDOM_ACCESS:
      if (n_bins < 1) { rc = BSHMEM_ERR_INVALID; break; }
      k_ft_random<<<wgs, wg_size, 0, stream>>>(st, t, a, n_bins);
      break;
    case FT_BARRIER_ALL: case FT_SYNC_ALL: case FT_SYNC:
      if (wgs > BSHMEM_MAX_COLL_CTAS) { rc = BSHMEM_ERR_INVALID; break; }
      k_ft_sync<<<wgs, wg_size, 0, stream>>>(st, t, a);
      break;
    case FT_REDUCTION: case FT_TEAM_REDUCTION: case FT_BROADCAST: case FT_TEAM_BROADCAST: case FT_FCOLLECT: case FT_COLLECT:
    case FT_ALLTOALL: case FT_ALLTOALLS:
      if (wgs != 1 || size % 4 || wg_size > 256) { rc = BSHMEM_ERR_INVALID; break; }
      ft::launch_coll((type == FT_REDUCTION || type == FT_TEAM_REDUCTION) ? 0 : (type == FT_BROADCAST || type == FT_TEAM_BROADCAST) ? 1
                      : (type == FT_FCOLLECT || type == FT_COLLECT) ? 2 : 3, wg_size, stream, e0, st, t, a);
      break;
    case FT_INIT: case FT_SHMEM_PTR: case FT_TEAM_CTX_INFRA: k_ft_ptr<<<wgs, wg_size, 0, stream>>>(st, t, a); break;
    default: k_ft_amo<<<wgs, wg_size, 0, stream>>>(st, t, a); break;
  }
  cudaEventRecord(e1, stream);
  if (rc == BSHMEM_OK && cudaGetLastError() != cudaSuccess) rc = BSHMEM_ERR_CUDA;
  if (cudaStreamSynchronize(stream) != cudaSuccess) rc = BSHMEM_ERR_CUDA;
  float ms = 0.f;
  if (rc == BSHMEM_OK && cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess) rc = BSHMEM_ERR_CUDA;
  if (kernel_ms) *kernel_ms = ms;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return rc;
}

}  // extern "C"
