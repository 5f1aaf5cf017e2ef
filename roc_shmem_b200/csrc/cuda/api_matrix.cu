// api_matrix.cu — ONE functional matrix of the device API, instantiated for both transports and run with either a
// default (world) context or a team context:
//   direct  — dev:: / coll:: (loads, stores and atomics on the NVLink peer mapping)
//   proxy   — proxy:: (every operation is a descriptor executed by the PE's CPU service thread)
// p / g, the 15 atomics, put / get at thread, warp and block scope (blocking and nbi), put-with-signal, fence, quiet,
// context queries, and the work-group collectives of the context's team.  PE arguments are relative to the context's
// team.  Each check writes 1 (pass) or 0 into results[]; -1 terminates the list.
//
// Parity: the reference's functional tester types 0-12, 20-31, 36-51 (clients/functional_tests/tester.hpp:34-87),
// which it runs once per backend build and per context type; here the same kernel body serves all four combinations.
#include <cuda_runtime.h>

#include "../host/runtime.h"
#include "../include/bshmem_coll.cuh"
#include "../include/bshmem_gpu.h"
#include "../include/bshmem_proxy_device.cuh"

using namespace bshmem;
using dev::State;
using DTeam = bshmem::dev::Team;

namespace {

struct MatrixArgs {
  int* sym_i;                  // >= 4 ints
  unsigned long long* sym_u;   // >= 4 words
  float* sym_f;                // >= 4 floats
  char* data_sym;              // >= 3 * nbytes, symmetric
  char* local;                 // >= 6 * nbytes, device memory of this PE
  float* coll_src;             // symmetric, 64 * MAX_PES floats
  float* coll_dst;             // symmetric, 64 * MAX_PES floats
  int nbytes;                  // payload of each RMA check (multiple of 16)
  int peer;                    // target, relative to the context's team
};

// A is `dev` or `proxy`; C is the namespace of the context collectives (`coll` or `proxy`).
#define BSHMEM_API_MATRIX_BODY(A, C)                                                                                          \
  __shared__ dev::Ctx ctx;                                                                                                    \
  __shared__ int block_ok;                                                                                                    \
  dev::wg_init();                                                                                                             \
  dev::wg_team_create_ctx(s, team, BSHMEM_CTX_WG_PRIVATE, &ctx);                                                              \
  const int peer = m.peer, n = m.nbytes;                                                                                      \
  const int tid = threadIdx.x;                                                                                                \
  int r = 0;                                                                                                                  \
  /* ---- single-thread section: p / g, atomics, context queries ---- */                                                     \
  if (tid == 0) {                                                                                                             \
    results[r++] = dev::ctx_my_pe(ctx) == team.my_idx && dev::ctx_n_pes(ctx) == team.size;                                    \
    A::ctx_p<int>(s, ctx, m.sym_i, 1234, peer);                                                                               \
    A::ctx_quiet(s, ctx);                                                                                                     \
    results[r++] = A::ctx_g<int>(s, ctx, m.sym_i, peer) == 1234;                                                              \
    A::ctx_atomic_set<unsigned long long>(s, ctx, m.sym_u, 10ull, peer);                                                      \
    results[r++] = A::ctx_atomic_fetch_add<unsigned long long>(s, ctx, m.sym_u, 5ull, peer) == 10ull;                         \
    results[r++] = A::ctx_atomic_fetch_inc<unsigned long long>(s, ctx, m.sym_u, peer) == 15ull;                               \
    results[r++] = A::ctx_atomic_fetch<unsigned long long>(s, ctx, m.sym_u, peer) == 16ull;                                   \
    results[r++] = A::ctx_atomic_compare_swap<unsigned long long>(s, ctx, m.sym_u, 16ull, 100ull, peer) == 16ull;             \
    results[r++] = A::ctx_atomic_compare_swap<unsigned long long>(s, ctx, m.sym_u, 16ull, 7ull, peer) == 100ull;              \
    results[r++] = A::ctx_atomic_swap<unsigned long long>(s, ctx, m.sym_u, 0xF0ull, peer) == 100ull;                          \
    A::ctx_atomic_add<unsigned long long>(s, ctx, m.sym_u, 0ull, peer);                                                       \
    A::ctx_atomic_inc<unsigned long long>(s, ctx, m.sym_u + 1, peer);                                                         \
    results[r++] = A::ctx_atomic_fetch_and<unsigned long long>(s, ctx, m.sym_u, 0x3Cull, peer) == 0xF0ull;                    \
    results[r++] = A::ctx_atomic_fetch_or<unsigned long long>(s, ctx, m.sym_u, 0x03ull, peer) == 0x30ull;                     \
    results[r++] = A::ctx_atomic_fetch_xor<unsigned long long>(s, ctx, m.sym_u, 0xFFull, peer) == 0x33ull;                    \
    A::ctx_atomic_and<unsigned long long>(s, ctx, m.sym_u, 0xF0ull, peer);                                                    \
    A::ctx_atomic_or<unsigned long long>(s, ctx, m.sym_u, 0x01ull, peer);                                                     \
    A::ctx_atomic_xor<unsigned long long>(s, ctx, m.sym_u, 0x10ull, peer);                                                    \
    results[r++] = A::ctx_atomic_fetch<unsigned long long>(s, ctx, m.sym_u, peer) == 0xD1ull;                                 \
    /* 4-byte atomics and float extended atomics */                                                                          \
    A::ctx_atomic_set<int>(s, ctx, m.sym_i + 1, 7, peer);                                                                     \
    results[r++] = A::ctx_atomic_fetch_add<int>(s, ctx, m.sym_i + 1, 3, peer) == 7;                                           \
    results[r++] = A::ctx_atomic_fetch<int>(s, ctx, m.sym_i + 1, peer) == 10;                                                 \
    A::ctx_atomic_set<float>(s, ctx, m.sym_f, 1.5f, peer);                                                                    \
    results[r++] = A::ctx_atomic_swap<float>(s, ctx, m.sym_f, 2.5f, peer) == 1.5f;                                            \
    results[r++] = A::ctx_atomic_fetch<float>(s, ctx, m.sym_f, peer) == 2.5f;                                                 \
    A::ctx_fence(s, ctx);                                                                                                     \
  }                                                                                                                           \
  r = 16;                                                                                                                     \
  /* ---- RMA at block, warp and thread scope: put local[0:n) -> peer, get it back into local[k*n..), compare ---- */         \
  for (int i = tid; i < n; i += blockDim.x) m.local[i] = (char)(i * 7 + 3 + team.my_idx);                                     \
  if (tid == 0) block_ok = 1;                                                                                                 \
  __syncthreads();                                                                                                            \
  A::ctx_putmem<dev::BLOCK>(s, ctx, m.data_sym, m.local, n, peer);                                                            \
  if (tid == 0) A::ctx_quiet(s, ctx);                                                                                         \
  __syncthreads();                                                                                                            \
  A::ctx_getmem<dev::BLOCK>(s, ctx, m.local + n, m.data_sym, n, peer);                                                        \
  __syncthreads();                                                                                                            \
  for (int i = tid; i < n; i += blockDim.x)                                                                                   \
    if (reinterpret_cast<volatile char*>(m.local)[n + i] != m.local[i]) block_ok = 0;                                         \
  __syncthreads();                                                                                                            \
  if (tid == 0) { results[r] = block_ok; block_ok = 1; }                                                                      \
  ++r;                                                                                                                        \
  __syncthreads();                                                                                                            \
  if (tid < 32) {                                                                                                             \
    A::ctx_putmem_nbi<dev::WARP>(s, ctx, m.data_sym + n, m.local, n, peer);                                                   \
    if (tid == 0) A::ctx_quiet(s, ctx);                                                                                       \
    __syncwarp();                                                                                                             \
    A::ctx_getmem_nbi<dev::WARP>(s, ctx, m.local + 2 * n, m.data_sym + n, n, peer);                                           \
    if (tid == 0) A::ctx_quiet(s, ctx);                                                                                       \
    __syncwarp();                                                                                                             \
    for (int i = tid; i < n; i += 32)                                                                                         \
      if (reinterpret_cast<volatile char*>(m.local)[2 * n + i] != m.local[i]) block_ok = 0;                                   \
  }                                                                                                                           \
  __syncthreads();                                                                                                            \
  if (tid == 0) {                                                                                                             \
    results[r] = block_ok;                                                                                                    \
    A::ctx_putmem<dev::THREAD>(s, ctx, m.data_sym + 2 * n, m.local, n, peer);                                                 \
    A::ctx_quiet(s, ctx);                                                                                                     \
    A::ctx_getmem<dev::THREAD>(s, ctx, m.local + 3 * n, m.data_sym + 2 * n, n, peer);                                         \
    int same = 1;                                                                                                             \
    for (int i = 0; i < n; ++i) same &= reinterpret_cast<volatile char*>(m.local)[3 * n + i] == m.local[i];                   \
    results[r + 1] = same;                                                                                                    \
    block_ok = 1;                                                                                                             \
  }                                                                                                                           \
  r += 2;                                                                                                                     \
  __syncthreads();                                                                                                            \
  /* ---- put-with-signal (block scope): payload then signal += 5 on the peer; read both back ---- */                         \
  for (int i = tid; i < n; i += blockDim.x) m.local[4 * n + i] = (char)(i * 5 + 1);                                           \
  __syncthreads();                                                                                                            \
  A::ctx_putmem_signal<dev::BLOCK>(s, ctx, m.data_sym, m.local + 4 * n, n, reinterpret_cast<uint64_t*>(m.sym_u + 2), 5ull,    \
                                   BSHMEM_SIGNAL_ADD, peer);                                                                  \
  __syncthreads();                                                                                                            \
  if (tid == 0) {                                                                                                             \
    results[r] = A::ctx_atomic_fetch<unsigned long long>(s, ctx, m.sym_u + 2, peer) % 5ull == 0ull &&                         \
                 A::ctx_atomic_fetch<unsigned long long>(s, ctx, m.sym_u + 2, peer) >= 5ull;                                  \
  }                                                                                                                           \
  ++r;                                                                                                                        \
  A::ctx_getmem<dev::BLOCK>(s, ctx, m.local + 5 * n, m.data_sym, n, peer);                                                    \
  __syncthreads();                                                                                                            \
  for (int i = tid; i < n; i += blockDim.x)                                                                                   \
    if (reinterpret_cast<volatile char*>(m.local)[5 * n + i] != m.local[4 * n + i]) block_ok = 0;                             \
  __syncthreads();                                                                                                            \
  if (tid == 0) results[r] = block_ok;                                                                                        \
  ++r;                                                                                                                        \
  /* ---- work-group collectives on the context's team ---- */                                                               \
  const int P = team.size, me = team.my_idx;                                                                                  \
  for (int i = tid; i < 64 * P; i += blockDim.x) { m.coll_src[i] = (float)((me + 1) * ((i % 64) + 1)); m.coll_dst[i] = -1.f; } \
  __syncthreads();                                                                                                            \
  int rc = C::ctx_wg_team_sync(s, ctx);                                                                                       \
  if (rc == BSHMEM_OK) rc = C::ctx_wg_to_all<float>(s, ctx, BSHMEM_SUM, m.coll_dst, m.coll_src, 64);                          \
  if (tid == 0) {                                                                                                             \
    int good = rc == BSHMEM_OK;                                                                                               \
    for (int i = 0; i < 64; ++i) good &= reinterpret_cast<volatile float*>(m.coll_dst)[i] == (float)((i + 1) * P * (P + 1) / 2); \
    results[r] = good;                                                                                                        \
  }                                                                                                                           \
  ++r;                                                                                                                        \
  __syncthreads();                                                                                                            \
  rc = C::ctx_wg_fcollect<float>(s, ctx, m.coll_dst, m.coll_src, 64);                                                         \
  if (tid == 0) {                                                                                                             \
    int good = rc == BSHMEM_OK;                                                                                               \
    for (int k = 0; k < P; ++k)                                                                                               \
      for (int i = 0; i < 64; ++i) good &= reinterpret_cast<volatile float*>(m.coll_dst)[k * 64 + i] == (float)((k + 1) * (i + 1)); \
    results[r] = good;                                                                                                        \
  }                                                                                                                           \
  ++r;                                                                                                                        \
  __syncthreads();                                                                                                            \
  /* alltoall: block j of my source carries (me + 1) * 1000 + j */                                                           \
  for (int i = tid; i < 64 * P; i += blockDim.x) m.coll_src[i] = (float)((me + 1) * 1000 + i / 64);                           \
  __syncthreads();                                                                                                            \
  rc = C::ctx_wg_alltoall<float>(s, ctx, m.coll_dst, m.coll_src, 64);                                                         \
  if (tid == 0) {                                                                                                             \
    int good = rc == BSHMEM_OK;                                                                                               \
    for (int k = 0; k < P; ++k) good &= reinterpret_cast<volatile float*>(m.coll_dst)[k * 64 + 5] == (float)((k + 1) * 1000 + me); \
    results[r] = good;                                                                                                        \
  }                                                                                                                           \
  ++r;                                                                                                                        \
  __syncthreads();                                                                                                            \
  /* broadcast from the team's last member: the root's dest stays as it was */                                               \
  for (int i = tid; i < 64; i += blockDim.x) { m.coll_src[i] = (float)(me * 10 + 1); m.coll_dst[i] = -3.f; }                  \
  __syncthreads();                                                                                                            \
  rc = C::ctx_wg_broadcast<float>(s, ctx, m.coll_dst, m.coll_src, 64, P - 1);                                                 \
  if (tid == 0) {                                                                                                             \
    const float want = me == P - 1 ? -3.f : (float)((P - 1) * 10 + 1);                                                        \
    results[r] = rc == BSHMEM_OK && reinterpret_cast<volatile float*>(m.coll_dst)[63] == want;                                \
    results[r + 1] = -1;                                                                                                      \
  }                                                                                                                           \
  dev::wg_ctx_destroy(&ctx);                                                                                                  \
  dev::wg_finalize();

__global__ void __launch_bounds__(128) k_api_matrix_direct(State s, DTeam team, MatrixArgs m, int* results) {
  BSHMEM_API_MATRIX_BODY(dev, coll)
}
__global__ void __launch_bounds__(128) k_api_matrix_proxy(State s, DTeam team, MatrixArgs m, int* results) {
  BSHMEM_API_MATRIX_BODY(proxy, proxy)
}

}  // namespace

extern "C" {

// Runs the matrix on this PE (every member of `team_slot` must make the same call: the collectives inside are
// team-wide).  ring_dev == null: direct transport; otherwise the device pointer of the PE's proxy ring descriptor.
// Buffers: sym_* and data_sym / coll_sym are symmetric; local_dev is ordinary device memory of >= 6 * nbytes;
// coll_sym holds 2 * 64 * BSHMEM_MAX_PES floats.  results_dev: >= 40 ints.
int bshmem_gpu_api_matrix(bshmem_handle_t h, void* ring_dev, int team_slot, void* sym_i, void* sym_u, void* sym_f, void* data_sym,
                          void* local_dev, void* coll_sym, int nbytes, int peer, int* results_dev) {
  State st;
  int rc = bshmem_gpu_get_state(h, &st);
  if (rc != BSHMEM_OK) return rc;
  if (nbytes <= 0 || nbytes % 16) return BSHMEM_ERR_INVALID;
  DTeam t;
  t.my_idx = bshmem_team_my_pe(h, team_slot);
  t.size = bshmem_team_n_pes(h, team_slot);
  if (t.my_idx < 0 || t.size < 1 || peer < 0 || peer >= t.size) return BSHMEM_ERR_INVALID;
  t.slot = team_slot; t.reserved = 0; t.psync = nullptr;
  t.pe_start = bshmem_team_translate_pe(h, team_slot, 0, BSHMEM_TEAM_WORLD);
  t.stride = t.size > 1 ? bshmem_team_translate_pe(h, team_slot, 1, BSHMEM_TEAM_WORLD) - t.pe_start : 1;
  st.proxy = ring_dev;
  void* sv = nullptr;
  bshmem_gpu_get_stream(h, &sv);
  cudaStream_t stream = static_cast<cudaStream_t>(sv);
  MatrixArgs m;
  m.sym_i = static_cast<int*>(sym_i); m.sym_u = static_cast<unsigned long long*>(sym_u); m.sym_f = static_cast<float*>(sym_f);
  m.data_sym = static_cast<char*>(data_sym); m.local = static_cast<char*>(local_dev);
  m.coll_src = static_cast<float*>(coll_sym); m.coll_dst = m.coll_src + 64 * BSHMEM_MAX_PES;
  m.nbytes = nbytes; m.peer = peer;
  if (ring_dev) k_api_matrix_proxy<<<1, 128, 0, stream>>>(st, t, m, results_dev);
  else k_api_matrix_direct<<<1, 128, 0, stream>>>(st, t, m, results_dev);
  if (cudaGetLastError() != cudaSuccess) return BSHMEM_ERR_CUDA;
  return cudaStreamSynchronize(stream) == cudaSuccess ? BSHMEM_OK : BSHMEM_ERR_CUDA;
}

}  // extern "C"
