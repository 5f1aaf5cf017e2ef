// fused_tp.cu — tensor-parallel GEMMs with the collective inside the kernel (sm_100a).
//
//   GEMM → reduce-scatter (MLP down-projection):  every PE multiplies its K shard,
//     out_q = sum_r (X_r · W_r^T)[rows of q].  The epilogue of each 256x256 tile TMA-stores
//     the bf16 partial straight into the owner PE's staging slot over NVLink and bumps
//     the tile's signal word there (putmem_signal semantics); tiles are ordered so that at
//     any time the P ranks write to P different owners.  After its last tile every CTA
//     turns into a reducer: it waits for the signals of the tiles it owns, sums the P
//     partials in fp32 in a fixed order and writes the bf16 result.
//
//   all-gather → GEMM (gate/up projection):  X is row-sharded, out = gather(X) · W^T.
//     The gathered buffer is symmetric; a PE's own rows already sit in it.  While the
//     tensor core works, the epilogue warps of all CTAs pull the peers' rows piece by
//     piece over NVLink (plain peer loads → local stores) in the order the tile schedule
//     needs them and count arrivals per 256-row block; the TMA producer of a tile waits
//     for its block's counter before loading A from *local* memory.
//
// No TMA load ever reads another GPU's memory, nothing uses cluster multicast, and
// every wait (signals, ready/done flags, arrival counters, mbarriers) is bounded.
// Staging is double-buffered by call parity and all flags are monotonic counters, so
// back-to-back calls need no extra barrier.  No counterpart in the reference (it has
// neither GEMMs nor fused collectives); the signalling follows its put + flag idiom
// (library/src/gpu_ib/context_ib_tmpl_device.hpp:184-236).
#include <cstdlib>
#include <memory>
#include <vector>

#include "../include/bshmem_device.cuh"
#include "gemm_pair.cuh"
#include "tma_host.h"

using namespace bshmem;
using namespace bshmem::gemm2;
using gemm::wait_ge;

namespace {

constexpr int kMaxPes = BSHMEM_MAX_PES;

// =====================================================================================
// GEMM -> reduce-scatter
// =====================================================================================
struct RsParams {
  CoreParams core;
  CUtensorMap map_a, map_b;
  CUtensorMap map_stage[kMaxPes];               // owner q's staging slot of this rank: [rows_per_owner, N]
  CUtensorMap map_out;                          // this rank's reduced rows: [rows_per_owner, N] (ldo)
  int P, my_rank, blocks_per_owner, rows_per_owner;
  unsigned long long* sig_remote[kMaxPes];      // owner q's signal words, one per (row-block, n-block, 128-row half)
  const unsigned long long* sig_local;
  unsigned long long expect;                    // value of a signal once the P-1 peers' partials of this call landed
  const __nv_bfloat16* staging_local;           // [P][rows_per_owner][N] (this call's parity)
};

struct GemmRs : PolicyDefaults {
  using Params = RsParams;
  // deferred publication of the previous tile this warp sent to a peer
  struct EpiState { int pending, owner, idx, ord; };
  __device__ static __forceinline__ const CoreParams& core(const Params& p) { return p.core; }
  __device__ static __forceinline__ const CUtensorMap* map_a(const Params& p) { return &p.map_a; }
  __device__ static __forceinline__ const CUtensorMap* map_b(const Params& p) { return &p.map_b; }
  // First every tile whose rows another PE owns: in sub-round s every rank visits the owners me+1, me+2, ...,
  // me-1 and computes row-block s of each, so the P ranks always send to P different owners.  Then the tiles of
  // this PE's own rows, whose epilogue adds the P-1 partials that arrived meanwhile and writes the result.
  // Tile order.  First the tiles of rows that other PEs own, then this PE's own rows.  Row blocks are taken in groups;
  // inside a group the owner changes slowest (step s: every rank sends to owner me+1+s, so the P ranks always send to
  // P different owners), then the column block, and the row block of the group fastest: the CTA pairs that run side by
  // side share a few A row blocks and a few B column blocks, which keeps both in L2.  A group is at most 8 row blocks
  // and at most half of an owner's rows, so there are at least two groups: the partials of a PE's first group have all
  // been sent by the time the senders start their second one, long before the PE's own tiles (same group order) need
  // them.
  __device__ static __forceinline__ int group_rows(int bpo) {
    const int half = bpo >> 1;
    return half < 1 ? 1 : (half > 8 ? 8 : half);
  }
  __device__ static __forceinline__ void tile_coords(const Params& p, int tile, int* m_blk, int* n_blk) {
    const int num_n = p.core.num_n_blocks;
    const int bpo = p.blocks_per_owner;
    const int gm = group_rows(bpo);
    const int send_tiles = (p.P - 1) * bpo * num_n;
    int t = tile, owners = p.P - 1;
    const bool own = tile >= send_tiles;
    if (own) { t = tile - send_tiles; owners = 1; }
    const int per_group = owners * gm * num_n;               // only the last group can be smaller
    const int sg = t / per_group;
    const int first = sg * gm;
    const int rows = min(gm, bpo - first);
    const int rem = t - sg * per_group;
    const int per_step = rows * num_n;
    const int step = rem / per_step, r2 = rem - step * per_step;
    *n_blk = r2 / rows;
    const int owner = own ? p.my_rank : (p.my_rank + 1 + step) % p.P;
    *m_blk = owner * bpo + first + r2 % rows;
  }
  __device__ static __forceinline__ void out_target(const Params& p, int row, int col, const CUtensorMap** map, int* x, int* y) {
    int owner = row / p.rows_per_owner;
    *map = owner == p.my_rank ? &p.map_out : &p.map_stage[owner];
    *x = col;
    *y = row - owner * p.rows_per_owner;
  }
  // The warp's TMA stores of the tile it sent last are complete: count it on the CTA's counter of that tile; the
  // last of the CTA's eight warps publishes the CTA's half of the tile with ONE system-scope fence and ONE signal.
  // Counters are monotonic and keyed by the tile ordinal (mod 4); warps of a CTA are never more than two tiles
  // apart (two accumulators), so a counter is only shared by tiles whose counts cannot overlap in time.
  __device__ static __forceinline__ void flush(const Params& p, const Smem& L, EpiState& st, int lane) {
    if (!st.pending) return;
    st.pending = 0;
    if (lane == 0) {
      ptx::tma_wait_group<0>();
      ptx::fence_proxy_async_all();
      __threadfence();
      unsigned int old = atomicAdd(&L.scratch()[st.ord & 3], 1u);
      if (((old + 1) & (NUM_EPI_WARPS - 1)) == 0) {
        ptx::fence_acq_rel_sys();
        ptx::red_release_sys_add_u64(reinterpret_cast<uint64_t*>(p.sig_remote[st.owner] + st.idx), 1);
      }
    }
  }
  __device__ static __forceinline__ bool tile_begin(const Params& p, const Smem& L, EpiState& st, const Chunk& ck, int, int lane, Guard& g) {
    flush(p, L, st, lane);
    const int owner = ck.m_blk / p.blocks_per_owner;
    if (owner != p.my_rank || p.P == 1) return true;
    // own tile: the P-1 partials of this CTA's 128 rows must have landed in the local staging
    const int idx = ((ck.m_blk - owner * p.blocks_per_owner) * p.core.num_n_blocks + ck.n_blk) * 2 + ck.half;
    int ok = 1;
    if (lane == 0) ok = wait_ge<true>(p.sig_local + idx, p.expect, g, ERR_PEER_SIGNAL) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
  }
  // Own tile: add the peers' bf16 partials of this 32x64 chunk to the fp32 accumulators, in source order
  // (fixed, so results are reproducible run to run); see gemm::add_partial_chunks.
  __device__ static __forceinline__ void adjust(const Params& p, const Smem& L, EpiState&, const Chunk& ck, float (&f)[64], int ew, int lane) {
    const int owner = ck.m_blk / p.blocks_per_owner;
    if (owner != p.my_rank || p.P == 1) return;
    const long long N = p.core.N;
    const int r_local = ck.row0 - owner * p.rows_per_owner;
    const __nv_bfloat16* src0 = p.staging_local + (long long)(r_local + (lane >> 3)) * N + ck.col0 + (lane & 7) * 8;
    gemm::add_partial_chunks(f, src0, (long long)p.rows_per_owner * N, N, p.P, p.my_rank, L.epi(ew), lane);
  }
  __device__ static __forceinline__ void tile_end(const Params& p, const Smem&, EpiState& st, const Chunk& ck, int, int) {
    const int owner = ck.m_blk / p.blocks_per_owner;
    if (owner == p.my_rank) return;
    st.pending = 1;
    st.owner = owner;
    st.idx = ((ck.m_blk - owner * p.blocks_per_owner) * p.core.num_n_blocks + ck.n_blk) * 2 + ck.half;
    st.ord = ck.ordinal;
  }
  __device__ static __forceinline__ void epilogue_drain(const Params& p, const Smem& L, EpiState& st, int, int lane, Guard&) {
    flush(p, L, st, lane);
  }
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1) gemm_rs_kernel(const __grid_constant__ RsParams prm) {
  extern __shared__ uint8_t smem_raw[];
  gemm_mainloop<GemmRs>(prm, smem_raw);
}

// =====================================================================================
// all-gather -> GEMM
// =====================================================================================
constexpr int kPieceBytes = 16384;

struct AgParams {
  CoreParams core;                              // M = all tokens, N = local output features
  CUtensorMap map_a, map_b, map_c;              // A over the local gathered buffer
  int P, my_rank, blocks_per_rank, pieces_per_row;
  int pieces_per_block, pieces_per_src, total_pieces, pad;
  unsigned long long row_bytes;
  const char* xg_peer[kMaxPes];                 // every PE's gathered buffer as mapped here
  char* xg_local;
  unsigned long long* arrived;                  // local [num_m_blocks]: pieces landed (monotonic over calls)
  unsigned long long* src_pulled;               // local [P]: pieces pulled per source (monotonic)
  unsigned int* ticket;                         // local [2]: work counter of this call's parity
  unsigned long long* ready_remote[kMaxPes];    // peer's ready[P]; this rank writes entry my_rank
  const unsigned long long* ready_local;
  unsigned long long* done_remote[kMaxPes];     // peer's done[P]; this rank writes entry my_rank
  const unsigned long long* done_local;
  unsigned long long call;
};

struct AgGemm : PolicyDefaults {
  using Params = AgParams;
  __device__ static __forceinline__ const CoreParams& core(const Params& p) { return p.core; }
  __device__ static __forceinline__ const CUtensorMap* map_a(const Params& p) { return &p.map_a; }
  __device__ static __forceinline__ const CUtensorMap* map_b(const Params& p) { return &p.map_b; }
  // Source-major: first my own rows, then the rows of rank me+1, me+2, ... (the pull order).
  __device__ static __forceinline__ void tile_coords(const Params& p, int tile, int* m_blk, int* n_blk) {
    int per_src = p.blocks_per_rank * p.core.num_n_blocks;
    int step = tile / per_src, rem = tile - step * per_src;
    int src = (p.my_rank + step) % p.P;
    *m_blk = src * p.blocks_per_rank + rem % p.blocks_per_rank;
    *n_blk = rem / p.blocks_per_rank;
  }
  __device__ static __forceinline__ void out_target(const Params& p, int row, int col, const CUtensorMap** map, int* x, int* y) {
    *map = (row < p.core.M && col < p.core.N) ? &p.map_c : nullptr;
    *x = col;
    *y = row;
  }
  // One thread of CTA 0: recycle the other parity's ticket counter and tell every peer that this
  // rank's rows are in place for this call (they were written by earlier work on the stream).
  __device__ static __forceinline__ void prologue(const Params& p, Guard&) {
    if (blockIdx.x != 0) return;
    p.ticket[(p.call + 1) & 1] = 0;
    ptx::fence_acq_rel_sys();
    for (int q = 0; q < p.P; ++q)
      if (q != p.my_rank) ptx::st_release_sys_u64(reinterpret_cast<uint64_t*>(p.ready_remote[q] + p.my_rank), p.call);
  }
  // The producer may load A rows of block m_blk once all of their pieces have landed locally.
  __device__ static __forceinline__ bool a_ready(const Params& p, int m_blk, Guard& g) {
    if (m_blk / p.blocks_per_rank == p.my_rank) return true;
    if (!wait_ge<false>(p.arrived + m_blk, (unsigned long long)p.pieces_per_block * p.call, g, ERR_A_READY)) return false;
    ptx::fence_proxy_async_all();     // generic-proxy stores (the pull) before async-proxy reads (TMA)
    return true;
  }
  // A warp pulls one piece (<= 16 KiB of one row) of a peer's rows into the local gathered buffer.
  __device__ static __forceinline__ bool idle_work(const Params& p, int, int lane, Guard& g, int = 0, volatile int* = nullptr) {
    if (p.P == 1) return false;
    unsigned int t = 0;
    if (lane == 0) t = atomicAdd(&p.ticket[p.call & 1], 1u);
    t = __shfl_sync(0xffffffffu, t, 0);
    if (t >= (unsigned)p.total_pieces) return false;
    int step = t / p.pieces_per_src, rem = t - step * p.pieces_per_src;
    int blk_in_src = rem / p.pieces_per_block, piece = rem - blk_in_src * p.pieces_per_block;
    int src = (p.my_rank + 1 + step) % p.P;
    int row = piece / p.pieces_per_row, seg = piece - row * p.pieces_per_row;
    int m_blk = src * p.blocks_per_rank + blk_in_src;
    unsigned long long off = ((unsigned long long)m_blk * BM + row) * p.row_bytes + (unsigned long long)seg * kPieceBytes;
    unsigned long long left = p.row_bytes - (unsigned long long)seg * kPieceBytes;
    int nvec = (int)((left < (unsigned long long)kPieceBytes ? left : (unsigned long long)kPieceBytes) >> 4);
    int ok = 1;
    if (lane == 0) ok = wait_ge<true>(p.ready_local + src, p.call, g, ERR_PEER_READY) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) return false;
    const uint4* s4 = reinterpret_cast<const uint4*>(p.xg_peer[src] + off);
    uint4* d4 = reinterpret_cast<uint4*>(p.xg_local + off);
    int i = lane;
    for (; i + 96 < nvec; i += 128) {     // four independent 16-byte peer loads in flight per lane
      uint4 a = ptx::ld_relaxed_v4(s4 + i), b = ptx::ld_relaxed_v4(s4 + i + 32), c = ptx::ld_relaxed_v4(s4 + i + 64), d = ptx::ld_relaxed_v4(s4 + i + 96);
      d4[i] = a; d4[i + 32] = b; d4[i + 64] = c; d4[i + 96] = d;
    }
    for (; i < nvec; i += 32) d4[i] = ptx::ld_relaxed_v4(s4 + i);
    ptx::fence_proxy_async_all();
    __syncwarp();
    if (lane == 0) {
      __threadfence();
      asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p.arrived + m_blk), "l"(1ull) : "memory");
      unsigned long long pulled = atomicAdd(p.src_pulled + src, 1ull) + 1;
      if (pulled == (unsigned long long)p.pieces_per_src * p.call) {
        // everything of `src` is here: it may overwrite its rows once every PE said so
        ptx::fence_acq_rel_sys();
        ptx::st_release_sys_u64(reinterpret_cast<uint64_t*>(p.done_remote[src] + p.my_rank), p.call);
      }
    }
    return true;
  }
  __device__ static __forceinline__ void epilogue_drain(const Params& p, const Smem&, EpiState&, int ew, int lane, Guard& g) {
    while (idle_work(p, ew, lane, g, 0)) {}
  }
  // Before the kernel ends, CTA 0 makes sure every peer has finished pulling this rank's rows.
  __device__ static __forceinline__ void tail(const Params& p, const Smem&, Guard& g) {
    if (blockIdx.x == 0 && threadIdx.x < p.P && (int)threadIdx.x != p.my_rank)
      wait_ge<true>(p.done_local + threadIdx.x, p.call, g, ERR_PEER_DONE);
  }
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1) ag_gemm_kernel(const __grid_constant__ AgParams prm) {
  extern __shared__ uint8_t smem_raw[];
  gemm_mainloop<AgGemm>(prm, smem_raw);
}

// =====================================================================================
// host side
// =====================================================================================
struct Plan {
  int kind = 0;             // 0 = gemm->rs, 1 = ag->gemm
  int device = 0, pairs = 0;
  bshmem_dev_state_t st;
  int M = 0, N = 0, K = 0;
  unsigned long long call = 0;
  int* err = nullptr;
  // rs
  char* staging_local = nullptr;   // symmetric, 2 parities
  unsigned long long* sig_local = nullptr;
  // ag
  char* xg_local = nullptr;
  unsigned long long* flags_local = nullptr;   // symmetric: ready[P] then done[P]
  unsigned long long* arrived = nullptr;
  unsigned long long* src_pulled = nullptr;
  unsigned int* ticket = nullptr;
  ~Plan() {
    if (err) cudaFree(err);
    if (arrived) cudaFree(arrived);
    if (src_pulled) cudaFree(src_pulled);
    if (ticket) cudaFree(ticket);
  }
};

template <typename T> T* peer_ptr(const bshmem_dev_state_t& st, T* local, int pe) {
  return reinterpret_cast<T*>(st.heap_base[pe] + (reinterpret_cast<char*>(local) - st.heap_base[st.my_pe]));
}

int common_init(Plan* p) {
  int sms = 0;
  BSHMEM_CUDA_TRY(cudaGetDevice(&p->device));
  BSHMEM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, p->device));
  BSHMEM_CUDA_TRY(cudaMalloc(&p->err, sizeof(int)));
  BSHMEM_CUDA_TRY(cudaMemset(p->err, 0, sizeof(int)));
  BSHMEM_CUDA_TRY(cudaFuncSetAttribute(gemm_rs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
  BSHMEM_CUDA_TRY(cudaFuncSetAttribute(ag_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
  p->pairs = p->kind == 0 ? max_resident_pairs(gemm_rs_kernel, sms) : max_resident_pairs(ag_gemm_kernel, sms);
  return 0;
}

bool in_heap(const bshmem_dev_state_t& st, const void* p, uint64_t n) {
  const char* c = static_cast<const char*>(p);
  const char* b = st.heap_base[st.my_pe];
  return c >= b && (uint64_t)(c - b) + n <= st.heap_bytes;
}

int grid_ctas(const Plan* p, int tiles, int max_ctas) {
  int pairs = p->pairs;
  if (max_ctas > 1 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
  if (tiles < pairs) pairs = tiles;
  return 2 * pairs;
}

}  // namespace

extern "C" {

const char* bshmem_fused_last_error() { return host::last_error().c_str(); }

// Bytes of symmetric memory the GEMM->RS plan needs: staging (2 parities x P slots x M/P x N bf16) and one signal
// word per owned tile half.
uint64_t bshmem_fused_rs_staging_bytes(int M, int N) { return 2ull * (uint64_t)M * N * 2; }
uint64_t bshmem_fused_rs_signal_bytes(int M, int N, int P) { return (uint64_t)(M / P / BM) * (N / BN) * 2 * 8; }

int bshmem_fused_rs_plan(const bshmem_dev_state_t* st, int M, int N, int K, void* staging_local, void* sig_local, void** out) {
  if (!st || !out) return 1;
  int P = st->n_pes;
  if (M <= 0 || N <= 0 || K <= 0 || M % (P * BM) || N % BN || K % 8) {
    host::last_error() = "gemm_rs: needs M % (P*256) == 0, N % 256 == 0, K % 8 == 0";
    return 1;
  }
  if (!in_heap(*st, staging_local, bshmem_fused_rs_staging_bytes(M, N)) ||
      !in_heap(*st, sig_local, bshmem_fused_rs_signal_bytes(M, N, P))) {
    host::last_error() = "gemm_rs: staging / signal buffers must be symmetric allocations of the stated sizes";
    return 4;
  }
  std::unique_ptr<Plan> p(new Plan());
  p->kind = 0; p->st = *st; p->M = M; p->N = N; p->K = K;
  p->staging_local = static_cast<char*>(staging_local);
  p->sig_local = static_cast<unsigned long long*>(sig_local);
  int rc = common_init(p.get());
  if (rc) return rc;
  *out = p.release();
  return 0;
}

// x: [M, K] bf16 (ldx), w: [N, K] bf16 (ldw), out: [M/P, N] bf16 (ldo): this PE's rows of the reduced product.
int bshmem_fused_rs_run(void* plan, const void* x, int ldx, const void* w, int ldw, void* out, int ldo, void* stream,
                        int timeout_ms, int max_ctas) {
  Plan* p = static_cast<Plan*>(plan);
  if (!p || p->kind != 0) return 1;
  const int P = p->st.n_pes, me = p->st.my_pe;
  const int rows = p->M / P;
  RsParams prm;
  memset(&prm, 0, sizeof(prm));
  prm.core.M = p->M; prm.core.N = p->N; prm.core.K = p->K;
  prm.core.num_m_blocks = p->M / BM; prm.core.num_n_blocks = p->N / BN;
  prm.core.group_m = 8;
  prm.core.timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 2000) * 1000000ull;
  prm.core.err = p->err;
  prm.P = P; prm.my_rank = me; prm.blocks_per_owner = rows / BM; prm.rows_per_owner = rows;
  int rc = host::make_tmap_2d(&prm.map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, p->M, p->K, ldx, CTA_M, 64);
  if (rc) return rc;
  rc = host::make_tmap_2d(&prm.map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, p->N, p->K, ldw, CTA_NLOAD, 64);
  if (rc) return rc;
  rc = host::make_tmap_2d(&prm.map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, out, rows, p->N, ldo, 32, EPI_COLS);
  if (rc) return rc;
  const unsigned long long call = p->call + 1;
  const uint64_t parity_bytes = (uint64_t)p->M * p->N * 2;          // P slots x rows x N
  const uint64_t slot_bytes = (uint64_t)rows * p->N * 2;
  char* stage_par = p->staging_local + (call & 1) * parity_bytes;
  for (int q = 0; q < P; ++q) {
    // my slot (index me) inside owner q's staging of this parity
    char* dst = peer_ptr(p->st, stage_par, q) + (uint64_t)me * slot_bytes;
    rc = host::make_tmap_2d(&prm.map_stage[q], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dst, rows, p->N, p->N, 32, EPI_COLS);
    if (rc) return rc;
    prm.sig_remote[q] = peer_ptr(p->st, p->sig_local, q);
  }
  prm.sig_local = p->sig_local;
  prm.expect = (unsigned long long)(P - 1) * call;
  prm.staging_local = reinterpret_cast<const __nv_bfloat16*>(stage_par);
  const int tiles = prm.core.num_m_blocks * prm.core.num_n_blocks;
  const int ctas = grid_ctas(p, tiles, max_ctas);
  gemm_rs_kernel<<<ctas, NUM_THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(prm);
  BSHMEM_CUDA_TRY(cudaGetLastError());
  p->call = call;      // counted only once the kernel that sends this call's signals is enqueued
  return 0;
}

// Symmetric memory of the AG->GEMM plan: the gathered activations [M, K] bf16 and 2*P flag words.
uint64_t bshmem_fused_ag_flag_bytes(int P) { return 2ull * P * 8; }

int bshmem_fused_ag_plan(const bshmem_dev_state_t* st, int M, int N, int K, void* xg_local, void* flags_local, void** out) {
  if (!st || !out) return 1;
  int P = st->n_pes;
  if (M <= 0 || N <= 0 || K <= 0 || M % (P * BM) || K % 8 || N % 8) {
    host::last_error() = "ag_gemm: needs M % (P*256) == 0, K % 8 == 0, N % 8 == 0";
    return 1;
  }
  if (!in_heap(*st, xg_local, (uint64_t)M * K * 2) || !in_heap(*st, flags_local, bshmem_fused_ag_flag_bytes(P))) {
    host::last_error() = "ag_gemm: the gathered buffer and the flags must be symmetric allocations";
    return 4;
  }
  std::unique_ptr<Plan> p(new Plan());
  p->kind = 1; p->st = *st; p->M = M; p->N = N; p->K = K;
  p->xg_local = static_cast<char*>(xg_local);
  p->flags_local = static_cast<unsigned long long*>(flags_local);
  int rc = common_init(p.get());
  if (rc) return rc;
  int nblk = M / BM;
  BSHMEM_CUDA_TRY(cudaMalloc(&p->arrived, sizeof(unsigned long long) * nblk));
  BSHMEM_CUDA_TRY(cudaMemset(p->arrived, 0, sizeof(unsigned long long) * nblk));
  BSHMEM_CUDA_TRY(cudaMalloc(&p->src_pulled, sizeof(unsigned long long) * kMaxPes));
  BSHMEM_CUDA_TRY(cudaMemset(p->src_pulled, 0, sizeof(unsigned long long) * kMaxPes));
  BSHMEM_CUDA_TRY(cudaMalloc(&p->ticket, sizeof(unsigned int) * 2));
  BSHMEM_CUDA_TRY(cudaMemset(p->ticket, 0, sizeof(unsigned int) * 2));
  *out = p.release();
  return 0;
}

// This PE's rows must already be in xg_local[my_pe * M/P : (my_pe+1) * M/P].  w: [N, K] (ldw), out: [M, N] (ldo).
int bshmem_fused_ag_run(void* plan, const void* w, int ldw, void* out, int ldo, void* stream, int timeout_ms, int max_ctas) {
  Plan* p = static_cast<Plan*>(plan);
  if (!p || p->kind != 1) return 1;
  const int P = p->st.n_pes, me = p->st.my_pe;
  const unsigned long long call = p->call + 1;
  AgParams prm;
  memset(&prm, 0, sizeof(prm));
  prm.core.M = p->M; prm.core.N = p->N; prm.core.K = p->K;
  prm.core.num_m_blocks = p->M / BM; prm.core.num_n_blocks = (p->N + BN - 1) / BN;
  prm.core.group_m = 8;
  prm.core.timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 2000) * 1000000ull;
  prm.core.err = p->err;
  prm.P = P; prm.my_rank = me; prm.blocks_per_rank = p->M / P / BM;
  prm.row_bytes = (unsigned long long)p->K * 2;
  prm.pieces_per_row = (int)((prm.row_bytes + kPieceBytes - 1) / kPieceBytes);
  prm.pieces_per_block = BM * prm.pieces_per_row;
  prm.pieces_per_src = prm.blocks_per_rank * prm.pieces_per_block;
  prm.total_pieces = (P - 1) * prm.pieces_per_src;
  int rc = host::make_tmap_2d(&prm.map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p->xg_local, p->M, p->K, p->K, CTA_M, 64);
  if (rc) return rc;
  rc = host::make_tmap_2d(&prm.map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, p->N, p->K, ldw, CTA_NLOAD, 64);
  if (rc) return rc;
  rc = host::make_tmap_2d(&prm.map_c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, out, p->M, p->N, ldo, 32, EPI_COLS);
  if (rc) return rc;
  for (int q = 0; q < P; ++q) {
    prm.xg_peer[q] = peer_ptr(p->st, p->xg_local, q);
    prm.ready_remote[q] = peer_ptr(p->st, p->flags_local, q);
    prm.done_remote[q] = peer_ptr(p->st, p->flags_local, q) + P;
  }
  prm.xg_local = p->xg_local;
  prm.arrived = p->arrived;
  prm.src_pulled = p->src_pulled;
  prm.ticket = p->ticket;
  prm.ready_local = p->flags_local;
  prm.done_local = p->flags_local + P;
  prm.call = call;
  const int tiles = prm.core.num_m_blocks * prm.core.num_n_blocks;
  const int ctas = grid_ctas(p, tiles, max_ctas);
  ag_gemm_kernel<<<ctas, NUM_THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(prm);
  BSHMEM_CUDA_TRY(cudaGetLastError());
  p->call = call;
  return 0;
}

int bshmem_fused_error_site(void* plan, int clear) {
  Plan* p = static_cast<Plan*>(plan);
  int v = 0;
  if (!p || !p->err) return 0;
  cudaMemcpy(&v, p->err, sizeof(int), cudaMemcpyDeviceToHost);
  if (clear && v) cudaMemset(p->err, 0, sizeof(int));
  return v;
}

int bshmem_fused_destroy(void* plan) {
  delete static_cast<Plan*>(plan);
  return 0;
}

}  // extern "C"
