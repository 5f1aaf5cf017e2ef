// gemm_fp8.cu — block-scaled fp8 (e4m3) tcgen05 GEMM for sm_100a:
//
//   C[M,N] (bf16) = sum over 128-wide k-blocks kb of
//                   sa[kb][m] * sb[kb][n/128] * ( A8[m, kb] · B8[n, kb]^T )
//
// A8: [M, K] e4m3 activations with one fp32 scale per row and 128 columns ("1x128"), stored
// k-block-major (sa[kb * M + m]) so that the 32 rows of a warp read 128 contiguous bytes;
// B8: [N, K] e4m3 weights with one fp32 scale per 128x128 block (sb[kb * (N/128) + n/128]).
//
// The scales differ from k-block to k-block, so the tensor core cannot keep one running
// accumulator.  Each k-block's product (M128 x N256 x K128, four tcgen05.mma kind::f8f6f4)
// goes into one of two 256-column TMEM buffers; sixteen epilogue warps read the buffer that
// just completed, multiply by the row's scale and add into fp32 registers (64 per thread,
// packed two-wide FMAs) while the tensor core fills the other buffer.  Four warps per SM
// sub-partition hide the TMEM load latency.  One CTA per SM, persistent over 128x256 tiles:
//   warp 0      TMA producer: 3-stage ring of 48 KiB (A 128 rows + B 256 rows of 128 bytes)
//   warp 1      MMA issuer, commits each k-block to the stage's and the buffer's mbarrier
//   warps 2-17  promote partial products (32 rows x 64 columns each), then convert, stage in
//               swizzled smem and TMA-store
// Every wait is bounded (see gemm_core.cuh); there is no counterpart in the reference.
#include <cuda_fp8.h>

#include "../include/bshmem_device.cuh"
#include "gemm_core.cuh"
#include "tma_host.h"

using namespace bshmem;
using namespace bshmem::gemm;

namespace {

constexpr int FBM = 128, FBN = 256, FBK = 128;          // tile and k-block in elements (= bytes)
constexpr int FSTAGES = 3;
constexpr int FEPI_WARPS = 16;
constexpr int FNUM_THREADS = 32 * (2 + FEPI_WARPS);
constexpr uint32_t FA_BYTES = FBM * FBK, FB_BYTES = FBN * FBK, FSTAGE_BYTES = FA_BYTES + FB_BYTES;
constexpr uint32_t FEPI_BYTES = 32 * 128;               // one warp: 32 rows x 64 bf16
constexpr uint32_t FSMEM_TILES = FSTAGES * FSTAGE_BYTES + FEPI_WARPS * FEPI_BYTES;
constexpr uint32_t FSMEM_BYTES = FSMEM_TILES + 256 + 1024;
constexpr uint32_t kIdescFp8 = ptx::umma_idesc(0, 0, 128, 256);   // e4m3 x e4m3 -> fp32, M128 N256

enum : int { ERR_F8_PART_FULL = 121, ERR_F8_PART_EMPTY = 122 };

constexpr int kMaxPes = BSHMEM_MAX_PES;
constexpr int kPieceBytes = 16384;
constexpr int FPULL_WARPS = 2;                          // all-gather variant: warps 18-19 pull the peers' rows

// All-gather state (all-gather -> GEMM variant): the activations A8 [M, K] and their scales [K/128][M] live in
// symmetric memory; every PE owns M/P rows.  Pull warps copy the peers' rows and scale columns into the local
// buffers piece by piece (a piece = up to 16 KiB of one row, or the scale columns of one 128-row block) and bump
// the block's arrival counter; producers and epilogue warps wait on that counter before they touch the block.
struct Fp8Ag {
  int P, my_rank, blocks_per_rank, pieces_per_row;
  int pieces_per_block, pieces_per_src, total_pieces, num_kb;
  unsigned long long row_bytes;
  const char* xq_peer[kMaxPes];
  char* xq_local;
  const float* sa_peer[kMaxPes];
  float* sa_local;
  unsigned long long* arrived;                  // local [M/128]: pieces landed (monotonic over calls)
  unsigned long long* src_pulled;               // local [P]
  unsigned int* ticket;                         // local [2]: work counter of this call's parity
  unsigned long long* ready_remote[kMaxPes];    // peer's ready[P]; this rank writes entry my_rank
  const unsigned long long* ready_local;
  unsigned long long* done_remote[kMaxPes];
  const unsigned long long* done_local;
  unsigned long long call;
};

// Reduce-scatter state (GEMM -> reduce-scatter variant): every PE multiplies its K shard, rounds the 128x256 partial
// tiles of rows another PE owns to bf16 and TMA-stores them into the staging slot [parity][source PE] of that owner,
// then bumps the tile's signal word there.  The tiles of its own rows come last: their epilogue waits for the P-1
// partials that arrived meanwhile, adds them to the fp32 accumulators and writes the result (no reduction pass).
struct Fp8Rs {
  int P, my_rank, blocks_per_rank, pad;         // blocks_per_rank: 128-row blocks per owner
  CUtensorMap map_stage[kMaxPes];               // owner q's slot for (parity, source = this PE): [M/P, N] bf16
  CUtensorMap map_out;                          // this PE's reduced rows [M/P, N] (ldo)
  unsigned long long* sig_remote[kMaxPes];      // owner q's signal words [blocks_per_rank * N/256] (monotonic over calls)
  const unsigned long long* sig_local;
  const __nv_bfloat16* stage_local;             // this PE's staging of this call's parity: [P][M/P][N]
  __nv_bfloat16* out;                           // [M/P, N]
  int ldo, pad2;
  unsigned long long call;
};

struct Fp8Params {
  CoreParams core;             // num_m_blocks counts 128-row blocks
  CUtensorMap map_a, map_b, map_c;
  const float* sa;             // [K/128][M]
  const float* sb;             // [K/128][N/128]
  Fp8Ag ag;                    // used by the all-gather variant only
};
struct Fp8RsParams {
  Fp8Params base;
  Fp8Rs rs;
};
enum : int { F8_PLAIN = 0, F8_AG = 1, F8_RS = 2 };

enum : int { ERR_F8_A_READY = 123, ERR_F8_PEER_READY = 124, ERR_F8_PEER_DONE = 125, ERR_F8_RS_SIGNAL = 126 };

// Tile order: grouped raster, or (all-gather) source-major starting with this PE's own rows, then the rows of
// rank me+1, me+2, ... which is also the order in which the pull warps fetch them.
template <int kMode>
__device__ __forceinline__ void f8_tile_coords(const Fp8Params& p, const Fp8Rs* rs, int tile, int* m_blk, int* n_blk) {
  if constexpr (kMode == F8_PLAIN) {
    raster_coords(p.core, tile, m_blk, n_blk);
  } else if constexpr (kMode == F8_RS) {
    // owner-major, owners visited in the order me+1, me+2, ..., me: the P ranks always write to P different owners
    const int per_owner = rs->blocks_per_rank * p.core.num_n_blocks;
    const int step = tile / per_owner, rem = tile - step * per_owner;
    const int owner = (rs->my_rank + 1 + step) % rs->P;
    *m_blk = owner * rs->blocks_per_rank + rem % rs->blocks_per_rank;
    *n_blk = rem / rs->blocks_per_rank;
  } else {
    const int per_src = p.ag.blocks_per_rank * p.core.num_n_blocks;
    const int step = tile / per_src, rem = tile - step * per_src;
    const int src = (p.ag.my_rank + step) % p.ag.P;
    *m_blk = src * p.ag.blocks_per_rank + rem % p.ag.blocks_per_rank;
    *n_blk = rem / p.ag.blocks_per_rank;
  }
}

// One pull warp fetches one piece; returns false when no work is left (or the CTA is aborting).
__device__ __forceinline__ bool f8_pull_piece(const Fp8Params& prm, int lane, Guard& g) {
  const Fp8Ag& p = prm.ag;
  unsigned int t = 0;
  if (lane == 0) t = atomicAdd(&p.ticket[p.call & 1], 1u);
  t = __shfl_sync(0xffffffffu, t, 0);
  if (t >= (unsigned)p.total_pieces) return false;
  const int step = t / p.pieces_per_src, rem = t - step * p.pieces_per_src;
  const int blk_in_src = rem / p.pieces_per_block, piece = rem - blk_in_src * p.pieces_per_block;
  const int src = (p.my_rank + 1 + step) % p.P;
  const int m_blk = src * p.blocks_per_rank + blk_in_src;
  int ok = 1;
  if (lane == 0) ok = wait_ge<true>(p.ready_local + src, p.call, g, ERR_F8_PEER_READY) ? 1 : 0;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  if (!ok) return false;
  if (piece < p.pieces_per_block - 1) {
    // up to 16 KiB of one activation row
    const int row = piece / p.pieces_per_row, seg = piece - row * p.pieces_per_row;
    const unsigned long long off = ((unsigned long long)m_blk * FBM + row) * p.row_bytes + (unsigned long long)seg * kPieceBytes;
    const unsigned long long left = p.row_bytes - (unsigned long long)seg * kPieceBytes;
    const int nvec = (int)((left < (unsigned long long)kPieceBytes ? left : (unsigned long long)kPieceBytes) >> 4);
    const uint4* s4 = reinterpret_cast<const uint4*>(p.xq_peer[src] + off);
    uint4* d4 = reinterpret_cast<uint4*>(p.xq_local + off);
    int i = lane;
    for (; i + 224 < nvec; i += 256) {                  // eight independent 16-byte peer loads in flight per lane
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = ptx::ld_relaxed_v4(s4 + i + 32 * u);
#pragma unroll
      for (int u = 0; u < 8; ++u) d4[i + 32 * u] = v[u];
    }
    for (; i < nvec; i += 32) d4[i] = ptx::ld_relaxed_v4(s4 + i);
  } else {
    // the block's scale columns: 128 floats (512 bytes) of every k-block row of the [K/128][M] scale matrix
    const size_t col0 = (size_t)m_blk * FBM;
    int kb = 0;
    for (; kb + 8 <= p.num_kb; kb += 8) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        v[u] = ptx::ld_relaxed_v4(reinterpret_cast<const uint4*>(p.sa_peer[src] + (size_t)(kb + u) * prm.core.M + col0) + lane);
#pragma unroll
      for (int u = 0; u < 8; ++u) reinterpret_cast<uint4*>(p.sa_local + (size_t)(kb + u) * prm.core.M + col0)[lane] = v[u];
    }
    for (; kb < p.num_kb; ++kb)
      reinterpret_cast<uint4*>(p.sa_local + (size_t)kb * prm.core.M + col0)[lane] =
          ptx::ld_relaxed_v4(reinterpret_cast<const uint4*>(p.sa_peer[src] + (size_t)kb * prm.core.M + col0) + lane);
  }
  ptx::fence_proxy_async_all();           // generic-proxy stores (the pull) before async-proxy reads (TMA)
  __syncwarp();
  if (lane == 0) {
    __threadfence();
    asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p.arrived + m_blk), "l"(1ull) : "memory");
    const unsigned long long pulled = atomicAdd(p.src_pulled + src, 1ull) + 1;
    if (pulled == (unsigned long long)p.pieces_per_src * p.call) {
      // everything of `src` is here: it may overwrite its rows once every PE said so
      ptx::fence_acq_rel_sys();
      ptx::st_release_sys_u64(reinterpret_cast<uint64_t*>(p.done_remote[src] + p.my_rank), p.call);
    }
  }
  return true;
}

struct FSmem {
  uint32_t base;
  uint8_t* gen;
  __device__ __forceinline__ uint32_t a(int s) const { return base + s * FSTAGE_BYTES; }
  __device__ __forceinline__ uint32_t b(int s) const { return base + s * FSTAGE_BYTES + FA_BYTES; }
  __device__ __forceinline__ uint32_t epi(int w) const { return base + FSTAGES * FSTAGE_BYTES + w * FEPI_BYTES; }
  __device__ __forceinline__ uint32_t bars() const { return base + FSMEM_TILES; }
  __device__ __forceinline__ uint32_t full(int s) const { return bars() + 8 * s; }
  __device__ __forceinline__ uint32_t empty(int s) const { return bars() + 8 * (FSTAGES + s); }
  __device__ __forceinline__ uint32_t part_full(int b) const { return bars() + 8 * (2 * FSTAGES + b); }
  __device__ __forceinline__ uint32_t part_empty(int b) const { return bars() + 8 * (2 * FSTAGES + 2 + b); }
  __device__ __forceinline__ uint32_t tmem_slot() const { return bars() + 8 * (2 * FSTAGES + 4); }
  __device__ __forceinline__ volatile int* abort_flag() const {
    return reinterpret_cast<volatile int*>(gen + FSMEM_TILES + 8 * (2 * FSTAGES + 4) + 8);
  }
  // reduce-scatter variant: epilogue warps that have completed their store of a tile, counted monotonically on the
  // counter (tile ordinal & 3)
  __device__ __forceinline__ unsigned int* rs_count(int which) const {
    return reinterpret_cast<unsigned int*>(gen + FSMEM_TILES + 8 * (2 * FSTAGES + 4) + 16) + which;
  }
};

// Called by lane 0 of an epilogue warp once its own TMA store of a tile is complete: the last of the 16 warps to
// arrive publishes the whole tile with ONE system-scope fence and ONE signal; no warp ever waits for another.
// The counters only ever grow (a multiple of 16 means "tile complete") and there are four of them, indexed by the
// tile ordinal: the two partial-product buffers bound the skew between epilogue warps to two k-blocks, which is at
// most two tiles even when a tile is a single k-block, and a warp publishes one tile late, so the tiles that can be
// in the publishing stage at the same time are at most three apart and never share a counter.
__device__ __forceinline__ void rs_publish(unsigned int* count, uint64_t* sig) {
  __threadfence();
  if (((atomicAdd(count, 1u) + 1u) & (FEPI_WARPS - 1)) == 0u) {
    ptx::fence_proxy_async_all();
    ptx::fence_acq_rel_sys();
    ptx::red_release_sys_add_u64(sig, 1);
  }
}

template <int kMode>
__device__ __forceinline__ void gemm_fp8_body(const Fp8Params& prm, const Fp8Rs* rs, uint8_t* smem_raw) {
  constexpr bool kAG = kMode == F8_AG;
  constexpr bool kRS = kMode == F8_RS;
  FSmem L;
  {
    uint32_t r = ptx::smem_u32(smem_raw);
    L.base = (r + 1023u) & ~1023u;
    L.gen = smem_raw + (L.base - r);
  }
  const CoreParams& cp = prm.core;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = cp.num_m_blocks * cp.num_n_blocks;
  const int num_kb = cp.K / FBK;
  Guard g{cp.err, L.abort_flag(), cp.timeout_ns};

  if (threadIdx.x == 0) {
    *L.abort_flag() = 0;
    for (int i = 0; i < 4; ++i) *L.rs_count(i) = 0;
    for (int s = 0; s < FSTAGES; ++s) { ptx::mbar_init(L.full(s), 1); ptx::mbar_init(L.empty(s), 1); }
    for (int b = 0; b < 2; ++b) { ptx::mbar_init(L.part_full(b), 1); ptx::mbar_init(L.part_empty(b), FEPI_WARPS); }
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&prm.map_a);
    ptx::prefetch_tensormap(&prm.map_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(L.tmem_slot(), TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(L.tmem_slot()));
  if constexpr (kAG) {
    // one thread of CTA 0: recycle the other parity's ticket counter and tell every peer that this PE's rows and
    // scales are in place for this call (they were written by earlier work on the stream)
    if (blockIdx.x == 0 && threadIdx.x == 64) {
      prm.ag.ticket[(prm.ag.call + 1) & 1] = 0;
      ptx::fence_acq_rel_sys();
      for (int q = 0; q < prm.ag.P; ++q)
        if (q != prm.ag.my_rank)
          ptx::st_release_sys_u64(reinterpret_cast<uint64_t*>(prm.ag.ready_remote[q] + prm.ag.my_rank), prm.ag.call);
    }
  }

  if (warp >= 2 + FEPI_WARPS) {
    // ------------------------------ pull warps (all-gather variant) ------------
    if constexpr (kAG) {
      if (prm.ag.P > 1)
        while (f8_pull_piece(prm, lane, g)) {}
    }
  } else if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int s = 0; uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk;
        f8_tile_coords<kMode>(prm, rs, tile, &m_blk, &n_blk);
        if constexpr (kAG) {
          if (m_blk / prm.ag.blocks_per_rank != prm.ag.my_rank) {
            if (!wait_ge<false>(prm.ag.arrived + m_blk, (unsigned long long)prm.ag.pieces_per_block * prm.ag.call, g, ERR_F8_A_READY)) break;
            ptx::fence_proxy_async_all();
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(L.empty(s), ph ^ 1, g, ERR_PRODUCER_EMPTY)) { ok = false; break; }
          ptx::mbar_arrive_expect_tx(L.full(s), FSTAGE_BYTES);
          ptx::tma_load_2d(L.a(s), &prm.map_a, L.full(s), kb * FBK, m_blk * FBM);
          ptx::tma_load_2d(L.b(s), &prm.map_b, L.full(s), kb * FBK, n_blk * FBN);
          if (++s == FSTAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    if (lane == 0) {
      int s = 0; uint32_t ph = 0;
      uint32_t it = 0;                       // k-blocks issued so far: buffer = it & 1, use count = it >> 1
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int buf = it & 1;
          // the epilogue must have drained this buffer's previous product
          if (!mbar_wait(L.part_empty(buf), ((it >> 1) & 1) ^ 1, g, ERR_F8_PART_EMPTY)) { ok = false; break; }
          if (!mbar_wait(L.full(s), ph, g, ERR_MMA_FULL)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t a0 = L.a(s), b0 = L.b(s);
#pragma unroll
          for (int k = 0; k < FBK / UMMA_K_BYTES; ++k)
            ptx::umma_f8f6f4(tmem_base + buf * FBN, ptx::umma_desc_sw128(a0 + k * UMMA_K_BYTES),
                             ptx::umma_desc_sw128(b0 + k * UMMA_K_BYTES), kIdescFp8, k != 0 ? 1u : 0u);
          ptx::umma_commit(L.empty(s));            // smem stage reusable once these MMAs retire
          ptx::umma_commit(L.part_full(buf));      // product of this k-block complete
          if (++s == FSTAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else {
    // ------------------------------ promotion + epilogue -------------------------
    const int ew = warp - 2;               // 0..15
    const int quarter = warp & 3;          // TMEM lanes 32*quarter.. belong to this warp
    const int cg = ew >> 2;                // columns [64*cg, 64*cg + 64) of the tile
    uint64_t* pend_sig = nullptr;          // reduce-scatter variant: signal word of the tile whose store is in flight
    int pend_par = 0, tiles_done = 0;      // ... and which of the four arrival counters that tile uses
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m_blk, n_blk;
      f8_tile_coords<kMode>(prm, rs, tile, &m_blk, &n_blk);
      if constexpr (kAG) {
        // the block's scale columns are pulled like its rows: wait for them before the first scale load
        if (m_blk / prm.ag.blocks_per_rank != prm.ag.my_rank) {
          int arrived_ok = 1;
          if (lane == 0)
            arrived_ok = wait_ge<false>(prm.ag.arrived + m_blk, (unsigned long long)prm.ag.pieces_per_block * prm.ag.call, g, ERR_F8_A_READY) ? 1 : 0;
          arrived_ok = __shfl_sync(0xffffffffu, arrived_ok, 0);
          if (!arrived_ok) { ok = false; break; }
        }
      }
      const int row = m_blk * FBM + quarter * 32 + lane;
      const float* sa = prm.sa + row;
      const float* sb = prm.sb + (n_blk * (FBN / 128) + (cg >> 1));
      const int sb_stride = cp.N / 128;
      float2 acc[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = make_float2(0.f, 0.f);
      // scales are fetched three k-blocks ahead of their use (an L2 round trip is longer than a k-block)
      auto scale_at = [&](int kb) -> float {
        if (kb >= num_kb) return 0.f;
        // pulled scales were written during this kernel: no non-coherent load for them
        const float a = kAG ? *reinterpret_cast<const volatile float*>(sa + (size_t)kb * cp.M) : __ldg(sa + (size_t)kb * cp.M);
        return a * __ldg(sb + (size_t)kb * sb_stride);
      };
      float s0 = scale_at(0), s1 = scale_at(1), s2n = scale_at(2);
#pragma unroll 1
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const float s3 = scale_at(kb + 3);
        const int buf = it & 1;
        if (!mbar_wait(L.part_full(buf), (it >> 1) & 1, g, ERR_F8_PART_FULL)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * FBN + cg * 64;
        const float2 sc = make_float2(s0, s0);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[16];
          ptx::tmem_ld_32x32b_x16(taddr + c * 16, v);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i)
            acc[c * 8 + i] = __ffma2_rn(sc, make_float2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1])), acc[c * 8 + i]);
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(L.part_empty(buf));
        s0 = s1; s1 = s2n; s2n = s3;
      }
      if (!ok) break;
      // ---- tile output: one 64-column chunk per warp through its swizzled staging buffer ----
      if constexpr (kRS) {
        // the previous tile's store has had a whole tile of promotion work to land: complete it and publish it now
        if (lane == 0) {
          ptx::tma_wait_group<0>();
          if (pend_sig != nullptr) {
            rs_publish(L.rs_count(pend_par), pend_sig);
            pend_sig = nullptr;
          }
        }
      } else {
        if (lane == 0) ptx::tma_wait_group_read<0>();
      }
      __syncwarp();
      if constexpr (kRS) {
        const int owner = m_blk / rs->blocks_per_rank;
        if (owner == rs->my_rank && rs->P > 1) {
          // own rows: the P-1 partials of this tile must have landed; add them (source order, fixed) to the accumulators
          const int m_in = m_blk - owner * rs->blocks_per_rank;
          int sig_ok = 1;
          if (lane == 0)
            sig_ok = wait_ge<true>(rs->sig_local + (size_t)m_in * cp.num_n_blocks + n_blk, (unsigned long long)(rs->P - 1) * rs->call, g,
                                   ERR_F8_RS_SIGNAL) ? 1 : 0;
          sig_ok = __shfl_sync(0xffffffffu, sig_ok, 0);
          if (!sig_ok) { ok = false; break; }
          const long long N = cp.N;
          const __nv_bfloat16* src0 = rs->stage_local + (long long)(m_in * FBM + quarter * 32 + (lane >> 3)) * N +
                                      (long long)n_blk * FBN + cg * 64 + (lane & 7) * 8;
          add_partial_chunks<false>(reinterpret_cast<float(&)[64]>(acc), src0, (long long)(cp.M / rs->P) * N, N, rs->P, rs->my_rank, L.epi(ew), lane);
        }
      }
      const uint32_t rowbase = L.epi(ew) + lane * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2* src = &acc[j * 4];
        uint32_t w0 = pack_bf16(src[0].x, src[0].y), w1 = pack_bf16(src[1].x, src[1].y);
        uint32_t w2 = pack_bf16(src[2].x, src[2].y), w3 = pack_bf16(src[3].x, src[3].y);
        uint32_t dst = rowbase + ((j ^ (lane & 7)) << 4);
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if constexpr (!kRS) {
        if (lane == 0) {
          ptx::tma_store_2d(&prm.map_c, L.epi(ew), n_blk * FBN + cg * 64, m_blk * FBM + quarter * 32);
          ptx::tma_commit_group();
        }
      } else {
        if (lane == 0) {
          const int owner = m_blk / rs->blocks_per_rank, m_in = m_blk - owner * rs->blocks_per_rank;
          if (owner == rs->my_rank) {
            // the reduced chunk of this PE's own rows goes straight to the output
            ptx::tma_store_2d(&rs->map_out, L.epi(ew), n_blk * FBN + cg * 64, m_in * FBM + quarter * 32);
            ptx::tma_commit_group();
          } else {
            // partial chunk -> the owner's staging slot (peer memory), then one signal per tile
            ptx::tma_store_2d(&rs->map_stage[owner], L.epi(ew), n_blk * FBN + cg * 64, m_in * FBM + quarter * 32);
            ptx::tma_commit_group();
            // the tile's signal is sent once every warp's store is complete: at the next tile's output stage
            pend_sig = reinterpret_cast<uint64_t*>(rs->sig_remote[owner] + (size_t)m_in * cp.num_n_blocks + n_blk);
            pend_par = tiles_done & 3;
          }
        }
      }
      ++tiles_done;
    }
    if (lane == 0) {
      ptx::tma_wait_group<0>();
      if constexpr (kRS) {
        if (pend_sig != nullptr) rs_publish(L.rs_count(pend_par), pend_sig);
      }
    }
    __syncwarp();
  }

  // ------------------------------ teardown ---------------------------------------
  ptx::tc_fence_before();
  __syncthreads();
  if constexpr (kAG) {
    // before the kernel ends, CTA 0 makes sure every peer has finished pulling this PE's rows
    if (!*L.abort_flag() && blockIdx.x == 0 && (int)threadIdx.x < prm.ag.P && (int)threadIdx.x != prm.ag.my_rank)
      wait_ge<true>(prm.ag.done_local + threadIdx.x, prm.ag.call, g, ERR_F8_PEER_DONE);
    __syncthreads();
  }
  if (*L.abort_flag()) {
    // let copies and MMAs that are still in flight land before smem/TMEM go away
    unsigned long long t0 = ptx::globaltimer();
    while (ptx::globaltimer() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

__global__ void __launch_bounds__(FNUM_THREADS, 1) gemm_fp8_blockscale_kernel(const __grid_constant__ Fp8Params prm) {
  extern __shared__ uint8_t smem_raw[];
  gemm_fp8_body<F8_PLAIN>(prm, nullptr, smem_raw);
}
// all-gather -> GEMM: two more warps per CTA pull the peers' rows and scales while the tensor core runs
__global__ void __launch_bounds__(FNUM_THREADS + 32 * FPULL_WARPS, 1) ag_gemm_fp8_kernel(const __grid_constant__ Fp8Params prm) {
  extern __shared__ uint8_t smem_raw[];
  gemm_fp8_body<F8_AG>(prm, nullptr, smem_raw);
}
// GEMM -> reduce-scatter: partial tiles go to their owner's staging over NVLink, owned tiles are reduced at the end
__global__ void __launch_bounds__(FNUM_THREADS, 1) gemm_rs_fp8_kernel(const __grid_constant__ Fp8RsParams prm) {
  extern __shared__ uint8_t smem_raw[];
  gemm_fp8_body<F8_RS>(prm.base, &prm.rs, smem_raw);
}

// ---- quantisers ------------------------------------------------------------------------------
__device__ __forceinline__ uint8_t to_e4m3(float x) {
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

// Activations: one scale per row and 128 columns.  One warp per (row, k-block); lane l owns 4 elements.
// q: [M, K] e4m3, scales: [K/128][M] fp32 with  x ≈ q * scale,  scale = absmax / 448 (1 if the block is all zero).
__global__ void quant_act_1x128_kernel(const __nv_bfloat16* __restrict__ x, int M, int K, int ldx, uint8_t* __restrict__ q,
                                       float* __restrict__ scales, int scale_ld) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long nblk = (long long)M * (K / 128);
  for (long long w = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); w < nblk; w += (long long)gridDim.x * warps_per_block) {
    const int kb = (int)(w % (K / 128));
    const int m = (int)(w / (K / 128));
    const uint2 raw = *reinterpret_cast<const uint2*>(x + (size_t)m * ldx + kb * 128 + lane * 4);
    const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    float v[4] = {__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1)};
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = amax > 0.f ? amax / 448.f : 1.f;
    const float inv = 1.f / scale;
    uint32_t packed = to_e4m3(v[0] * inv) | (to_e4m3(v[1] * inv) << 8) | (to_e4m3(v[2] * inv) << 16) | ((uint32_t)to_e4m3(v[3] * inv) << 24);
    *reinterpret_cast<uint32_t*>(q + (size_t)m * K + kb * 128 + lane * 4) = packed;
    if (lane == 0) scales[(size_t)kb * scale_ld + m] = scale;
  }
}

// Weights: one scale per 128x128 block.  One CTA (256 threads) per block; scales: [K/128][N/128].
__global__ void quant_w_128x128_kernel(const __nv_bfloat16* __restrict__ w, int N, int K, int ldw, uint8_t* __restrict__ q,
                                       float* __restrict__ scales) {
  __shared__ float red[8];
  __shared__ float s_scale;
  const int kb = blockIdx.x, nb = blockIdx.y;
  const int t = threadIdx.x;
  // thread t: row (t >> 1) + 0 of the block ... 64 elements of one row: rows = 128, two threads per row
  const int r = t >> 1, c0 = (t & 1) * 64;
  const __nv_bfloat16* src = w + (size_t)(nb * 128 + r) * ldw + kb * 128 + c0;
  float v[64];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint4 raw = reinterpret_cast<const uint4*>(src)[i];
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[i * 8 + 2 * j] = __low2float(p[j]);
      v[i * 8 + 2 * j + 1] = __high2float(p[j]);
      amax = fmaxf(amax, fmaxf(fabsf(v[i * 8 + 2 * j]), fabsf(v[i * 8 + 2 * j + 1])));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((t & 31) == 0) red[t >> 5] = amax;
  __syncthreads();
  if (t == 0) {
    float a = red[0];
    for (int i = 1; i < 8; ++i) a = fmaxf(a, red[i]);
    s_scale = a > 0.f ? a / 448.f : 1.f;
    scales[(size_t)kb * (N / 128) + nb] = s_scale;
  }
  __syncthreads();
  const float inv = 1.f / s_scale;
  uint8_t* dst = q + (size_t)(nb * 128 + r) * K + kb * 128 + c0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float* e = &v[i * 16 + j * 4];
      o[j] = to_e4m3(e[0] * inv) | (to_e4m3(e[1] * inv) << 8) | (to_e4m3(e[2] * inv) << 16) | ((uint32_t)to_e4m3(e[3] * inv) << 24);
    }
    reinterpret_cast<uint4*>(dst)[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

int* g_err_dev[64] = {};
int g_sms[64] = {};

struct AgPlan {
  bshmem_dev_state_t st;
  int M, N, K, device;
  unsigned long long call = 0;
  int* err = nullptr;
  char* xq_local = nullptr;                    // symmetric [M, K] e4m3
  float* sa_local = nullptr;                   // symmetric [K/128][M]
  unsigned long long* flags_local = nullptr;   // symmetric: ready[P] then done[P]
  unsigned long long* arrived = nullptr;
  unsigned long long* src_pulled = nullptr;
  unsigned int* ticket = nullptr;
};

struct RsPlan {
  bshmem_dev_state_t st;
  int M, N, K, device;
  unsigned long long call = 0;
  int* err = nullptr;
  char* staging_local = nullptr;               // symmetric: [2 parities][P sources][M/P][N] bf16
  unsigned long long* sig_local = nullptr;     // symmetric: [M/P/128 * N/256]
};

template <typename T> T* peer_ptr(const bshmem_dev_state_t& st, T* local, int pe) {
  return reinterpret_cast<T*>(st.heap_base[pe] + (reinterpret_cast<char*>(local) - st.heap_base[st.my_pe]));
}
bool in_heap(const bshmem_dev_state_t& st, const void* p, uint64_t n) {
  const char* c = static_cast<const char*>(p);
  const char* b = st.heap_base[st.my_pe];
  return c >= b && (uint64_t)(c - b) + n <= st.heap_bytes;
}

int ensure(int dev) {
  if (g_err_dev[dev]) return 0;
  BSHMEM_CUDA_TRY(cudaMalloc(&g_err_dev[dev], sizeof(int)));
  BSHMEM_CUDA_TRY(cudaMemset(g_err_dev[dev], 0, sizeof(int)));
  BSHMEM_CUDA_TRY(cudaDeviceGetAttribute(&g_sms[dev], cudaDevAttrMultiProcessorCount, dev));
  BSHMEM_CUDA_TRY(cudaFuncSetAttribute(gemm_fp8_blockscale_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FSMEM_BYTES));
  BSHMEM_CUDA_TRY(cudaFuncSetAttribute(ag_gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FSMEM_BYTES));
  BSHMEM_CUDA_TRY(cudaFuncSetAttribute(gemm_rs_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FSMEM_BYTES));
  return 0;
}

}  // namespace

extern "C" {

const char* bshmem_fp8_last_error() { return host::last_error().c_str(); }

// C[M,N] bf16 = block-scaled A8[M,K] · B8[N,K]^T.  M % 128 == 0, N % 256 == 0, K % 128 == 0; A8/B8 dense
// (row pitch K bytes), scale_a: [K/128][M], scale_b: [K/128][N/128], ldc in elements (% 8 == 0).
int bshmem_gemm_fp8_blockscale(const void* A8, const float* scale_a, const void* B8, const float* scale_b, void* C, int M, int N,
                               int K, int ldc, void* stream, int max_ctas, int timeout_ms) {
  if (M <= 0 || N <= 0 || K <= 0 || M % FBM || N % FBN || K % FBK || ldc % 8) {
    host::last_error() = "fp8 gemm: needs M % 128 == 0, N % 256 == 0, K % 128 == 0, ldc % 8 == 0";
    return 1;
  }
  int dev = 0;
  BSHMEM_CUDA_TRY(cudaGetDevice(&dev));
  int rc = ensure(dev);
  if (rc) return rc;
  Fp8Params p;
  memset(&p, 0, sizeof(p));
  p.core.M = M; p.core.N = N; p.core.K = K;
  p.core.num_m_blocks = M / FBM; p.core.num_n_blocks = N / FBN;
  p.core.group_m = 32;
  p.core.timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 4000) * 1000000ull;
  p.core.err = g_err_dev[dev];
  p.sa = scale_a; p.sb = scale_b;
  rc = host::make_tmap_2d(&p.map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A8, M, K, K, FBM, FBK);
  if (rc) return rc;
  rc = host::make_tmap_2d(&p.map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B8, N, K, K, FBN, FBK);
  if (rc) return rc;
  rc = host::make_tmap_2d(&p.map_c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, M, N, ldc, 32, 64);
  if (rc) return rc;
  int ctas = g_sms[dev];
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  const int tiles = p.core.num_m_blocks * p.core.num_n_blocks;
  if (ctas > tiles) ctas = tiles;
  gemm_fp8_blockscale_kernel<<<ctas, FNUM_THREADS, FSMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(p);
  BSHMEM_CUDA_TRY(cudaGetLastError());
  return 0;
}

// x: [M, K] bf16 (ldx elements, % 4 == 0, 8-byte aligned rows) -> q [M, K] e4m3 + scales; the scale of row m and
// k-block kb goes to scales[kb * scale_ld + m] (scale_ld >= M: a shard can write its columns of a wider matrix).
int bshmem_fp8_quant_act_ld(const void* x, int M, int K, int ldx, void* q, float* scales, int scale_ld, void* stream) {
  if (K % 128 || ldx % 4 || scale_ld < M) { host::last_error() = "fp8 quant: K % 128 != 0, ldx % 4 != 0 or scale_ld < M"; return 1; }
  long long nblk = (long long)M * (K / 128);
  int blocks = (int)((nblk + 7) / 8 < 148 * 16 ? (nblk + 7) / 8 : 148 * 16);
  if (blocks < 1) blocks = 1;
  quant_act_1x128_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x), M, K, ldx,
                                                                                static_cast<uint8_t*>(q), scales, scale_ld);
  BSHMEM_CUDA_TRY(cudaGetLastError());
  return 0;
}
int bshmem_fp8_quant_act(const void* x, int M, int K, int ldx, void* q, float* scales, void* stream) {
  return bshmem_fp8_quant_act_ld(x, M, K, ldx, q, scales, M, stream);
}

// ---- all-gather -> fp8 GEMM -------------------------------------------------------------------------------
// Symmetric memory of a plan: xq [M, K] bytes, sa [K/128][M] floats, 2*P flag words (zeroed, then a barrier).
uint64_t bshmem_fp8_ag_flag_bytes(int P) { return 2ull * P * 8; }

int bshmem_fp8_ag_plan(const bshmem_dev_state_t* st, int M, int N, int K, void* xq_local, void* sa_local, void* flags_local, void** out) {
  if (!st || !out) return 1;
  const int P = st->n_pes;
  if (P > kMaxPes || M % (P * FBM) || N % FBN || K % FBK) {
    host::last_error() = "ag_gemm_fp8: needs M % (P*128) == 0, N % 256 == 0, K % 128 == 0";
    return 1;
  }
  if (!in_heap(*st, xq_local, (uint64_t)M * K) || !in_heap(*st, sa_local, (uint64_t)(K / 128) * M * 4) ||
      !in_heap(*st, flags_local, bshmem_fp8_ag_flag_bytes(P))) {
    host::last_error() = "ag_gemm_fp8: the gathered activations, their scales and the flags must be symmetric allocations";
    return 4;
  }
  AgPlan* p = new AgPlan();
  p->st = *st; p->M = M; p->N = N; p->K = K;
  p->xq_local = static_cast<char*>(xq_local);
  p->sa_local = static_cast<float*>(sa_local);
  p->flags_local = static_cast<unsigned long long*>(flags_local);
  BSHMEM_CUDA_TRY(cudaGetDevice(&p->device));
  int rc = ensure(p->device);
  if (rc) { delete p; return rc; }
  const int nblk = M / FBM;
  BSHMEM_CUDA_TRY(cudaMalloc(&p->err, sizeof(int)));
  BSHMEM_CUDA_TRY(cudaMemset(p->err, 0, sizeof(int)));
  BSHMEM_CUDA_TRY(cudaMalloc(&p->arrived, sizeof(unsigned long long) * nblk));
  BSHMEM_CUDA_TRY(cudaMemset(p->arrived, 0, sizeof(unsigned long long) * nblk));
  BSHMEM_CUDA_TRY(cudaMalloc(&p->src_pulled, sizeof(unsigned long long) * kMaxPes));
  BSHMEM_CUDA_TRY(cudaMemset(p->src_pulled, 0, sizeof(unsigned long long) * kMaxPes));
  BSHMEM_CUDA_TRY(cudaMalloc(&p->ticket, sizeof(unsigned int) * 2));
  BSHMEM_CUDA_TRY(cudaMemset(p->ticket, 0, sizeof(unsigned int) * 2));
  *out = p;
  return 0;
}

// This PE's quantised rows and scale columns must already be in place (bshmem_fp8_quant_act_ld into the shard's slice).
// B8: [N, K] e4m3, scale_b: [K/128][N/128], C: [M, N] bf16 (ldc).
int bshmem_fp8_ag_run(void* plan, const void* B8, const float* scale_b, void* C, int ldc, void* stream, int timeout_ms, int max_ctas) {
  AgPlan* p = static_cast<AgPlan*>(plan);
  if (!p || ldc % 8) return 1;
  const int P = p->st.n_pes, me = p->st.my_pe;
  p->call += 1;
  Fp8Params prm;
  memset(&prm, 0, sizeof(prm));
  prm.core.M = p->M; prm.core.N = p->N; prm.core.K = p->K;
  prm.core.num_m_blocks = p->M / FBM; prm.core.num_n_blocks = p->N / FBN;
  prm.core.group_m = 32;
  prm.core.timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 2000) * 1000000ull;
  prm.core.err = p->err;
  prm.sa = p->sa_local; prm.sb = scale_b;
  Fp8Ag& a = prm.ag;
  a.P = P; a.my_rank = me; a.blocks_per_rank = p->M / P / FBM;
  a.row_bytes = (unsigned long long)p->K;
  a.num_kb = p->K / FBK;
  a.pieces_per_row = (int)((a.row_bytes + kPieceBytes - 1) / kPieceBytes);
  a.pieces_per_block = FBM * a.pieces_per_row + 1;                 // + the block's scale columns
  a.pieces_per_src = a.blocks_per_rank * a.pieces_per_block;
  a.total_pieces = (P - 1) * a.pieces_per_src;
  int rc = host::make_tmap_2d(&prm.map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p->xq_local, p->M, p->K, p->K, FBM, FBK);
  if (rc) return rc;
  rc = host::make_tmap_2d(&prm.map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B8, p->N, p->K, p->K, FBN, FBK);
  if (rc) return rc;
  rc = host::make_tmap_2d(&prm.map_c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, p->M, p->N, ldc, 32, 64);
  if (rc) return rc;
  for (int q = 0; q < P; ++q) {
    a.xq_peer[q] = peer_ptr(p->st, p->xq_local, q);
    a.sa_peer[q] = peer_ptr(p->st, p->sa_local, q);
    a.ready_remote[q] = peer_ptr(p->st, p->flags_local, q);
    a.done_remote[q] = peer_ptr(p->st, p->flags_local, q) + P;
  }
  a.xq_local = p->xq_local; a.sa_local = p->sa_local;
  a.arrived = p->arrived; a.src_pulled = p->src_pulled; a.ticket = p->ticket;
  a.ready_local = p->flags_local; a.done_local = p->flags_local + P;
  a.call = p->call;
  int ctas = g_sms[p->device];
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  const int tiles = prm.core.num_m_blocks * prm.core.num_n_blocks;
  if (ctas > tiles) ctas = tiles;
  ag_gemm_fp8_kernel<<<ctas, FNUM_THREADS + 32 * FPULL_WARPS, FSMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(prm);
  BSHMEM_CUDA_TRY(cudaGetLastError());
  return 0;
}

// ---- fp8 GEMM -> reduce-scatter ---------------------------------------------------------------------------
// out[M/P, N] (this PE's rows) = sum over PEs r of dequant(A8_r)[M, K] · dequant(B8_r)[N, K]^T (every PE holds a K shard).
// Symmetric memory of a plan: staging 2 * M * N bf16 (two call parities) and M/P/128 * N/256 signal words (zeroed,
// then a barrier before the first call).
uint64_t bshmem_fp8_rs_staging_bytes(int M, int N) { return 2ull * (uint64_t)M * N * 2; }
uint64_t bshmem_fp8_rs_signal_bytes(int M, int N, int P) { return (uint64_t)(M / P / FBM) * (N / FBN) * 8; }

int bshmem_fp8_rs_plan(const bshmem_dev_state_t* st, int M, int N, int K, void* staging_local, void* sig_local, void** out) {
  if (!st || !out) return 1;
  const int P = st->n_pes;
  if (P > kMaxPes || M % (P * FBM) || N % FBN || K % FBK) {
    host::last_error() = "gemm_rs_fp8: needs M % (P*128) == 0, N % 256 == 0, K % 128 == 0";
    return 1;
  }
  if (!in_heap(*st, staging_local, bshmem_fp8_rs_staging_bytes(M, N)) || !in_heap(*st, sig_local, bshmem_fp8_rs_signal_bytes(M, N, P))) {
    host::last_error() = "gemm_rs_fp8: staging and signal buffers must be symmetric allocations of the stated sizes";
    return 4;
  }
  RsPlan* p = new RsPlan();
  p->st = *st; p->M = M; p->N = N; p->K = K;
  p->staging_local = static_cast<char*>(staging_local);
  p->sig_local = static_cast<unsigned long long*>(sig_local);
  BSHMEM_CUDA_TRY(cudaGetDevice(&p->device));
  int rc = ensure(p->device);
  if (rc) { delete p; return rc; }
  BSHMEM_CUDA_TRY(cudaMalloc(&p->err, sizeof(int)));
  BSHMEM_CUDA_TRY(cudaMemset(p->err, 0, sizeof(int)));
  *out = p;
  return 0;
}

// A8: [M, K] e4m3 + scale_a [K/128][M]; B8: [N, K] e4m3 + scale_b [K/128][N/128]; out: [M/P, N] bf16 (ldo).
int bshmem_fp8_rs_run(void* plan, const void* A8, const float* scale_a, const void* B8, const float* scale_b, void* out, int ldo,
                      void* stream, int timeout_ms, int max_ctas) {
  RsPlan* p = static_cast<RsPlan*>(plan);
  if (!p || ldo % 8) return 1;
  const int P = p->st.n_pes, me = p->st.my_pe;
  p->call += 1;
  const int parity = (int)(p->call & 1);
  Fp8RsParams prm;
  memset(&prm, 0, sizeof(prm));
  Fp8Params& b = prm.base;
  b.core.M = p->M; b.core.N = p->N; b.core.K = p->K;
  b.core.num_m_blocks = p->M / FBM; b.core.num_n_blocks = p->N / FBN;
  b.core.group_m = 32;
  b.core.timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 2000) * 1000000ull;
  b.core.err = p->err;
  b.sa = scale_a; b.sb = scale_b;
  int rc = host::make_tmap_2d(&b.map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A8, p->M, p->K, p->K, FBM, FBK);
  if (rc) return rc;
  rc = host::make_tmap_2d(&b.map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B8, p->N, p->K, p->K, FBN, FBK);
  if (rc) return rc;
  Fp8Rs& r = prm.rs;
  r.P = P; r.my_rank = me; r.blocks_per_rank = p->M / P / FBM;
  const uint64_t rows = (uint64_t)p->M / P;
  const uint64_t slot_bytes = rows * p->N * 2;
  for (int q = 0; q < P; ++q) {
    char* slot = peer_ptr(p->st, p->staging_local, q) + ((uint64_t)parity * P + me) * slot_bytes;
    rc = host::make_tmap_2d(&r.map_stage[q], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, slot, rows, p->N, p->N, 32, 64);
    if (rc) return rc;
    r.sig_remote[q] = peer_ptr(p->st, p->sig_local, q);
  }
  r.sig_local = p->sig_local;
  r.stage_local = reinterpret_cast<const __nv_bfloat16*>(p->staging_local + (uint64_t)parity * P * slot_bytes);
  r.out = static_cast<__nv_bfloat16*>(out);
  r.ldo = ldo;
  rc = host::make_tmap_2d(&r.map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, out, rows, p->N, ldo, 32, 64);
  if (rc) return rc;
  r.call = p->call;
  int ctas = g_sms[p->device];
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  const int tiles = b.core.num_m_blocks * b.core.num_n_blocks;
  if (ctas > tiles) ctas = tiles;
  gemm_rs_fp8_kernel<<<ctas, FNUM_THREADS, FSMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(prm);
  BSHMEM_CUDA_TRY(cudaGetLastError());
  return 0;
}

int bshmem_fp8_rs_error_site(void* plan, int clear) {
  RsPlan* p = static_cast<RsPlan*>(plan);
  int v = 0;
  if (!p || !p->err) return 0;
  cudaMemcpy(&v, p->err, sizeof(int), cudaMemcpyDeviceToHost);
  if (clear && v) cudaMemset(p->err, 0, sizeof(int));
  return v;
}

int bshmem_fp8_rs_destroy(void* plan) {
  RsPlan* p = static_cast<RsPlan*>(plan);
  if (!p) return 0;
  cudaFree(p->err);
  delete p;
  return 0;
}

int bshmem_fp8_ag_error_site(void* plan, int clear) {
  AgPlan* p = static_cast<AgPlan*>(plan);
  int v = 0;
  if (!p || !p->err) return 0;
  cudaMemcpy(&v, p->err, sizeof(int), cudaMemcpyDeviceToHost);
  if (clear && v) cudaMemset(p->err, 0, sizeof(int));
  return v;
}

int bshmem_fp8_ag_destroy(void* plan) {
  AgPlan* p = static_cast<AgPlan*>(plan);
  if (!p) return 0;
  cudaFree(p->err); cudaFree(p->arrived); cudaFree(p->src_pulled); cudaFree(p->ticket);
  delete p;
  return 0;
}

// w: [N, K] bf16 (ldw % 8 == 0) -> q [N, K] e4m3 + scales [K/128][N/128].
int bshmem_fp8_quant_weight(const void* w, int N, int K, int ldw, void* q, float* scales, void* stream) {
  if (K % 128 || N % 128 || ldw % 8) { host::last_error() = "fp8 quant: N, K % 128 != 0 or ldw % 8 != 0"; return 1; }
  quant_w_128x128_kernel<<<dim3(K / 128, N / 128), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(w), N, K, ldw, static_cast<uint8_t*>(q), scales);
  BSHMEM_CUDA_TRY(cudaGetLastError());
  return 0;
}

int bshmem_fp8_error_site(int clear) {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || !g_err_dev[dev]) return 0;
  cudaMemcpy(&v, g_err_dev[dev], sizeof(int), cudaMemcpyDeviceToHost);
  if (clear && v) cudaMemset(g_err_dev[dev], 0, sizeof(int));
  return v;
}

}  // extern "C"
