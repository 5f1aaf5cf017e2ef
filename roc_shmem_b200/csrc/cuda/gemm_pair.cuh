// gemm_pair.cuh — persistent tcgen05 GEMM main loop on CTA PAIRS (cta_group::2) for
// sm_100a:  C[M,N] = A[M,K] · B[N,K]^T, bf16 operands, fp32 accumulation in TMEM.
//
// A thread-block cluster of two CTAs (two SMs of one TPC) owns a 256x256 output tile:
//   CTA r of the pair loads A rows [128r, 128r+128) and B rows [128r, 128r+128) of the
//   tile — 32 KiB per stage and CTA, plain (non-multicast) TMA loads from this GPU's own
//   memory — and holds the accumulator of its 128 output rows x 256 columns in its TMEM.
//   One thread of the pair's first CTA issues tcgen05.mma.cta_group::2 (M256 N256 K16);
//   the tensor cores of both SMs read both CTAs' shared memory.
// An accumulator is 256 TMEM columns, so the 512 columns hold TWO: the epilogue of tile
// i (tcgen05.ld -> bf16 -> swizzled smem -> TMA store, possibly to another GPU) runs
// while the tensor cores already work on tile i+1.  That is the point of this core: the
// single-CTA 256x256 loop (gemm_core.cuh) has to drain both of its accumulators before
// the next tile can start, which exposes the epilogue — and everything the epilogue
// waits for, e.g. NVLink stores — on the critical path.
//
//   warp 0      TMA producer (each CTA for its own halves), 6-stage ring
//   warp 1      first CTA: MMA issuer.  second CTA: relay — waits for its own stage to
//               fill, then arrives on the first CTA's `full` barrier of that stage, which
//               expects two arrivals (a load without the cta_group qualifier can only
//               signal a barrier of the CTA it writes to)
//   warps 2-9   epilogue: warp w drains TMEM lanes 32*(w%4).., columns 128*(w>=6)..
//
// tcgen05.commit (with its cluster-multicast form, a barrier arrival, not a load) hands
// stages and accumulators back to BOTH CTAs.
// Every wait is bounded by a %globaltimer deadline; on expiry the CTA records a site
// code in the error word and all roles leave their loops; both CTAs always reach the
// closing cluster barrier before TMEM is released.  Every load is a plain tiled TMA
// load of one CTA.  The reference has no GEMM, hence no counterpart.
#pragma once
#include "gemm_core.cuh"

namespace bshmem {
namespace gemm2 {

using gemm::CoreParams;
using gemm::Guard;
using gemm::guard_fail;
using gemm::pack_bf16;
using gemm::raster_coords;

constexpr int BM = 256, BN = 256;                 // tile of the CTA pair
constexpr int CTA_M = 128, CTA_NLOAD = 128;       // rows of A / of B one CTA loads
constexpr int BK_BYTES = 128;
constexpr int BK = 64;                            // bf16 elements per k-block
#ifndef BSHMEM_PAIR_STAGES
#define BSHMEM_PAIR_STAGES 6
#endif
constexpr int STAGES = BSHMEM_PAIR_STAGES;
constexpr int UMMA_K_BYTES = 32;
constexpr int NUM_EPI_WARPS = 8;
constexpr int NUM_THREADS = 32 * (2 + NUM_EPI_WARPS);
constexpr int EPI_COLS = 64;
constexpr uint32_t A_STAGE_BYTES = CTA_M * BK_BYTES;           // 16 KiB
constexpr uint32_t B_STAGE_BYTES = CTA_NLOAD * BK_BYTES;       // 16 KiB
constexpr uint32_t STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr uint32_t EPI_BUF_BYTES = 32 * EPI_COLS * 2;          // one warp: 32 rows x 128 B
constexpr uint32_t SMEM_TILES = STAGES * STAGE_BYTES + NUM_EPI_WARPS * EPI_BUF_BYTES;
constexpr uint32_t SMEM_BARS = 512;
constexpr uint32_t SMEM_BYTES = SMEM_TILES + SMEM_BARS + 1024 /*alignment slack*/;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t ACC_COLS = 256;
constexpr uint32_t kIdescBf16 = ptx::umma_idesc(1, 1, BM, BN);

enum ErrSite : int {
  ERR_PRODUCER_EMPTY = 201, ERR_MMA_FULL = 202, ERR_MMA_TMEM_EMPTY = 204, ERR_EPI_TMEM_FULL = 205,
  ERR_RELAY_FULL = 206, ERR_A_READY = 207, ERR_PEER_SIGNAL = 208, ERR_PEER_READY = 209, ERR_PEER_DONE = 210
};

// ---- cluster / cta_group::2 PTX --------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory byte in CTA `rank` of this cluster (shared::cluster window).
__device__ __forceinline__ uint32_t mapa(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Waits use the default (CTA-scope) acquire also for barriers the other CTA arrives on: what such an arrival
// announces is shared-memory or tensor-memory traffic of the async proxies (TMA, tcgen05), not generic-proxy
// stores, and a cluster-scope acquire on every poll made the MMA issuer the bottleneck (2.5x slower).
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) { return ptx::mbar_try_wait(bar, parity); }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_result, uint32_t ncols) {   // whole warp, in both CTAs
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One commit that arrives on the barrier at this offset in BOTH CTAs of the pair (two single-destination commits
// per k-block cost the issuing thread 6 % of the GEMM's throughput).
__device__ __forceinline__ void umma2_commit_both(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}

// Host side: how many CTA pairs of `kernel` the device can hold at once (at most one per two SMs).
template <class Kernel>
inline int max_resident_pairs(Kernel kernel, int sms) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(sms & ~1), 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = sms / 2; }
  return n < sms / 2 ? n : sms / 2;
}

__device__ __forceinline__ bool pair_wait(uint32_t bar, uint32_t parity, Guard& g, int site) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  unsigned long long t0 = ptx::globaltimer();
  uint32_t it = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if ((++it & 0x3F) == 0) {
      if (*g.abort_flag) return false;
      if (ptx::globaltimer() - t0 > g.timeout_ns) return guard_fail(g, site);
    }
  }
  return true;
}

// Shared-memory carve-up (shared-window byte addresses).
struct Smem {
  uint32_t base;        // 1024-byte aligned
  uint8_t* gen;         // generic pointer to the same byte
  __device__ __forceinline__ uint32_t a(int s) const { return base + s * STAGE_BYTES; }
  __device__ __forceinline__ uint32_t b(int s) const { return base + s * STAGE_BYTES + A_STAGE_BYTES; }
  __device__ __forceinline__ uint32_t epi(int w) const { return base + STAGES * STAGE_BYTES + w * EPI_BUF_BYTES; }
  __device__ __forceinline__ uint8_t* epi_gen(int w) const { return gen + STAGES * STAGE_BYTES + w * EPI_BUF_BYTES; }
  __device__ __forceinline__ uint32_t bars() const { return base + SMEM_TILES; }
  __device__ __forceinline__ uint32_t full(int s) const { return bars() + 8 * s; }
  __device__ __forceinline__ uint32_t empty(int s) const { return bars() + 8 * (2 * STAGES + s); }
  __device__ __forceinline__ uint32_t tmem_full(int a) const { return bars() + 8 * (3 * STAGES + a); }
  __device__ __forceinline__ uint32_t tmem_empty(int a) const { return bars() + 8 * (3 * STAGES + 2 + a); }
  __device__ __forceinline__ uint32_t tmem_slot() const { return bars() + 8 * (3 * STAGES + 4); }
  __device__ __forceinline__ volatile int* abort_flag() const {
    return reinterpret_cast<volatile int*>(gen + SMEM_TILES + 8 * (3 * STAGES + 4) + 8);
  }
  // 8 words of policy scratch per CTA (zeroed at kernel start), e.g. per-tile arrival counters
  __device__ __forceinline__ unsigned int* scratch() const {
    return reinterpret_cast<unsigned int*>(gen + SMEM_TILES + 256);
  }
  // one word of private state per warp, zeroed at kernel start
  __device__ __forceinline__ volatile int* warp_state(int w) const {
    return reinterpret_cast<volatile int*>(gen + SMEM_TILES + 320 + 4 * w);
  }
};

__device__ __forceinline__ Smem carve_smem(uint8_t* raw) {
  Smem L;
  uint32_t r = ptx::smem_u32(raw);
  L.base = (r + 1023u) & ~1023u;
  L.gen = raw + (L.base - r);
  return L;
}

// What an epilogue warp knows about the chunk it is draining.
struct Chunk {
  int m_blk, n_blk;     // tile
  int row0;             // first of the warp's 32 output rows (row of lane l = row0 + l)
  int col0;             // first of the chunk's 64 output columns
  int ordinal;          // how many tiles this CTA pair has finished before this one
  int half;             // which 128-row half of the tile this CTA holds (its rank in the pair)
};

struct PolicyDefaults {
  struct EpiState {};
  // Gated epilogue: inside every 64-column chunk of the accumulator, columns 0-31 are gate pre-activations and 32-63
  // the matching up-projections; the epilogue writes silu(gate) * up, i.e. half as many output columns (the two
  // chunks of a warp make one 32 x 64 output box; out_target gets the OUTPUT column).
  static constexpr bool kGated = false;
  // Operand layout.  Default: both operands K-major, one 128-row x 128-byte TMA box per operand, CTA and stage, and
  // shared-memory descriptors that step 32 bytes along K inside the swizzle atom.  A policy with MN-major operands
  // overrides the instruction descriptor, the stage-0 descriptors, the step per MMA and the loads.
  static constexpr uint32_t kIdesc = kIdescBf16;
  static constexpr uint32_t kKStepBytes = UMMA_K_BYTES;
  __device__ static __forceinline__ uint64_t desc_a0(uint32_t a0) { return ptx::umma_desc_sw128(a0); }
  __device__ static __forceinline__ uint64_t desc_b0(uint32_t b0) { return ptx::umma_desc_sw128(b0); }
  // a_row / b_row: first row this CTA loads (its rank's half included); kb: k-block of the tile
  template <class Params>
  __device__ static __forceinline__ void load_stage(const Params&, const CUtensorMap* ma, const CUtensorMap* mb, uint32_t a_smem,
                                                    uint32_t b_smem, uint32_t bar, int kb, int a_row, int b_row, int, int, int) {
    ptx::tma_load_2d(a_smem, ma, bar, kb * BK, a_row);
    ptx::tma_load_2d(b_smem, mb, bar, kb * BK, b_row);
  }
  // k-blocks of the tile's reduction (ragged per group in the grouped weight-gradient GEMM); at least 1
  template <class Params> __device__ static __forceinline__ int num_kb(const Params& p, int) { return (p.core.K + BK - 1) / BK; }
  // first row of the 256-row block of A / of the 256-row block of B that tile (m_blk, n_blk) multiplies
  template <class Params> __device__ static __forceinline__ int a_row(const Params&, int m_blk) { return m_blk * BM; }
  template <class Params> __device__ static __forceinline__ int b_row(const Params&, int, int n_blk) { return n_blk * BN; }
  template <class Params> __device__ static __forceinline__ bool a_ready(const Params&, int, Guard&) { return true; }
  template <class Params> __device__ static __forceinline__ int num_tiles(const Params& p) {
    return p.core.num_m_blocks * p.core.num_n_blocks;
  }
  template <class Params> __device__ static __forceinline__ bool idle_work(const Params&, int, int, Guard&, int, volatile int*) { return false; }
  // epilogue warp, accumulator of the tile is complete, before the first chunk; false aborts
  template <class Params, class St> __device__ static __forceinline__ bool tile_begin(const Params&, const Smem&, St&, const Chunk&, int, int, Guard&) { return true; }
  // the warp's 64 accumulators of this chunk (row = lane) may be changed before they are packed and stored;
  // the warp's staging buffer is free to use here (the previous store has finished reading it)
  template <class Params, class St> __device__ static __forceinline__ void adjust(const Params&, const Smem&, St&, const Chunk&, float (&)[64], int, int) {}
  // after the warp issued (not completed) its stores of the tile
  template <class Params, class St> __device__ static __forceinline__ void tile_end(const Params&, const Smem&, St&, const Chunk&, int, int) {}
  // after an epilogue warp's last tile, all of its stores complete
  template <class Params, class St> __device__ static __forceinline__ void epilogue_drain(const Params&, const Smem&, St&, int, int, Guard&) {}
  template <class Params> __device__ static __forceinline__ void tail(const Params&, const Smem&, Guard&) {}
  template <class Params> __device__ static __forceinline__ void prologue(const Params&, Guard&) {}
};

// Policy contract (static __device__ members; P::Params is the kernel's by-value parameter):
//   core(prm) -> const CoreParams&        map_a(prm), map_b(prm) -> const CUtensorMap*
//   tile_coords(prm, tile, &m_blk, &n_blk)     tile = index in the pair's schedule (pair id + k * pairs)
//   a_ready(prm, m_blk, guard)            producer lane, before a tile's first A load (rows of the whole 256-row block)
//   out_target(prm, row, col, &map, &x, &y)    where the 32x64 chunk starting at C[row, col] goes (map may be null)
//   a_row(prm, m_blk), b_row(prm, m_blk, n_blk), kGated                          (defaults in PolicyDefaults)
//   the hooks of PolicyDefaults
template <class P>
__device__ __forceinline__ void gemm_mainloop(const typename P::Params& prm, uint8_t* smem_raw) {
  const CoreParams& cp = P::core(prm);
  const Smem L = carve_smem(smem_raw);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();            // 0 issues the MMAs
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_tiles = P::num_tiles(prm);
  Guard g{cp.err, L.abort_flag(), cp.timeout_ns};

  if (threadIdx.x == 0) {
    *L.abort_flag() = 0;
    for (int w = 0; w < NUM_THREADS / 32; ++w) *L.warp_state(w) = 0;
    for (int i = 0; i < 8; ++i) L.scratch()[i] = 0;
    for (int s = 0; s < STAGES; ++s) {
      // first CTA: its own producer's expect_tx arrival plus the relay's arrival for the second CTA's stage
      ptx::mbar_init(L.full(s), rank == 0 ? 2 : 1);
      ptx::mbar_init(L.empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(L.tmem_full(a), 1);
      ptx::mbar_init(L.tmem_empty(a), 2 * NUM_EPI_WARPS);     // every epilogue warp of both CTAs
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(P::map_a(prm));
    ptx::prefetch_tensormap(P::map_b(prm));
  }
  if (warp == 1) {
    tmem_alloc2(L.tmem_slot(), TMEM_COLS);
    tmem_relinquish2();
  }
  ptx::tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                 // the peer's barriers exist before anyone arrives on them
  ptx::tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(L.tmem_slot()));
  if (threadIdx.x == 64) P::prologue(prm, g);

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int s = 0; uint32_t ph = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int m_blk, n_blk;
        P::tile_coords(prm, tile, &m_blk, &n_blk);
        if (!P::a_ready(prm, m_blk, g)) break;
        const int num_kb = P::num_kb(prm, m_blk);
        const int a_row = P::a_row(prm, m_blk) + (int)rank * CTA_M;
        const int b_row = P::b_row(prm, m_blk, n_blk) + (int)rank * CTA_NLOAD;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!pair_wait(L.empty(s), ph ^ 1, g, ERR_PRODUCER_EMPTY)) { ok = false; break; }
          ptx::mbar_arrive_expect_tx(L.full(s), STAGE_BYTES);
          P::load_stage(prm, P::map_a(prm), P::map_b(prm), L.a(s), L.b(s), L.full(s), kb, a_row, b_row, m_blk, n_blk, (int)rank);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ------------------------------ MMA issuer (first CTA) ---------------------------------
      int s = 0; uint32_t ph = 0;
      uint32_t acc_ph = 0;          // bit a = phase of accumulator a
      int ord = 0;
      bool ok = true;
      const uint64_t desc_a0 = P::desc_a0(L.a(0)), desc_b0 = P::desc_b0(L.b(0));
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++ord) {
        const int acc = ord & 1;
        int m_blk, n_blk;
        P::tile_coords(prm, tile, &m_blk, &n_blk);
        const int num_kb = P::num_kb(prm, m_blk);
        // the epilogue warps of both CTAs must have drained this accumulator (two tiles ago)
        if (!pair_wait(L.tmem_empty(acc), ((acc_ph >> acc) & 1) ^ 1, g, ERR_MMA_TMEM_EMPTY)) break;
        acc_ph ^= 1u << acc;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!pair_wait(L.full(s), ph, g, ERR_MMA_FULL)) { ok = false; break; }
          ptx::tc_fence_after();
          // descriptors differ only in the 16-byte-unit start address (low 14 bits; shared memory is < 256 KiB)
          const uint64_t da = desc_a0 + (uint64_t)((s * STAGE_BYTES) >> 4);
          const uint64_t db = desc_b0 + (uint64_t)((s * STAGE_BYTES) >> 4);
#pragma unroll
          for (int k = 0; k < BK_BYTES / UMMA_K_BYTES; ++k)
            umma2_f16(d_tmem, da + (uint64_t)((k * P::kKStepBytes) >> 4), db + (uint64_t)((k * P::kKStepBytes) >> 4), P::kIdesc,
                      (kb | k) != 0 ? 1u : 0u);
          umma2_commit_both(L.empty(s));       // stage reusable in both CTAs once these MMAs retire
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        umma2_commit_both(L.tmem_full(acc));
      }
    }
    else if (lane == 0) {
      // ------------------------------ relay (second CTA) --------------------------------------
      int s = 0; uint32_t ph = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int m_blk, n_blk;
        P::tile_coords(prm, tile, &m_blk, &n_blk);
        const int num_kb = P::num_kb(prm, m_blk);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!pair_wait(L.full(s), ph, g, ERR_RELAY_FULL)) { ok = false; break; }
          mbar_arrive_cluster(mapa(L.full(s), 0));
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------------------------
    const int ew = warp - 2;               // 0..7
    const int quarter = warp & 3;          // TMEM lanes 32*quarter.. belong to this warp
    const int colhalf = ew >> 2;           // columns 128*colhalf.. of the accumulator
    uint32_t full_ph = 0;           // bit a = phase of accumulator a
    typename P::EpiState st{};
    bool ok = true;
    int ord = 0;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++ord) {
      const int acc = ord & 1;
      Chunk ck;
      P::tile_coords(prm, tile, &ck.m_blk, &ck.n_blk);
      ck.ordinal = ord;
      ck.half = (int)rank;
      ck.row0 = P::a_row(prm, ck.m_blk) + (int)rank * CTA_M + quarter * 32;
      ck.col0 = ck.n_blk * BN + colhalf * 128;
      // the tensor core is busy with this tile: do useful work until the accumulator is ready
      while (!mbar_try_wait_cluster(L.tmem_full(acc), ((full_ph >> acc) & 1))) {
        if (!P::idle_work(prm, ew, lane, g, tile, L.warp_state(warp))) {
          if (!pair_wait(L.tmem_full(acc), ((full_ph >> acc) & 1), g, ERR_EPI_TMEM_FULL)) ok = false;
          break;
        }
      }
      if (!ok) break;
      full_ph ^= 1u << acc;
      ptx::tc_fence_after();
      if (!P::tile_begin(prm, L, st, ck, ew, lane, g)) { ok = false; break; }
      if constexpr (!P::kGated) {
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t v[2][32];
          uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * ACC_COLS + colhalf * 128 + c * EPI_COLS;
          ptx::tmem_ld_32x32b_x32(taddr, v[0]);
          ptx::tmem_ld_32x32b_x32(taddr + 32, v[1]);
          ptx::tmem_ld_wait();
          if (c == 1) {
            // all TMEM reads of this warp are done: hand the accumulator back to the MMA issuer
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa(L.tmem_empty(acc), 0));
          }
          float f[64];
#pragma unroll
          for (int i = 0; i < 64; ++i) f[i] = __uint_as_float(v[i >> 5][i & 31]);
          // the previous chunk's TMA store must have finished reading the staging buffer
          if (lane == 0) ptx::tma_wait_group_read<0>();
          __syncwarp();
          Chunk cc = ck;
          cc.col0 = ck.col0 + c * EPI_COLS;
          P::adjust(prm, L, st, cc, f, ew, lane);
          // row = lane; 8 x 16-byte pieces, piece j lives at (j ^ (row & 7)) under the 128-byte swizzle
          const uint32_t rowbase = L.epi(ew) + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint32_t w0 = pack_bf16(f[j * 8 + 0], f[j * 8 + 1]);
            uint32_t w1 = pack_bf16(f[j * 8 + 2], f[j * 8 + 3]);
            uint32_t w2 = pack_bf16(f[j * 8 + 4], f[j * 8 + 5]);
            uint32_t w3 = pack_bf16(f[j * 8 + 6], f[j * 8 + 7]);
            uint32_t dst = rowbase + ((j ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
          }
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const CUtensorMap* map; int x, y;
            P::out_target(prm, cc.row0, cc.col0, &map, &x, &y);
            if (map != nullptr) ptx::tma_store_2d(map, L.epi(ew), x, y);
            ptx::tma_commit_group();
          }
        }
      } else {
        // the warp's two 64-column chunks (32 gate + 32 up each) make one 64-column output chunk
        if (lane == 0) ptx::tma_wait_group_read<0>();     // the previous tile's store has read the staging buffer
        __syncwarp();
        const uint32_t rowbase = L.epi(ew) + lane * 128;
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {
          uint32_t v[2][32];
          uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * ACC_COLS + colhalf * 128 + hc * EPI_COLS;
          ptx::tmem_ld_32x32b_x32(taddr, v[0]);        // gate
          ptx::tmem_ld_32x32b_x32(taddr + 32, v[1]);   // up
          ptx::tmem_ld_wait();
          if (hc == 1) {
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa(L.tmem_empty(acc), 0));
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float g0 = __uint_as_float(v[0][j * 8 + 2 * q]), g1 = __uint_as_float(v[0][j * 8 + 2 * q + 1]);
              float u0 = __uint_as_float(v[1][j * 8 + 2 * q]), u1 = __uint_as_float(v[1][j * 8 + 2 * q + 1]);
              float h0 = g0 / (1.f + __expf(-g0)) * u0, h1 = g1 / (1.f + __expf(-g1)) * u1;
              w[q] = pack_bf16(h0, h1);
            }
            uint32_t dst = rowbase + (((hc * 4 + j) ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
          }
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const CUtensorMap* map; int x, y;
          P::out_target(prm, ck.row0, ck.col0 / 2, &map, &x, &y);     // output column = half the accumulator column
          if (map != nullptr) ptx::tma_store_2d(map, L.epi(ew), x, y);
          ptx::tma_commit_group();
        }
      }
      P::tile_end(prm, L, st, ck, ew, lane);
    }
    if (lane == 0) ptx::tma_wait_group<0>();
    __syncwarp();
    if (ok) P::epilogue_drain(prm, L, st, ew, lane, g);
  }

  // ------------------------------ tail + teardown ---------------------------------------
  ptx::tc_fence_before();
  __syncthreads();
  if (!*L.abort_flag()) P::tail(prm, L, g);
  __syncthreads();
  if (*L.abort_flag()) {
    // let copies and MMAs that are still in flight land before smem/TMEM go away
    unsigned long long t0 = ptx::globaltimer();
    while (ptx::globaltimer() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  // neither CTA may leave (its shared memory and TMEM are read by the pair's MMAs and written by the
  // other CTA's arrivals) before both are done
  cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm2
}  // namespace bshmem
