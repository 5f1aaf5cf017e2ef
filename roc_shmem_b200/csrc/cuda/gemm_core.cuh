// gemm_core.cuh — persistent, warp-specialised tcgen05 GEMM main loop for
// sm_100a:  C[M,N] = A[M,K] · B[N,K]^T, bf16 (or fp8) operands, fp32 accumulation
// in tensor memory.
//
// One CTA per SM owns a 256x256 output tile at a time:
//   warp 0      TMA producer: A (256 rows) and B (256 rows) stages of 128 bytes of K,
//               128-byte swizzle, 3-stage ring of 64 KiB, plain (non-multicast) tiled loads
//   warp 1      MMA issuer: per k-block 2 x 4 tcgen05.mma (M128,N256,K 32 bytes);
//               rows 0-127 accumulate in TMEM columns 0-255, rows 128-255 in 256-511
//   warps 2-9   epilogue: tcgen05.ld -> convert -> swizzled smem -> TMA store
// A 256x256 tile needs 128 FLOP per byte of smem fill, which keeps the L2->SM
// traffic of 148 concurrently running tiles within what the L2 can deliver; the
// price is that both accumulators are busy, so the epilogue of a tile only
// overlaps the next tile's TMA prefetch, not its MMAs.
//
// The main loop is parameterised by a Policy so that the fused compute+collective
// kernels reuse it.  The policy decides the tile order, when an A row-block may be
// loaded (all-gather → GEMM waits for the block's arrival counter), where an output
// chunk goes (GEMM → reduce-scatter stores into the owner PE's memory), what the
// epilogue warps do while they wait for the tensor core (pull peer data), and what
// the whole CTA does after its last tile (reduce the partials that arrived).
//
// Every wait is bounded by a %globaltimer deadline; on expiry the CTA records a
// site code in the error word, lets in-flight copies land, frees its TMEM and
// returns.  There is no counterpart in the reference (it has no GEMM).
#pragma once
#include "ptx.cuh"

namespace bshmem {
namespace gemm {

constexpr int BM = 256, BN = 256;
constexpr int BK_BYTES = 128;                     // one 128-byte swizzle atom of K per stage row
constexpr int STAGES = 3;
constexpr int UMMA_M = 128, UMMA_N = 256;
constexpr int UMMA_K_BYTES = 32;                  // K extent of one tcgen05.mma in bytes (16 bf16 / 32 fp8)
constexpr int NUM_EPI_WARPS = 8;
constexpr int NUM_THREADS = 32 * (2 + NUM_EPI_WARPS);
constexpr int EPI_COLS = 64;                      // columns per epilogue chunk (128 B of bf16)
constexpr uint32_t A_STAGE_BYTES = BM * BK_BYTES;
constexpr uint32_t B_STAGE_BYTES = BN * BK_BYTES;
constexpr uint32_t STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr uint32_t EPI_BUF_BYTES = 32 * EPI_COLS * 2;          // one warp: 32 rows x 128 B
constexpr uint32_t SMEM_TILES = STAGES * STAGE_BYTES + NUM_EPI_WARPS * EPI_BUF_BYTES;
constexpr uint32_t SMEM_BYTES = SMEM_TILES + 256 /*barriers*/ + 1024 /*alignment slack*/;
constexpr uint32_t TMEM_COLS = 512;

enum ErrSite : int {
  ERR_NONE = 0, ERR_PRODUCER_EMPTY = 101, ERR_MMA_FULL = 102, ERR_MMA_TMEM_EMPTY = 103, ERR_EPI_TMEM_FULL = 104,
  ERR_A_READY = 105, ERR_PEER_SIGNAL = 106, ERR_PEER_READY = 107, ERR_PEER_DONE = 108
};

struct CoreParams {
  int M, N, K;
  int num_m_blocks, num_n_blocks;
  int group_m;             // m-blocks per raster group (L2 reuse)
  unsigned long long timeout_ns;
  int* err;                // device word: first error site, 0 = none
};

struct Guard {
  int* err;
  volatile int* abort_flag;   // shared memory
  unsigned long long timeout_ns;
};

__device__ __forceinline__ bool guard_fail(Guard& g, int site) {
  *g.abort_flag = 1;
  atomicCAS(g.err, 0, site);
  return false;
}

// Bounded mbarrier wait.  Returns false if the CTA is aborting.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, Guard& g, int site) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = ptx::globaltimer();
  uint32_t it = 0;
  while (!ptx::mbar_try_wait(bar, parity)) {
    if ((++it & 0x3F) == 0) {
      if (*g.abort_flag) return false;
      if (ptx::globaltimer() - t0 > g.timeout_ns) return guard_fail(g, site);
    }
  }
  return true;
}

// Bounded wait until *p >= target (acquire at gpu or system scope).
template <bool kSys>
__device__ __forceinline__ bool wait_ge(const unsigned long long* p, unsigned long long target, Guard& g, int site) {
  unsigned long long t0 = 0;
  uint32_t it = 0;
  while (true) {
    unsigned long long v;
    if (kSys) asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    else asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    if (v >= target) return true;
    if ((++it & 0xF) == 0) {
      if (*g.abort_flag) return false;
      unsigned long long now = ptx::globaltimer();
      if (t0 == 0) t0 = now;
      else if (now - t0 > g.timeout_ns) return guard_fail(g, site);
      __nanosleep(100);
    }
  }
}

// Grouped raster: consecutive tile ids walk down `group_m` row-blocks before
// moving to the next column-block, so concurrently running CTAs share A and B.
__device__ __forceinline__ void raster_coords(const CoreParams& p, int tile, int* m_blk, int* n_blk) {
  int per_group = p.group_m * p.num_n_blocks;
  int g = tile / per_group;
  int first_m = g * p.group_m;
  int rows = min(p.group_m, p.num_m_blocks - first_m);
  int in_g = tile - g * per_group;
  *m_blk = first_m + in_g % rows;
  *n_blk = in_g / rows;
}

// Shared-memory carve-up (all addresses are shared-window byte addresses).
struct Smem {
  uint32_t base;        // 1024-byte aligned
  uint8_t* gen;         // generic pointer to the same byte
  __device__ __forceinline__ uint32_t a(int s) const { return base + s * STAGE_BYTES; }
  __device__ __forceinline__ uint32_t b(int s) const { return base + s * STAGE_BYTES + A_STAGE_BYTES; }
  __device__ __forceinline__ uint32_t epi(int w) const { return base + STAGES * STAGE_BYTES + w * EPI_BUF_BYTES; }
  __device__ __forceinline__ uint32_t bars() const { return base + SMEM_TILES; }
  __device__ __forceinline__ uint32_t full(int s) const { return bars() + 8 * s; }
  __device__ __forceinline__ uint32_t empty(int s) const { return bars() + 8 * (STAGES + s); }
  __device__ __forceinline__ uint32_t tmem_full(int h) const { return bars() + 8 * (2 * STAGES + h); }
  __device__ __forceinline__ uint32_t tmem_empty(int h) const { return bars() + 8 * (2 * STAGES + 2 + h); }
  __device__ __forceinline__ uint32_t tmem_slot() const { return bars() + 8 * (2 * STAGES + 4); }
  __device__ __forceinline__ volatile int* abort_flag() const {
    return reinterpret_cast<volatile int*>(gen + SMEM_TILES + 8 * (2 * STAGES + 4) + 8);
  }
  // 16 bytes of policy scratch (e.g. a broadcast slot for the tail phase)
  // one word of private state per warp (10 warps), zeroed at kernel start
  __device__ __forceinline__ volatile int* warp_state(int w) const {
    return reinterpret_cast<volatile int*>(gen + SMEM_TILES + 128 + 4 * w);
  }
  __device__ __forceinline__ volatile int* scratch() const {
    return reinterpret_cast<volatile int*>(gen + SMEM_TILES + 8 * (2 * STAGES + 4) + 16);
  }
};

__device__ __forceinline__ Smem carve_smem(uint8_t* raw) {
  Smem L;
  uint32_t r = ptx::smem_u32(raw);
  L.base = (r + 1023u) & ~1023u;
  L.gen = raw + (L.base - r);
  return L;
}

// Pack two fp32 into one bf16x2 word (round to nearest even).
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Reduce-scatter epilogues: add the bf16 32x64 chunks of the other PEs' partial results to the warp's 64 fp32
// accumulators per lane (row = lane), in source order 0..P-1 skipping `skip` (fixed order: reproducible bits).
// `src0` points at (row lane/8, column 8*(lane%8)) of the chunk in source slot 0, `slot` is the distance between
// source slots and `ld` the row pitch, both in elements.  A chunk is fetched with fully coalesced 16-byte loads
// (lane -> row lane/8 + 4i, piece lane%8), parked in the warp's swizzled 4 KiB staging buffer `buf` (free at this
// point) and read back row-per-lane; the next source's loads are already in flight meanwhile.
// kPrefetch = true keeps the next source's eight loads in flight while the current one is added (32 more registers);
// false fetches four at a time and suits kernels that are short of registers.
template <bool kPrefetch = true>
__device__ __forceinline__ void add_partial_chunks(float (&f)[64], const __nv_bfloat16* src0, long long slot, long long ld, int P, int skip,
                                                   uint32_t buf, int lane) {
  const int pr = lane >> 3, pc = lane & 7;
  auto park = [&](const uint4& v, int i) {
    const int row = pr + 4 * i;
    const uint32_t dst = buf + row * 128 + ((pc ^ (row & 7)) << 4);
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  };
  auto add_row = [&]() {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint4 y;
      const uint32_t a = buf + lane * 128 + ((j ^ (lane & 7)) << 4);
      asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(y.x), "=r"(y.y), "=r"(y.z), "=r"(y.w) : "r"(a) : "memory");
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 v = __bfloat1622float2(h[e]);
        f[j * 8 + 2 * e] += v.x;
        f[j * 8 + 2 * e + 1] += v.y;
      }
    }
  };
  int s = skip == 0 ? 1 : 0;
  if (s >= P) return;
  if constexpr (kPrefetch) {
    uint4 x[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = ptx::ld_relaxed_v4(src0 + s * slot + (long long)(4 * i) * ld);
    while (true) {
#pragma unroll
      for (int i = 0; i < 8; ++i) park(x[i], i);
      __syncwarp();
      int next = s + 1;
      if (next == skip) ++next;
      if (next < P) {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = ptx::ld_relaxed_v4(src0 + next * slot + (long long)(4 * i) * ld);
      }
      add_row();
      __syncwarp();
      if (next >= P) break;
      s = next;
    }
  } else {
    for (; s < P; ++s) {
      if (s == skip) continue;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint4 x[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = ptx::ld_relaxed_v4(src0 + s * slot + (long long)(4 * (half * 4 + i)) * ld);
#pragma unroll
        for (int i = 0; i < 4; ++i) park(x[i], half * 4 + i);
      }
      __syncwarp();
      add_row();
      __syncwarp();
    }
  }
}

// Defaults a policy can inherit.
struct PolicyDefaults {
  static constexpr bool kWaitStoresPerTile = false;
  // Gated epilogue: inside every 64-column chunk, columns 0-31 are gate pre-activations and 32-63 the
  // matching up-projections; the epilogue writes silu(gate) * up, i.e. half as many output columns.
  static constexpr bool kGated = false;
  template <class Params> __device__ static __forceinline__ int b_row(const Params&, int, int n_blk) { return n_blk * BN; }
  // K-major operands: one TMA box per operand and stage (256 rows x 128 bytes of K) ...
  template <class Params>
  __device__ static __forceinline__ void load_stage(const Params&, const CUtensorMap* ma, const CUtensorMap* mb, uint32_t a_smem,
                                                    uint32_t b_smem, uint32_t bar, int k_elem, int a_row, int b_row) {
    ptx::tma_load_2d(a_smem, ma, bar, k_elem, a_row);
    ptx::tma_load_2d(b_smem, mb, bar, k_elem, b_row);
  }
  // ... and shared-memory descriptors that step 32 bytes along K inside the swizzle atom.
  __device__ static __forceinline__ uint64_t desc_a(uint32_t a0, int half, int k) {
    return ptx::umma_desc_sw128(a0 + half * (UMMA_M * BK_BYTES) + k * UMMA_K_BYTES);
  }
  __device__ static __forceinline__ uint64_t desc_b(uint32_t b0, int k) { return ptx::umma_desc_sw128(b0 + k * UMMA_K_BYTES); }
  template <class Params> __device__ static __forceinline__ bool a_ready(const Params&, int, Guard&) { return true; }
  // k-blocks of the tile's reduction (ragged per group in the grouped weight-gradient GEMM)
  template <class Params> __device__ static __forceinline__ int num_kb(const Params& p, int, int bk) {
    return (p.core.K + bk - 1) / bk;
  }
  template <class Params> __device__ static __forceinline__ int num_tiles(const Params& p) {
    return p.core.num_m_blocks * p.core.num_n_blocks;
  }
  template <class Params> __device__ static __forceinline__ void tile_done(const Params&, int, int, int, int) {}
  // work for an epilogue warp while the tensor core is busy; false = nothing to do
  // `tile` is the tile this CTA is working on (lets a policy order its side work by schedule progress)
  template <class Params> __device__ static __forceinline__ bool idle_work(const Params&, int, int, Guard&, int, volatile int*) { return false; }
  // after an epilogue warp's last tile
  template <class Params> __device__ static __forceinline__ void epilogue_drain(const Params&, int, int, Guard&) {}
  // whole CTA, after all roles have finished (before TMEM is released)
  template <class Params> __device__ static __forceinline__ void tail(const Params&, const Smem&, Guard&) {}
  // one-time work of one thread of the CTA at kernel start
  template <class Params> __device__ static __forceinline__ void prologue(const Params&, Guard&) {}
};

// Policy contract (static __device__ members; P::Params is the kernel's by-value parameter):
//   core(prm) -> const CoreParams&        map_a(prm), map_b(prm) -> const CUtensorMap*
//   kElemBytes, kIdesc                    mma(d_tmem, adesc, bdesc, idesc, accumulate)
//   tile_coords(prm, tile, &m_blk, &n_blk)
//   a_ready(prm, m_blk, guard)            producer lane, before a tile's first A load
//   a_row(prm, m_blk) -> int              row coordinate of the A block in map_a
//   pack(lo_bits, hi_bits, prm, row, col) -> uint32   two accumulators -> one output word
//   out_target(prm, row, col, &map, &x, &y)  where the 32x64 chunk starting at C[row, col] goes
//   tile_done(prm, m_blk, n_blk, epi_warp, lane)  after the warp's stores (complete if kWaitStoresPerTile)
//   idle_work / epilogue_drain / tail / prologue as in PolicyDefaults
template <class P>
__device__ __forceinline__ void gemm_mainloop(const typename P::Params& prm, uint8_t* smem_raw) {
  const CoreParams& cp = P::core(prm);
  const Smem L = carve_smem(smem_raw);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = P::num_tiles(prm);
  constexpr int BK = BK_BYTES / P::kElemBytes;   // k-block in elements
  Guard g{cp.err, L.abort_flag(), cp.timeout_ns};

  if (threadIdx.x == 0) {
    *L.abort_flag() = 0;
    for (int w = 0; w < NUM_THREADS / 32; ++w) *L.warp_state(w) = 0;
    for (int s = 0; s < STAGES; ++s) { ptx::mbar_init(L.full(s), 1); ptx::mbar_init(L.empty(s), 1); }
    for (int h = 0; h < 2; ++h) { ptx::mbar_init(L.tmem_full(h), 1); ptx::mbar_init(L.tmem_empty(h), NUM_EPI_WARPS / 2); }
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(P::map_a(prm));
    ptx::prefetch_tensormap(P::map_b(prm));
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
  if (threadIdx.x == 64) P::prologue(prm, g);      // first epilogue warp's lane 0

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int s = 0; uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk;
        P::tile_coords(prm, tile, &m_blk, &n_blk);
        if (!P::a_ready(prm, m_blk, g)) break;
        const int a_row = P::a_row(prm, m_blk);
        const int b_row = P::b_row(prm, m_blk, n_blk);
        const int num_kb = P::num_kb(prm, m_blk, BK);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(L.empty(s), ph ^ 1, g, ERR_PRODUCER_EMPTY)) { ok = false; break; }
          ptx::mbar_arrive_expect_tx(L.full(s), STAGE_BYTES);
          P::load_stage(prm, P::map_a(prm),P::map_b(prm), L.a(s), L.b(s), L.full(s), kb * BK, a_row, b_row);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = P::kIdesc;
      int s = 0; uint32_t ph = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        // both accumulators must have been drained by the epilogue of the previous tile
        if (!mbar_wait(L.tmem_empty(0), acc_ph ^ 1, g, ERR_MMA_TMEM_EMPTY)) break;
        if (!mbar_wait(L.tmem_empty(1), acc_ph ^ 1, g, ERR_MMA_TMEM_EMPTY)) break;
        ptx::tc_fence_after();
        int m_blk, n_blk;
        P::tile_coords(prm, tile, &m_blk, &n_blk);
        const int num_kb = P::num_kb(prm, m_blk, BK);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(L.full(s), ph, g, ERR_MMA_FULL)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t a0 = L.a(s), b0 = L.b(s);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int k = 0; k < BK_BYTES / UMMA_K_BYTES; ++k) {
              uint64_t da = P::desc_a(a0, half, k);
              uint64_t db = P::desc_b(b0, k);
              P::mma(tmem_base + half * UMMA_N, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
            }
          }
          ptx::umma_commit(L.empty(s));       // stage reusable once these MMAs retire
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        ptx::umma_commit(L.tmem_full(0));
        ptx::umma_commit(L.tmem_full(1));
        acc_ph ^= 1;
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------------
    const int ew = warp - 2;               // 0..7
    const int quarter = warp & 3;          // TMEM lanes 32*quarter.. are this warp's
    const int half = ew >> 2;              // 0: rows 0-127 (cols 0-255), 1: rows 128-255 (cols 256-511)
    uint32_t acc_ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m_blk, n_blk;
      P::tile_coords(prm, tile, &m_blk, &n_blk);
      // the tensor core is busy with this tile: do useful work until the accumulator is ready
      while (!ptx::mbar_try_wait(L.tmem_full(half), acc_ph)) {
        if (!P::idle_work(prm, ew, lane, g, tile, L.warp_state(warp))) {
          if (!mbar_wait(L.tmem_full(half), acc_ph, g, ERR_EPI_TMEM_FULL)) ok = false;
          break;
        }
      }
      if (!ok) break;
      ptx::tc_fence_after();
      const int row0 = m_blk * BM + half * UMMA_M + quarter * 32;
      if constexpr (!P::kGated) {
#pragma unroll 1
        for (int c = 0; c < BN / EPI_COLS; ++c) {
          uint32_t v[2][32];
          uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * UMMA_N + c * EPI_COLS;
          ptx::tmem_ld_32x32b_x32(taddr, v[0]);
          ptx::tmem_ld_32x32b_x32(taddr + 32, v[1]);
          ptx::tmem_ld_wait();
          // the previous chunk's TMA store must have finished reading the staging buffer
          if (lane == 0) ptx::tma_wait_group_read<0>();
          __syncwarp();
          // row = lane; 8 x 16-byte pieces, piece j lives at (j ^ (row & 7)) under the 128-byte swizzle
          const uint32_t rowbase = L.epi(ew) + lane * 128;
          const int col0 = n_blk * BN + c * EPI_COLS;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t* src = &v[j >> 2][(j & 3) * 8];
            uint32_t w0 = P::pack(src[0], src[1], prm, row0 + lane, col0 + j * 8);
            uint32_t w1 = P::pack(src[2], src[3], prm, row0 + lane, col0 + j * 8 + 2);
            uint32_t w2 = P::pack(src[4], src[5], prm, row0 + lane, col0 + j * 8 + 4);
            uint32_t w3 = P::pack(src[6], src[7], prm, row0 + lane, col0 + j * 8 + 6);
            uint32_t dst = rowbase + ((j ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
          }
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const CUtensorMap* map; int x, y;
            P::out_target(prm, row0, col0, &map, &x, &y);
            if (map != nullptr) ptx::tma_store_2d(map, L.epi(ew), x, y);
            ptx::tma_commit_group();
          }
        }
      } else {
        // two 64-column chunks (32 gate + 32 up each) make one 64-column output chunk
#pragma unroll 1
        for (int c2 = 0; c2 < BN / (2 * EPI_COLS); ++c2) {
          if (lane == 0) ptx::tma_wait_group_read<0>();
          __syncwarp();
          const uint32_t rowbase = L.epi(ew) + lane * 128;
#pragma unroll
          for (int hc = 0; hc < 2; ++hc) {
            uint32_t v[2][32];
            uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * UMMA_N + (2 * c2 + hc) * EPI_COLS;
            ptx::tmem_ld_32x32b_x32(taddr, v[0]);        // gate
            ptx::tmem_ld_32x32b_x32(taddr + 32, v[1]);   // up
            ptx::tmem_ld_wait();
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
            // output column index is half the accumulator column index
            P::out_target(prm, row0, (n_blk * BN + c2 * 2 * EPI_COLS) / 2, &map, &x, &y);
            if (map != nullptr) ptx::tma_store_2d(map, L.epi(ew), x, y);
            ptx::tma_commit_group();
          }
        }
      }
      // all TMEM reads of this warp are done: hand the accumulator half back (4 warps share it)
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(L.tmem_empty(half));
      if (P::kWaitStoresPerTile) {
        if (lane == 0) ptx::tma_wait_group<0>();
        __syncwarp();
      }
      P::tile_done(prm, m_blk, n_blk, ew, lane);
      acc_ph ^= 1;
    }
    if (lane == 0) ptx::tma_wait_group<0>();
    __syncwarp();
    if (ok) P::epilogue_drain(prm, ew, lane, g);
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
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm
}  // namespace bshmem
