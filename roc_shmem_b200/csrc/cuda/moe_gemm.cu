// moe_gemm.cu — grouped (per-expert) tcgen05 GEMM for the MoE layer.  The K-major forms (gate/up, down and the two
// data-gradient GEMMs) run on the CTA-pair main loop of gemm_pair.cuh (cta_group::2, the epilogue of one tile overlaps
// the MMAs of the next); the weight-gradient form on token-major operands and the ragged-K form run on the
// single-CTA main loop of gemm_core.cuh.
//
//   C_g = A_g · B_g^T  for every local expert g, all operands K-major bf16:
//     rows mode   A: [G][cap rows][K]   B: [G][N][K]    C: [G][cap][N]
//                 the row count of group g is read from device memory (tokens that arrived),
//                 so no host synchronisation is needed between dispatch and the GEMM;
//     ragged-K    A: [G][M][cap]        B: [G][N][cap]  C: [G][M][N]
//                 the reduction length of group g is the device-side token count (weight
//                 gradients over transposed, zero-padded activations).
//   Optional gated epilogue (SwiGLU fused: interleaved gate/up columns → silu(g)·u) and an
//   optional wait on the dispatch arrival words before the first A load.
// There is no grouped GEMM in the reference; the layout conventions are those of
// moe_kernels.cu.
#include <cstdlib>

#include "gemm_pair.cuh"
#include "moe_common.h"
#include "tma_host.h"

using namespace bshmem;
using namespace bshmem::gemm;

namespace {

struct GroupedParams {
  CoreParams core;                 // N = output columns of the accumulator, K = full reduction length
  CUtensorMap map_a, map_b, map_c;
  const int* rows;                 // [G] valid rows per group (rows mode) or null (all `fixed_rows`)
  const int* klen;                 // [G] reduction length per group (ragged-K mode) or null
  int G, fixed_rows;
  int a_blocks_per_group;          // 256-row blocks between consecutive groups in A and C
  int b_rows_per_group;            // rows between consecutive groups in B
  int k_rows_per_group;            // token rows between consecutive groups of A and B (transposed-operand mode)
  int tn3d;                        // transposed-operand mode: maps are 3-D column-block views, one copy per operand
  int group_m;
  int P;                           // arrival wait: number of words, 0 = no wait
  const unsigned long long* arrive;
  const int* expected;
};

template <bool kGatedEpi>
struct Grouped : PolicyDefaults {
  using Params = GroupedParams;
  static constexpr int kElemBytes = 2;
  static constexpr uint32_t kIdesc = ptx::umma_idesc(1, 1, UMMA_M, UMMA_N);
  static constexpr bool kGated = kGatedEpi;
  __device__ static __forceinline__ const CoreParams& core(const Params& p) { return p.core; }
  __device__ static __forceinline__ const CUtensorMap* map_a(const Params& p) { return &p.map_a; }
  __device__ static __forceinline__ const CUtensorMap* map_b(const Params& p) { return &p.map_b; }
  __device__ static __forceinline__ int group_rows(const Params& p, int g) { return p.rows ? p.rows[g] : p.fixed_rows; }
  __device__ static __forceinline__ int num_tiles(const Params& p) {
    int t = 0;
    for (int g = 0; g < p.G; ++g) t += ((group_rows(p, g) + BM - 1) / BM) * p.core.num_n_blocks;
    return t;
  }
  // m_blk is a virtual block index: group * a_blocks_per_group + block inside the group
  __device__ static __forceinline__ void tile_coords(const Params& p, int tile, int* m_blk, int* n_blk) {
    int g = 0, mb_g = 0;
    for (; g < p.G; ++g) {
      mb_g = (group_rows(p, g) + BM - 1) / BM;
      int tg = mb_g * p.core.num_n_blocks;
      if (tile < tg) break;
      tile -= tg;
    }
    int per = p.group_m * p.core.num_n_blocks;
    int sg = tile / per, first = sg * p.group_m;
    int rows = min(p.group_m, mb_g - first);
    int in = tile - sg * per;
    *m_blk = g * p.a_blocks_per_group + first + in % rows;
    *n_blk = in / rows;
  }
  __device__ static __forceinline__ int a_row(const Params&, int m_blk) { return m_blk * BM; }
  __device__ static __forceinline__ int b_row(const Params& p, int m_blk, int n_blk) {
    return (m_blk / p.a_blocks_per_group) * p.b_rows_per_group + n_blk * BN;
  }
  __device__ static __forceinline__ int num_kb(const Params& p, int m_blk, int bk) {
    int k = p.klen ? p.klen[m_blk / p.a_blocks_per_group] : p.core.K;
    int n = (k + bk - 1) / bk;
    return n < 1 ? 1 : n;     // an empty group still runs one (all-zero) k-block so that C becomes 0
  }
  __device__ static __forceinline__ bool a_ready(const Params& p, int, Guard& g) {
    for (int s = 0; s < p.P; ++s)
      if (!wait_ge<true>(p.arrive + s, (unsigned long long)p.expected[s], g, ERR_PEER_SIGNAL)) return false;
    if (p.P) ptx::fence_proxy_async_all();   // peer stores (generic proxy) before the TMA reads
    return true;
  }
  __device__ static __forceinline__ void mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    ptx::umma_f16(d, a, b, idesc, acc);
  }
  __device__ static __forceinline__ uint32_t pack(uint32_t lo, uint32_t hi, const Params&, int, int) {
    return pack_bf16(__uint_as_float(lo), __uint_as_float(hi));
  }
  __device__ static __forceinline__ void out_target(const Params& p, int row, int col, const CUtensorMap** map, int* x, int* y) {
    *map = &p.map_c;       // rows beyond a group's count are scratch inside the group's own region
    *x = col;
    *y = row;
  }
};

// Weight-gradient flavour: C_g[M, N] = A_g^T · B_g with A_g stored [tokens_g][M] and B_g stored [tokens_g][N]
// (the token-major activations as they are), i.e. both operands MN-major; the reduction runs over the
// ragged token dimension.  A stage holds, per operand, four 64-wide MN blocks of 64 tokens each (8 KiB per
// block, 128-byte swizzle): inside a block 8 tokens form one 1 KiB swizzle atom (SBO), blocks are 8 KiB apart
// (LBO).  Tokens in [count, next multiple of 64) of every group must be zero (bshmem_moe_zero_pad_rows).
struct GroupedTN : Grouped<false> {
  static constexpr uint32_t kIdesc = ptx::umma_idesc_mn_major(1, 1, UMMA_M, UMMA_N);
  static constexpr uint32_t kBlock = 64 * BK_BYTES;            // one 64 (MN) x 64 (tokens) block: 8 KiB
  // the "row" values handed to load_stage are the tile's block indices; the token row comes from the group
  __device__ static __forceinline__ int a_row(const Params&, int m_blk) { return m_blk; }
  __device__ static __forceinline__ int b_row(const Params&, int, int n_blk) { return n_blk; }
  __device__ static __forceinline__ void load_stage(const Params& p, const CUtensorMap* ma, const CUtensorMap* mb, uint32_t a_smem,
                                                    uint32_t b_smem, uint32_t bar, int k_elem, int m_blk, int n_blk) {
    const int g = m_blk / p.a_blocks_per_group;
    const int tok = g * p.k_rows_per_group + k_elem;
    const int m0 = (m_blk - g * p.a_blocks_per_group) * BM, n0 = n_blk * BN;
    if (p.tn3d) {                  // one 32 KiB copy per operand: {64, 64 tokens, 4 column blocks}
      ptx::tma_load_3d(a_smem, ma, bar, 0, tok, m0 / 64);
      ptx::tma_load_3d(b_smem, mb, bar, 0, tok, n0 / 64);
      return;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ptx::tma_load_2d(a_smem + i * kBlock, ma, bar, m0 + i * 64, tok);
      ptx::tma_load_2d(b_smem + i * kBlock, mb, bar, n0 + i * 64, tok);
    }
  }
  // one MMA consumes 16 tokens = two swizzle atoms (2 KiB) of every MN block
  __device__ static __forceinline__ uint64_t desc_a(uint32_t a0, int half, int k) {
    return ptx::umma_desc_sw128_ex(a0 + half * 2 * kBlock + k * 2048, kBlock, 1024);
  }
  __device__ static __forceinline__ uint64_t desc_b(uint32_t b0, int k) { return ptx::umma_desc_sw128_ex(b0 + k * 2048, kBlock, 1024); }
};

__global__ void __launch_bounds__(NUM_THREADS, 1) grouped_gemm_kernel(const __grid_constant__ GroupedParams prm) {
  extern __shared__ uint8_t smem_raw[];
  gemm_mainloop<Grouped<false>>(prm, smem_raw);
}
__global__ void __launch_bounds__(NUM_THREADS, 1) grouped_gemm_gated_kernel(const __grid_constant__ GroupedParams prm) {
  extern __shared__ uint8_t smem_raw[];
  gemm_mainloop<Grouped<true>>(prm, smem_raw);
}
__global__ void __launch_bounds__(NUM_THREADS, 1) grouped_gemm_tn_kernel(const __grid_constant__ GroupedParams prm) {
  extern __shared__ uint8_t smem_raw[];
  gemm_mainloop<GroupedTN>(prm, smem_raw);
}

// ---- the K-major rows mode on CTA pairs ---------------------------------------------------------------------------
// Same tile schedule (a tile is 256 rows of one group x 256 accumulator columns) and the same parameters; each CTA of
// the pair loads 128 rows of the A block and 128 rows of the B block, so the tensor maps have 128-row boxes.
namespace g2 = bshmem::gemm2;

template <bool kGatedEpi>
struct GroupedPair : g2::PolicyDefaults {
  using Params = GroupedParams;
  using Base = Grouped<kGatedEpi>;
  static constexpr bool kGated = kGatedEpi;
  __device__ static __forceinline__ const CoreParams& core(const Params& p) { return p.core; }
  __device__ static __forceinline__ const CUtensorMap* map_a(const Params& p) { return &p.map_a; }
  __device__ static __forceinline__ const CUtensorMap* map_b(const Params& p) { return &p.map_b; }
  __device__ static __forceinline__ int num_tiles(const Params& p) { return Base::num_tiles(p); }
  __device__ static __forceinline__ void tile_coords(const Params& p, int tile, int* m_blk, int* n_blk) {
    Base::tile_coords(p, tile, m_blk, n_blk);
  }
  __device__ static __forceinline__ int a_row(const Params&, int m_blk) { return m_blk * g2::BM; }
  __device__ static __forceinline__ int b_row(const Params& p, int m_blk, int n_blk) {
    return (m_blk / p.a_blocks_per_group) * p.b_rows_per_group + n_blk * g2::BN;
  }
  // runs in the producer lane of BOTH CTAs: each loads its own half of the block
  __device__ static __forceinline__ bool a_ready(const Params& p, int, Guard& g) {
    for (int s = 0; s < p.P; ++s)
      if (!wait_ge<true>(p.arrive + s, (unsigned long long)p.expected[s], g, g2::ERR_PEER_SIGNAL)) return false;
    if (p.P) ptx::fence_proxy_async_all();   // peer stores (generic proxy) before the TMA reads
    return true;
  }
  __device__ static __forceinline__ void out_target(const Params& p, int row, int col, const CUtensorMap** map, int* x, int* y) {
    *map = &p.map_c;       // rows beyond a group's count are scratch inside the group's own region
    *x = col;
    *y = row;
  }
};

// Weight-gradient flavour on CTA pairs: both operands MN-major (token-major activations as they are), ragged
// reduction over the group's tokens.  Per CTA and stage, each operand is two 64-wide MN blocks of 64 tokens (8 KiB per
// block, 128-byte swizzle), i.e. the CTA's 128 of the tile's 256 rows / columns.
struct GroupedPairTN : GroupedPair<false> {
  static constexpr uint32_t kIdesc = ptx::umma_idesc_mn_major(1, 1, g2::BM, g2::BN);
  static constexpr uint32_t kBlock = 64 * g2::BK_BYTES;         // one 64 (MN) x 64 (tokens) block: 8 KiB
  static constexpr uint32_t kKStepBytes = 2048;                 // one MMA consumes 16 tokens = two swizzle atoms
  __device__ static __forceinline__ uint64_t desc_a0(uint32_t a0) { return ptx::umma_desc_sw128_ex(a0, kBlock, 1024); }
  __device__ static __forceinline__ uint64_t desc_b0(uint32_t b0) { return ptx::umma_desc_sw128_ex(b0, kBlock, 1024); }
  __device__ static __forceinline__ int num_kb(const Params& p, int m_blk) {
    const int n = (p.klen[m_blk / p.a_blocks_per_group] + 63) / 64;
    return n < 1 ? 1 : n;     // an empty group still runs one (all-zero) k-block so that C becomes 0
  }
  __device__ static __forceinline__ bool a_ready(const Params&, int, Guard&) { return true; }
  __device__ static __forceinline__ void load_stage(const Params& p, const CUtensorMap* ma, const CUtensorMap* mb, uint32_t a_smem,
                                                    uint32_t b_smem, uint32_t bar, int kb, int, int, int m_blk, int n_blk, int rank) {
    const int g = m_blk / p.a_blocks_per_group;
    const int tok = g * p.k_rows_per_group + kb * 64;
    const int m0 = (m_blk - g * p.a_blocks_per_group) * g2::BM + rank * g2::CTA_M, n0 = n_blk * g2::BN + rank * g2::CTA_NLOAD;
    if (p.tn3d) {                  // one 16 KiB copy per operand: {64, 64 tokens, 2 column blocks}
      ptx::tma_load_3d(a_smem, ma, bar, 0, tok, m0 / 64);
      ptx::tma_load_3d(b_smem, mb, bar, 0, tok, n0 / 64);
      return;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ptx::tma_load_2d(a_smem + i * kBlock, ma, bar, m0 + i * 64, tok);
      ptx::tma_load_2d(b_smem + i * kBlock, mb, bar, n0 + i * 64, tok);
    }
  }
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(g2::NUM_THREADS, 1)
grouped_gemm_pair_kernel(const __grid_constant__ GroupedParams prm) {
  extern __shared__ uint8_t smem_raw[];
  g2::gemm_mainloop<GroupedPair<false>>(prm, smem_raw);
}
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(g2::NUM_THREADS, 1)
grouped_gemm_pair_gated_kernel(const __grid_constant__ GroupedParams prm) {
  extern __shared__ uint8_t smem_raw[];
  g2::gemm_mainloop<GroupedPair<true>>(prm, smem_raw);
}
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(g2::NUM_THREADS, 1)
grouped_gemm_pair_tn_kernel(const __grid_constant__ GroupedParams prm) {
  extern __shared__ uint8_t smem_raw[];
  g2::gemm_mainloop<GroupedPairTN>(prm, smem_raw);
}

// Zero the token rows [count_g, next multiple of 64) — rows [0, 64) of an empty group — of every group of a
// [G][cap][cols] bf16 buffer.
__global__ void zero_pad_rows_kernel(__nv_bfloat16* buf, const int* counts, int cap, int cols) {
  const int g = blockIdx.y;
  const int c = counts[g];
  int end = c == 0 ? 64 : (c + 63) / 64 * 64;      // an empty group still feeds one (all-zero) block to the GEMM
  if (end > cap) end = cap;
  const int vec_per_row = cols / 8;
  const long long n = (long long)(end - c) * vec_per_row;
  uint4* base = reinterpret_cast<uint4*>(buf + ((size_t)g * cap + c) * cols);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    base[i] = make_uint4(0, 0, 0, 0);
}

int* g_err_dev[64] = {};
int g_sms[64] = {};
int g_pairs[64] = {};

int ensure(int dev) {
  if (g_err_dev[dev]) return 0;
  BSHMEM_CUDA_TRY(cudaMalloc(&g_err_dev[dev], sizeof(int)));
  BSHMEM_CUDA_TRY(cudaMemset(g_err_dev[dev], 0, sizeof(int)));
  BSHMEM_CUDA_TRY(cudaDeviceGetAttribute(&g_sms[dev], cudaDevAttrMultiProcessorCount, dev));
  BSHMEM_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
  BSHMEM_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_gated_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
  BSHMEM_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
  BSHMEM_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g2::SMEM_BYTES));
  BSHMEM_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_pair_gated_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g2::SMEM_BYTES));
  BSHMEM_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_pair_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g2::SMEM_BYTES));
  g_pairs[dev] = g2::max_resident_pairs(grouped_gemm_pair_kernel, g_sms[dev]);
  return 0;
}

}  // namespace

extern "C" {

const char* bshmem_moe_gemm_last_error() { return host::last_error().c_str(); }

// Grouped GEMM.  A: [G * a_rows_per_group, K] (lda), B: [G * b_rows_per_group, K] (ldb), C: [G * a_rows_per_group, N_out] (ldc).
//   rows_dev   per-group valid row counts on the device, or null → every group has `fixed_rows` rows
//   klen_dev   per-group reduction lengths on the device, or null → K
//   gated      1: accumulator columns are interleaved gate/up, C gets N/2 columns of silu(gate)*up
//   arrive/expected/P  optional arrival words to wait for before the first load (P = 0: none)
int bshmem_moe_grouped_gemm(const void* A, const void* B, void* C, int G, int a_rows_per_group, int b_rows_per_group, int N, int K,
                            int lda, int ldb, int ldc, const int* rows_dev, int fixed_rows, const int* klen_dev, int gated,
                            const void* arrive, const int* expected, int P, void* stream, int timeout_ms, int max_ctas) {
  if (G < 1 || a_rows_per_group % BM || N % BN || K % 8 || lda % 8 || ldb % 8 || ldc % 8) {
    host::last_error() = "grouped gemm: needs rows-per-group % 256 == 0, N % 256 == 0, K and leading dimensions % 8 == 0";
    return 1;
  }
  int dev = 0;
  BSHMEM_CUDA_TRY(cudaGetDevice(&dev));
  int rc = ensure(dev);
  if (rc) return rc;
  GroupedParams p;
  memset(&p, 0, sizeof(p));
  p.core.M = G * a_rows_per_group; p.core.N = N; p.core.K = K;
  p.core.num_m_blocks = p.core.M / BM; p.core.num_n_blocks = N / BN;
  p.core.group_m = 16;
  p.core.timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 4000) * 1000000ull;
  p.core.err = g_err_dev[dev];
  p.rows = rows_dev; p.klen = klen_dev; p.G = G; p.fixed_rows = fixed_rows > 0 ? fixed_rows : a_rows_per_group;
  p.a_blocks_per_group = a_rows_per_group / BM;
  p.b_rows_per_group = b_rows_per_group;
  p.group_m = 16;
  p.P = P; p.arrive = static_cast<const unsigned long long*>(arrive); p.expected = expected;
  // K-major rows mode with a uniform reduction length: CTA pairs; a ragged reduction length (legacy weight-gradient
  // form on transposed copies) stays on the single-CTA loop
  const bool pair = klen_dev == nullptr && g_pairs[dev] > 0;
  const int box_rows_a = pair ? g2::CTA_M : BM, box_rows_b = pair ? g2::CTA_NLOAD : BN;
  rc = host::make_tmap_2d(&p.map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, (uint64_t)G * a_rows_per_group, K, lda, box_rows_a, 64);
  if (rc) return rc;
  rc = host::make_tmap_2d(&p.map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, (uint64_t)G * b_rows_per_group, K, ldb, box_rows_b, 64);
  if (rc) return rc;
  rc = host::make_tmap_2d(&p.map_c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, (uint64_t)G * a_rows_per_group, gated ? N / 2 : N, ldc, 32, EPI_COLS);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (pair) {
    int pairs = g_pairs[dev];
    if (max_ctas > 1 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
    if (gated) grouped_gemm_pair_gated_kernel<<<2 * pairs, g2::NUM_THREADS, g2::SMEM_BYTES, st>>>(p);
    else grouped_gemm_pair_kernel<<<2 * pairs, g2::NUM_THREADS, g2::SMEM_BYTES, st>>>(p);
  } else {
    int ctas = g_sms[dev];
    if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
    if (gated) grouped_gemm_gated_kernel<<<ctas, NUM_THREADS, SMEM_BYTES, st>>>(p);
    else grouped_gemm_kernel<<<ctas, NUM_THREADS, SMEM_BYTES, st>>>(p);
  }
  BSHMEM_CUDA_TRY(cudaGetLastError());
  return 0;
}

// Weight-gradient GEMM on token-major operands: C_g[M, N] = A_g^T · B_g for every group.
//   A: [G * cap, M] (lda), B: [G * cap, N] (ldb), C: [G * M, N] (ldc); the number of tokens of group g is
//   klen_dev[g] (<= cap).  Token rows [klen, next multiple of 64) must be zero in A and B.
int bshmem_moe_grouped_gemm_tn(const void* A, const void* B, void* C, int G, int cap, int M, int N, int lda, int ldb, int ldc,
                               const int* klen_dev, void* stream, int timeout_ms, int max_ctas) {
  if (G < 1 || M % BM || N % BN || cap % 64 || lda % 8 || ldb % 8 || ldc % 8 || !klen_dev) {
    host::last_error() = "grouped gemm (transposed operands): needs M % 256 == 0, N % 256 == 0, capacity % 64 == 0, leading dimensions % 8 == 0";
    return 1;
  }
  int dev = 0;
  BSHMEM_CUDA_TRY(cudaGetDevice(&dev));
  int rc = ensure(dev);
  if (rc) return rc;
  GroupedParams p;
  memset(&p, 0, sizeof(p));
  p.core.M = G * M; p.core.N = N; p.core.K = cap;
  p.core.num_m_blocks = p.core.M / BM; p.core.num_n_blocks = N / BN;
  p.core.group_m = 16;
  p.core.timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 4000) * 1000000ull;
  p.core.err = g_err_dev[dev];
  p.rows = nullptr; p.klen = klen_dev; p.G = G; p.fixed_rows = M;
  p.a_blocks_per_group = M / BM;
  p.k_rows_per_group = cap;
  p.group_m = 16;
  // CTA pairs (a CTA then loads two 64-wide column blocks per operand and stage instead of four); the single-CTA loop
  // only if the device cannot hold a pair of this kernel
  const bool pair = g_pairs[dev] > 0;
  const uint32_t blocks = pair ? 2 : 4;
  // preferred: one 3-D copy per operand and stage; if the driver refuses that view, boxes of 64 MN-elements
  // (128 bytes, the swizzle span) by 64 tokens, one per column block
  static const bool no3d = getenv("B200SHMEM_TN_2D") != nullptr;
  p.tn3d = 0;
  if (!no3d && host::make_tmap_colblocks_3d(&p.map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, A, (uint64_t)G * cap, M, lda, 64, blocks) == 0 &&
      host::make_tmap_colblocks_3d(&p.map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, B, (uint64_t)G * cap, N, ldb, 64, blocks) == 0)
    p.tn3d = 1;
  if (!p.tn3d) {
    rc = host::make_tmap_2d(&p.map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, (uint64_t)G * cap, M, lda, 64, 64);
    if (rc) return rc;
    rc = host::make_tmap_2d(&p.map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, (uint64_t)G * cap, N, ldb, 64, 64);
    if (rc) return rc;
  }
  rc = host::make_tmap_2d(&p.map_c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, (uint64_t)G * M, N, ldc, 32, EPI_COLS);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (pair) {
    int pairs = g_pairs[dev];
    if (max_ctas > 1 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
    grouped_gemm_pair_tn_kernel<<<2 * pairs, g2::NUM_THREADS, g2::SMEM_BYTES, st>>>(p);
  } else {
    int ctas = g_sms[dev];
    if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
    grouped_gemm_tn_kernel<<<ctas, NUM_THREADS, SMEM_BYTES, st>>>(p);
  }
  BSHMEM_CUDA_TRY(cudaGetLastError());
  return 0;
}

// buf: [G][cap][cols] bf16, cols % 8 == 0: zero rows [counts[g], next multiple of 64) of every group.
int bshmem_moe_zero_pad_rows(void* buf, const int* counts_dev, int G, int cap, int cols, void* stream) {
  if (cols % 8 || G < 1) { host::last_error() = "zero_pad_rows: cols % 8 != 0"; return 1; }
  zero_pad_rows_kernel<<<dim3(8, G), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<__nv_bfloat16*>(buf), counts_dev, cap, cols);
  BSHMEM_CUDA_TRY(cudaGetLastError());
  return 0;
}

int bshmem_moe_gemm_error_site(int clear) {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || !g_err_dev[dev]) return 0;
  cudaMemcpy(&v, g_err_dev[dev], sizeof(int), cudaMemcpyDeviceToHost);
  if (clear && v) cudaMemset(g_err_dev[dev], 0, sizeof(int));
  return v;
}

int* bshmem_moe_gemm_error_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || ensure(dev)) return nullptr;
  return g_err_dev[dev];
}

}  // extern "C"
