// gemm_bf16.cu — stand-alone tcgen05 bf16 GEMM:  C[M,N] = A[M,K] · B[N,K]^T
// (both operands K-major, i.e. activations times a torch Linear weight), fp32
// accumulation in TMEM, bf16 output through TMA stores; CTA pairs (cta_group::2) with
// two accumulator stages, see gemm_pair.cuh.  This is the compute core
// that the fused all-gather→GEMM and GEMM→reduce-scatter kernels build on; it has
// no counterpart in the reference, which contains no GEMM.
#include "gemm_pair.cuh"
#include "tma_host.h"

using namespace bshmem;
using namespace bshmem::gemm2;

namespace {

struct PlainParams {
  CoreParams core;
  CUtensorMap map_a, map_b, map_c;
};

struct PlainBf16 : PolicyDefaults {
  using Params = PlainParams;
  __device__ static __forceinline__ const CoreParams& core(const Params& p) { return p.core; }
  __device__ static __forceinline__ const CUtensorMap* map_a(const Params& p) { return &p.map_a; }
  __device__ static __forceinline__ const CUtensorMap* map_b(const Params& p) { return &p.map_b; }
  __device__ static __forceinline__ void tile_coords(const Params& p, int tile, int* m_blk, int* n_blk) {
    raster_coords(p.core, tile, m_blk, n_blk);
  }
  __device__ static __forceinline__ void out_target(const Params& p, int row, int col, const CUtensorMap** map, int* x, int* y) {
    *map = (row < p.core.M && col < p.core.N) ? &p.map_c : nullptr;
    *x = col;
    *y = row;
  }
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1) gemm_bf16_kernel(const __grid_constant__ PlainParams prm) {
  extern __shared__ uint8_t smem_raw[];
  gemm_mainloop<PlainBf16>(prm, smem_raw);
}

int* g_err_dev[64] = {};
int g_pairs[64] = {};

int ensure_device_state(int dev) {
  if (g_err_dev[dev]) return 0;
  int sms = 0;
  BSHMEM_CUDA_TRY(cudaMalloc(&g_err_dev[dev], sizeof(int)));
  BSHMEM_CUDA_TRY(cudaMemset(g_err_dev[dev], 0, sizeof(int)));
  BSHMEM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  BSHMEM_CUDA_TRY(cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
  g_pairs[dev] = max_resident_pairs(gemm_bf16_kernel, sms);
  return 0;
}

}  // namespace

extern "C" {

const char* bshmem_gemm_last_error() { return host::last_error().c_str(); }

// C = A · B^T.  A: [M, K] row-major (lda elements), B: [N, K] row-major (ldb), C: [M, N] (ldc), all bf16.
// K, lda, ldb, ldc must be multiples of 8 and the bases 16-byte aligned (TMA).
// The kernel runs as CTA pairs (clusters of two); max_ctas <= 1 uses every pair the device can hold.  timeout_ms bounds every in-kernel wait.
int bshmem_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                     void* stream, int max_ctas, int timeout_ms) {
  if (M <= 0 || N <= 0 || K <= 0) { host::last_error() = "gemm: empty problem"; return 1; }
  if ((K % 8) || (lda % 8) || (ldb % 8) || (ldc % 8)) { host::last_error() = "gemm: K and leading dimensions must be multiples of 8"; return 1; }
  int dev = 0;
  BSHMEM_CUDA_TRY(cudaGetDevice(&dev));
  int rc = ensure_device_state(dev);
  if (rc) return rc;
  PlainParams p;
  p.core.M = M; p.core.N = N; p.core.K = K;
  p.core.num_m_blocks = (M + BM - 1) / BM;
  p.core.num_n_blocks = (N + BN - 1) / BN;
  p.core.group_m = 8;
  p.core.timeout_ns = (unsigned long long)(timeout_ms > 0 ? timeout_ms : 2000) * 1000000ull;
  p.core.err = g_err_dev[dev];
  rc = host::make_tmap_2d(&p.map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, M, K, lda, CTA_M, 64);
  if (rc) return rc;
  rc = host::make_tmap_2d(&p.map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, N, K, ldb, CTA_NLOAD, 64);
  if (rc) return rc;
  rc = host::make_tmap_2d(&p.map_c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, M, N, ldc, 32, EPI_COLS);
  if (rc) return rc;
  int tiles = p.core.num_m_blocks * p.core.num_n_blocks;
  int pairs = g_pairs[dev];
  if (max_ctas > 1 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
  if (tiles < pairs) pairs = tiles;
  const int ctas = 2 * pairs;
  gemm_bf16_kernel<<<ctas, NUM_THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(p);
  BSHMEM_CUDA_TRY(cudaGetLastError());
  return 0;
}

// Reads (and clears) the device error word of the current device: 0 = no bounded wait ran out.
int bshmem_gemm_error_site(int clear) {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || !g_err_dev[dev]) return 0;
  cudaMemcpy(&v, g_err_dev[dev], sizeof(int), cudaMemcpyDeviceToHost);
  if (clear && v) cudaMemset(g_err_dev[dev], 0, sizeof(int));
  return v;
}

}  // extern "C"
