// tma_host.h — host helpers shared by the kernel libraries: encoding TMA tensor
// maps through the driver entry point (no link-time dependency on libcuda, so the
// libraries also load on a machine without a driver), and error plumbing.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <stdint.h>

#include <cstdio>
#include <mutex>
#include <string>

namespace bshmem {
namespace host {

inline std::string& last_error() {
  static thread_local std::string e;
  return e;
}

#define BSHMEM_CUDA_TRY(expr)                                                                   \
  do {                                                                                          \
    cudaError_t _e = (expr);                                                                    \
    if (_e != cudaSuccess) {                                                                    \
      ::bshmem::host::last_error() = std::string(#expr) + ": " + cudaGetErrorString(_e);        \
      return 7; /* BSHMEM_ERR_CUDA */                                                           \
    }                                                                                           \
  } while (0)

inline PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

// 2-D row-major tensor [rows, cols] with row pitch `ld` elements; box = [box_rows, box_cols],
// 128-byte swizzle (box_cols * elem_bytes must be 128).
inline int make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t rows,
                        uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_cols,
                        CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B,
                        CUtensorMapL2promotion l2 = CU_TENSOR_MAP_L2_PROMOTION_L2_256B) {
  auto fn = encode_fn();
  if (!fn) { last_error() = "cuTensorMapEncodeTiled entry point not available"; return 7; }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * elem_bytes) & 15)) {
    last_error() = "TMA needs a 16-byte aligned base and row pitch";
    return 1;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  l2, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    last_error() = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r);
    return 7;
  }
  return 0;
}

// 3-D view of a row-major [rows, cols] 2-byte tensor for MN-major operands: dim0 = 64 elements inside a 64-wide
// column block, dim1 = rows, dim2 = column block (128 bytes apart).  One box {64, box_rows, box_blocks} lands in
// shared memory as box_blocks consecutive [box_rows][64] blocks with the 128-byte swizzle, i.e. what several 2-D
// {64, box_rows} boxes would write, in one copy.  Returns non-zero if the driver refuses the (non-monotonic) strides.
inline int make_tmap_colblocks_3d(CUtensorMap* out, CUtensorMapDataType dt, const void* base, uint64_t rows, uint64_t cols,
                                  uint64_t ld, uint32_t box_rows, uint32_t box_blocks) {
  auto fn = encode_fn();
  if (!fn) { last_error() = "cuTensorMapEncodeTiled entry point not available"; return 7; }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15) || cols % 64) {
    last_error() = "TMA needs a 16-byte aligned base and row pitch, and a column count that is a multiple of 64";
    return 1;
  }
  cuuint64_t dims[3] = {64, rows, cols / 64};
  cuuint64_t strides[2] = {ld * 2, 128};
  cuuint32_t box[3] = {64, box_rows, box_blocks};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    last_error() = "cuTensorMapEncodeTiled (3-D column blocks) failed with CUresult " + std::to_string((int)r);
    return 7;
  }
  return 0;
}

}  // namespace host
}  // namespace bshmem
