// Picks the collective-kernel unit for a call (see coll_kernels.h).
#include "../include/bshmem_gpu.h"
#include "coll_kernels.h"

namespace bshmem {
namespace collk {
namespace {
enum Unit { U_MOVE, U_F32, U_F16, U_I32, U_I8, U_NONE };
Unit unit_of(const CollArgs& a) {
  if (a.kind != BSHMEM_COLL_REDUCE && a.kind != BSHMEM_COLL_REDUCE_SCATTER && a.kind != BSHMEM_COLL_REDUCE_ROOT) return U_MOVE;
  switch (a.dtype) {
    case BSHMEM_FLOAT: case BSHMEM_DOUBLE: return U_F32;
    case BSHMEM_BF16: case BSHMEM_FP16: return U_F16;
    case BSHMEM_INT32: case BSHMEM_UINT32: case BSHMEM_INT64: case BSHMEM_UINT64: return U_I32;
    case BSHMEM_INT8: case BSHMEM_UINT8: case BSHMEM_INT16: case BSHMEM_UINT16: return U_I8;
    default: return U_NONE;
  }
}
}  // namespace

cudaError_t launch(const State& s, const DTeam& t, const CollArgs& a, int ctas, int* status, cudaStream_t stream) {
  switch (unit_of(a)) {
    case U_MOVE: return launch_move(s, t, a, ctas, status, stream);
    case U_F32: return launch_f32(s, t, a, ctas, status, stream);
    case U_F16: return launch_f16(s, t, a, ctas, status, stream);
    case U_I32: return launch_i32(s, t, a, ctas, status, stream);
    case U_I8: return launch_i8(s, t, a, ctas, status, stream);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_group(const State* states, const DTeam* teams, const CollArgs& a, int ctas, int n, int* status,
                         cudaStream_t stream) {
  switch (unit_of(a)) {
    case U_MOVE: return launch_group_move(states, teams, a, ctas, n, status, stream);
    case U_F32: return launch_group_f32(states, teams, a, ctas, n, status, stream);
    case U_F16: return launch_group_f16(states, teams, a, ctas, n, status, stream);
    case U_I32: return launch_group_i32(states, teams, a, ctas, n, status, stream);
    case U_I8: return launch_group_i8(states, teams, a, ctas, n, status, stream);
    default: return cudaErrorInvalidValue;
  }
}

void preload() {
  preload_move(); preload_f32(); preload_f16(); preload_i32(); preload_i8();
}

}  // namespace collk
}  // namespace bshmem
