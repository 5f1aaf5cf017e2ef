// coll_kernels.h — host launchers of the collective kernels.
//
// The device collectives of bshmem_coll.cuh are templates over the element type and the operator; instantiating all
// of them in one translation unit takes many minutes.  The kernels are therefore split by element class into
// translation units of their own (built in parallel): data movement and synchronisation, 4/8-byte floats, 2-byte
// floats, 4/8-byte integers, 1/2-byte integers.  Each unit has one kernel for a PE per launch and one for all PEs
// of a local group in a single cooperative launch (blockIdx.y = PE), and the host picks the unit by (kind, dtype).
// Parity: these are the bodies behind library/src/roc_shmem.cpp's host collectives (:1033-1128), which the
// reference forwards to MPI.
#pragma once
#include <cuda_runtime.h>

#include "../include/bshmem_device.cuh"

namespace bshmem {
namespace collk {

using State = bshmem_dev_state_t;
using DTeam = bshmem_team_dev_t;

struct CollArgs {
  int kind;            // BSHMEM_COLL_*
  int dtype, op, root;
  uint64_t dst_off, src_off, n;   // n: elements for reductions, bytes otherwise
  uint64_t psync_off;  // active set
  int use_nvls;
  unsigned long long ll_epoch;   // != 0: epoch of a host-launched low-latency allreduce (same on every PE)
  unsigned long long stage_seq;  // != 0: one-exchange form through the staging region, call number (same on every PE)
  int stage_oneshot;             // allreduce with stage_seq: 1 = every PE reduces the whole vector (one exchange), 0 = two-shot
};

// Threads per block: 512 for the data-movement unit; 256 for the reduction units, whose unrolled multi-source loops
// then have 255 registers per thread and compile without spills.
constexpr int kMoveThreads = 512;
constexpr int kReduceThreads = 256;

// Bytes a collective reads at src_off and writes at dst_off on every member (count: elements for reductions,
// bytes otherwise), for range checks on the host.
inline void extent(int kind, int dtype, uint64_t count, int team_size, uint64_t* src_bytes, uint64_t* dst_bytes) {
  const uint64_t es = bshmem_dtype_size(dtype);
  switch (kind) {
    case 3 /* BSHMEM_COLL_REDUCE */: *src_bytes = *dst_bytes = count * es; break;
    case 8 /* BSHMEM_COLL_REDUCE_ROOT */: *src_bytes = *dst_bytes = count * es; break;
    case 4 /* BSHMEM_COLL_REDUCE_SCATTER */: *src_bytes = count * es * team_size; *dst_bytes = count * es; break;
    case 5 /* BSHMEM_COLL_FCOLLECT */: *src_bytes = count; *dst_bytes = count * team_size; break;
    case 6 /* BSHMEM_COLL_ALLTOALL */: *src_bytes = *dst_bytes = count * team_size; break;
    case 2 /* BSHMEM_COLL_BROADCAST */: *src_bytes = *dst_bytes = count; break;
    default: *src_bytes = *dst_bytes = 0;
  }
}

// One PE: `ctas` blocks on `stream`; a non-zero device status lands in *status (first one wins).
cudaError_t launch(const State& s, const DTeam& t, const CollArgs& a, int ctas, int* status, cudaStream_t stream);
// All PEs of a local group at once: states / teams are device arrays of n entries (a team with my_idx < 0 sits out).
cudaError_t launch_group(const State* states, const DTeam* teams, const CollArgs& a, int ctas, int n, int* status,
                         cudaStream_t stream);
// Loads every kernel module now (a lazy first load from another thread could need a device-wide quiet point).
void preload();

// per element class (defined by coll_kernels_impl.cuh in each unit)
#define BSHMEM_COLL_UNIT(name)                                                                                          \
  cudaError_t launch_##name(const State&, const DTeam&, const CollArgs&, int, int*, cudaStream_t);                       \
  cudaError_t launch_group_##name(const State*, const DTeam*, const CollArgs&, int, int, int*, cudaStream_t);           \
  void preload_##name();
BSHMEM_COLL_UNIT(move)
BSHMEM_COLL_UNIT(f32)
BSHMEM_COLL_UNIT(f16)
BSHMEM_COLL_UNIT(i32)
BSHMEM_COLL_UNIT(i8)
#undef BSHMEM_COLL_UNIT

}  // namespace collk
}  // namespace bshmem
