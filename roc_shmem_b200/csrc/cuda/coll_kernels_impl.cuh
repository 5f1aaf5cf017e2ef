// coll_kernels_impl.cuh — body of one collective-kernel translation unit.  The including .cu defines
//   COLL_UNIT        name of the unit (move, f32, ...)
//   COLL_TYPES(X)    X(dtype code, C type) for every element type the unit reduces (empty for `move`)
// and gets a per-PE kernel, a local-group kernel and their launchers (see coll_kernels.h).
#include "../include/bshmem_coll.cuh"
#include "../include/bshmem_gpu.h"
#include "coll_kernels.h"

namespace bshmem {
namespace collk {
namespace {

#ifdef COLL_UNIT_MOVE
constexpr int kThreads = kMoveThreads;
#else
constexpr int kThreads = kReduceThreads;
#endif

#define COLL_CAT2(a, b) a##b
#define COLL_CAT(a, b) COLL_CAT2(a, b)

// dynamic shared memory of the reduction kernels: the staging ring of coll::reduce_bulk
#ifndef COLL_UNIT_MOVE
constexpr uint32_t kDynSmem = coll::kBulkSmemBytes;
#else
constexpr uint32_t kDynSmem = 0;
#endif

template <typename T>
__device__ int reduce_typed(const State& s, const DTeam& t, const CollArgs& a, int cta, int ncta) {
  extern __shared__ __align__(128) char coll_dyn_smem[];
  char* bulk = kDynSmem ? coll_dyn_smem : nullptr;
  T* d = reinterpret_cast<T*>(s.heap_base[s.my_pe] + a.dst_off);
  const T* src = reinterpret_cast<const T*>(s.heap_base[s.my_pe] + a.src_off);
  if (a.kind == BSHMEM_COLL_REDUCE_ROOT) return coll::team_reduce_root<T>(s, t, a.op, d, src, a.n, a.root, cta, ncta, bulk);
  if (a.kind == BSHMEM_COLL_REDUCE_SCATTER) {
    if constexpr (std::is_same<T, float>::value || std::is_same<T, __nv_bfloat16>::value) {
      // large sums on the whole world: the switch reduces (see the allreduce below)
      if (a.use_nvls && s.mc_base && t.size == s.n_pes && a.op == BSHMEM_SUM && ((a.dst_off | a.src_off) & 15) == 0 &&
          (a.n * sizeof(T)) % 16 == 0 && !a.stage_seq)
        return coll::team_reduce_scatter_nvls<T>(s, t, d, src, a.n, cta, ncta);
    }
    if (a.stage_seq) return coll::team_reduce_scatter_staged<T>(s, t, a.op, d, src, a.n, a.stage_seq, cta, ncta, bulk);
    return coll::team_reduce_scatter<T>(s, t, a.op, d, src, a.n, cta, ncta, bulk);
  }
  if constexpr (std::is_same<T, float>::value || std::is_same<T, __nv_bfloat16>::value) {
    // the multicast mapping spans every PE, so the in-switch reduction only fits a team that is the whole world
    // (small vectors stay on the one-exchange slots: a switch round trip per vector only pays off in bandwidth)
    if (a.use_nvls && s.mc_base && t.size == s.n_pes && a.op == BSHMEM_SUM && ((a.dst_off | a.src_off) & 15) == 0 &&
        (a.n * sizeof(T)) % 16 == 0 && a.ll_epoch == 0 && a.n * sizeof(T) > BSHMEM_LLB_PAYLOAD_BYTES)
      return coll::team_reduce_nvls<T>(s, t, d, src, a.n, cta, ncta);
  }
  if (a.stage_seq && a.stage_oneshot) return coll::team_reduce_staged_oneshot<T>(s, t, a.op, d, src, a.n, a.stage_seq, cta, ncta, bulk);
  if (a.stage_seq) return coll::team_reduce_staged<T>(s, t, a.op, d, src, a.n, a.stage_seq, cta, ncta, bulk);
  return coll::team_reduce<T>(s, t, a.op, d, src, a.n, cta, ncta, a.ll_epoch, bulk);
}

__device__ __noinline__ int run_coll(const State& s, DTeam t, const CollArgs& a, int cta, int ncta) {
  char* base = s.heap_base[s.my_pe];
  if (t.slot < 0) t.psync = reinterpret_cast<long*>(base + a.psync_off);
  switch (a.kind) {
#ifdef COLL_UNIT_MOVE
    case BSHMEM_COLL_SYNC: return coll::team_sync(s, t, cta);
    case BSHMEM_COLL_BARRIER: return coll::team_barrier(s, t, cta);
    case BSHMEM_COLL_BROADCAST: return coll::team_broadcast(s, t, base + a.dst_off, base + a.src_off, a.n, a.root, cta, ncta);
    case BSHMEM_COLL_FCOLLECT:
      if (a.stage_seq) return coll::team_fcollect_staged(s, t, base + a.dst_off, base + a.src_off, a.n, a.stage_seq, a.use_nvls, cta, ncta);
      return coll::team_fcollect(s, t, base + a.dst_off, base + a.src_off, a.n, cta, ncta);
    case BSHMEM_COLL_ALLTOALL:
      if (a.stage_seq) return coll::team_alltoall_staged(s, t, base + a.dst_off, base + a.src_off, a.n, a.stage_seq, cta, ncta);
      return coll::team_alltoall(s, t, base + a.dst_off, base + a.src_off, a.n, cta, ncta);
    case BSHMEM_COLL_EXCHANGE: {
      // publish one u64 (held in a.n) in every member's exchange row, sync, leave the row for the host
      if (threadIdx.x < t.size) {
        uint64_t* row = reinterpret_cast<uint64_t*>(s.heap_base[dev::team_pe(t, threadIdx.x)] + BSHMEM_OFF_XCHG) +
                        (size_t)t.slot * BSHMEM_MAX_PES;
        row[t.my_idx] = a.n;
      }
      int rc = coll::team_barrier(s, t, cta);
      if (rc != BSHMEM_OK) return rc;
      return coll::team_sync(s, t, cta);   // nobody overwrites a row that is still being read... by the next exchange
    }
#endif
    case BSHMEM_COLL_REDUCE: case BSHMEM_COLL_REDUCE_SCATTER: case BSHMEM_COLL_REDUCE_ROOT:
      switch (a.dtype) {
#define COLL_CASE(code, T) case code: return reduce_typed<T>(s, t, a, cta, ncta);
        COLL_TYPES(COLL_CASE)
#undef COLL_CASE
      }
      return BSHMEM_ERR_UNSUPPORTED;
  }
  return BSHMEM_ERR_INVALID;
}

__global__ void __launch_bounds__(kThreads) COLL_CAT(k_coll_, COLL_UNIT)(State s, DTeam t, CollArgs a, int* status) {
  int rc = run_coll(s, t, a, blockIdx.x, gridDim.x);
  if (rc != BSHMEM_OK && threadIdx.x == 0) atomicCAS(status, 0, rc);
}

// All PEs of a local group in ONE cooperative launch: blockIdx.y is the PE.  Used to exercise the multi-PE
// algorithms on a single GPU (kernels that wait on one another must not be separate launches on one device).
__global__ void __launch_bounds__(kThreads) COLL_CAT(k_coll_group_, COLL_UNIT)(const State* states, const DTeam* teams,
                                                                                CollArgs a, int* status) {
  State s = states[blockIdx.y];
  DTeam t = teams[blockIdx.y];
  if (t.my_idx < 0) return;
  int rc = run_coll(s, t, a, blockIdx.x, gridDim.x);
  if (rc != BSHMEM_OK && threadIdx.x == 0) atomicCAS(status, 0, rc);
}

}  // namespace

cudaError_t COLL_CAT(launch_, COLL_UNIT)(const State& s, const DTeam& t, const CollArgs& a, int ctas, int* status, cudaStream_t stream) {
  COLL_CAT(k_coll_, COLL_UNIT)<<<ctas, kThreads, kDynSmem, stream>>>(s, t, a, status);
  return cudaGetLastError();
}

cudaError_t COLL_CAT(launch_group_, COLL_UNIT)(const State* states, const DTeam* teams, const CollArgs& a, int ctas, int n,
                                               int* status, cudaStream_t stream) {
  CollArgs args_copy = a;
  void* args[] = {&states, &teams, &args_copy, &status};
  return cudaLaunchCooperativeKernel((void*)COLL_CAT(k_coll_group_, COLL_UNIT), dim3(ctas, n), dim3(kThreads), args, kDynSmem, stream);
}

void COLL_CAT(preload_, COLL_UNIT)() {
  cudaFuncAttributes fa;
  cudaFuncGetAttributes(&fa, COLL_CAT(k_coll_, COLL_UNIT));
  cudaFuncGetAttributes(&fa, COLL_CAT(k_coll_group_, COLL_UNIT));
  if (kDynSmem) {      // per device: the caller has made the PE's device current
    cudaFuncSetAttribute(COLL_CAT(k_coll_, COLL_UNIT), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDynSmem);
    cudaFuncSetAttribute(COLL_CAT(k_coll_group_, COLL_UNIT), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDynSmem);
  }
}

}  // namespace collk
}  // namespace bshmem
