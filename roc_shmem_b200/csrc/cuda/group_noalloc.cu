// group_noalloc.cu — bshmem_gpu_group_collective_noalloc(): the group collective for
// callers that must not allocate device memory.  See bshmem_gpu_noalloc.h for who those
// callers are and for the limits; this file holds the fixed scratch array, its one-time
// address look-up and the launch.
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>
#include <string>

#include "../include/bshmem_coll.cuh"
#include "../include/bshmem_gpu_noalloc.h"

using namespace bshmem;
using dev::State;
using DTeam = bshmem::dev::Team;

namespace {

// Per-GPU scratch that lives in the library image: [State x 16][Team x 16][status word].
// In host code this name is only a stand-in for the symbol; the device address comes from
// cudaGetSymbolAddress() below and is what the kernel receives.
static __device__ __align__(256) unsigned char g_group_scratch[BSHMEM_NOALLOC_SCRATCH_BYTES];

constexpr size_t kStatesBytes = sizeof(State) * BSHMEM_NOALLOC_MAX_PES;
constexpr size_t kTeamsBytes = sizeof(DTeam) * BSHMEM_NOALLOC_MAX_PES;
constexpr size_t kStatusOffset = kStatesBytes + kTeamsBytes;
static_assert(kStatusOffset + sizeof(int) <= BSHMEM_NOALLOC_SCRATCH_BYTES, "scratch array too small for 16 PEs");

struct Args {
  int kind, dtype, op, root;
  uint64_t dst_off, src_off, n;
};

template <typename T>
__device__ int reduce_as(const State& s, const DTeam& t, const Args& a, int cta, int ncta) {
  T* d = reinterpret_cast<T*>(s.heap_base[s.my_pe] + a.dst_off);
  const T* src = reinterpret_cast<const T*>(s.heap_base[s.my_pe] + a.src_off);
  if (a.kind == BSHMEM_COLL_REDUCE_SCATTER) return coll::team_reduce_scatter<T>(s, t, a.op, d, src, a.n, cta, ncta);
  return coll::team_reduce<T>(s, t, a.op, d, src, a.n, cta, ncta);
}

__device__ int run_one(const State& s, const DTeam& t, const Args& a, int cta, int ncta) {
  char* base = s.heap_base[s.my_pe];
  switch (a.kind) {
    case BSHMEM_COLL_SYNC: return coll::team_sync(s, t, cta);
    case BSHMEM_COLL_BARRIER: return coll::team_barrier(s, t, cta);
    case BSHMEM_COLL_BROADCAST: return coll::team_broadcast(s, t, base + a.dst_off, base + a.src_off, a.n, a.root, cta, ncta);
    case BSHMEM_COLL_FCOLLECT: return coll::team_fcollect(s, t, base + a.dst_off, base + a.src_off, a.n, cta, ncta);
    case BSHMEM_COLL_ALLTOALL: return coll::team_alltoall(s, t, base + a.dst_off, base + a.src_off, a.n, cta, ncta);
    case BSHMEM_COLL_REDUCE: case BSHMEM_COLL_REDUCE_SCATTER:
      switch (a.dtype) {
        case BSHMEM_INT8: return reduce_as<int8_t>(s, t, a, cta, ncta);
        case BSHMEM_UINT8: return reduce_as<uint8_t>(s, t, a, cta, ncta);
        case BSHMEM_INT16: return reduce_as<int16_t>(s, t, a, cta, ncta);
        case BSHMEM_UINT16: return reduce_as<uint16_t>(s, t, a, cta, ncta);
        case BSHMEM_INT32: return reduce_as<int32_t>(s, t, a, cta, ncta);
        case BSHMEM_UINT32: return reduce_as<uint32_t>(s, t, a, cta, ncta);
        case BSHMEM_INT64: return reduce_as<long long>(s, t, a, cta, ncta);
        case BSHMEM_UINT64: return reduce_as<unsigned long long>(s, t, a, cta, ncta);
        case BSHMEM_FLOAT: return reduce_as<float>(s, t, a, cta, ncta);
        case BSHMEM_DOUBLE: return reduce_as<double>(s, t, a, cta, ncta);
        case BSHMEM_BF16: return reduce_as<__nv_bfloat16>(s, t, a, cta, ncta);
        case BSHMEM_FP16: return reduce_as<__half>(s, t, a, cta, ncta);
      }
      return BSHMEM_ERR_UNSUPPORTED;
  }
  return BSHMEM_ERR_INVALID;
}

// Same shape as the allocating entry's kernel: one cooperative launch, blockIdx.y is the PE.
__global__ void __launch_bounds__(512) k_group_static(const State* states, const DTeam* teams, Args a, int* status) {
  State s = states[blockIdx.y];
  DTeam t = teams[blockIdx.y];
  if (t.my_idx < 0) return;
  int rc = run_one(s, t, a, blockIdx.x, gridDim.x);
  if (rc != BSHMEM_OK && threadIdx.x == 0) atomicCAS(status, 0, rc);
}

thread_local std::string g_err;
std::mutex g_mu;
unsigned char* g_scratch_addr[64] = {};   // device address of g_group_scratch, per device

// Once per device, with that device current: resolve the array's device address.
int scratch_for_current_device(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) { g_err = "cudaGetDevice failed or device index out of range"; return BSHMEM_ERR_CUDA; }
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_scratch_addr[dev]) {
    unsigned char* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_group_scratch);
    if (e != cudaSuccess || !p) {
      g_err = std::string("cudaGetSymbolAddress(g_group_scratch): ") + cudaGetErrorString(e);
      return BSHMEM_ERR_CUDA;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return BSHMEM_OK;
}

}  // namespace

extern "C" {

const char* bshmem_gpu_noalloc_last_error(void) { return g_err.c_str(); }

int bshmem_gpu_group_collective_noalloc(bshmem_handle_t* handles, int n, int team_slot, int kind, int dtype, int op,
                                        int root, uint64_t dst_off, uint64_t src_off, uint64_t count, int ctas) {
  g_err.clear();
  if (!handles || n < 1) { g_err = "no handles"; return BSHMEM_ERR_INVALID; }
  if (n > BSHMEM_NOALLOC_MAX_PES) {
    g_err = "group of " + std::to_string(n) + " PEs exceeds the fixed scratch array (at most " +
            std::to_string(BSHMEM_NOALLOC_MAX_PES) + " PEs); use bshmem_gpu_group_collective()";
    return BSHMEM_ERR_LIMIT;
  }
  if (kind < BSHMEM_COLL_SYNC || kind > BSHMEM_COLL_ALLTOALL) { g_err = "unknown collective kind"; return BSHMEM_ERR_INVALID; }

  // Host image of the scratch: states, teams, and a zero status word (the array keeps the
  // previous call's contents, so everything the kernel reads is rewritten here).
  alignas(16) unsigned char image[BSHMEM_NOALLOC_SCRATCH_BYTES];
  memset(image, 0, sizeof(image));
  State* hs = reinterpret_cast<State*>(image);
  DTeam* ht = reinterpret_cast<DTeam*>(image + kStatesBytes);
  void* stream_v = nullptr;
  for (int i = 0; i < n; ++i) {
    int rc = bshmem_gpu_get_state(handles[i], &hs[i]);
    if (rc != BSHMEM_OK) { g_err = "handle " + std::to_string(i) + " is not a GPU runtime"; return rc; }
    DTeam& t = ht[i];
    t.my_idx = bshmem_team_my_pe(handles[i], team_slot);
    t.size = bshmem_team_n_pes(handles[i], team_slot);
    t.slot = team_slot;
    t.reserved = 0;
    t.psync = nullptr;
    if (t.my_idx < 0 || t.size < 1) { t.my_idx = -1; t.size = 0; t.pe_start = 0; t.stride = 1; continue; }
    t.pe_start = bshmem_team_translate_pe(handles[i], team_slot, 0, BSHMEM_TEAM_WORLD);
    t.stride = t.size > 1 ? bshmem_team_translate_pe(handles[i], team_slot, 1, BSHMEM_TEAM_WORLD) - t.pe_start : 1;
  }
  if (bshmem_gpu_get_stream(handles[0], &stream_v) != BSHMEM_OK) { g_err = "cannot get the PE's stream"; return BSHMEM_ERR_STATE; }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  unsigned char* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != BSHMEM_OK) return rc;
  cudaError_t e = cudaMemcpyAsync(scratch, image, kStatusOffset + sizeof(int), cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) { g_err = std::string("copy of the PE table: ") + cudaGetErrorString(e); return BSHMEM_ERR_CUDA; }

  const State* d_states = reinterpret_cast<const State*>(scratch);
  const DTeam* d_teams = reinterpret_cast<const DTeam*>(scratch + kStatesBytes);
  int* d_status = reinterpret_cast<int*>(scratch + kStatusOffset);
  Args a{kind, dtype, op, root, dst_off, src_off, count};
  if (ctas < 1) ctas = 1;
  void* args[] = {&d_states, &d_teams, &a, &d_status};
  e = cudaLaunchCooperativeKernel((void*)k_group_static, dim3(ctas, n), dim3(512), args, 0, stream);
  if (e != cudaSuccess) { g_err = std::string("cooperative launch: ") + cudaGetErrorString(e); return BSHMEM_ERR_CUDA; }
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) { g_err = std::string("stream synchronize: ") + cudaGetErrorString(e); return BSHMEM_ERR_CUDA; }
  int st = 0;
  e = cudaMemcpy(&st, d_status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) { g_err = std::string("status read: ") + cudaGetErrorString(e); return BSHMEM_ERR_CUDA; }
  if (st != 0) g_err = "a device-side wait of the collective ran out";
  return st;
}

}  // extern "C"
