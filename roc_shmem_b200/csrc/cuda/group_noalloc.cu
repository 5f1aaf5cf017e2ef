// group_noalloc.cu — bshmem_gpu_group_collective_noalloc(): the group collective for
// callers that must not allocate device memory.  See bshmem_gpu_noalloc.h for who those
// callers are and for the limits; this file holds the fixed scratch array, its one-time
// address look-up and the launch (of the same cooperative kernels the allocating entry runs,
// coll_kernels.h, handed pointers into the array).
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>
#include <string>

#include "../include/bshmem_gpu.h"
#include "../include/bshmem_gpu_noalloc.h"
#include "coll_kernels.h"

using namespace bshmem;
using State = bshmem_dev_state_t;
using DTeam = bshmem_team_dev_t;

namespace {

// Per-GPU scratch that lives in the library image: [State x 16][Team x 16][status word].
// In host code this name is only a stand-in for the symbol; the device address comes from
// cudaGetSymbolAddress() below and is what the kernel receives.
static __device__ __align__(256) unsigned char g_group_scratch[BSHMEM_NOALLOC_SCRATCH_BYTES];

constexpr size_t kStatesBytes = sizeof(State) * BSHMEM_NOALLOC_MAX_PES;
constexpr size_t kTeamsBytes = sizeof(DTeam) * BSHMEM_NOALLOC_MAX_PES;
constexpr size_t kStatusOffset = kStatesBytes + kTeamsBytes;
static_assert(kStatusOffset + sizeof(int) <= BSHMEM_NOALLOC_SCRATCH_BYTES, "scratch array too small for 16 PEs");

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
  // The array that is resolved and written below belongs to the CURRENT device, so that must be the handles' device.
  int cur = -1, hdev = -1;
  if (cudaGetDevice(&cur) != cudaSuccess || bshmem_gpu_get_device(handles[0], &hdev) != BSHMEM_OK) {
    g_err = "cannot determine the current device or the handles' device";
    return BSHMEM_ERR_STATE;
  }
  if (cur != hdev) {
    g_err = "the current CUDA device (" + std::to_string(cur) + ") is not the device of the group's heaps (" + std::to_string(hdev) +
            "); call cudaSetDevice first";
    return BSHMEM_ERR_STATE;
  }

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
  for (int i = 0; i < n; ++i) {
    if (ht[i].my_idx < 0) continue;
    uint64_t sb = 0, db = 0;
    collk::extent(kind, dtype, count, ht[i].size, &sb, &db);
    if (src_off > hs[i].heap_bytes || sb > hs[i].heap_bytes - src_off || dst_off > hs[i].heap_bytes || db > hs[i].heap_bytes - dst_off) {
      g_err = "source or destination range lies outside the symmetric heap";
      return BSHMEM_ERR_RANGE;
    }
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
  collk::CollArgs a{};
  a.kind = kind; a.dtype = dtype; a.op = op; a.root = root; a.dst_off = dst_off; a.src_off = src_off; a.n = count;
  if (ctas < 1) ctas = 1;
  if (ctas > BSHMEM_MAX_COLL_CTAS) ctas = BSHMEM_MAX_COLL_CTAS;     // one flag row per channel exists, no more
  e = collk::launch_group(d_states, d_teams, a, ctas, n, d_status, stream);
  if (e != cudaSuccess) { g_err = std::string("cooperative launch: ") + cudaGetErrorString(e); return BSHMEM_ERR_CUDA; }
  // the status word comes back on the PE's own stream: nothing here touches any other stream of the device
  int st = 0;
  e = cudaMemcpyAsync(&st, d_status, sizeof(int), cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) { g_err = std::string("status read: ") + cudaGetErrorString(e); return BSHMEM_ERR_CUDA; }
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) { g_err = std::string("stream synchronize: ") + cudaGetErrorString(e); return BSHMEM_ERR_CUDA; }
  if (st != 0) g_err = "a device-side wait of the collective ran out";
  return st;
}

}  // extern "C"
