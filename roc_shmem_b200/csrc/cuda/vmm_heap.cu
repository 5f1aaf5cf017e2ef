// vmm_heap.cu — the symmetric heap in GPU memory and its mapping into every peer.
//
// Each PE creates one physical allocation with the CUDA virtual-memory API
// (shareable as a POSIX file descriptor), reserves one virtual range of
// n_pes * heap_bytes and maps PE p's allocation at base + p * heap_bytes, so the
// remote address of a symmetric object is pure arithmetic.  Descriptors travel
// between processes over a Unix socket (done by the Python bootstrap).  Where the
// driver refuses shareable VMM allocations the heap falls back to cudaMalloc +
// cudaIpc handles (peers then sit at unrelated addresses; the base table hides it).
// Optionally the allocations are also bound to an NVLink multicast object, which
// gives the `mc_base` mapping used by multimem reductions and broadcasts.
//
// Parity: the reference's heap is fine-grained hipExtMallocWithFlags memory whose
// bases are all-gathered over MPI (library/src/memory/remote_heap_info.hpp:142-152)
// and IPC-mapped per node (ipc_policy.cpp:34-111).  The driver API is reached
// through cudaGetDriverEntryPoint, so this library has no link-time dependency on
// libcuda and loads on machines without a driver.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <unistd.h>

#include <cstring>
#include <mutex>
#include <string>

#include "../include/bshmem_device.cuh"
#include "gpu_heap.h"

namespace bshmem {
namespace gpu {

std::string& heap_error() {
  static thread_local std::string e;
  return e;
}

namespace {

struct Driver {
  PFN_cuMemCreate_v10020 MemCreate = nullptr;
  PFN_cuMemRelease_v10020 MemRelease = nullptr;
  PFN_cuMemAddressReserve_v10020 MemAddressReserve = nullptr;
  PFN_cuMemAddressFree_v10020 MemAddressFree = nullptr;
  PFN_cuMemMap_v10020 MemMap = nullptr;
  PFN_cuMemUnmap_v10020 MemUnmap = nullptr;
  PFN_cuMemSetAccess_v10020 MemSetAccess = nullptr;
  PFN_cuMemGetAllocationGranularity_v10020 MemGetAllocationGranularity = nullptr;
  PFN_cuMemExportToShareableHandle_v10020 MemExportToShareableHandle = nullptr;
  PFN_cuMemImportFromShareableHandle_v10020 MemImportFromShareableHandle = nullptr;
  PFN_cuMulticastCreate_v12010 MulticastCreate = nullptr;
  PFN_cuMulticastAddDevice_v12010 MulticastAddDevice = nullptr;
  PFN_cuMulticastBindMem_v12010 MulticastBindMem = nullptr;
  PFN_cuMulticastGetGranularity_v12010 MulticastGetGranularity = nullptr;
  PFN_cuDeviceGetAttribute_v2000 DeviceGetAttribute = nullptr;
  PFN_cuGetErrorString_v6000 GetErrorString = nullptr;
  bool ok = false;
};

template <typename F> bool load_sym(const char* name, F* out) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p)
    return false;
  *out = reinterpret_cast<F>(p);
  return true;
}

Driver& drv() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    bool ok = true;
    ok &= load_sym("cuMemCreate", &d.MemCreate);
    ok &= load_sym("cuMemRelease", &d.MemRelease);
    ok &= load_sym("cuMemAddressReserve", &d.MemAddressReserve);
    ok &= load_sym("cuMemAddressFree", &d.MemAddressFree);
    ok &= load_sym("cuMemMap", &d.MemMap);
    ok &= load_sym("cuMemUnmap", &d.MemUnmap);
    ok &= load_sym("cuMemSetAccess", &d.MemSetAccess);
    ok &= load_sym("cuMemGetAllocationGranularity", &d.MemGetAllocationGranularity);
    ok &= load_sym("cuMemExportToShareableHandle", &d.MemExportToShareableHandle);
    ok &= load_sym("cuMemImportFromShareableHandle", &d.MemImportFromShareableHandle);
    ok &= load_sym("cuDeviceGetAttribute", &d.DeviceGetAttribute);
    ok &= load_sym("cuGetErrorString", &d.GetErrorString);
    // multicast is optional
    load_sym("cuMulticastCreate", &d.MulticastCreate);
    load_sym("cuMulticastAddDevice", &d.MulticastAddDevice);
    load_sym("cuMulticastBindMem", &d.MulticastBindMem);
    load_sym("cuMulticastGetGranularity", &d.MulticastGetGranularity);
    d.ok = ok;
  });
  return d;
}

int cu_fail(const char* what, CUresult r) {
  const char* s = nullptr;
  if (drv().GetErrorString) drv().GetErrorString(r, &s);
  heap_error() = std::string(what) + " failed: " + (s ? s : "?") + " (CUresult " + std::to_string((int)r) + ")";
  return BSHMEM_ERR_CUDA;
}
int rt_fail(const char* what, cudaError_t e) {
  heap_error() = std::string(what) + " failed: " + cudaGetErrorString(e);
  return BSHMEM_ERR_CUDA;
}
#define CU_TRY(call) do { CUresult _r = (call); if (_r != CUDA_SUCCESS) return cu_fail(#call, _r); } while (0)
#define RT_TRY(call) do { cudaError_t _e = (call); if (_e != cudaSuccess) return rt_fail(#call, _e); } while (0)

CUmemAllocationProp alloc_prop(int device) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

int map_at(Heap* h, int pe, CUmemGenericAllocationHandle handle) {
  CUdeviceptr va = h->va_base + (CUdeviceptr)pe * h->heap_bytes;
  CU_TRY(drv().MemMap(va, h->heap_bytes, 0, handle, 0));
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = h->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CU_TRY(drv().MemSetAccess(va, h->heap_bytes, &acc, 1));
  h->base[pe] = reinterpret_cast<char*>(va);
  h->mapped[pe] = true;
  return BSHMEM_OK;
}

}  // namespace

int heap_create(int my_pe, int n_pes, uint64_t heap_bytes, int device, int mode, Heap** out) {
  if (!out || n_pes < 1 || n_pes > BSHMEM_MAX_PES || my_pe < 0 || my_pe >= n_pes) return BSHMEM_ERR_INVALID;
  RT_TRY(cudaSetDevice(device));
  RT_TRY(cudaFree(nullptr));   // make sure the primary context exists
  Heap* h = new Heap();
  h->my_pe = my_pe; h->n_pes = n_pes; h->device = device; h->mode = mode;
  if (heap_bytes < BSHMEM_INTERNAL_BYTES * 2) heap_bytes = BSHMEM_INTERNAL_BYTES * 2;
  if (mode == HEAP_VMM) {
    if (!drv().ok) { delete h; heap_error() = "CUDA VMM driver entry points unavailable"; return BSHMEM_ERR_UNSUPPORTED; }
    CUmemAllocationProp prop = alloc_prop(device);
    size_t gran = 0;
    CUresult r = drv().MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
    if (r != CUDA_SUCCESS) { delete h; return cu_fail("cuMemGetAllocationGranularity", r); }
    if (gran < (2u << 20)) gran = 2u << 20;
    h->heap_bytes = (heap_bytes + gran - 1) / gran * gran;
    h->granularity = gran;
    r = drv().MemAddressReserve(&h->va_base, h->heap_bytes * (uint64_t)n_pes, gran, 0, 0);
    if (r != CUDA_SUCCESS) { delete h; return cu_fail("cuMemAddressReserve", r); }
    r = drv().MemCreate(&h->handles[my_pe], h->heap_bytes, &prop, 0);
    if (r != CUDA_SUCCESS) {
      drv().MemAddressFree(h->va_base, h->heap_bytes * (uint64_t)n_pes);
      delete h;
      return cu_fail("cuMemCreate", r);
    }
    h->own_handle[my_pe] = true;
    int rc = map_at(h, my_pe, h->handles[my_pe]);
    if (rc != BSHMEM_OK) { heap_destroy(h); return rc; }
  } else {
    h->heap_bytes = (heap_bytes + (2u << 20) - 1) / (2u << 20) * (2u << 20);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, h->heap_bytes);
    if (e != cudaSuccess) { delete h; return rt_fail("cudaMalloc(heap)", e); }
    h->base[my_pe] = static_cast<char*>(p);
    h->mapped[my_pe] = true;
  }
  // The internal region (flags, epochs) must start at zero.
  cudaError_t e = cudaMemset(h->base[my_pe], 0, BSHMEM_INTERNAL_BYTES);
  if (e != cudaSuccess) { heap_destroy(h); return rt_fail("cudaMemset(internal region)", e); }
  RT_TRY(cudaDeviceSynchronize());
  *out = h;
  return BSHMEM_OK;
}

int heap_export_fd(Heap* h, int* fd) {
  if (!h || h->mode != HEAP_VMM || !fd) return BSHMEM_ERR_INVALID;
  int out = -1;
  CU_TRY(drv().MemExportToShareableHandle(&out, h->handles[h->my_pe], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *fd = out;
  return BSHMEM_OK;
}

int heap_import_fd(Heap* h, int pe, int fd) {
  if (!h || h->mode != HEAP_VMM || pe < 0 || pe >= h->n_pes || pe == h->my_pe) return BSHMEM_ERR_INVALID;
  CU_TRY(drv().MemImportFromShareableHandle(&h->handles[pe], (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  h->own_handle[pe] = true;
  return map_at(h, pe, h->handles[pe]);
}

int heap_export_ipc(Heap* h, void* handle64) {
  if (!h || h->mode != HEAP_IPC || !handle64) return BSHMEM_ERR_INVALID;
  cudaIpcMemHandle_t ih;
  RT_TRY(cudaIpcGetMemHandle(&ih, h->base[h->my_pe]));
  memcpy(handle64, &ih, sizeof(ih));
  return BSHMEM_OK;
}

int heap_import_ipc(Heap* h, int pe, const void* handle64) {
  if (!h || h->mode != HEAP_IPC || pe < 0 || pe >= h->n_pes || pe == h->my_pe) return BSHMEM_ERR_INVALID;
  cudaIpcMemHandle_t ih;
  memcpy(&ih, handle64, sizeof(ih));
  void* p = nullptr;
  RT_TRY(cudaIpcOpenMemHandle(&p, ih, cudaIpcMemLazyEnablePeerAccess));
  h->base[pe] = static_cast<char*>(p);
  h->mapped[pe] = true;
  h->ipc_opened[pe] = true;
  return BSHMEM_OK;
}

// All PEs of a group live in this process on one device (single-GPU emulation of a
// multi-PE job for tests): n allocations, one shared base table.
int heap_create_local_group(int n_pes, uint64_t heap_bytes, int device, Heap** out /*[n_pes]*/) {
  if (!out || n_pes < 1 || n_pes > BSHMEM_MAX_PES) return BSHMEM_ERR_INVALID;
  RT_TRY(cudaSetDevice(device));
  if (heap_bytes < BSHMEM_INTERNAL_BYTES * 2) heap_bytes = BSHMEM_INTERNAL_BYTES * 2;
  uint64_t hb = (heap_bytes + (2u << 20) - 1) / (2u << 20) * (2u << 20);
  char* all = nullptr;
  RT_TRY(cudaMalloc(&all, hb * (uint64_t)n_pes));
  RT_TRY(cudaMemset(all, 0, hb * (uint64_t)n_pes));
  RT_TRY(cudaDeviceSynchronize());
  for (int p = 0; p < n_pes; ++p) {
    Heap* h = new Heap();
    h->my_pe = p; h->n_pes = n_pes; h->device = device; h->mode = HEAP_LOCAL_GROUP;
    h->heap_bytes = hb;
    for (int q = 0; q < n_pes; ++q) { h->base[q] = all + (uint64_t)q * hb; h->mapped[q] = true; }
    h->group_alloc = (p == 0) ? all : nullptr;
    out[p] = h;
  }
  return BSHMEM_OK;
}

// ---- NVLink multicast (NVLS) -----------------------------------------------------------------
int heap_multicast_supported(int device) {
  if (!drv().ok || !drv().MulticastCreate) return 0;
  int v = 0;
  if (drv().DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device) != CUDA_SUCCESS) return 0;
  return v;
}

static CUmulticastObjectProp mc_prop(Heap* h) {
  CUmulticastObjectProp p;
  memset(&p, 0, sizeof(p));
  p.numDevices = h->n_pes;
  p.size = h->heap_bytes;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

// PE 0 creates the multicast object and exports it; the others import the descriptor.
int heap_multicast_create(Heap* h, int* fd) {
  if (!h || h->mode != HEAP_VMM || !heap_multicast_supported(h->device)) return BSHMEM_ERR_UNSUPPORTED;
  CUmulticastObjectProp p = mc_prop(h);
  size_t gran = 0;
  CU_TRY(drv().MulticastGetGranularity(&gran, &p, CU_MULTICAST_GRANULARITY_MINIMUM));
  if (h->heap_bytes % gran) {
    heap_error() = "heap size " + std::to_string(h->heap_bytes) + " is not a multiple of the multicast granularity " + std::to_string(gran);
    return BSHMEM_ERR_UNSUPPORTED;
  }
  CU_TRY(drv().MulticastCreate(&h->mc_handle, &p));
  h->mc_created = true;
  int out = -1;
  CU_TRY(drv().MemExportToShareableHandle(&out, h->mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *fd = out;
  return BSHMEM_OK;
}

int heap_multicast_import(Heap* h, int fd) {
  if (!h || h->mode != HEAP_VMM) return BSHMEM_ERR_UNSUPPORTED;
  CU_TRY(drv().MemImportFromShareableHandle(&h->mc_handle, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  h->mc_created = true;
  return BSHMEM_OK;
}

// Every PE: add its device (all PEs must have done so before anyone binds), then bind + map.
int heap_multicast_add_device(Heap* h) {
  if (!h || !h->mc_created) return BSHMEM_ERR_STATE;
  CU_TRY(drv().MulticastAddDevice(h->mc_handle, h->device));
  return BSHMEM_OK;
}

int heap_multicast_bind(Heap* h) {
  if (!h || !h->mc_created) return BSHMEM_ERR_STATE;
  CU_TRY(drv().MulticastBindMem(h->mc_handle, 0, h->handles[h->my_pe], 0, h->heap_bytes, 0));
  CU_TRY(drv().MemAddressReserve(&h->mc_va, h->heap_bytes, h->granularity, 0, 0));
  CU_TRY(drv().MemMap(h->mc_va, h->heap_bytes, 0, h->mc_handle, 0));
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = h->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CU_TRY(drv().MemSetAccess(h->mc_va, h->heap_bytes, &acc, 1));
  h->mc_base = reinterpret_cast<char*>(h->mc_va);
  return BSHMEM_OK;
}

int heap_destroy(Heap* h) {
  if (!h) return BSHMEM_OK;
  cudaSetDevice(h->device);
  cudaDeviceSynchronize();
  if (h->mode == HEAP_VMM) {
    if (h->mc_base) { drv().MemUnmap(h->mc_va, h->heap_bytes); drv().MemAddressFree(h->mc_va, h->heap_bytes); }
    if (h->mc_created) drv().MemRelease(h->mc_handle);
    for (int p = 0; p < h->n_pes; ++p) {
      if (h->mapped[p]) drv().MemUnmap(h->va_base + (CUdeviceptr)p * h->heap_bytes, h->heap_bytes);
      if (h->own_handle[p]) drv().MemRelease(h->handles[p]);
    }
    if (h->va_base) drv().MemAddressFree(h->va_base, h->heap_bytes * (uint64_t)h->n_pes);
  } else if (h->mode == HEAP_IPC) {
    for (int p = 0; p < h->n_pes; ++p)
      if (h->ipc_opened[p]) cudaIpcCloseMemHandle(h->base[p]);
    if (h->base[h->my_pe]) cudaFree(h->base[h->my_pe]);
  } else if (h->mode == HEAP_LOCAL_GROUP) {
    if (h->group_alloc) cudaFree(h->group_alloc);
  }
  delete h;
  return BSHMEM_OK;
}

}  // namespace gpu
}  // namespace bshmem
