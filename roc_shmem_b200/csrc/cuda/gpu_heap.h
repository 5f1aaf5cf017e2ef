// gpu_heap.h — the GPU symmetric heap object shared by vmm_heap.cu (mapping) and
// gpu_backend.cu (transport).  See vmm_heap.cu for the design.
#pragma once
#include <cuda.h>
#include <stdint.h>

#include <string>

#include "../include/bshmem_types.h"

namespace bshmem {
namespace gpu {

enum HeapMode { HEAP_VMM = 0, HEAP_IPC = 1, HEAP_LOCAL_GROUP = 2 };

struct Heap {
  int my_pe = 0, n_pes = 1, device = 0, mode = HEAP_VMM;
  uint64_t heap_bytes = 0;
  size_t granularity = 0;
  CUdeviceptr va_base = 0;
  CUmemGenericAllocationHandle handles[BSHMEM_MAX_PES] = {};
  bool own_handle[BSHMEM_MAX_PES] = {};
  bool mapped[BSHMEM_MAX_PES] = {};
  bool ipc_opened[BSHMEM_MAX_PES] = {};
  char* base[BSHMEM_MAX_PES] = {};
  char* group_alloc = nullptr;
  // NVLink multicast
  CUmemGenericAllocationHandle mc_handle = 0;
  bool mc_created = false;
  CUdeviceptr mc_va = 0;
  char* mc_base = nullptr;
};

std::string& heap_error();
int heap_create(int my_pe, int n_pes, uint64_t heap_bytes, int device, int mode, Heap** out);
int heap_create_local_group(int n_pes, uint64_t heap_bytes, int device, Heap** out);
int heap_export_fd(Heap* h, int* fd);
int heap_import_fd(Heap* h, int pe, int fd);
int heap_export_ipc(Heap* h, void* handle64);
int heap_import_ipc(Heap* h, int pe, const void* handle64);
int heap_multicast_supported(int device);
int heap_multicast_create(Heap* h, int* fd);
int heap_multicast_import(Heap* h, int fd);
int heap_multicast_add_device(Heap* h);
int heap_multicast_bind(Heap* h);
int heap_destroy(Heap* h);

}  // namespace gpu
}  // namespace bshmem
