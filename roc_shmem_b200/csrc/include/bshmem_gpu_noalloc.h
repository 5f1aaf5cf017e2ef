/* bshmem_gpu_noalloc.h — a group collective that allocates nothing.
 *
 * This entry point has no counterpart in the reference.
 *
 * bshmem_gpu_group_collective() builds a small table of per-PE state on the device for
 * every call, with cudaMalloc before the launch and cudaFree after it.  Some callers
 * must not allocate: code that runs between other frameworks' stream-ordered work and
 * cannot afford the device-wide synchronisation an allocation implies, latency-critical
 * serving loops whose memory budget was fixed at start-up, and hosts that run with a
 * capped or fully pre-reserved device heap where a late cudaMalloc simply fails.  For
 * them this variant keeps the table in a fixed array that is part of the library image:
 *
 *   - the array is 4 KiB per GPU, holds the table for at most BSHMEM_MAX_PES (16) PEs,
 *     and stays resident on every GPU that loads the library until the process exits;
 *   - the call performs no cudaMalloc / cudaFree and calls no allocating library routine;
 *     inputs and outputs are still the caller's symmetric buffers, named by heap offset
 *     exactly as for bshmem_gpu_group_collective();
 *   - more than 16 PEs is rejected with BSHMEM_ERR_LIMIT and a message available from
 *     bshmem_gpu_noalloc_last_error();
 *   - the array belongs to the CURRENT device, which therefore has to be the device the
 *     group's heaps live on (anything else is refused with BSHMEM_ERR_STATE); offsets and
 *     counts that leave the symmetric heap are refused with BSHMEM_ERR_RANGE, and the
 *     number of CTAs is capped at BSHMEM_MAX_COLL_CTAS;
 *   - the first call on a device looks the array's device address up (once per device,
 *     with that device current).  Make that first call outside any stream capture;
 *   - the status word is read back on the PE's own stream, so the call synchronises
 *     with that stream only;
 *   - every call on a device reuses the same array and it keeps the previous call's
 *     contents, so the entry rewrites the table and clears the status word each time.
 *     Two calls that overlap on the GPU (different streams, or different host threads
 *     driving the same device) would race on it: serialise them.
 *
 * Arguments are those of bshmem_gpu_group_collective(): the group's runtime handles, the
 * team slot, the collective kind (BSHMEM_COLL_*), element type / operator / root where they
 * apply, symmetric heap offsets of destination and source, the count (elements for
 * reductions, bytes otherwise) and the number of CTAs per PE.
 */
#ifndef BSHMEM_GPU_NOALLOC_H_
#define BSHMEM_GPU_NOALLOC_H_

#include "bshmem_gpu.h"

#define BSHMEM_NOALLOC_MAX_PES BSHMEM_MAX_PES
#define BSHMEM_NOALLOC_SCRATCH_BYTES 4096

#ifdef __cplusplus
extern "C" {
#endif

int bshmem_gpu_group_collective_noalloc(bshmem_handle_t* handles, int n, int team_slot, int kind, int dtype, int op,
                                        int root, uint64_t dst_off, uint64_t src_off, uint64_t count, int ctas);
const char* bshmem_gpu_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* BSHMEM_GPU_NOALLOC_H_ */
