/* bshmem_gpu.h — C entry points of the NVLink (GPU) runtime library.
 *
 * Bring-up order for one PE per process:
 *   heap_create → export descriptor → (exchange through the bootstrap) → import every
 *   peer → [multicast create/import → add_device → barrier → bind] → gpu_init.
 * For single-GPU tests a "local group" puts all PEs of a job into one process on
 * one device; their collectives run as ONE cooperative launch (group_collective).
 */
#ifndef BSHMEM_GPU_H_
#define BSHMEM_GPU_H_

#include "bshmem.h"
#include "bshmem_device.cuh"

enum {
  BSHMEM_COLL_SYNC = 0,
  BSHMEM_COLL_BARRIER = 1,
  BSHMEM_COLL_BROADCAST = 2,
  BSHMEM_COLL_REDUCE = 3,
  BSHMEM_COLL_REDUCE_SCATTER = 4,
  BSHMEM_COLL_FCOLLECT = 5,
  BSHMEM_COLL_ALLTOALL = 6,
  BSHMEM_COLL_EXCHANGE = 7,
  BSHMEM_COLL_REDUCE_ROOT = 8
};

#ifdef __cplusplus
extern "C" {
#endif

const char* bshmem_gpu_last_error(void);
/* mode: 0 = CUDA VMM (fd-shareable), 1 = cudaMalloc + cudaIpc handles */
int bshmem_gpu_heap_create(int my_pe, int n_pes, uint64_t heap_bytes, int device, int mode, void** heap);
int bshmem_gpu_heap_create_local_group(int n_pes, uint64_t heap_bytes, int device, void** heaps);
int bshmem_gpu_heap_export_fd(void* heap, int* fd);
int bshmem_gpu_heap_import_fd(void* heap, int pe, int fd);
int bshmem_gpu_heap_export_ipc(void* heap, void* handle64);
int bshmem_gpu_heap_import_ipc(void* heap, int pe, const void* handle64);
int bshmem_gpu_multicast_supported(int device);
int bshmem_gpu_multicast_create(void* heap, int* fd);
int bshmem_gpu_multicast_import(void* heap, int fd);
int bshmem_gpu_multicast_add_device(void* heap);
int bshmem_gpu_multicast_bind(void* heap);
int bshmem_gpu_heap_destroy(void* heap);
uint64_t bshmem_gpu_heap_bytes(void* heap);

int bshmem_gpu_init(void* heap, const bshmem_config_t* cfg, int coll_ctas, int own_heap, bshmem_handle_t* out);
int bshmem_gpu_set_stream(bshmem_handle_t h, void* stream);
int bshmem_gpu_get_stream(bshmem_handle_t h, void** stream);
int bshmem_gpu_get_device(bshmem_handle_t h, int* device);
int bshmem_gpu_bind_thread_ctx(bshmem_handle_t h, int ctx);
int bshmem_gpu_synchronize(bshmem_handle_t h);
int bshmem_gpu_set_blocking(bshmem_handle_t h, int blocking);
/* micro-benchmarks and device-API test kernels (p2p_kernels.cu); times in ns from %globaltimer */
int bshmem_gpu_bench_pingpong(bshmem_handle_t h, void* flag_sym, int peer, int iters, int initiator, uint64_t* ns);
int bshmem_gpu_bench_put_signal(bshmem_handle_t h, void* data_sym, void* sig_sym, uint64_t nbytes, int peer, int iters,
                                int initiator, int threads, uint64_t* ns);
int bshmem_gpu_bench_amo(bshmem_handle_t h, void* target_sym, int peer, int iters, int op, uint64_t* ns);
int bshmem_gpu_bench_msgrate(bshmem_handle_t h, void* dest_sym, const void* src, uint64_t size, int peer, int windows,
                             int ctas, int threads, uint64_t* ns);
int bshmem_gpu_bench_amo_rate(bshmem_handle_t h, void* target_sym, int words, int peer, int iters, int ctas, int threads, uint64_t* ns);
int bshmem_gpu_put_signal_stream(bshmem_handle_t h, void* data_sym, const void* src, void* sig_sym, uint64_t nbytes, int peer,
                                 int iters, int ctas, int threads);
int bshmem_gpu_swarm_get(bshmem_handle_t h, void* local, const void* sym, uint64_t size, int peer, int ctas, int threads);
int bshmem_gpu_api_selftest(bshmem_handle_t h, void* sym_i, void* sym_u, void* sym_f, int peer, int* results_dev);
int bshmem_gpu_api_matrix(bshmem_handle_t h, void* ring_dev, int team_slot, void* sym_i, void* sym_u, void* sym_f, void* data_sym,
                          void* local_dev, void* coll_sym, int nbytes, int peer, int* results_dev);
int bshmem_gpu_wg_collectives(bshmem_handle_t h, void* dst_sym, void* src_sym, int n, int* status_out);
/* One launch of the functional test driver's kernel for test `type` (numbers as in roc_shmem_b200/bench/functional.py). */
int bshmem_gpu_functional_run(bshmem_handle_t h, int type, int team_slot, int peer, int wgs, int wg_size, int loops, int skip,
                              uint64_t size, void* sym_a, void* sym_b, void* local_dev, void* words, void* timers_dev, int* status_dev,
                              long ctx_options, int initiator, unsigned n_bins, float* kernel_ms);
int bshmem_gpu_set_coll_ctas(bshmem_handle_t h, int n);
int bshmem_gpu_set_nvls(bshmem_handle_t h, int on);
int bshmem_gpu_get_state(bshmem_handle_t h, bshmem_dev_state_t* out);
int bshmem_gpu_check_error(bshmem_handle_t h);
int bshmem_gpu_get_device_stats(bshmem_handle_t h, uint64_t* out, int n);
int bshmem_gpu_reset_device_stats(bshmem_handle_t h);
/* Device timeline (event ring behind the counters): capacity 0 = off, at most BSHMEM_TRACE_MAX_EVENTS. */
int bshmem_gpu_trace_enable(bshmem_handle_t h, int capacity);
int bshmem_gpu_trace_read(bshmem_handle_t h, uint64_t* out, int max_events, int* n_out, uint64_t* total);
int bshmem_gpu_rma_kernel(bshmem_handle_t h, void* sym, void* local, uint64_t n, int pe, int is_put, int scope,
                          int ctas, int threads);
int bshmem_gpu_group_collective(bshmem_handle_t* handles, int n, int team_slot, int kind, int dtype, int op, int root,
                                uint64_t dst_off, uint64_t src_off, uint64_t count, int ctas);
int bshmem_gpu_group_team_split(bshmem_handle_t* handles, int n, int parent_slot, int start, int stride, int size,
                                int* out_slots);

#ifdef __cplusplus
}
#endif
#endif /* BSHMEM_GPU_H_ */
