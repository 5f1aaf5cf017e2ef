/* bshmem.h — host-side public C API of the runtime.
 *
 * One PE (processing element) is one runtime handle.  On a GPU node that is one
 * process per GPU; with the CPU backend several PEs may live in one process as
 * threads, which is why every call takes the handle explicitly.  The typed,
 * handle-free OpenSHMEM-style names (bshmem_int_put, bshmem_long_sum_to_all,
 * ...) in bshmem_typed.h act on the calling thread's *current* handle.
 *
 * API-shape parity: library/include/roc_shmem.hpp:144-460 (host functions) and
 * library/src/roc_shmem.cpp (semantics: collective malloc = alloc + barrier,
 * free = barrier + release, finalize destroys leftover contexts and teams).
 * Additions the reference does not have: putmem_signal, reduce_scatter, host
 * alltoall/fcollect, bounded waits that return BSHMEM_ERR_TIMEOUT.
 *
 * Every function returns a bshmem_status_t unless stated otherwise.
 */
#ifndef BSHMEM_H_
#define BSHMEM_H_

#include "bshmem_types.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct bshmem_runtime* bshmem_handle_t;

typedef struct {
  uint64_t heap_bytes;       /* symmetric heap per PE (default 1 GiB)            */
  uint64_t timeout_us;       /* bound of every blocking wait (default 30 s)      */
  int32_t max_teams;         /* <= BSHMEM_MAX_TEAMS                              */
  int32_t max_ctxs;          /* <= BSHMEM_MAX_CTXS                               */
  int32_t debug;             /* bounds checks + verbose errors                   */
  int32_t profile;           /* count API calls                                  */
  int32_t requested_thread_level;
  int32_t reserved0;
} bshmem_config_t;

void bshmem_config_default(bshmem_config_t* cfg);

/* ---- CPU backend worlds (threads or processes over shared memory) -------- */
/* name == NULL: anonymous in-process world for thread PEs.  Otherwise a POSIX
 * shared-memory object of that name that other processes open.               */
int bshmem_cpu_world_create(const char* name, int n_pes, uint64_t heap_bytes, void** world);
int bshmem_cpu_world_open(const char* name, void** world);
int bshmem_cpu_world_destroy(void* world);
int bshmem_cpu_init(void* world, int pe, const bshmem_config_t* cfg, bshmem_handle_t* out);
/* Host-side fault injection: mark a PE failed so that peers' waits return
 * BSHMEM_ERR_PEER_DEAD instead of running into their timeout.                */
int bshmem_cpu_world_mark_dead(void* world, int pe);

/* ---- lifecycle ------------------------------------------------------------ */
int bshmem_finalize(bshmem_handle_t h);
int bshmem_query_thread(bshmem_handle_t h, int* provided);
int bshmem_my_pe(bshmem_handle_t h);            /* returns the PE number      */
int bshmem_n_pes(bshmem_handle_t h);            /* returns the PE count       */
int bshmem_global_exit(bshmem_handle_t h, int status);
const char* bshmem_last_error(bshmem_handle_t h);
int bshmem_get_error_record(bshmem_handle_t h, bshmem_error_record_t* out, int clear);
const char* bshmem_status_string(int status);
/* Bound of every blocking wait of this PE, host and device side. */
int bshmem_set_timeout_us(bshmem_handle_t h, uint64_t timeout_us);
uint64_t bshmem_get_timeout_us(bshmem_handle_t h);
void bshmem_set_current(bshmem_handle_t h);     /* thread-local default handle */
bshmem_handle_t bshmem_get_current(void);

/* ---- symmetric memory ------------------------------------------------------ */
void* bshmem_malloc(bshmem_handle_t h, size_t size);            /* collective */
void* bshmem_align(bshmem_handle_t h, size_t alignment, size_t size);
void* bshmem_calloc(bshmem_handle_t h, size_t count, size_t size);
int bshmem_free(bshmem_handle_t h, void* ptr);                  /* collective */
/* Non-collective forms (no barrier) for callers that synchronise themselves. */
void* bshmem_malloc_local(bshmem_handle_t h, size_t size, size_t alignment);
int bshmem_free_local(bshmem_handle_t h, void* ptr);
void* bshmem_ptr(bshmem_handle_t h, const void* dest, int pe);
void* bshmem_heap_base(bshmem_handle_t h);
uint64_t bshmem_heap_bytes(bshmem_handle_t h);
int bshmem_heap_usage(bshmem_handle_t h, uint64_t out[9]);
int bshmem_addr_accessible(bshmem_handle_t h, const void* addr, int pe);

/* ---- contexts -------------------------------------------------------------- */
int bshmem_ctx_create(bshmem_handle_t h, long options, bshmem_ctx_t* ctx);
int bshmem_team_create_ctx(bshmem_handle_t h, bshmem_team_t team, long options, bshmem_ctx_t* ctx);
int bshmem_ctx_destroy(bshmem_handle_t h, bshmem_ctx_t ctx);

/* ---- teams ----------------------------------------------------------------- */
int bshmem_team_split_strided(bshmem_handle_t h, bshmem_team_t parent, int start, int stride,
                              int size, bshmem_team_t* new_team);
int bshmem_team_destroy(bshmem_handle_t h, bshmem_team_t team);
int bshmem_team_n_pes(bshmem_handle_t h, bshmem_team_t team);   /* -1 if invalid */
int bshmem_team_my_pe(bshmem_handle_t h, bshmem_team_t team);   /* -1 if invalid */
int bshmem_team_translate_pe(bshmem_handle_t h, bshmem_team_t src, int src_pe, bshmem_team_t dst);

/* ---- RMA -------------------------------------------------------------------- */
int bshmem_ctx_putmem(bshmem_handle_t h, bshmem_ctx_t c, void* dest, const void* src, size_t n, int pe);
int bshmem_ctx_getmem(bshmem_handle_t h, bshmem_ctx_t c, void* dest, const void* src, size_t n, int pe);
int bshmem_ctx_putmem_nbi(bshmem_handle_t h, bshmem_ctx_t c, void* dest, const void* src, size_t n, int pe);
int bshmem_ctx_getmem_nbi(bshmem_handle_t h, bshmem_ctx_t c, void* dest, const void* src, size_t n, int pe);
int bshmem_ctx_putmem_signal(bshmem_handle_t h, bshmem_ctx_t c, void* dest, const void* src, size_t n,
                             uint64_t* sig_addr, uint64_t signal, int sig_op, int pe);
int bshmem_ctx_putmem_signal_nbi(bshmem_handle_t h, bshmem_ctx_t c, void* dest, const void* src, size_t n,
                                 uint64_t* sig_addr, uint64_t signal, int sig_op, int pe);
uint64_t bshmem_signal_fetch(bshmem_handle_t h, const uint64_t* sig_addr);

/* ---- atomics: one generic entry, typed wrappers in bshmem_typed.h ---------- */
/* value/cond/fetched carry the operand bit pattern in the low bytes.          */
int bshmem_ctx_amo(bshmem_handle_t h, bshmem_ctx_t c, int dtype, int op, void* dest, uint64_t value,
                   uint64_t cond, int pe, uint64_t* fetched);

/* ---- ordering / point-to-point sync ---------------------------------------- */
int bshmem_ctx_fence(bshmem_handle_t h, bshmem_ctx_t c);
int bshmem_ctx_quiet(bshmem_handle_t h, bshmem_ctx_t c);
int bshmem_wait_until(bshmem_handle_t h, int dtype, void* ivar, int cmp, uint64_t value);
int bshmem_test(bshmem_handle_t h, int dtype, void* ivar, int cmp, uint64_t value, int* result);

/* ---- collectives (team form) ------------------------------------------------ */
int bshmem_barrier_all(bshmem_handle_t h);
int bshmem_sync_all(bshmem_handle_t h);
int bshmem_team_sync(bshmem_handle_t h, bshmem_team_t team);
int bshmem_team_barrier(bshmem_handle_t h, bshmem_team_t team);
int bshmem_team_broadcast(bshmem_handle_t h, bshmem_team_t team, void* dest, const void* src,
                          size_t nbytes, int root);
int bshmem_team_reduce(bshmem_handle_t h, bshmem_team_t team, int dtype, int op, void* dest,
                       const void* src, size_t nelems);         /* allreduce */
/* rooted reduce: only member `root` of the team receives op over all members' src (the others' dest is untouched) */
int bshmem_team_reduce_root(bshmem_handle_t h, bshmem_team_t team, int dtype, int op, void* dest,
                            const void* src, size_t nelems, int root);
int bshmem_team_reduce_scatter(bshmem_handle_t h, bshmem_team_t team, int dtype, int op, void* dest,
                               const void* src, size_t nelems_per_pe);
int bshmem_team_fcollect(bshmem_handle_t h, bshmem_team_t team, void* dest, const void* src, size_t nbytes);
int bshmem_team_alltoall(bshmem_handle_t h, bshmem_team_t team, void* dest, const void* src, size_t nbytes);

/* ---- collectives (legacy active-set form; pSync holds BSHMEM_SYNC_VALUE
 *      before and after each call) ------------------------------------------- */
int bshmem_barrier(bshmem_handle_t h, int pe_start, int log_stride, int pe_size, long* psync);
int bshmem_sync(bshmem_handle_t h, int pe_start, int log_stride, int pe_size, long* psync);
int bshmem_broadcast(bshmem_handle_t h, void* dest, const void* src, size_t nbytes, int root,
                     int pe_start, int log_stride, int pe_size, long* psync);
int bshmem_to_all(bshmem_handle_t h, int dtype, int op, void* dest, const void* src, size_t nelems,
                  int pe_start, int log_stride, int pe_size, void* pwrk, long* psync);

/* ---- statistics -------------------------------------------------------------- */
int bshmem_stats_count(void);
const char* bshmem_stats_name(int idx);
int bshmem_get_stats(bshmem_handle_t h, uint64_t* out, int n);
int bshmem_reset_stats(bshmem_handle_t h);
int bshmem_dump_stats(bshmem_handle_t h);   /* prints a table to stdout */

#ifdef __cplusplus
}
#endif
#endif /* BSHMEM_H_ */
