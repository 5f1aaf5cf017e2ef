/* bshmem_proxy.h — the reverse-offload command ring shared by the device
 * producers (bshmem_proxy_device.cuh), the host service thread (host/proxy.cc) and
 * host-side producers used in tests.
 *
 * A producer reserves a slot with a ticket — only while the ring has room, so a
 * producer that gives up on a full ring leaves no hole in the ticket sequence —
 * fills a 128-byte descriptor, publishes it by storing ticket+1 to the descriptor's
 * `valid` word (on its own cache line) and, for blocking operations, waits — bounded
 * — for the same value in the slot's completion word, reads the result word and
 * acknowledges in the slot's `consumed` word.  The consumer executes descriptors
 * strictly in ticket order, publishes its read index for back-pressure, and does not
 * overwrite a slot's result before the blocking producer that owned the slot one lap
 * earlier has acknowledged (or its wait has run out).
 *
 * Parity: library/src/reverse_offload/queue_proxy.hpp:40-131 (queue_element_t with
 * the valid flag on its own cache line, 512-slot rings), commands_types.hpp:29-48
 * (18 commands), queue_desc_proxy.hpp:30-57 (read/write indices and status words).
 * Differences: one ring per PE instead of one per work-group (tickets make slot
 * reservation lock-free), completion words per slot instead of per thread, and
 * every wait is bounded.
 */
#ifndef BSHMEM_PROXY_H_
#define BSHMEM_PROXY_H_

#include "bshmem_types.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  BSHMEM_PROXY_NOP = 0,
  BSHMEM_PROXY_PUT = 1,
  BSHMEM_PROXY_GET = 2,
  BSHMEM_PROXY_PUT_NBI = 3,
  BSHMEM_PROXY_GET_NBI = 4,
  BSHMEM_PROXY_P = 5,            /* value carried inline                       */
  BSHMEM_PROXY_G = 6,            /* result returned through the result word    */
  BSHMEM_PROXY_AMO = 7,          /* amo_op selects one of the 15 flavours      */
  BSHMEM_PROXY_PUT_SIGNAL = 8,
  BSHMEM_PROXY_FENCE = 9,
  BSHMEM_PROXY_QUIET = 10,
  BSHMEM_PROXY_BARRIER_ALL = 11,
  BSHMEM_PROXY_SYNC_ALL = 12,
  BSHMEM_PROXY_TEAM_SYNC = 13,
  BSHMEM_PROXY_TO_ALL = 14,
  BSHMEM_PROXY_BROADCAST = 15,
  BSHMEM_PROXY_ALLTOALL = 16,
  BSHMEM_PROXY_FCOLLECT = 17,
  BSHMEM_PROXY_FINALIZE = 18,
  BSHMEM_PROXY_OP_COUNT = 19
} bshmem_proxy_op_t;

#define BSHMEM_PROXY_FLAG_BLOCKING 1u      /* producer waits for the completion word   */
#define BSHMEM_PROXY_FLAG_SRC_IS_OFFSET 2u /* `local` is a heap offset, not a pointer  */

typedef struct {
  /* ---- the command (72 bytes) ---- */
  uint32_t op;          /* bshmem_proxy_op_t                                      */
  int32_t pe;           /* target PE (world numbering)                            */
  uint32_t dtype;       /* element type for AMO / P / G / reductions              */
  uint32_t sub_op;      /* AMO flavour, reduction operator, or signal operator    */
  uint64_t sym_off;     /* heap offset of the symmetric operand                   */
  uint64_t local;       /* local buffer: pointer or heap offset (see flags)       */
  uint64_t nbytes;      /* payload bytes / element count for reductions           */
  uint64_t value;       /* inline value (P, AMO operand, signal value)            */
  uint64_t cond;        /* AMO compare value / signal heap offset                 */
  uint32_t flags;
  int32_t team;         /* team slot for collectives                              */
  uint32_t root;
  uint32_t block_id;    /* producer's block, for statistics                       */
  /* ---- publication (second cache line of the 128-byte slot) ---- */
  uint64_t ticket;
  uint64_t pad[5];
  volatile uint64_t valid;   /* ticket + 1 once the command above is complete     */
} bshmem_proxy_desc_t;   /* 128 bytes */

typedef struct {
  uint64_t capacity;                 /* power of two                                    */
  bshmem_proxy_desc_t* slots;        /* [capacity], host memory visible to the producer */
  volatile uint64_t* completion;     /* [capacity]: ticket + 1 when executed            */
  volatile uint64_t* result;         /* [capacity]: fetched value / status              */
  volatile uint64_t* consumed;       /* [capacity]: ticket + 1 once a blocking producer has read its result */
  volatile uint64_t* read_index;     /* consumer progress, for back-pressure            */
  unsigned long long* write_index;   /* ticket counter in the producers' memory         */
  unsigned long long timeout_ns;
} bshmem_proxy_ring_t;

/* ---- host control of the service thread ------------------------------------------- */
typedef struct bshmem_proxy bshmem_proxy_t;

/* Ring in ordinary host memory, commands executed through the handle's own backend
 * (CPU backend, or any backend when the producers are host threads).               */
struct bshmem_runtime;
int bshmem_proxy_create_host(struct bshmem_runtime* h, uint64_t capacity, uint64_t timeout_us, bshmem_proxy_t** out);
int bshmem_proxy_set_timeout_us(bshmem_proxy_t* px, uint64_t timeout_us);

/* Host-side producer (CPU tests and CPU "proxy" mode): same protocol as the device code.
 * Returns BSHMEM_OK / BSHMEM_ERR_TIMEOUT; *result gets the fetched value if non-null.  */
int bshmem_proxy_host_submit(bshmem_proxy_t* px, const bshmem_proxy_desc_t* cmd, uint64_t* result);

/* Fault injection, host side only: pause the service thread / drop the next n commands
 * (they are consumed but neither executed nor completed).                              */
int bshmem_proxy_pause(bshmem_proxy_t* px, int paused);
int bshmem_proxy_drop_next(bshmem_proxy_t* px, int n);
int bshmem_proxy_get_counters(bshmem_proxy_t* px, uint64_t out[8]);
int bshmem_proxy_get_ring(bshmem_proxy_t* px, bshmem_proxy_ring_t* out);
int bshmem_proxy_stop(bshmem_proxy_t* px);

#ifdef __cplusplus
}
#endif
#endif /* BSHMEM_PROXY_H_ */
