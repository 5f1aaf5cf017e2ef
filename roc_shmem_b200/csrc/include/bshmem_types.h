/* bshmem_types.h — enums and plain-old-data shared by the host runtime, the
 * device API and the Python layer.
 *
 * API-shape parity with the reference's public header
 * (library/include/roc_shmem.hpp:52-130): comparison constants, thread levels,
 * context option bits, collective scratch sizes, opaque ctx/team handles.
 * Everything here is C so that ctypes, g++ and nvcc all read the same file.
 */
#ifndef BSHMEM_TYPES_H_
#define BSHMEM_TYPES_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- limits ------------------------------------------------------------ */
#define BSHMEM_MAX_PES 16            /* one NVSwitch node (8) with head-room     */
#define BSHMEM_MAX_TEAMS 40          /* incl. TEAM_WORLD in slot 0 (team_tracker) */
#define BSHMEM_MAX_CTXS 40           /* host contexts per PE                      */
#define BSHMEM_MAX_COLL_CTAS 160     /* CTAs per PE taking part in one collective */
#define BSHMEM_ALIGNMENT 128         /* smallest heap block, bytes                */

/* ---- status codes (every call returns one; nothing aborts) -------------- */
typedef enum {
  BSHMEM_OK = 0,
  BSHMEM_ERR_INVALID = 1,   /* bad argument                                  */
  BSHMEM_ERR_NOMEM = 2,     /* symmetric heap exhausted                      */
  BSHMEM_ERR_TIMEOUT = 3,   /* a bounded wait ran out                        */
  BSHMEM_ERR_RANGE = 4,     /* address not inside the symmetric heap         */
  BSHMEM_ERR_STATE = 5,     /* not initialised / already finalised           */
  BSHMEM_ERR_LIMIT = 6,     /* out of team / context slots                   */
  BSHMEM_ERR_CUDA = 7,      /* a CUDA call failed (see last_error string)    */
  BSHMEM_ERR_UNSUPPORTED = 8,
  BSHMEM_ERR_ABORTED = 9,   /* another PE called global_exit                 */
  BSHMEM_ERR_PEER_DEAD = 10 /* a peer was marked failed by the host          */
} bshmem_status_t;

/* ---- comparison operators for wait_until / test ------------------------- */
typedef enum {
  BSHMEM_CMP_EQ = 0,
  BSHMEM_CMP_NE = 1,
  BSHMEM_CMP_GT = 2,
  BSHMEM_CMP_GE = 3,
  BSHMEM_CMP_LT = 4,
  BSHMEM_CMP_LE = 5
} bshmem_cmp_t;

/* ---- thread levels ------------------------------------------------------ */
typedef enum {
  BSHMEM_THREAD_SINGLE = 0,
  BSHMEM_THREAD_FUNNELED = 1,
  BSHMEM_THREAD_WG_FUNNELED = 2,
  BSHMEM_THREAD_SERIALIZED = 3,
  BSHMEM_THREAD_MULTIPLE = 4
} bshmem_thread_level_t;

/* ---- context option bits (same values as the reference) ----------------- */
#define BSHMEM_CTX_ZERO 0L
#define BSHMEM_CTX_NOSTORE 1L     /* caller has no plain stores to publish  */
#define BSHMEM_CTX_SERIALIZED 2L
#define BSHMEM_CTX_WG_PRIVATE 4L  /* used by one thread block only          */
#define BSHMEM_CTX_PRIVATE BSHMEM_CTX_WG_PRIVATE  /* host side: used only by the thread that created it (refused from
                                                     any other thread when debug checks are on) */
#define BSHMEM_CTX_SHARED 8L      /* shareable between blocks (locks on)    */

/* ---- active-set scratch sizes (elements) -------------------------------- */
#define BSHMEM_REDUCE_MIN_WRKDATA_SIZE 1024
#define BSHMEM_ATA_MAX_WRKDATA_SIZE (4 * 1024 * 1024)
#define BSHMEM_BARRIER_SYNC_SIZE 256
#define BSHMEM_REDUCE_SYNC_SIZE 256
#define BSHMEM_BCAST_SYNC_SIZE 256
#define BSHMEM_SYNC_VALUE 0

/* ---- element types ------------------------------------------------------ */
typedef enum {
  BSHMEM_INT8 = 0,
  BSHMEM_UINT8 = 1,
  BSHMEM_INT16 = 2,
  BSHMEM_UINT16 = 3,
  BSHMEM_INT32 = 4,
  BSHMEM_UINT32 = 5,
  BSHMEM_INT64 = 6,
  BSHMEM_UINT64 = 7,
  BSHMEM_FLOAT = 8,
  BSHMEM_DOUBLE = 9,
  BSHMEM_BF16 = 10,
  BSHMEM_FP16 = 11,
  BSHMEM_DTYPE_COUNT = 12
} bshmem_dtype_t;

/* ---- reduction operators ------------------------------------------------ */
typedef enum {
  BSHMEM_SUM = 0,
  BSHMEM_MIN = 1,
  BSHMEM_MAX = 2,
  BSHMEM_PROD = 3,
  BSHMEM_AND = 4,
  BSHMEM_OR = 5,
  BSHMEM_XOR = 6
} bshmem_redop_t;

/* ---- atomic memory operations (the reference's 15 flavours) ------------- */
typedef enum {
  BSHMEM_AMO_FETCH_ADD = 0,
  BSHMEM_AMO_FETCH_INC = 1,
  BSHMEM_AMO_FETCH = 2,
  BSHMEM_AMO_FETCH_CSWAP = 3,
  BSHMEM_AMO_ADD = 4,
  BSHMEM_AMO_INC = 5,
  BSHMEM_AMO_CSWAP = 6,
  BSHMEM_AMO_SET = 7,
  BSHMEM_AMO_SWAP = 8,
  BSHMEM_AMO_FETCH_AND = 9,
  BSHMEM_AMO_FETCH_OR = 10,
  BSHMEM_AMO_FETCH_XOR = 11,
  BSHMEM_AMO_AND = 12,
  BSHMEM_AMO_OR = 13,
  BSHMEM_AMO_XOR = 14,
  BSHMEM_AMO_COUNT = 15
} bshmem_amo_t;

/* ---- signal operators for putmem_signal (OpenSHMEM 1.5 semantics) ------- */
typedef enum { BSHMEM_SIGNAL_SET = 0, BSHMEM_SIGNAL_ADD = 1 } bshmem_sigop_t;

/* ---- opaque handles ----------------------------------------------------- */
typedef int32_t bshmem_team_t;             /* slot index; -1 = invalid      */
#define BSHMEM_TEAM_WORLD ((bshmem_team_t)0)
#define BSHMEM_TEAM_INVALID ((bshmem_team_t)-1)

typedef int32_t bshmem_ctx_t;              /* host ctx index; 0 = default   */
#define BSHMEM_CTX_DEFAULT ((bshmem_ctx_t)0)
#define BSHMEM_CTX_INVALID ((bshmem_ctx_t)-1)

/* ---- error record written by a bounded device or host wait -------------- */
typedef struct {
  uint32_t code;      /* bshmem_status_t; 0 = no error recorded              */
  int32_t pe;         /* peer the wait was for, -1 if n/a                    */
  uint32_t where;     /* BSHMEM_WHERE_* site id                              */
  uint32_t count;     /* number of errors since the last clear               */
  uint64_t addr;      /* address (or heap offset) that was polled            */
  uint64_t expected;  /* value waited for                                    */
  uint64_t seen;      /* last value observed                                 */
} bshmem_error_record_t;

enum {
  BSHMEM_WHERE_NONE = 0,
  BSHMEM_WHERE_WAIT_UNTIL = 1,
  BSHMEM_WHERE_BARRIER = 2,
  BSHMEM_WHERE_COLL_SIGNAL = 3,
  BSHMEM_WHERE_PROXY_SLOT = 4,
  BSHMEM_WHERE_PROXY_DONE = 5,
  BSHMEM_WHERE_FUSED_CHUNK = 6,
  BSHMEM_WHERE_MOE_SIGNAL = 7,
  BSHMEM_WHERE_MBARRIER = 8,
  BSHMEM_WHERE_BOUNDS = 9,
  BSHMEM_WHERE_MUTEX = 10
};

#if defined(__CUDACC__)
__host__ __device__
#endif
static inline size_t bshmem_dtype_size(int dt) {
  switch (dt) {
    case BSHMEM_INT8: case BSHMEM_UINT8: return 1;
    case BSHMEM_INT16: case BSHMEM_UINT16: case BSHMEM_BF16: case BSHMEM_FP16: return 2;
    case BSHMEM_INT32: case BSHMEM_UINT32: case BSHMEM_FLOAT: return 4;
    case BSHMEM_INT64: case BSHMEM_UINT64: case BSHMEM_DOUBLE: return 8;
    default: return 0;
  }
}

#ifdef __cplusplus
}
#endif
#endif /* BSHMEM_TYPES_H_ */
