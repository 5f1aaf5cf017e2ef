/* bshmem_typed.h — the type-suffixed, handle-free OpenSHMEM-style host API.
 *
 * Every name is generated from the type tables below, so adding a type or an
 * operation is a one-line change.  The functions act on the calling thread's
 * current handle (bshmem_set_current); a PE thread sets it once after init.
 *
 * API-shape parity: the macro-generated families of
 * library/include/roc_shmem.hpp:837-1163 and their instantiations :1190-2020
 * (13 standard C types + 10 fixed-width aliases for RMA, the AMO type lists,
 * 7 reductions on integers and 4 on floating types).
 */
#ifndef BSHMEM_TYPED_H_
#define BSHMEM_TYPED_H_

#include "bshmem.h"

/* X(ctype, name, dtype enum) */
#define BSHMEM_RMA_TYPES(X)                       \
  X(float, float, BSHMEM_FLOAT)                   \
  X(double, double, BSHMEM_DOUBLE)                \
  X(char, char, BSHMEM_INT8)                      \
  X(signed char, schar, BSHMEM_INT8)              \
  X(short, short, BSHMEM_INT16)                   \
  X(int, int, BSHMEM_INT32)                       \
  X(long, long, BSHMEM_INT64)                     \
  X(long long, longlong, BSHMEM_INT64)            \
  X(unsigned char, uchar, BSHMEM_UINT8)           \
  X(unsigned short, ushort, BSHMEM_UINT16)        \
  X(unsigned int, uint, BSHMEM_UINT32)            \
  X(unsigned long, ulong, BSHMEM_UINT64)          \
  X(unsigned long long, ulonglong, BSHMEM_UINT64) \
  X(int8_t, int8, BSHMEM_INT8)                    \
  X(int16_t, int16, BSHMEM_INT16)                 \
  X(int32_t, int32, BSHMEM_INT32)                 \
  X(int64_t, int64, BSHMEM_INT64)                 \
  X(uint8_t, uint8, BSHMEM_UINT8)                 \
  X(uint16_t, uint16, BSHMEM_UINT16)              \
  X(uint32_t, uint32, BSHMEM_UINT32)              \
  X(uint64_t, uint64, BSHMEM_UINT64)              \
  X(size_t, size, BSHMEM_UINT64)                  \
  X(ptrdiff_t, ptrdiff, BSHMEM_INT64)

/* standard AMOs (add / inc / cswap families) */
#define BSHMEM_AMO_STD_TYPES(X)                   \
  X(int, int, BSHMEM_INT32)                       \
  X(long, long, BSHMEM_INT64)                     \
  X(long long, longlong, BSHMEM_INT64)            \
  X(unsigned int, uint, BSHMEM_UINT32)            \
  X(unsigned long, ulong, BSHMEM_UINT64)          \
  X(unsigned long long, ulonglong, BSHMEM_UINT64) \
  X(int32_t, int32, BSHMEM_INT32)                 \
  X(int64_t, int64, BSHMEM_INT64)                 \
  X(uint32_t, uint32, BSHMEM_UINT32)              \
  X(uint64_t, uint64, BSHMEM_UINT64)              \
  X(size_t, size, BSHMEM_UINT64)                  \
  X(ptrdiff_t, ptrdiff, BSHMEM_INT64)

/* extended AMOs (fetch / set / swap) additionally cover float and double */
#define BSHMEM_AMO_EXT_TYPES(X) \
  BSHMEM_AMO_STD_TYPES(X)       \
  X(float, float, BSHMEM_FLOAT) \
  X(double, double, BSHMEM_DOUBLE)

/* bitwise AMOs */
#define BSHMEM_AMO_BIT_TYPES(X)                   \
  X(unsigned int, uint, BSHMEM_UINT32)            \
  X(unsigned long, ulong, BSHMEM_UINT64)          \
  X(unsigned long long, ulonglong, BSHMEM_UINT64) \
  X(int32_t, int32, BSHMEM_INT32)                 \
  X(int64_t, int64, BSHMEM_INT64)                 \
  X(uint32_t, uint32, BSHMEM_UINT32)              \
  X(uint64_t, uint64, BSHMEM_UINT64)

#define BSHMEM_REDUCE_INT_TYPES(X)     \
  X(short, short, BSHMEM_INT16)        \
  X(int, int, BSHMEM_INT32)            \
  X(long, long, BSHMEM_INT64)          \
  X(long long, longlong, BSHMEM_INT64)

#define BSHMEM_REDUCE_FP_TYPES(X) \
  X(float, float, BSHMEM_FLOAT)   \
  X(double, double, BSHMEM_DOUBLE)

/* Y(name, op enum) */
#define BSHMEM_ARITH_OPS(Y) Y(sum, BSHMEM_SUM) Y(min, BSHMEM_MIN) Y(max, BSHMEM_MAX) Y(prod, BSHMEM_PROD)
#define BSHMEM_BIT_OPS(Y) Y(and, BSHMEM_AND) Y(or, BSHMEM_OR) Y(xor, BSHMEM_XOR)

#ifdef __cplusplus
extern "C" {
#endif

/* handle-free generic forms (default context) */
int bshmem_putmem(void* dest, const void* src, size_t n, int pe);
int bshmem_getmem(void* dest, const void* src, size_t n, int pe);
int bshmem_putmem_nbi(void* dest, const void* src, size_t n, int pe);
int bshmem_getmem_nbi(void* dest, const void* src, size_t n, int pe);
int bshmem_putmem_signal(void* dest, const void* src, size_t n, uint64_t* sig, uint64_t value, int sig_op, int pe);
int bshmem_fence(void);
int bshmem_quiet(void);

#define BSHMEM_DECL_RMA(T, N, D)                                                              \
  int bshmem_##N##_put(T* dest, const T* src, size_t nelems, int pe);                         \
  int bshmem_##N##_get(T* dest, const T* src, size_t nelems, int pe);                         \
  int bshmem_##N##_put_nbi(T* dest, const T* src, size_t nelems, int pe);                     \
  int bshmem_##N##_get_nbi(T* dest, const T* src, size_t nelems, int pe);                     \
  int bshmem_##N##_p(T* dest, T value, int pe);                                               \
  T bshmem_##N##_g(const T* src, int pe);                                                     \
  int bshmem_ctx_##N##_put(bshmem_ctx_t c, T* dest, const T* src, size_t nelems, int pe);     \
  int bshmem_ctx_##N##_get(bshmem_ctx_t c, T* dest, const T* src, size_t nelems, int pe);     \
  int bshmem_ctx_##N##_put_nbi(bshmem_ctx_t c, T* dest, const T* src, size_t nelems, int pe); \
  int bshmem_ctx_##N##_get_nbi(bshmem_ctx_t c, T* dest, const T* src, size_t nelems, int pe); \
  int bshmem_ctx_##N##_p(bshmem_ctx_t c, T* dest, T value, int pe);                           \
  T bshmem_ctx_##N##_g(bshmem_ctx_t c, const T* src, int pe);                                 \
  int bshmem_##N##_wait_until(T* ivar, int cmp, T value);                                     \
  int bshmem_##N##_test(T* ivar, int cmp, T value);                                           \
  int bshmem_##N##_broadcast(bshmem_team_t team, T* dest, const T* src, size_t nelems, int root); \
  int bshmem_##N##_fcollect(bshmem_team_t team, T* dest, const T* src, size_t nelems);        \
  int bshmem_##N##_alltoall(bshmem_team_t team, T* dest, const T* src, size_t nelems);        \
  /* put-with-signal, OpenSHMEM 1.5 (not in the reference): the signal update is visible after the data */ \
  int bshmem_##N##_put_signal(T* dest, const T* src, size_t nelems, uint64_t* sig_addr, uint64_t signal, int sig_op, int pe);     \
  int bshmem_##N##_put_signal_nbi(T* dest, const T* src, size_t nelems, uint64_t* sig_addr, uint64_t signal, int sig_op, int pe); \
  int bshmem_ctx_##N##_put_signal(bshmem_ctx_t c, T* dest, const T* src, size_t nelems, uint64_t* sig_addr, uint64_t signal, int sig_op, int pe); \
  int bshmem_ctx_##N##_put_signal_nbi(bshmem_ctx_t c, T* dest, const T* src, size_t nelems, uint64_t* sig_addr, uint64_t signal, int sig_op, int pe);
BSHMEM_RMA_TYPES(BSHMEM_DECL_RMA)
#undef BSHMEM_DECL_RMA

#define BSHMEM_DECL_AMO_STD(T, N, D)                                         \
  T bshmem_##N##_atomic_fetch_add(T* dest, T value, int pe);                 \
  T bshmem_##N##_atomic_fetch_inc(T* dest, int pe);                          \
  T bshmem_##N##_atomic_compare_swap(T* dest, T cond, T value, int pe);      \
  int bshmem_##N##_atomic_add(T* dest, T value, int pe);                     \
  int bshmem_##N##_atomic_inc(T* dest, int pe);                              \
  T bshmem_ctx_##N##_atomic_fetch_add(bshmem_ctx_t c, T* dest, T value, int pe);            \
  T bshmem_ctx_##N##_atomic_fetch_inc(bshmem_ctx_t c, T* dest, int pe);                     \
  T bshmem_ctx_##N##_atomic_compare_swap(bshmem_ctx_t c, T* dest, T cond, T value, int pe); \
  int bshmem_ctx_##N##_atomic_add(bshmem_ctx_t c, T* dest, T value, int pe);                \
  int bshmem_ctx_##N##_atomic_inc(bshmem_ctx_t c, T* dest, int pe);
BSHMEM_AMO_STD_TYPES(BSHMEM_DECL_AMO_STD)
#undef BSHMEM_DECL_AMO_STD

#define BSHMEM_DECL_AMO_EXT(T, N, D)                                  \
  T bshmem_##N##_atomic_fetch(T* src, int pe);                        \
  int bshmem_##N##_atomic_set(T* dest, T value, int pe);              \
  T bshmem_##N##_atomic_swap(T* dest, T value, int pe);               \
  T bshmem_ctx_##N##_atomic_fetch(bshmem_ctx_t c, T* src, int pe);    \
  int bshmem_ctx_##N##_atomic_set(bshmem_ctx_t c, T* dest, T value, int pe); \
  T bshmem_ctx_##N##_atomic_swap(bshmem_ctx_t c, T* dest, T value, int pe);
BSHMEM_AMO_EXT_TYPES(BSHMEM_DECL_AMO_EXT)
#undef BSHMEM_DECL_AMO_EXT

#define BSHMEM_DECL_AMO_BIT(T, N, D)                              \
  T bshmem_##N##_atomic_fetch_and(T* dest, T value, int pe);      \
  T bshmem_##N##_atomic_fetch_or(T* dest, T value, int pe);       \
  T bshmem_##N##_atomic_fetch_xor(T* dest, T value, int pe);      \
  int bshmem_##N##_atomic_and(T* dest, T value, int pe);          \
  int bshmem_##N##_atomic_or(T* dest, T value, int pe);           \
  int bshmem_##N##_atomic_xor(T* dest, T value, int pe);
BSHMEM_AMO_BIT_TYPES(BSHMEM_DECL_AMO_BIT)
#undef BSHMEM_DECL_AMO_BIT

/* reductions: team form  bshmem_<type>_<op>_reduce(team, dest, src, n)
 *             active set bshmem_<type>_<op>_to_all(dest, src, n, start, logstride, size, pWrk, pSync) */
#define BSHMEM_DECL_RED_ONE(T, N, OPN)                                                      \
  int bshmem_##N##_##OPN##_reduce(bshmem_team_t team, T* dest, const T* src, size_t nreduce); \
  int bshmem_##N##_##OPN##_to_all(T* dest, const T* src, size_t nreduce, int pe_start,      \
                                  int log_stride, int pe_size, T* pwrk, long* psync);
#define BSHMEM_DECL_RED_ARITH(T, N, D) \
  BSHMEM_DECL_RED_ONE(T, N, sum) BSHMEM_DECL_RED_ONE(T, N, min) BSHMEM_DECL_RED_ONE(T, N, max) BSHMEM_DECL_RED_ONE(T, N, prod)
#define BSHMEM_DECL_RED_BIT(T, N, D) \
  BSHMEM_DECL_RED_ONE(T, N, and) BSHMEM_DECL_RED_ONE(T, N, or) BSHMEM_DECL_RED_ONE(T, N, xor)
BSHMEM_REDUCE_INT_TYPES(BSHMEM_DECL_RED_ARITH)
BSHMEM_REDUCE_INT_TYPES(BSHMEM_DECL_RED_BIT)
BSHMEM_REDUCE_FP_TYPES(BSHMEM_DECL_RED_ARITH)
#undef BSHMEM_DECL_RED_ARITH
#undef BSHMEM_DECL_RED_BIT
#undef BSHMEM_DECL_RED_ONE

#ifdef __cplusplus
}
#endif
#endif /* BSHMEM_TYPED_H_ */
