// typed_api.cc — expands the type tables of bshmem_typed.h into C symbols.
// Each wrapper forwards to the generic, handle-taking entry of bshmem.h using
// the calling thread's current handle.  Parity: the per-type macro expansion
// in library/src/roc_shmem.cpp:758-1246.
#include <cstring>

#include "../include/bshmem_typed.h"

namespace {
inline bshmem_handle_t cur() { return bshmem_get_current(); }
template <typename T> inline uint64_t bits(T v) { uint64_t b = 0; memcpy(&b, &v, sizeof(T)); return b; }
template <typename T> inline T unbits(uint64_t b) { T v; memcpy(&v, &b, sizeof(T)); return v; }
template <typename T> inline T amo_fetching(bshmem_ctx_t c, int dtype, int op, T* dest, T value, T cond, int pe) {
  uint64_t f = 0;
  bshmem_ctx_amo(cur(), c, dtype, op, dest, bits(value), bits(cond), pe, &f);
  return unbits<T>(f);
}
}  // namespace

extern "C" {

int bshmem_putmem(void* d, const void* s, size_t n, int pe) { return bshmem_ctx_putmem(cur(), BSHMEM_CTX_DEFAULT, d, s, n, pe); }
int bshmem_getmem(void* d, const void* s, size_t n, int pe) { return bshmem_ctx_getmem(cur(), BSHMEM_CTX_DEFAULT, d, s, n, pe); }
int bshmem_putmem_nbi(void* d, const void* s, size_t n, int pe) { return bshmem_ctx_putmem_nbi(cur(), BSHMEM_CTX_DEFAULT, d, s, n, pe); }
int bshmem_getmem_nbi(void* d, const void* s, size_t n, int pe) { return bshmem_ctx_getmem_nbi(cur(), BSHMEM_CTX_DEFAULT, d, s, n, pe); }
int bshmem_putmem_signal(void* d, const void* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) {
  return bshmem_ctx_putmem_signal(cur(), BSHMEM_CTX_DEFAULT, d, s, n, sig, v, op, pe);
}
int bshmem_fence(void) { return bshmem_ctx_fence(cur(), BSHMEM_CTX_DEFAULT); }
int bshmem_quiet(void) { return bshmem_ctx_quiet(cur(), BSHMEM_CTX_DEFAULT); }

#define DEF_RMA(T, N, D)                                                                                   \
  int bshmem_ctx_##N##_put(bshmem_ctx_t c, T* d, const T* s, size_t n, int pe) { return bshmem_ctx_putmem(cur(), c, d, s, n * sizeof(T), pe); } \
  int bshmem_ctx_##N##_get(bshmem_ctx_t c, T* d, const T* s, size_t n, int pe) { return bshmem_ctx_getmem(cur(), c, d, s, n * sizeof(T), pe); } \
  int bshmem_ctx_##N##_put_nbi(bshmem_ctx_t c, T* d, const T* s, size_t n, int pe) { return bshmem_ctx_putmem_nbi(cur(), c, d, s, n * sizeof(T), pe); } \
  int bshmem_ctx_##N##_get_nbi(bshmem_ctx_t c, T* d, const T* s, size_t n, int pe) { return bshmem_ctx_getmem_nbi(cur(), c, d, s, n * sizeof(T), pe); } \
  int bshmem_ctx_##N##_p(bshmem_ctx_t c, T* d, T v, int pe) { return bshmem_ctx_putmem_nbi(cur(), c, d, &v, sizeof(T), pe); } \
  T bshmem_ctx_##N##_g(bshmem_ctx_t c, const T* s, int pe) { T v = (T)0; bshmem_ctx_getmem(cur(), c, &v, s, sizeof(T), pe); return v; } \
  int bshmem_##N##_put(T* d, const T* s, size_t n, int pe) { return bshmem_ctx_##N##_put(BSHMEM_CTX_DEFAULT, d, s, n, pe); } \
  int bshmem_##N##_get(T* d, const T* s, size_t n, int pe) { return bshmem_ctx_##N##_get(BSHMEM_CTX_DEFAULT, d, s, n, pe); } \
  int bshmem_##N##_put_nbi(T* d, const T* s, size_t n, int pe) { return bshmem_ctx_##N##_put_nbi(BSHMEM_CTX_DEFAULT, d, s, n, pe); } \
  int bshmem_##N##_get_nbi(T* d, const T* s, size_t n, int pe) { return bshmem_ctx_##N##_get_nbi(BSHMEM_CTX_DEFAULT, d, s, n, pe); } \
  int bshmem_##N##_p(T* d, T v, int pe) { return bshmem_ctx_##N##_p(BSHMEM_CTX_DEFAULT, d, v, pe); }       \
  T bshmem_##N##_g(const T* s, int pe) { return bshmem_ctx_##N##_g(BSHMEM_CTX_DEFAULT, s, pe); }           \
  int bshmem_##N##_wait_until(T* ivar, int cmp, T v) { return bshmem_wait_until(cur(), D, ivar, cmp, bits(v)); } \
  int bshmem_##N##_test(T* ivar, int cmp, T v) { int r = 0; bshmem_test(cur(), D, ivar, cmp, bits(v), &r); return r; } \
  int bshmem_##N##_broadcast(bshmem_team_t t, T* d, const T* s, size_t n, int root) { return bshmem_team_broadcast(cur(), t, d, s, n * sizeof(T), root); } \
  int bshmem_##N##_fcollect(bshmem_team_t t, T* d, const T* s, size_t n) { return bshmem_team_fcollect(cur(), t, d, s, n * sizeof(T)); } \
  int bshmem_##N##_alltoall(bshmem_team_t t, T* d, const T* s, size_t n) { return bshmem_team_alltoall(cur(), t, d, s, n * sizeof(T)); } \
  int bshmem_ctx_##N##_put_signal(bshmem_ctx_t c, T* d, const T* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { return bshmem_ctx_putmem_signal(cur(), c, d, s, n * sizeof(T), sig, v, op, pe); } \
  int bshmem_ctx_##N##_put_signal_nbi(bshmem_ctx_t c, T* d, const T* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { return bshmem_ctx_putmem_signal_nbi(cur(), c, d, s, n * sizeof(T), sig, v, op, pe); } \
  int bshmem_##N##_put_signal(T* d, const T* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { return bshmem_ctx_##N##_put_signal(BSHMEM_CTX_DEFAULT, d, s, n, sig, v, op, pe); } \
  int bshmem_##N##_put_signal_nbi(T* d, const T* s, size_t n, uint64_t* sig, uint64_t v, int op, int pe) { return bshmem_ctx_##N##_put_signal_nbi(BSHMEM_CTX_DEFAULT, d, s, n, sig, v, op, pe); }
BSHMEM_RMA_TYPES(DEF_RMA)

#define DEF_AMO_STD(T, N, D)                                                                                        \
  T bshmem_ctx_##N##_atomic_fetch_add(bshmem_ctx_t c, T* d, T v, int pe) { return amo_fetching<T>(c, D, BSHMEM_AMO_FETCH_ADD, d, v, (T)0, pe); } \
  T bshmem_ctx_##N##_atomic_fetch_inc(bshmem_ctx_t c, T* d, int pe) { return amo_fetching<T>(c, D, BSHMEM_AMO_FETCH_INC, d, (T)0, (T)0, pe); }    \
  T bshmem_ctx_##N##_atomic_compare_swap(bshmem_ctx_t c, T* d, T cond, T v, int pe) { return amo_fetching<T>(c, D, BSHMEM_AMO_FETCH_CSWAP, d, v, cond, pe); } \
  int bshmem_ctx_##N##_atomic_add(bshmem_ctx_t c, T* d, T v, int pe) { return bshmem_ctx_amo(cur(), c, D, BSHMEM_AMO_ADD, d, bits(v), 0, pe, nullptr); } \
  int bshmem_ctx_##N##_atomic_inc(bshmem_ctx_t c, T* d, int pe) { return bshmem_ctx_amo(cur(), c, D, BSHMEM_AMO_INC, d, 0, 0, pe, nullptr); }   \
  T bshmem_##N##_atomic_fetch_add(T* d, T v, int pe) { return bshmem_ctx_##N##_atomic_fetch_add(BSHMEM_CTX_DEFAULT, d, v, pe); }                \
  T bshmem_##N##_atomic_fetch_inc(T* d, int pe) { return bshmem_ctx_##N##_atomic_fetch_inc(BSHMEM_CTX_DEFAULT, d, pe); }                        \
  T bshmem_##N##_atomic_compare_swap(T* d, T cond, T v, int pe) { return bshmem_ctx_##N##_atomic_compare_swap(BSHMEM_CTX_DEFAULT, d, cond, v, pe); } \
  int bshmem_##N##_atomic_add(T* d, T v, int pe) { return bshmem_ctx_##N##_atomic_add(BSHMEM_CTX_DEFAULT, d, v, pe); }                          \
  int bshmem_##N##_atomic_inc(T* d, int pe) { return bshmem_ctx_##N##_atomic_inc(BSHMEM_CTX_DEFAULT, d, pe); }
BSHMEM_AMO_STD_TYPES(DEF_AMO_STD)

#define DEF_AMO_EXT(T, N, D)                                                                                       \
  T bshmem_ctx_##N##_atomic_fetch(bshmem_ctx_t c, T* s, int pe) { return amo_fetching<T>(c, D, BSHMEM_AMO_FETCH, s, (T)0, (T)0, pe); } \
  int bshmem_ctx_##N##_atomic_set(bshmem_ctx_t c, T* d, T v, int pe) { return bshmem_ctx_amo(cur(), c, D, BSHMEM_AMO_SET, d, bits(v), 0, pe, nullptr); } \
  T bshmem_ctx_##N##_atomic_swap(bshmem_ctx_t c, T* d, T v, int pe) { return amo_fetching<T>(c, D, BSHMEM_AMO_SWAP, d, v, (T)0, pe); } \
  T bshmem_##N##_atomic_fetch(T* s, int pe) { return bshmem_ctx_##N##_atomic_fetch(BSHMEM_CTX_DEFAULT, s, pe); }   \
  int bshmem_##N##_atomic_set(T* d, T v, int pe) { return bshmem_ctx_##N##_atomic_set(BSHMEM_CTX_DEFAULT, d, v, pe); } \
  T bshmem_##N##_atomic_swap(T* d, T v, int pe) { return bshmem_ctx_##N##_atomic_swap(BSHMEM_CTX_DEFAULT, d, v, pe); }
BSHMEM_AMO_EXT_TYPES(DEF_AMO_EXT)

#define DEF_AMO_BIT(T, N, D)                                                                                            \
  T bshmem_##N##_atomic_fetch_and(T* d, T v, int pe) { return amo_fetching<T>(BSHMEM_CTX_DEFAULT, D, BSHMEM_AMO_FETCH_AND, d, v, (T)0, pe); } \
  T bshmem_##N##_atomic_fetch_or(T* d, T v, int pe) { return amo_fetching<T>(BSHMEM_CTX_DEFAULT, D, BSHMEM_AMO_FETCH_OR, d, v, (T)0, pe); }   \
  T bshmem_##N##_atomic_fetch_xor(T* d, T v, int pe) { return amo_fetching<T>(BSHMEM_CTX_DEFAULT, D, BSHMEM_AMO_FETCH_XOR, d, v, (T)0, pe); } \
  int bshmem_##N##_atomic_and(T* d, T v, int pe) { return bshmem_ctx_amo(cur(), BSHMEM_CTX_DEFAULT, D, BSHMEM_AMO_AND, d, bits(v), 0, pe, nullptr); } \
  int bshmem_##N##_atomic_or(T* d, T v, int pe) { return bshmem_ctx_amo(cur(), BSHMEM_CTX_DEFAULT, D, BSHMEM_AMO_OR, d, bits(v), 0, pe, nullptr); }   \
  int bshmem_##N##_atomic_xor(T* d, T v, int pe) { return bshmem_ctx_amo(cur(), BSHMEM_CTX_DEFAULT, D, BSHMEM_AMO_XOR, d, bits(v), 0, pe, nullptr); }
BSHMEM_AMO_BIT_TYPES(DEF_AMO_BIT)

#define DEF_RED_ONE(T, N, D, OPN, OPE)                                                                              \
  int bshmem_##N##_##OPN##_reduce(bshmem_team_t t, T* d, const T* s, size_t n) { return bshmem_team_reduce(cur(), t, D, OPE, d, s, n); } \
  int bshmem_##N##_##OPN##_to_all(T* d, const T* s, size_t n, int st, int ls, int sz, T* pwrk, long* psync) {       \
    return bshmem_to_all(cur(), D, OPE, d, s, n, st, ls, sz, pwrk, psync);                                          \
  }
#define DEF_RED_ARITH(T, N, D) \
  DEF_RED_ONE(T, N, D, sum, BSHMEM_SUM) DEF_RED_ONE(T, N, D, min, BSHMEM_MIN) DEF_RED_ONE(T, N, D, max, BSHMEM_MAX) DEF_RED_ONE(T, N, D, prod, BSHMEM_PROD)
#define DEF_RED_BIT(T, N, D) \
  DEF_RED_ONE(T, N, D, and, BSHMEM_AND) DEF_RED_ONE(T, N, D, or, BSHMEM_OR) DEF_RED_ONE(T, N, D, xor, BSHMEM_XOR)
BSHMEM_REDUCE_INT_TYPES(DEF_RED_ARITH)
BSHMEM_REDUCE_INT_TYPES(DEF_RED_BIT)
BSHMEM_REDUCE_FP_TYPES(DEF_RED_ARITH)

}  // extern "C"
