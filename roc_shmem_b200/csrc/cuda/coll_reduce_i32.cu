// Reductions (allreduce, reduce-scatter) on 4- and 8-byte integers.
#define COLL_UNIT i32
#define COLL_TYPES(X) X(BSHMEM_INT32, int32_t) X(BSHMEM_UINT32, uint32_t) X(BSHMEM_INT64, long long) X(BSHMEM_UINT64, unsigned long long)
#include "coll_kernels_impl.cuh"
