// Reductions (allreduce, reduce-scatter) on 1- and 2-byte integers.
#define COLL_UNIT i8
#define COLL_TYPES(X) X(BSHMEM_INT8, int8_t) X(BSHMEM_UINT8, uint8_t) X(BSHMEM_INT16, int16_t) X(BSHMEM_UINT16, uint16_t)
#include "coll_kernels_impl.cuh"
