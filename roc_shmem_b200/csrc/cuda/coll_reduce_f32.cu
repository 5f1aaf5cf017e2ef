// Reductions (allreduce, reduce-scatter) on float and double.
#define COLL_UNIT f32
#define COLL_TYPES(X) X(BSHMEM_FLOAT, float) X(BSHMEM_DOUBLE, double)
#include "coll_kernels_impl.cuh"
