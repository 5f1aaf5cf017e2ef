// Reductions (allreduce, reduce-scatter) on bf16 and fp16, accumulated in fp32.
#define COLL_UNIT f16
#define COLL_TYPES(X) X(BSHMEM_BF16, __nv_bfloat16) X(BSHMEM_FP16, __half)
#include "coll_kernels_impl.cuh"
