// Collective kernels without arithmetic: sync, barrier, broadcast, fcollect, alltoall, host exchange.
#define COLL_UNIT move
#define COLL_UNIT_MOVE 1
#define COLL_TYPES(X)
#include "coll_kernels_impl.cuh"
