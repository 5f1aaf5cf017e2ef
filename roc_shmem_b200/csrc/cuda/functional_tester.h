// functional_tester.h — what the translation units of the functional test driver share: the argument block of every
// test kernel and the launcher of the collective kernels (which live in their own unit so that the register budget of
// the reduction body is set by their 256-thread launch bound alone).
#pragma once
#include <cuda_runtime.h>

#include "../include/bshmem_coll.cuh"

namespace bshmem {
namespace ft {

struct FtArgs {
  int type, loops, skip, peer;       // peer: relative to the context's team
  unsigned long long size;           // message bytes (element count x 4 for the typed collectives)
  char* sym_a;                       // symmetric: remote side of put / get, collective source
  char* sym_b;                       // symmetric: collective destination
  char* local;                       // this PE's private buffer (source of put, destination of get)
  unsigned long long* words;         // symmetric: AMO targets, flags, signals (>= 2 * wgs * wg_size + 64 words)
  unsigned long long* timers;        // device: [wgs]
  int* status;                       // device: first error code
  long ctx_options;
  int initiator;                     // ping-pong and put-with-signal: 1 on the PE that sends first
};

inline __device__ void ft_fail(const FtArgs& a, int rc) { if (rc != BSHMEM_OK) atomicCAS(a.status, 0, rc); }

// kind: 0 reduction (float sum), 1 broadcast from PE 0, 2 fcollect, 3 alltoall; one work-group of <= 256 threads.
// Enqueues a.skip untimed and a.loops timed launches; `timed_from` is recorded before the first timed one and
// timers[0] (zeroed by the caller) receives the sum of the timed calls' device times.
void launch_coll(int kind, int wg_size, cudaStream_t stream, cudaEvent_t timed_from, const dev::State& s, const dev::Team& t,
                 const FtArgs& a);

}  // namespace ft
}  // namespace bshmem
