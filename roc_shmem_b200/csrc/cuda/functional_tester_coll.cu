// functional_tester_coll.cu — the collective kernels of the functional test driver (types 5, 20-24, 36, 37): one
// work-group per PE calls the context form of the work-group collective once per launch; `skip` untimed launches are
// followed by `loops` timed ones.
// Parity: clients/functional_tests/reduction_tester.cpp:74-104, broadcast_tester.cpp, alltoall_tester.cpp,
// fcollect_tester.cpp and their team variants.
#include "functional_tester.h"

using namespace bshmem;
using dev::State;
using DTeam = bshmem::dev::Team;
using ft::FtArgs;
using ft::ft_fail;

namespace {

// ---- work-group collectives through a context (types 5, 20, 22, 23, 36, 37): one work-group per PE -----------------
// One call of the collective per launch; the host repeats the launch (untimed ones first) and the kernel adds the time
// of a timed call to timers[0].  (A kernel with several call sites of a reduction collective makes the compiler build
// the reduction body as a callable function with a small register budget, which spills; one call site does not.)
// kKind: 0 reduction, 1 broadcast, 2 fcollect, 3 alltoall.  The work-group is capped at 256 threads, as in the
// library's own collective kernels.
template <int kKind>
__global__ void __launch_bounds__(256) k_ft_coll(State s, DTeam team, FtArgs a) {
  __shared__ dev::Ctx ctx;
  dev::wg_team_create_ctx(s, team, a.ctx_options, &ctx);
  const size_t n = a.size / 4;
  const unsigned long long t0 = dev::timer();
  int rc;
  if (kKind == 0)
    rc = coll::ctx_wg_to_all<float>(s, ctx, BSHMEM_SUM, reinterpret_cast<float*>(a.sym_b), reinterpret_cast<const float*>(a.sym_a), n);
  else if (kKind == 1)
    rc = coll::ctx_wg_broadcast<int>(s, ctx, reinterpret_cast<int*>(a.sym_b), reinterpret_cast<const int*>(a.sym_a), n, 0);
  else if (kKind == 2)
    rc = coll::ctx_wg_fcollect<int>(s, ctx, reinterpret_cast<int*>(a.sym_b), reinterpret_cast<const int*>(a.sym_a), n);
  else
    rc = coll::ctx_wg_alltoall<int>(s, ctx, reinterpret_cast<int*>(a.sym_b), reinterpret_cast<const int*>(a.sym_a), n);
  if (threadIdx.x == 0) {
    if (a.skip == 0) a.timers[0] += dev::timer() - t0;
    ft_fail(a, rc);
  }
}

}  // namespace

namespace bshmem {
namespace ft {

void launch_coll(int kind, int wg_size, cudaStream_t stream, cudaEvent_t timed_from, const State& s, const DTeam& t, const FtArgs& args) {
  FtArgs a = args;
  for (int i = 0; i < args.skip + args.loops; ++i) {
    if (i == args.skip) cudaEventRecord(timed_from, stream);
    a.skip = i < args.skip ? 1 : 0;        // 1: an untimed call
    if (kind == 0) k_ft_coll<0><<<1, wg_size, 0, stream>>>(s, t, a);
    else if (kind == 1) k_ft_coll<1><<<1, wg_size, 0, stream>>>(s, t, a);
    else if (kind == 2) k_ft_coll<2><<<1, wg_size, 0, stream>>>(s, t, a);
    else k_ft_coll<3><<<1, wg_size, 0, stream>>>(s, t, a);
  }
}

}  // namespace ft
}  // namespace bshmem
