// bshmem_coll.cuh — device collectives over peer-mapped heaps.
//
// Every routine is a *block collective*: all threads of the calling block take
// part, and the block identifies itself as channel `cta` of `ncta` so that a
// host-launched kernel can stripe one collective over many CTAs (channel c of PE
// i only ever synchronises with channel c of the other PEs).  A user kernel that
// calls them roc_shmem-style from one block passes cta = 0, ncta = 1.
//
// NVSwitch gives every pair of GPUs full bandwidth, so all algorithms are direct
// (one hop): barrier = all-to-all epoch flags; allreduce = one-shot pull for small
// vectors, two-shot (reduce my slice from all peers, push the result to all peers)
// for large ones; reduce-scatter = the first half of that; fcollect / alltoall =
// direct pushes; broadcast = pull from the root.  With an NVLink multicast mapping
// the allreduce can instead use multimem.ld_reduce / multimem.st.
//
// Parity: library/src/gpu_ib/context_ib_device_coll.cpp:30-120 (barriers),
// context_ib_tmpl_device.hpp:120-307 (direct and ring allreduce, selection),
// :455-519 (broadcast), :521-558 (alltoall), :836-876 (fcollect).  Unlike the
// reference's reset-to-zero flags (context_ib_device_coll.cpp:38-52), barrier
// flags carry a monotonically increasing epoch, which is safe for back-to-back
// collectives; the log-step variants (Bruck, gcen) are not needed on a full mesh.
#pragma once
#include <type_traits>

#include "bshmem_device.cuh"

#ifdef __CUDACC__
namespace bshmem {
namespace coll {

using dev::State;
using dev::Team;

__device__ __forceinline__ uint64_t* flag_addr(const State& s, int pe, int slot, int cta, int src_idx) {
  return reinterpret_cast<uint64_t*>(s.heap_base[pe] + BSHMEM_OFF_FLAGS) +
         ((size_t)slot * BSHMEM_MAX_COLL_CTAS + cta) * BSHMEM_MAX_PES + src_idx;
}
__device__ __forceinline__ uint64_t* epoch_addr(const State& s, int slot, int cta) {
  return reinterpret_cast<uint64_t*>(s.heap_base[s.my_pe] + BSHMEM_OFF_EPOCHS) + (size_t)slot * BSHMEM_MAX_COLL_CTAS + cta;
}

// Active-set sync on the caller's pSync (single block per PE): members count in on the
// first member's pSync[0]; that member resets the counter and releases everyone through
// pSync[1], which each member resets itself, so both words end at BSHMEM_SYNC_VALUE.
// (Same protocol as the flat barrier of context_ib_device_coll.cpp:30-55.)
__device__ __forceinline__ int active_set_sync(const State& s, const Team& t) {
  __shared__ int as_status;
  if (threadIdx.x == 0) as_status = BSHMEM_OK;
  __syncthreads();
  if (threadIdx.x == 0) {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    int root = dev::team_pe(t, 0);
    unsigned long long* root_count = reinterpret_cast<unsigned long long*>(dev::ptr(s, t.psync, root));
    atomicAdd_system(root_count, 1ull);
    if (t.my_idx == 0) {
      int rc = dev::wait_until<uint64_t>(s, reinterpret_cast<const uint64_t*>(t.psync), BSHMEM_CMP_EQ, (uint64_t)t.size,
                                         BSHMEM_WHERE_BARRIER, -1);
      if (rc == BSHMEM_OK) {
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(t.psync), "l"((uint64_t)BSHMEM_SYNC_VALUE) : "memory");
        for (int i = 1; i < t.size; ++i) {
          long* rel = dev::ptr(s, t.psync, dev::team_pe(t, i)) + 1;
          asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(rel), "l"(1ull) : "memory");
        }
      } else {
        as_status = rc;
      }
    } else {
      int rc = dev::wait_until<uint64_t>(s, reinterpret_cast<const uint64_t*>(t.psync + 1), BSHMEM_CMP_EQ, 1ull,
                                         BSHMEM_WHERE_BARRIER, root);
      if (rc == BSHMEM_OK)
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(t.psync + 1), "l"((uint64_t)BSHMEM_SYNC_VALUE) : "memory");
      else
        as_status = rc;
    }
  }
  __syncthreads();
  int rc = as_status;
  __syncthreads();
  return rc;
}

// sync: every member's channel `cta` has arrived.  Does not complete RMA by itself,
// but publishes the calling block's earlier stores (fence before the flag stores).
// Returns BSHMEM_OK or BSHMEM_ERR_TIMEOUT (same value in every thread of the block).
// World team with an NVLink multicast mapping: every PE adds 1 to channel `cta`'s counter in ALL heaps with one
// multimem.red (the switch replicates it) and waits until its own copy has counted every member of this epoch.
// One store per PE instead of size-1 flag stores; counters are monotonic.
__device__ __forceinline__ int team_sync_mc(const State& s, const Team& t, int cta) {
  __shared__ int mc_status;
  unsigned long long t0 = s.stats ? dev::timer() : 0;
  __syncthreads();                       // all stores of the block precede the release below
  if (threadIdx.x == 0) {
    unsigned long long* ep = reinterpret_cast<unsigned long long*>(s.heap_base[s.my_pe] + BSHMEM_OFF_MCBAR) + BSHMEM_MAX_COLL_CTAS + cta;
    const unsigned long long epoch = *ep + 1;
    const uint64_t off = BSHMEM_OFF_MCBAR + (uint64_t)cta * 8;
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    asm volatile("multimem.red.release.sys.global.add.u64 [%0], %1;" ::"l"(s.mc_base + off), "l"(1ull) : "memory");
    mc_status = dev::wait_until<uint64_t>(s, reinterpret_cast<const uint64_t*>(s.heap_base[s.my_pe] + off), BSHMEM_CMP_GE,
                                          epoch * (uint64_t)t.size, BSHMEM_WHERE_BARRIER, -1);
    *ep = epoch;
    if (s.stats) {
      dev::stat(s, BSHMEM_DSTAT_BARRIER);
      dev::stat(s, BSHMEM_DSTAT_BARRIER_NS, dev::timer() - t0);
      dev::trace(s, BSHMEM_TRACE_BARRIER, s.my_pe, dev::timer() - t0);
    }
  }
  __syncthreads();
  int rc = mc_status;
  __syncthreads();
  return rc;
}

__device__ __forceinline__ int team_sync(const State& s, const Team& t, int cta = 0) {
  if (t.slot < 0) return active_set_sync(s, t);
  if (t.slot == 0 && t.size == s.n_pes && s.mc_base != nullptr && s.n_pes > 1) return team_sync_mc(s, t, cta);
  __shared__ int sync_status;
  const int tid = threadIdx.x;
  unsigned long long t0 = s.stats ? dev::timer() : 0;
  if (tid == 0) sync_status = BSHMEM_OK;
  __syncthreads();                       // all stores of the block precede the release below
  uint64_t epoch = *epoch_addr(s, t.slot, cta) + 1;
  if (tid < t.size) {
    // release pattern: one system fence per signalling thread, then the flag.  The block barrier above makes every
    // thread's earlier stores (remote ones included) precede this fence, so they are visible to whoever sees the flag.
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    uint64_t* remote = flag_addr(s, dev::team_pe(t, tid), t.slot, cta, t.my_idx);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(remote), "l"(epoch) : "memory");
    const uint64_t* mine = flag_addr(s, s.my_pe, t.slot, cta, tid);
    int rc = dev::wait_until<uint64_t>(s, mine, BSHMEM_CMP_GE, epoch, BSHMEM_WHERE_BARRIER, dev::team_pe(t, tid));
    if (rc != BSHMEM_OK) sync_status = rc;
  }
  __syncthreads();
  if (tid == 0) {
    *epoch_addr(s, t.slot, cta) = epoch;
    if (s.stats) {
      dev::stat(s, BSHMEM_DSTAT_BARRIER);
      dev::stat(s, BSHMEM_DSTAT_BARRIER_NS, dev::timer() - t0);
      dev::trace(s, BSHMEM_TRACE_BARRIER, s.my_pe, dev::timer() - t0);
    }
  }
  int rc = sync_status;
  __syncthreads();
  return rc;
}
// barrier = quiet + sync.  The sync's own release (block barrier, then a system fence by each signalling thread before
// its flag store) already orders every earlier store of the calling block, puts to peers included, before the flags;
// a second fence by all threads of the block would only add system-scope fences that contend across blocks.
__device__ __forceinline__ int team_barrier(const State& s, const Team& t, int cta = 0) {
  return team_sync(s, t, cta);
}
__device__ __forceinline__ int wg_barrier_all(const State& s) { return team_barrier(s, dev::team_world(s)); }
__device__ __forceinline__ int wg_sync_all(const State& s) { return team_sync(s, dev::team_world(s)); }
__device__ __forceinline__ int wg_team_sync(const State& s, const Team& t) { return team_sync(s, t); }

// ---- element-wise reduction on 16-byte vectors ------------------------------------------------
template <typename T> struct Acc { using type = T; };
template <> struct Acc<__nv_bfloat16> { using type = float; };
template <> struct Acc<__half> { using type = float; };

template <typename A> __device__ __forceinline__ A apply(int op, A a, A b) {
  if constexpr (std::is_floating_point<A>::value) {
    switch (op) {
      case BSHMEM_SUM: return a + b;
      case BSHMEM_MIN: return b < a ? b : a;
      case BSHMEM_MAX: return b > a ? b : a;
      default: return a * b;
    }
  } else {
    switch (op) {
      case BSHMEM_SUM: return (A)(a + b);
      case BSHMEM_MIN: return b < a ? b : a;
      case BSHMEM_MAX: return b > a ? b : a;
      case BSHMEM_PROD: return (A)(a * b);
      case BSHMEM_AND: return (A)(a & b);
      case BSHMEM_OR: return (A)(a | b);
      default: return (A)(a ^ b);
    }
  }
}
template <typename T> __device__ __forceinline__ typename Acc<T>::type to_acc(T v) { return (typename Acc<T>::type)v; }
template <> __device__ __forceinline__ float to_acc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_acc<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_acc(typename Acc<T>::type v) { return (T)v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_acc<__half>(float v) { return __float2half_rn(v); }

template <typename T> union Vec16 {
  uint4 raw;
  T e[16 / sizeof(T)];
};

// 16-byte vectors [v0, v1) of the reduction, striped over the block.  NS bounds the member count at compile
// time, U vectors per thread form a batch: all U x nsrc loads of a batch are issued before its first use, and the
// NEXT batch's loads are issued before the current batch is reduced and stored (two register sets), so a thread
// keeps up to 2 x U x nsrc 16-byte loads in flight across loop iterations.
template <typename T, int NS, int U>
__device__ __forceinline__ void reduce_vec_load(Vec16<T> (&in)[U][NS], const uint4* const (&sp)[NS], int nsrc, size_t base, size_t v1) {
  const size_t tid = threadIdx.x, nth = blockDim.x;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const size_t v = base + u * nth + tid;
    if (v < v1) {
#pragma unroll
      for (int k = 0; k < NS; ++k)
        if (k < nsrc) in[u][k].raw = sp[k][v];
    }
  }
}
template <typename T, int OP, int NS, int U>
__device__ __forceinline__ void reduce_vec_store(const Vec16<T> (&in)[U][NS], int nsrc, int ndst, T* const* dsts, size_t base, size_t v1) {
  using A = typename Acc<T>::type;
  constexpr int VE = 16 / sizeof(T);
  const size_t tid = threadIdx.x, nth = blockDim.x;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const size_t v = base + u * nth + tid;
    if (v < v1) {
      A acc[VE];
#pragma unroll
      for (int e = 0; e < VE; ++e) acc[e] = to_acc<T>(in[u][0].e[e]);
#pragma unroll
      for (int k = 1; k < NS; ++k) {
        if (k < nsrc) {
#pragma unroll
          for (int e = 0; e < VE; ++e) acc[e] = apply<A>(OP, acc[e], to_acc<T>(in[u][k].e[e]));
        }
      }
      Vec16<T> out;
#pragma unroll
      for (int e = 0; e < VE; ++e) out.e[e] = from_acc<T>(acc[e]);
      for (int d = 0; d < ndst; ++d) reinterpret_cast<uint4*>(dsts[d])[v] = out.raw;
    }
  }
}
template <typename T, int OP, int NS, int U>
__device__ __forceinline__ void reduce_vec_body(int nsrc, const T* const* srcs, int ndst, T* const* dsts, size_t v0, size_t v1) {
  const size_t step = (size_t)U * blockDim.x;
  const uint4* sp[NS];
#pragma unroll
  for (int k = 0; k < NS; ++k) sp[k] = reinterpret_cast<const uint4*>(srcs[k < nsrc ? k : 0]);
  if (v0 >= v1) return;
  Vec16<T> a[U][NS], b[U][NS];
  reduce_vec_load<T, NS, U>(a, sp, nsrc, v0, v1);
  for (size_t base = v0; base < v1; base += 2 * step) {
    if (base + step < v1) reduce_vec_load<T, NS, U>(b, sp, nsrc, base + step, v1);
    reduce_vec_store<T, OP, NS, U>(a, nsrc, ndst, dsts, base, v1);
    if (base + step >= v1) break;
    if (base + 2 * step < v1) reduce_vec_load<T, NS, U>(a, sp, nsrc, base + 2 * step, v1);
    reduce_vec_store<T, OP, NS, U>(b, nsrc, ndst, dsts, base + step, v1);
  }
}

// ---- large reductions through shared memory with bulk async copies ------------------------------------------------
// Plain loads are bounded by the outstanding-miss capacity of an SM's load/store unit: about 1.3 TB/s of local HBM
// and a few hundred GB/s over NVLink (3 us latency) however many loads a thread keeps in flight.  Here one thread
// fetches a chunk of EVERY source with cp.async.bulk (global -> shared, mbarrier completion; sources may be peer
// memory, nothing is multicast) into a ring of kBulkStages stages, all threads reduce the stage out of shared memory
// and write the result with ordinary (fire-and-forget) stores to the ndst destinations.
constexpr int kBulkStages = 3;
constexpr uint32_t kBulkStageBytes = 48 * 1024;
constexpr uint32_t kBulkSmemBytes = kBulkStages * kBulkStageBytes + 64;   // + mbarriers
// Range [begin, end) in elements, both multiples of 16 / sizeof(T); every pointer 16-byte aligned.  Returns false if
// a bounded wait ran out (the error record is filled).
template <typename T, int OP>
__device__ __forceinline__ bool reduce_bulk(const State& s, int nsrc, const T* const* srcs, int ndst, T* const* dsts, size_t begin,
                                            size_t end, char* smem) {
  using A = typename Acc<T>::type;
  constexpr int VE = 16 / sizeof(T);
  __shared__ int bulk_ok;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBulkStages * kBulkStageBytes);
  const uint32_t chunk = (kBulkStageBytes / nsrc) & ~127u;            // bytes per source and stage
  const size_t bytes = (end - begin) * sizeof(T);
  const size_t nchunks = (bytes + chunk - 1) / chunk;
  if (threadIdx.x == 0) {
    bulk_ok = 1;
    for (int i = 0; i < kBulkStages; ++i)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&bars[i])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  auto issue = [&](size_t c) {           // thread 0: chunk c of every source into stage c % kBulkStages
    const int st = (int)(c % kBulkStages);
    const uint32_t nb = (uint32_t)((c + 1) * (size_t)chunk <= bytes ? chunk : bytes - c * (size_t)chunk);
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&bars[st]);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(nb * (uint32_t)nsrc) : "memory");
    for (int k = 0; k < nsrc; ++k) {
      const uint32_t sm = (uint32_t)__cvta_generic_to_shared(smem + (size_t)st * kBulkStageBytes + (size_t)k * chunk);
      const char* g = reinterpret_cast<const char*>(srcs[k] + begin) + c * (size_t)chunk;
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(sm), "l"(g), "r"(nb), "r"(bar) : "memory");
    }
  };
  if (threadIdx.x == 0)
    for (size_t c = 0; c < nchunks && c < (size_t)kBulkStages; ++c) issue(c);
  const unsigned long long t0 = dev::timer();
  for (size_t c = 0; c < nchunks; ++c) {
    const int st = (int)(c % kBulkStages);
    const uint32_t parity = (uint32_t)((c / kBulkStages) & 1);
    const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&bars[st]);
    uint32_t done = 0, it = 0;
    while (true) {
      asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                   : "=r"(done) : "r"(bar), "r"(parity) : "memory");
      if (done) break;
      if ((++it & 63) == 0 && (bulk_ok == 0 || dev::timer() - t0 > s.timeout_ns)) {
        if (bulk_ok != 0 && threadIdx.x == 0) dev::record_error(s, BSHMEM_ERR_TIMEOUT, -1, BSHMEM_WHERE_MBARRIER, (uint64_t)srcs[0], c, 0);
        bulk_ok = 0;
        break;
      }
    }
    __syncthreads();                       // bulk_ok is the same for everybody from here
    if (!bulk_ok) break;
    const uint32_t nb = (uint32_t)((c + 1) * (size_t)chunk <= bytes ? chunk : bytes - c * (size_t)chunk);
    const char* stage = smem + (size_t)st * kBulkStageBytes;
    const size_t v_base = (begin * sizeof(T) + c * (size_t)chunk) >> 4;          // 16-byte vector index in the tensors
    for (uint32_t v = threadIdx.x; v < (nb >> 4); v += blockDim.x) {
      Vec16<T> in, out;
      in.raw = *reinterpret_cast<const uint4*>(stage + (size_t)v * 16);
      A acc[VE];
#pragma unroll
      for (int e = 0; e < VE; ++e) acc[e] = to_acc<T>(in.e[e]);
      for (int k = 1; k < nsrc; ++k) {
        in.raw = *reinterpret_cast<const uint4*>(stage + (size_t)k * chunk + (size_t)v * 16);
#pragma unroll
        for (int e = 0; e < VE; ++e) acc[e] = apply<A>(OP, acc[e], to_acc<T>(in.e[e]));
      }
#pragma unroll
      for (int e = 0; e < VE; ++e) out.e[e] = from_acc<T>(acc[e]);
      for (int d = 0; d < ndst; ++d) reinterpret_cast<uint4*>(dsts[d])[v_base + v] = out.raw;
    }
    __syncthreads();                       // the stage has been read by everybody: refill it
    if (threadIdx.x == 0 && c + kBulkStages < nchunks) issue(c + kBulkStages);
  }
  __syncthreads();
  return bulk_ok != 0;
}

// dst[i] = reduce over members k (in team order) of src_k[i], for i in [begin, end) elements;
// the result goes to `ndst` destinations.  Vector body + scalar edges, striped over the block.
template <typename T, int OP>
__device__ __forceinline__ void reduce_range_op(const State& s, int nsrc, const T* const* srcs, int ndst, T* const* dsts,
                                                size_t begin, size_t end, char* bulk) {
  constexpr int op = OP;      // compile-time operator: the per-element switch in apply() folds away
  using A = typename Acc<T>::type;
  constexpr int VE = 16 / sizeof(T);
  const int tid = threadIdx.x, nth = blockDim.x;
  size_t vbeg = (begin + VE - 1) / VE * VE, vend = end / VE * VE;
  // sources are usually the same symmetric offset on every member, but staged collectives mix a staging block per
  // sender with the local source, so every pointer is checked
  bool aligned = true;
  for (int k = 0; k < nsrc; ++k) aligned &= ((uintptr_t)srcs[k] & 15) == 0;
  for (int d = 0; d < ndst; ++d) aligned &= ((uintptr_t)dsts[d] & 15) == 0;
  if (!aligned || vbeg >= vend) { vbeg = vend = begin; }
  for (size_t i = begin + tid; i < vbeg; i += nth) {
    A acc = to_acc<T>(srcs[0][i]);
    for (int k = 1; k < nsrc; ++k) acc = apply<A>(op, acc, to_acc<T>(srcs[k][i]));
    for (int d = 0; d < ndst; ++d) dsts[d][i] = from_acc<T>(acc);
  }
  size_t v0 = vbeg / VE, v1 = vend / VE;
  // big aligned ranges go through shared memory with bulk async copies when the kernel provides the buffer
  if (bulk != nullptr && aligned && (v1 - v0) * 16 >= (size_t)64 * 1024 && nsrc <= 16 &&
      (OP == BSHMEM_SUM || OP == BSHMEM_MAX || OP == BSHMEM_MIN)) {
    if (reduce_bulk<T, OP>(s, nsrc, srcs, ndst, dsts, vbeg, vend, bulk)) v0 = v1;     // nothing left for the register path
    else return;
  }
  // the unrolled variants exist for the element types and operators of bulk reductions (sum / max / min of
  // float, double, half, bf16, int32, int64); everything else takes the generic body, which keeps the build short
  constexpr bool kHot = (OP == BSHMEM_SUM || OP == BSHMEM_MAX || OP == BSHMEM_MIN) &&
                        (std::is_same<T, float>::value || std::is_same<T, double>::value || std::is_same<T, __half>::value ||
                         std::is_same<T, __nv_bfloat16>::value || std::is_same<T, int32_t>::value || std::is_same<T, long long>::value);
  if constexpr (kHot) {
    // members x unroll = 16 independent 16-byte loads per batch and two batches in flight (128 registers; the
    // reduction kernels run 256-thread blocks, so nothing spills): ~100 blocks keep tens of megabytes in flight
    if (nsrc <= 2) reduce_vec_body<T, OP, 2, 8>(nsrc, srcs, ndst, dsts, v0, v1);
    else if (nsrc <= 4) reduce_vec_body<T, OP, 4, 4>(nsrc, srcs, ndst, dsts, v0, v1);
    else if (nsrc <= 8) reduce_vec_body<T, OP, 8, 2>(nsrc, srcs, ndst, dsts, v0, v1);
    else reduce_vec_body<T, OP, BSHMEM_MAX_PES, 1>(nsrc, srcs, ndst, dsts, v0, v1);
  } else {
    reduce_vec_body<T, OP, BSHMEM_MAX_PES, 1>(nsrc, srcs, ndst, dsts, v0, v1);
  }
  size_t tail = (vend > begin) ? vend : begin;
  for (size_t i = tail + tid; i < end; i += nth) {
    A acc = to_acc<T>(srcs[0][i]);
    for (int k = 1; k < nsrc; ++k) acc = apply<A>(op, acc, to_acc<T>(srcs[k][i]));
    for (int d = 0; d < ndst; ++d) dsts[d][i] = from_acc<T>(acc);
  }
}

// Run-time operator -> compile-time instantiation (bitwise operators exist for integer types only).
// Not inlined: one copy per element type is shared by every collective kernel of a translation unit,
// which keeps the kernels (and their compile time) small; the call happens once per CTA and collective.
// `bulk`: kBulkSmemBytes of 128-byte aligned dynamic shared memory for the large-range path, or null.
template <typename T>
__device__ __noinline__ void reduce_range(const State& s, int op, int nsrc, const T* const* srcs, int ndst, T* const* dsts,
                                          size_t begin, size_t end, char* bulk = nullptr) {
  switch (op) {
    case BSHMEM_SUM: reduce_range_op<T, BSHMEM_SUM>(s, nsrc, srcs, ndst, dsts, begin, end, bulk); break;
    case BSHMEM_MIN: reduce_range_op<T, BSHMEM_MIN>(s, nsrc, srcs, ndst, dsts, begin, end, bulk); break;
    case BSHMEM_MAX: reduce_range_op<T, BSHMEM_MAX>(s, nsrc, srcs, ndst, dsts, begin, end, bulk); break;
    case BSHMEM_PROD: reduce_range_op<T, BSHMEM_PROD>(s, nsrc, srcs, ndst, dsts, begin, end, bulk); break;
    default:
      if constexpr (!std::is_floating_point<typename Acc<T>::type>::value) {
        if (op == BSHMEM_AND) reduce_range_op<T, BSHMEM_AND>(s, nsrc, srcs, ndst, dsts, begin, end, bulk);
        else if (op == BSHMEM_OR) reduce_range_op<T, BSHMEM_OR>(s, nsrc, srcs, ndst, dsts, begin, end, bulk);
        else reduce_range_op<T, BSHMEM_XOR>(s, nsrc, srcs, ndst, dsts, begin, end, bulk);
      }
  }
}

// Contiguous share of [0, n) for part `idx` of `parts`, in units of `gran` elements.
__device__ __forceinline__ void split_range(size_t n, int parts, int idx, size_t gran, size_t* b, size_t* e) {
  size_t units = (n + gran - 1) / gran;
  size_t per = (units + parts - 1) / parts;
  size_t ub = per * idx, ue = ub + per;
  *b = ub * gran < n ? ub * gran : n;
  *e = ue * gran < n ? ue * gran : n;
}

constexpr size_t kOneShotBytes = 64 * 1024;   // below this every PE reduces the whole vector itself

static_assert(BSHMEM_OFF_SCRATCH + BSHMEM_SCRATCH_BYTES <= BSHMEM_OFF_MCBAR && BSHMEM_OFF_MCBAR + BSHMEM_MCBAR_BYTES <= BSHMEM_OFF_LL &&
              BSHMEM_OFF_LLT + (uint64_t)BSHMEM_MAX_TEAMS * BSHMEM_LLT_TEAM_BYTES <= BSHMEM_OFF_STAGE &&
              BSHMEM_OFF_STAGE + 2 * BSHMEM_STAGE_BYTES <= BSHMEM_INTERNAL_BYTES && BSHMEM_OFF_LL + BSHMEM_LL_BYTES <= BSHMEM_OFF_SLAB &&
              BSHMEM_OFF_SLAB + BSHMEM_SLAB_BYTES <= BSHMEM_OFF_LLB && BSHMEM_OFF_LLB + BSHMEM_LLB_BYTES <= BSHMEM_OFF_LLT &&
              BSHMEM_OFF_SCRATCH + BSHMEM_SCRATCH_BYTES <= BSHMEM_OFF_LL,
              "internal heap regions overlap");

// Low-latency allreduce for small vectors on the world team, single block: ONE NVLink exchange instead of
// sync + reduce + barrier.  Every PE pushes its vector into a per-sender slot on every PE as 8-byte words that carry
// 4 bytes of data and the 32-bit epoch, so data and "it has arrived" travel in the same store; receivers poll the
// words, reduce in team order (identical result on every PE) and return.  The source is reusable on return (it was
// copied out); slots alternate by epoch parity: a sender can only write epoch e+2 after it finished e+1, which needed
// this PE's data of e+1, which this PE sent after it had read every slot of e.
// `epoch_in` = 0: single block, the epoch is a counter in this PE's heap (any caller, device-initiated included);
// otherwise the host supplies the epoch of a multi-block launch (block `cta` of `ncta` takes a share of the words)
// and the larger slot region is used.
template <typename T>
__device__ __forceinline__ int team_reduce_ll(const State& s, const Team& t, int op, T* dest, const T* source, size_t n,
                                              unsigned long long epoch_in = 0, int cta = 0, int ncta = 1) {
  using A = typename Acc<T>::type;
  constexpr int kUnit = sizeof(T) > 4 ? (int)sizeof(T) : 4;        // bytes reduced together: whole elements
  constexpr int kWords = kUnit / 4, kElems = kUnit / (int)sizeof(T);
  __shared__ unsigned long long ll_epoch;
  __shared__ int ll_status;
  // world team: host-epoch region or the small region; any other team: that team's own block
  const size_t region = epoch_in ? BSHMEM_OFF_LLB : t.slot == 0 ? BSHMEM_OFF_LL : BSHMEM_OFF_LLT + (size_t)t.slot * BSHMEM_LLT_TEAM_BYTES;
  const size_t slot_bytes = epoch_in ? BSHMEM_LLB_SLOT_BYTES : t.slot == 0 ? BSHMEM_LL_SLOT_BYTES : BSHMEM_LLT_SLOT_BYTES;
  char* my_base = s.heap_base[s.my_pe] + region;
  if (threadIdx.x == 0) {
    ll_epoch = epoch_in ? epoch_in : *reinterpret_cast<unsigned long long*>(my_base) + 1;
    ll_status = BSHMEM_OK;
  }
  __syncthreads();
  const unsigned long long e = ll_epoch;
  const unsigned long long flag = (e & 0xFFFFFFFFull) << 32;
  const int nwords = (int)(n * sizeof(T) / 4);
  const size_t slot0 = (epoch_in ? 0 : 64) + (size_t)(e & 1) * BSHMEM_MAX_PES * slot_bytes;
  // this block's share, in whole units
  const int units_all = nwords / kWords;
  const int per = (units_all + ncta - 1) / ncta;
  const int u_begin = min(per * cta, units_all), u_end = min(u_begin + per, units_all);
  // ---- push: my words into slot [my_idx] of every member (myself included) ----
  const uint32_t* src32 = reinterpret_cast<const uint32_t*>(source);
  for (int w = u_begin * kWords + threadIdx.x; w < u_end * kWords; w += blockDim.x) {
    const unsigned long long packed = flag | src32[w];
    for (int k = 0; k < t.size; ++k) {
      char* peer = s.heap_base[dev::team_pe(t, k)] + region + slot0 + (size_t)t.my_idx * slot_bytes;
      asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(peer + (size_t)w * 8), "l"(packed) : "memory");
    }
  }
  // ---- receive + reduce: unit u = kWords consecutive words of every sender ----
  const unsigned long long t0 = dev::timer();
  constexpr int kBatch = 8;      // senders polled together: their loads are in flight at the same time
  for (int u = u_begin + threadIdx.x; u < u_end; u += blockDim.x) {
    A acc[kElems];
    for (int k0 = 0; k0 < t.size; k0 += kBatch) {
      unsigned long long v[kBatch][kWords];
      const char* slot[kBatch];
#pragma unroll
      for (int kk = 0; kk < kBatch; ++kk) {
        // senders beyond the team re-read the last one (keeps the batch branch-free; the value is not used)
        const int k = k0 + kk < t.size ? k0 + kk : t.size - 1;
        slot[kk] = my_base + slot0 + (size_t)k * slot_bytes + (size_t)u * kWords * 8;
#pragma unroll
        for (int w = 0; w < kWords; ++w)
          asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v[kk][w]) : "l"(slot[kk] + w * 8) : "memory");
      }
#pragma unroll
      for (int kk = 0; kk < kBatch; ++kk) {
        if (k0 + kk >= t.size) break;
        uint32_t raw[kWords];
#pragma unroll
        for (int w = 0; w < kWords; ++w) {
          unsigned it = 0;
          while ((v[kk][w] >> 32) != (e & 0xFFFFFFFFull)) {          // not there yet: poll this word alone
            if ((++it & 63) == 0 && dev::timer() - t0 > s.timeout_ns) {
              dev::record_error(s, BSHMEM_ERR_TIMEOUT, dev::team_pe(t, k0 + kk), BSHMEM_WHERE_BARRIER, (uint64_t)slot[kk], e, v[kk][w] >> 32);
              ll_status = BSHMEM_ERR_TIMEOUT;
              break;
            }
            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v[kk][w]) : "l"(slot[kk] + w * 8) : "memory");
          }
          raw[w] = (uint32_t)v[kk][w];
        }
        T vals[kElems];
        memcpy(vals, raw, kUnit);
#pragma unroll
        for (int i = 0; i < kElems; ++i)
          acc[i] = (k0 + kk) == 0 ? to_acc<T>(vals[i]) : apply<A>(op, acc[i], to_acc<T>(vals[i]));
      }
    }
    T out[kElems];
#pragma unroll
    for (int i = 0; i < kElems; ++i) out[i] = from_acc<T>(acc[i]);
    memcpy(reinterpret_cast<char*>(dest) + (size_t)u * kUnit, out, kUnit);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!epoch_in) *reinterpret_cast<unsigned long long*>(my_base) = e;
    if (cta == 0) {
      dev::stat(s, BSHMEM_DSTAT_COLL);
      dev::trace(s, BSHMEM_TRACE_COLL, s.my_pe, n * sizeof(T));
    }
  }
  const int rc = ll_status;
  __syncthreads();
  return rc;
}

// allreduce (`*_to_all`): dest and source are symmetric; dest may alias source.
template <typename T>
__device__ __forceinline__ int team_reduce(const State& s, const Team& t, int op, T* dest, const T* source, size_t n,
                                           int cta = 0, int ncta = 1, unsigned long long ll_epoch = 0, char* bulk = nullptr) {
  // small vectors on the world team: one exchange (the condition is the same on every PE: symmetric addresses)
  if ((n * sizeof(T)) % (sizeof(T) > 4 ? sizeof(T) : 4) == 0 && n > 0 &&
      ((reinterpret_cast<uintptr_t>(dest) | reinterpret_cast<uintptr_t>(source)) & (sizeof(T) > 4 ? 7 : 3)) == 0) {
    if (t.slot == 0 && t.size == s.n_pes) {
      if (ncta == 1 && n * sizeof(T) <= BSHMEM_LL_PAYLOAD_BYTES) return team_reduce_ll<T>(s, t, op, dest, source, n);
      if (ll_epoch != 0 && n * sizeof(T) <= BSHMEM_LLB_PAYLOAD_BYTES) return team_reduce_ll<T>(s, t, op, dest, source, n, ll_epoch, cta, ncta);
    } else if (t.slot > 0 && t.slot < BSHMEM_MAX_TEAMS && ncta == 1 && n * sizeof(T) <= BSHMEM_LLT_PAYLOAD_BYTES) {
      return team_reduce_ll<T>(s, t, op, dest, source, n);
    }
  }
  const T* srcs[BSHMEM_MAX_PES];
  T* dsts[BSHMEM_MAX_PES];
  for (int k = 0; k < t.size; ++k) {
    srcs[k] = dev::ptr(s, source, dev::team_pe(t, k));
    dsts[k] = dev::ptr(s, dest, dev::team_pe(t, k));
  }
  int rc = team_sync(s, t, cta);          // every member's source is ready
  if (rc != BSHMEM_OK) return rc;
  constexpr size_t VE = 16 / sizeof(T);
  bool one_shot = n * sizeof(T) <= kOneShotBytes && (const void*)dest != (const void*)source;
  if (one_shot) {
    size_t b, e;
    split_range(n, ncta, cta, VE, &b, &e);
    T* mine[1] = {dest};
    reduce_range<T>(s, op, t.size, srcs, 1, mine, b, e);
  } else {
    // two-shot: I own slice my_idx; reduce it from everyone, push the result to everyone
    size_t sb, se, b, e;
    split_range(n, t.size, t.my_idx, VE, &sb, &se);
    split_range(se - sb, ncta, cta, VE, &b, &e);
    reduce_range<T>(s, op, t.size, srcs, t.size, dsts, sb + b, sb + e, bulk);
  }
  if (cta == 0 && threadIdx.x == 0) { dev::stat(s, BSHMEM_DSTAT_COLL); dev::trace(s, BSHMEM_TRACE_COLL, s.my_pe, 0); }
  return team_barrier(s, t, cta);         // results delivered; sources reusable
}

// rooted reduce: member `root` pulls every member's source and writes op over all of them into its dest; the other
// members only take part in the entry sync (their source is ready) and the closing barrier (it has been read).
// dest may alias source.  The reference offers only the `*_to_all` form (library/include/roc_shmem.hpp:837-887).
template <typename T>
__device__ __forceinline__ int team_reduce_root(const State& s, const Team& t, int op, T* dest, const T* source, size_t n, int root,
                                                int cta = 0, int ncta = 1, char* bulk = nullptr) {
  int rc = team_sync(s, t, cta);
  if (rc != BSHMEM_OK) return rc;
  if (t.my_idx == root) {
    const T* srcs[BSHMEM_MAX_PES];
    for (int k = 0; k < t.size; ++k) srcs[k] = dev::ptr(s, source, dev::team_pe(t, k));
    size_t b, e;
    split_range(n, ncta, cta, 16 / sizeof(T), &b, &e);
    T* mine[1] = {dest};
    reduce_range<T>(s, op, t.size, srcs, 1, mine, b, e, bulk);
    if (cta == 0 && threadIdx.x == 0) { dev::stat(s, BSHMEM_DSTAT_COLL); dev::trace(s, BSHMEM_TRACE_COLL, s.my_pe, n * sizeof(T)); }
  }
  return team_barrier(s, t, cta);
}

// reduce-scatter: dest (n elements) = reduction of the members' source[my_idx*n : (my_idx+1)*n].
template <typename T>
__device__ __forceinline__ int team_reduce_scatter(const State& s, const Team& t, int op, T* dest, const T* source,
                                                   size_t n, int cta = 0, int ncta = 1, char* bulk = nullptr) {
  const T* srcs[BSHMEM_MAX_PES];
  for (int k = 0; k < t.size; ++k) srcs[k] = dev::ptr(s, source, dev::team_pe(t, k)) + (size_t)t.my_idx * n;
  int rc = team_sync(s, t, cta);
  if (rc != BSHMEM_OK) return rc;
  size_t b, e;
  split_range(n, ncta, cta, 16 / sizeof(T), &b, &e);
  T* mine[1] = {dest};
  reduce_range<T>(s, op, t.size, srcs, 1, mine, b, e, bulk);
  if (cta == 0 && threadIdx.x == 0) { dev::stat(s, BSHMEM_DSTAT_COLL); dev::trace(s, BSHMEM_TRACE_COLL, s.my_pe, 0); }
  return team_barrier(s, t, cta);
}

// broadcast: the root's source lands in every other member's dest (the root's dest is untouched).
__device__ __forceinline__ int team_broadcast(const State& s, const Team& t, void* dest, const void* source, size_t nbytes,
                                              int root, int cta = 0, int ncta = 1) {
  int rc = team_sync(s, t, cta);
  if (rc != BSHMEM_OK) return rc;
  if (t.my_idx != root) {
    size_t b, e;
    split_range(nbytes, ncta, cta, 16, &b, &e);
    const char* src = dev::ptr(s, reinterpret_cast<const char*>(source), dev::team_pe(t, root));
    dev::copy_bytes<dev::BLOCK>(reinterpret_cast<char*>(dest) + b, src + b, e - b);
  }
  if (cta == 0 && threadIdx.x == 0) { dev::stat(s, BSHMEM_DSTAT_COLL); dev::trace(s, BSHMEM_TRACE_COLL, s.my_pe, 0); }
  return team_barrier(s, t, cta);
}

// fcollect (all-gather): my source lands in block my_idx of every member's dest.
__device__ __forceinline__ int team_fcollect(const State& s, const Team& t, void* dest, const void* source, size_t nbytes,
                                             int cta = 0, int ncta = 1) {
  int rc = team_sync(s, t, cta);          // every member's dest may be overwritten
  if (rc != BSHMEM_OK) return rc;
  size_t b, e;
  split_range(nbytes, ncta, cta, 16, &b, &e);
  for (int k = 0; k < t.size; ++k) {
    int peer_idx = (t.my_idx + k) % t.size;   // stagger the targets so the PEs do not gang up on one peer
    char* d = dev::ptr(s, reinterpret_cast<char*>(dest), dev::team_pe(t, peer_idx)) + (size_t)t.my_idx * nbytes;
    dev::copy_bytes<dev::BLOCK>(d + b, reinterpret_cast<const char*>(source) + b, e - b);
  }
  if (cta == 0 && threadIdx.x == 0) { dev::stat(s, BSHMEM_DSTAT_COLL); dev::trace(s, BSHMEM_TRACE_COLL, s.my_pe, 0); }
  return team_barrier(s, t, cta);
}

// alltoall: block j of my source lands in block my_idx of member j's dest.
__device__ __forceinline__ int team_alltoall(const State& s, const Team& t, void* dest, const void* source, size_t nbytes,
                                             int cta = 0, int ncta = 1) {
  int rc = team_sync(s, t, cta);
  if (rc != BSHMEM_OK) return rc;
  size_t b, e;
  split_range(nbytes, ncta, cta, 16, &b, &e);
  for (int k = 0; k < t.size; ++k) {
    int j = (t.my_idx + k) % t.size;
    char* d = dev::ptr(s, reinterpret_cast<char*>(dest), dev::team_pe(t, j)) + (size_t)t.my_idx * nbytes;
    const char* sp = reinterpret_cast<const char*>(source) + (size_t)j * nbytes;
    dev::copy_bytes<dev::BLOCK>(d + b, sp + b, e - b);
  }
  if (cta == 0 && threadIdx.x == 0) { dev::stat(s, BSHMEM_DSTAT_COLL); dev::trace(s, BSHMEM_TRACE_COLL, s.my_pe, 0); }
  return team_barrier(s, t, cta);
}


// ---- one-exchange collectives through the staging region (world team, host-launched) -------------------------
// The sync + work + barrier forms above pay two flag exchanges because a PE may only write into a peer's `dest`
// once that peer has entered the call.  Here every PE pushes into a runtime-owned per-sender block on the peer
// instead (always writable: see the parity argument), then ONE barrier tells everybody that all blocks have landed,
// and each PE copies / reduces its staging into `dest` locally.  `seq` is a call sequence number the host supplies,
// the same on every PE; consecutive calls alternate between the two staging halves.  A PE writes half (seq & 1)
// again two staged calls later; it has then completed call seq+1, whose barrier needed every peer's kernel of call
// seq+1 to be running, and kernels of one PE run in stream order, so every peer has finished reading call seq's half.
__device__ __forceinline__ char* stage_half(const State& s, int pe, unsigned long long seq) {
  return s.heap_base[pe] + BSHMEM_OFF_STAGE + (seq & 1) * BSHMEM_STAGE_BYTES;
}
// 16-byte-vector copy of the block's range into the same offset of EVERY PE's heap through the multicast mapping
__device__ __forceinline__ void copy_bytes_mc(char* mc_dst, const char* src, size_t n) {
  const uint4* s4 = reinterpret_cast<const uint4*>(src);
  for (size_t v = threadIdx.x; v < (n >> 4); v += blockDim.x) {
    const uint4 x = s4[v];
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(mc_dst + v * 16), "r"(x.x), "r"(x.y), "r"(x.z), "r"(x.w) : "memory");
  }
}

__device__ __forceinline__ int team_fcollect_staged(const State& s, const Team& t, void* dest, const void* source, size_t nbytes,
                                                    unsigned long long seq, int use_mc, int cta, int ncta) {
  size_t b, e;
  split_range(nbytes, ncta, cta, 16, &b, &e);
  const char* src = reinterpret_cast<const char*>(source);
  const size_t mine = (size_t)t.my_idx * nbytes;
  if (use_mc && s.mc_base) {
    // one multicast store per vector lands in block my_idx of every PE's staging half (this PE's included)
    copy_bytes_mc(s.mc_base + BSHMEM_OFF_STAGE + (seq & 1) * BSHMEM_STAGE_BYTES + mine + b, src + b, e - b);
  } else {
    for (int k = 1; k < t.size; ++k) {
      const int idx = (t.my_idx + k) % t.size;
      dev::copy_bytes<dev::BLOCK>(stage_half(s, dev::team_pe(t, idx), seq) + mine + b, src + b, e - b);
    }
  }
  dev::copy_bytes<dev::BLOCK>(reinterpret_cast<char*>(dest) + mine + b, src + b, e - b);
  int rc = team_barrier(s, t, cta);
  if (rc != BSHMEM_OK) return rc;
  const char* st = stage_half(s, s.my_pe, seq);
  for (int k = 1; k < t.size; ++k) {
    const size_t o = (size_t)((t.my_idx + k) % t.size) * nbytes + b;
    dev::copy_bytes<dev::BLOCK>(reinterpret_cast<char*>(dest) + o, st + o, e - b);
  }
  if (cta == 0 && threadIdx.x == 0) { dev::stat(s, BSHMEM_DSTAT_COLL); dev::trace(s, BSHMEM_TRACE_COLL, s.my_pe, nbytes); }
  return BSHMEM_OK;
}

__device__ __forceinline__ int team_alltoall_staged(const State& s, const Team& t, void* dest, const void* source, size_t nbytes,
                                                    unsigned long long seq, int cta, int ncta) {
  size_t b, e;
  split_range(nbytes, ncta, cta, 16, &b, &e);
  const char* src = reinterpret_cast<const char*>(source);
  const size_t mine = (size_t)t.my_idx * nbytes;
  for (int k = 1; k < t.size; ++k) {
    const int j = (t.my_idx + k) % t.size;
    dev::copy_bytes<dev::BLOCK>(stage_half(s, dev::team_pe(t, j), seq) + mine + b, src + (size_t)j * nbytes + b, e - b);
  }
  dev::copy_bytes<dev::BLOCK>(reinterpret_cast<char*>(dest) + mine + b, src + mine + b, e - b);
  int rc = team_barrier(s, t, cta);
  if (rc != BSHMEM_OK) return rc;
  const char* st = stage_half(s, s.my_pe, seq);
  for (int k = 1; k < t.size; ++k) {
    const size_t o = (size_t)((t.my_idx + k) % t.size) * nbytes + b;
    dev::copy_bytes<dev::BLOCK>(reinterpret_cast<char*>(dest) + o, st + o, e - b);
  }
  if (cta == 0 && threadIdx.x == 0) { dev::stat(s, BSHMEM_DSTAT_COLL); dev::trace(s, BSHMEM_TRACE_COLL, s.my_pe, nbytes); }
  return BSHMEM_OK;
}

// reduce-scatter: every PE pushes slice j of its source into PE j's staging, one barrier, local reduction (own slice
// straight from `source`).  n elements per PE; n * sizeof(T) is a multiple of 16 and source is 16-byte aligned.
template <typename T>
__device__ __forceinline__ int team_reduce_scatter_staged(const State& s, const Team& t, int op, T* dest, const T* source, size_t n,
                                                          unsigned long long seq, int cta, int ncta, char* bulk = nullptr) {
  size_t b, e;
  split_range(n, ncta, cta, 16 / sizeof(T), &b, &e);
  const size_t slot = n * sizeof(T);
  for (int k = 1; k < t.size; ++k) {
    const int j = (t.my_idx + k) % t.size;
    dev::copy_bytes<dev::BLOCK>(stage_half(s, dev::team_pe(t, j), seq) + (size_t)t.my_idx * slot + b * sizeof(T),
                                reinterpret_cast<const char*>(source + (size_t)j * n + b), (e - b) * sizeof(T));
  }
  int rc = team_barrier(s, t, cta);
  if (rc != BSHMEM_OK) return rc;
  const T* srcs[BSHMEM_MAX_PES];
  const char* st = stage_half(s, s.my_pe, seq);
  for (int k = 0; k < t.size; ++k)
    srcs[k] = k == t.my_idx ? source + (size_t)t.my_idx * n : reinterpret_cast<const T*>(st + (size_t)k * slot);
  T* mine[1] = {dest};
  reduce_range<T>(s, op, t.size, srcs, 1, mine, b, e, bulk);
  if (cta == 0 && threadIdx.x == 0) { dev::stat(s, BSHMEM_DSTAT_COLL); dev::trace(s, BSHMEM_TRACE_COLL, s.my_pe, slot); }
  return BSHMEM_OK;
}

// allreduce, two exchanges: staged reduce-scatter of uneven 16-byte-granular slices, then every PE writes its reduced
// slice into every member's dest (safe: after the first barrier all members are in this call and have finished
// reading their sources, so dest may even alias source) and a closing barrier delivers the results.
template <typename T>
__device__ __forceinline__ int team_reduce_staged(const State& s, const Team& t, int op, T* dest, const T* source, size_t n,
                                                  unsigned long long seq, int cta, int ncta, char* bulk = nullptr) {
  constexpr size_t VE = 16 / sizeof(T);
  const size_t slot = (BSHMEM_STAGE_BYTES / t.size) & ~(size_t)15;   // room per sender; a slice is at most ceil(n / size) elements
  for (int k = 1; k < t.size; ++k) {
    const int j = (t.my_idx + k) % t.size;
    size_t sb, se, b, e;
    split_range(n, t.size, j, VE, &sb, &se);
    split_range(se - sb, ncta, cta, VE, &b, &e);
    dev::copy_bytes<dev::BLOCK>(stage_half(s, dev::team_pe(t, j), seq) + (size_t)t.my_idx * slot + b * sizeof(T),
                                reinterpret_cast<const char*>(source + sb + b), (e - b) * sizeof(T));
  }
  int rc = team_barrier(s, t, cta);
  if (rc != BSHMEM_OK) return rc;
  size_t sb, se, b, e;
  split_range(n, t.size, t.my_idx, VE, &sb, &se);
  split_range(se - sb, ncta, cta, VE, &b, &e);
  const T* srcs[BSHMEM_MAX_PES];
  T* dsts[BSHMEM_MAX_PES];
  const char* st = stage_half(s, s.my_pe, seq);
  for (int k = 0; k < t.size; ++k) {
    // index i of reduce_range runs over [sb + b, sb + e): staged blocks start at element 0 of the slice
    srcs[k] = k == t.my_idx ? source : reinterpret_cast<const T*>(st + (size_t)k * slot) - sb;
    dsts[k] = dev::ptr(s, dest, dev::team_pe(t, k));
  }
  reduce_range<T>(s, op, t.size, srcs, t.size, dsts, sb + b, sb + e, bulk);
  if (cta == 0 && threadIdx.x == 0) { dev::stat(s, BSHMEM_DSTAT_COLL); dev::trace(s, BSHMEM_TRACE_COLL, s.my_pe, n * sizeof(T)); }
  return team_barrier(s, t, cta);
}

// allreduce, ONE exchange: every PE pushes its whole vector into its block of every member's staging, one barrier,
// then every PE reduces all blocks locally (same order everywhere, so the results are identical).  Moves (size - 1)
// times the vector per PE instead of 2 (size - 1) / size times, which pays while the second exchange of the two-shot
// form costs more than the extra bytes (the host picks; the vector must fit a sender's block).  dest may alias source.
template <typename T>
__device__ __forceinline__ int team_reduce_staged_oneshot(const State& s, const Team& t, int op, T* dest, const T* source, size_t n,
                                                          unsigned long long seq, int cta, int ncta, char* bulk = nullptr) {
  constexpr size_t VE = 16 / sizeof(T);
  const size_t slot = (BSHMEM_STAGE_BYTES / t.size) & ~(size_t)15;
  size_t b, e;
  split_range(n, ncta, cta, VE, &b, &e);
  for (int k = 1; k < t.size; ++k) {
    const int j = (t.my_idx + k) % t.size;
    dev::copy_bytes<dev::BLOCK>(stage_half(s, dev::team_pe(t, j), seq) + (size_t)t.my_idx * slot + b * sizeof(T),
                                reinterpret_cast<const char*>(source + b), (e - b) * sizeof(T));
  }
  int rc = team_barrier(s, t, cta);
  if (rc != BSHMEM_OK) return rc;
  const T* srcs[BSHMEM_MAX_PES];
  const char* st = stage_half(s, s.my_pe, seq);
  for (int k = 0; k < t.size; ++k) srcs[k] = k == t.my_idx ? source : reinterpret_cast<const T*>(st + (size_t)k * slot);
  T* mine[1] = {dest};
  reduce_range<T>(s, op, t.size, srcs, 1, mine, b, e, bulk);
  if (cta == 0 && threadIdx.x == 0) { dev::stat(s, BSHMEM_DSTAT_COLL); dev::trace(s, BSHMEM_TRACE_COLL, s.my_pe, n * sizeof(T)); }
  return BSHMEM_OK;
}

// ---- NVLink-multicast (NVLS) allreduce: the switch reduces and broadcasts ----------------------
// Works on 16-byte vectors of fp32 / bf16 sum only; the caller falls back otherwise.
template <typename T>
__device__ __forceinline__ int team_reduce_nvls(const State& s, const Team& t, T* dest, const T* source, size_t n,
                                                int cta = 0, int ncta = 1) {
  static_assert(std::is_same<T, float>::value || std::is_same<T, __nv_bfloat16>::value, "fp32 / bf16 only");
  constexpr size_t VE = 16 / sizeof(T);
  int rc = team_sync(s, t, cta);
  if (rc != BSHMEM_OK) return rc;
  size_t sb, se, b, e;
  split_range(n, t.size, t.my_idx, VE, &sb, &se);
  split_range(se - sb, ncta, cta, VE, &b, &e);
  uint64_t soff = reinterpret_cast<const char*>(source) - s.heap_base[s.my_pe];
  uint64_t doff = reinterpret_cast<char*>(dest) - s.heap_base[s.my_pe];
  const char* mc_src = s.mc_base + soff;
  char* mc_dst = s.mc_base + doff;
  // eight in-switch reductions in flight per thread: each is a round trip through the NVSwitch
  constexpr int U = 8;
  const size_t v1 = (sb + e) / VE;
  for (size_t base = (sb + b) / VE; base < v1; base += (size_t)U * blockDim.x) {
    uint4 r[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = base + (size_t)u * blockDim.x + threadIdx.x;
      if (v < v1) {
        if constexpr (std::is_same<T, float>::value) {
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(r[u].x), "=r"(r[u].y), "=r"(r[u].z), "=r"(r[u].w) : "l"(mc_src + v * 16) : "memory");
        } else {
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                       : "=r"(r[u].x), "=r"(r[u].y), "=r"(r[u].z), "=r"(r[u].w) : "l"(mc_src + v * 16) : "memory");
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = base + (size_t)u * blockDim.x + threadIdx.x;
      if (v < v1)
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                     ::"l"(mc_dst + v * 16), "r"(r[u].x), "r"(r[u].y), "r"(r[u].z), "r"(r[u].w) : "memory");
    }
  }
  return team_barrier(s, t, cta);
}

// reduce-scatter through the switch: my slice of everybody's source is reduced by one multimem.ld_reduce per vector
// and stored to the local dest.  fp32 / bf16 sum; n * sizeof(T) a multiple of 16; source and dest 16-byte aligned.
template <typename T>
__device__ __forceinline__ int team_reduce_scatter_nvls(const State& s, const Team& t, T* dest, const T* source, size_t n,
                                                        int cta = 0, int ncta = 1) {
  static_assert(std::is_same<T, float>::value || std::is_same<T, __nv_bfloat16>::value, "fp32 / bf16 only");
  constexpr size_t VE = 16 / sizeof(T);
  int rc = team_sync(s, t, cta);
  if (rc != BSHMEM_OK) return rc;
  size_t b, e;
  split_range(n, ncta, cta, VE, &b, &e);
  const uint64_t soff = reinterpret_cast<const char*>(source + (size_t)t.my_idx * n) - s.heap_base[s.my_pe];
  const char* mc_src = s.mc_base + soff;
  uint4* out = reinterpret_cast<uint4*>(dest);
  constexpr int U = 8;
  const size_t v1 = e / VE;
  for (size_t base = b / VE; base < v1; base += (size_t)U * blockDim.x) {
    uint4 r[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = base + (size_t)u * blockDim.x + threadIdx.x;
      if (v < v1) {
        if constexpr (std::is_same<T, float>::value) {
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(r[u].x), "=r"(r[u].y), "=r"(r[u].z), "=r"(r[u].w) : "l"(mc_src + v * 16) : "memory");
        } else {
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                       : "=r"(r[u].x), "=r"(r[u].y), "=r"(r[u].z), "=r"(r[u].w) : "l"(mc_src + v * 16) : "memory");
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = base + (size_t)u * blockDim.x + threadIdx.x;
      if (v < v1) out[v] = r[u];
    }
  }
  return team_barrier(s, t, cta);       // every member has finished reading everybody's source
}

// roc_shmem-style names for single-block use ---------------------------------------------------------
template <typename T> __device__ __forceinline__ int wg_to_all(const State& s, const Team& t, int op, T* dest, const T* src, size_t n) {
  return team_reduce<T>(s, t, op, dest, src, n, 0, 1);
}
template <typename T> __device__ __forceinline__ int wg_broadcast(const State& s, const Team& t, T* dest, const T* src, size_t n, int root) {
  return team_broadcast(s, t, dest, src, n * sizeof(T), root, 0, 1);
}
template <typename T> __device__ __forceinline__ int wg_fcollect(const State& s, const Team& t, T* dest, const T* src, size_t n) {
  return team_fcollect(s, t, dest, src, n * sizeof(T), 0, 1);
}
template <typename T> __device__ __forceinline__ int wg_alltoall(const State& s, const Team& t, T* dest, const T* src, size_t n) {
  return team_alltoall(s, t, dest, src, n * sizeof(T), 0, 1);
}


// context forms (library/include/roc_shmem.hpp:754-795, 838-1160): the context's team is the team of the collective
__device__ __forceinline__ int ctx_wg_barrier_all(const State& s, const dev::Ctx&) { return wg_barrier_all(s); }
__device__ __forceinline__ int ctx_wg_sync_all(const State& s, const dev::Ctx&) { return wg_sync_all(s); }
__device__ __forceinline__ int ctx_wg_team_sync(const State& s, const dev::Ctx& c) { return team_sync(s, c.team); }
template <typename T> __device__ __forceinline__ int ctx_wg_to_all(const State& s, const dev::Ctx& c, int op, T* dest, const T* src, size_t n) {
  return wg_to_all<T>(s, c.team, op, dest, src, n);
}
template <typename T> __device__ __forceinline__ int ctx_wg_broadcast(const State& s, const dev::Ctx& c, T* dest, const T* src, size_t n, int root) {
  return wg_broadcast<T>(s, c.team, dest, src, n, root);
}
template <typename T> __device__ __forceinline__ int ctx_wg_fcollect(const State& s, const dev::Ctx& c, T* dest, const T* src, size_t n) {
  return wg_fcollect<T>(s, c.team, dest, src, n);
}
template <typename T> __device__ __forceinline__ int ctx_wg_alltoall(const State& s, const dev::Ctx& c, T* dest, const T* src, size_t n) {
  return wg_alltoall<T>(s, c.team, dest, src, n);
}

}  // namespace coll
}  // namespace bshmem
#endif  // __CUDACC__
