// moe_kernels.cu — expert-parallel MoE layer pieces for sm_100a: router + top-k, a
// deterministic dispatch plan, token dispatch and combine over NVLink with
// putmem + signal semantics, SwiGLU forward/backward and the transposes the
// weight-gradient GEMMs need.  The grouped expert GEMM itself is in moe_gemm.cu.
//
// Data flow (E experts over P PEs, E/P experts per PE, top-k routing):
//   router_topk   logits = x · Wr^T, softmax, top-k, renormalised weights
//   plan          per expert: position of every (token, k) entry in token order → `pos`, counts
//   (all-gather of the counts through the runtime's fcollect)
//   offsets       where this PE's entries start inside every destination expert's buffer
//                 (entries are laid out by source PE, then token order → reproducible bits)
//   dispatch      one warp per entry: putmem of the token row into the destination expert's
//                 receive buffer slot (peer stores), entry id into the meta array; one
//                 release-add per (CTA, destination) on the destination's arrival word
//   [grouped GEMM gate/up → SwiGLU → grouped GEMM down; waits on the arrival words]
//   combine_send  expert PE returns each output row to the source PE's per-entry buffer + signal
//   combine_reduce  out[token] = sum_k w[token,k] * y[entry]
// Backward runs the same flow with gradients (dispatch of w·d_out, combine of dX rows).
//
// Arrival words are double-buffered by call parity and zeroed one call ahead, every wait
// is bounded.  The reference has no MoE layer; the put + signal idiom is its
// put / fence / flag pattern (library/src/gpu_ib/context_ib_tmpl_device.hpp:184-236).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstring>
#include <string>

#include "../include/bshmem_device.cuh"
#include "moe_common.h"
#include "ptx.cuh"

using namespace bshmem;
using dev::State;

namespace {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------------------------------
// router: one warp per token; E <= 64 experts, top-k <= 8
// ---------------------------------------------------------------------------------------
__global__ void k_router_topk(const bf16* __restrict__ x, const bf16* __restrict__ wr, int T, int H, int E, int topk,
                              int* __restrict__ topk_idx, float* __restrict__ topk_w, float* __restrict__ probs) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)warp * H);
  float logit[64];
  for (int e0 = 0; e0 < E; e0 += 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int v = lane; v < H / 8; v += 32) {
      uint4 xv = xr[v];
      const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv);
      float2 xf[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) xf[q] = __bfloat1622float2(xh[q]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (e0 + j < E) {
          uint4 wv = __ldg(reinterpret_cast<const uint4*>(wr + (size_t)(e0 + j) * H) + v);
          const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float2 wf = __bfloat1622float2(wh[q]);
            acc[j] += xf[q].x * wf.x + xf[q].y * wf.y;
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float s = warp_sum(acc[j]);
      if (e0 + j < E) logit[e0 + j] = s;
    }
  }
  if (lane == 0) {
    float mx = -INFINITY;
    for (int e = 0; e < E; ++e) mx = fmaxf(mx, logit[e]);
    float den = 0.f;
    for (int e = 0; e < E; ++e) { logit[e] = __expf(logit[e] - mx); den += logit[e]; }
    for (int e = 0; e < E; ++e) { logit[e] /= den; if (probs) probs[(size_t)warp * E + e] = logit[e]; }
    float wsum = 0.f;
    int chosen[8];
    for (int k = 0; k < topk; ++k) {
      int best = -1;
      float bv = -1.f;
      for (int e = 0; e < E; ++e) {      // ties go to the lower expert index
        bool taken = false;
        for (int j = 0; j < k; ++j) taken |= (chosen[j] == e);
        if (!taken && logit[e] > bv) { bv = logit[e]; best = e; }
      }
      chosen[k] = best;
      topk_idx[(size_t)warp * topk + k] = best;
      topk_w[(size_t)warp * topk + k] = bv;
      wsum += bv;
    }
    for (int k = 0; k < topk; ++k) topk_w[(size_t)warp * topk + k] /= wsum;   // renormalise over the chosen experts
  }
}

// ---------------------------------------------------------------------------------------
// plan: CTA e assigns positions to the entries routed to expert e, in entry order
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) k_plan(const int* __restrict__ topk_idx, int n_entries, int* __restrict__ pos,
                                               int* __restrict__ counts) {
  __shared__ int warp_tot[32];
  __shared__ int base_sh;
  const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  if (tid == 0) base_sh = 0;
  __syncthreads();
  for (int start = 0; start < n_entries; start += blockDim.x) {
    int i = start + tid;
    bool mine = i < n_entries && topk_idx[i] == e;
    unsigned ballot = __ballot_sync(0xffffffffu, mine);
    int prefix = __popc(ballot & ((1u << lane) - 1));
    if (lane == 0) warp_tot[wid] = __popc(ballot);
    __syncthreads();
    int before = 0;
    for (int w = 0; w < wid; ++w) before += warp_tot[w];
    int base = base_sh;
    if (mine) pos[i] = base + before + prefix;
    __syncthreads();
    if (tid == 0) {
      int tot = 0;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += warp_tot[w];
      base_sh = base + tot;
    }
    __syncthreads();
  }
  if (tid == 0) counts[e] = base_sh;
}

// ---------------------------------------------------------------------------------------
// offsets: from the gathered counts [P][E] derive everything the data movement needs
// ---------------------------------------------------------------------------------------
__global__ void k_offsets(MoePlanDev pl, const int* __restrict__ counts_all, int parity) {
  const int P = pl.P, E = pl.E, Epr = E / P, me = pl.me, cap = pl.cap;
  const int tid = threadIdx.x;
  // start of my entries inside every expert's buffer
  for (int e = tid; e < E; e += blockDim.x) {
    int b = 0;
    for (int s = 0; s < me; ++s) b += counts_all[s * E + e];
    pl.base_me[e] = b;
  }
  // local experts: rows that will arrive (clamped to the capacity), and each source's share
  for (int el = tid; el < Epr; el += blockDim.x) {
    int e = me * Epr + el, run = 0;
    for (int s = 0; s < P; ++s) {
      pl.src_start[el * (P + 1) + s] = run;
      run += counts_all[s * E + e];
    }
    pl.src_start[el * (P + 1) + P] = run;
    pl.recv_count[el] = run < cap ? run : cap;
    if (run > cap) atomicAdd(pl.dropped, run - cap);
  }
  __syncthreads();
  for (int s = tid; s < P; s += blockDim.x) {
    // entries of source s that fit into my experts' buffers (what will arrive from s)
    int exp_in = 0;
    for (int el = 0; el < Epr; ++el) {
      int a = pl.src_start[el * (P + 1) + s], b = pl.src_start[el * (P + 1) + s + 1];
      a = a < cap ? a : cap;
      b = b < cap ? b : cap;
      exp_in += b - a;
    }
    pl.expect_from[s] = exp_in;
    // my entries that fit into PE s's experts (what comes back from s in the combine)
    int out = 0;
    for (int el = 0; el < Epr; ++el) {
      int e = s * Epr + el;
      int a = 0;
      for (int q = 0; q < me; ++q) a += counts_all[q * E + e];
      int b = a + counts_all[me * E + e];
      a = a < cap ? a : cap;
      b = b < cap ? b : cap;
      out += b - a;
    }
    pl.send_to[s] = out;
    // recycle the other parity's arrival words for the next call
    for (int which = 0; which < 4; ++which) pl.arrive_sig[(parity ^ 1) * 4 * P + which * P + s] = 0;
  }
}

// ---------------------------------------------------------------------------------------
// dispatch: entry i = token * topk + k  →  row of the destination expert's receive buffer
// ---------------------------------------------------------------------------------------
template <bool kScale>
__global__ void __launch_bounds__(256) k_dispatch(State st, MoePlanDev pl, const bf16* __restrict__ rows, const float* __restrict__ scale,
                                                  const int* __restrict__ topk_idx, const int* __restrict__ pos, int n_entries, int topk,
                                                  int H, char* recv_sym, int* meta_sym, int parity, int which_sig) {
  __shared__ int sent[BSHMEM_MAX_PES];
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int Epr = pl.E / pl.P;
  if (threadIdx.x < BSHMEM_MAX_PES) sent[threadIdx.x] = 0;
  __syncthreads();
  const size_t row_bytes = (size_t)H * 2;
  for (int i = blockIdx.x * warps_per_block + (threadIdx.x >> 5); i < n_entries; i += gridDim.x * warps_per_block) {
    int e = topk_idx[i];
    int slot = pl.base_me[e] + pos[i];
    if (slot >= pl.cap) continue;                       // over capacity: dropped (counted in k_offsets)
    int r = e / Epr, el = e - r * Epr;
    const char* src = reinterpret_cast<const char*>(rows) + (size_t)(i / topk) * row_bytes;
    char* dst = dev::ptr(st, recv_sym, r) + ((size_t)el * pl.cap + slot) * row_bytes;
    if (!kScale) {
      dev::copy_bytes<dev::WARP>(dst, src, row_bytes);
    } else {
      const float w = scale[i];
      const uint4* s4 = reinterpret_cast<const uint4*>(src);
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      for (int v = lane; v < H / 8; v += 32) {
        uint4 xv = s4[v];
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&xv);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float2 f = __bfloat1622float2(h[q]);
          h[q] = __floats2bfloat162_rn(f.x * w, f.y * w);
        }
        d4[v] = xv;
      }
    }
    if (lane == 0) {
      if (meta_sym) dev::ptr(st, meta_sym, r)[el * pl.cap + slot] = (pl.me << 26) | i;
      atomicAdd(&sent[r], 1);
    }
  }
  // publish: every warp's stores, then one release-add per destination from this CTA
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < pl.P && sent[threadIdx.x] > 0) {
    int r = threadIdx.x;
    unsigned long long* sig = dev::ptr(st, pl.arrive_sig, r) + (size_t)parity * 4 * pl.P + (size_t)which_sig * pl.P + pl.me;
    ptx::fence_acq_rel_sys();
    ptx::red_release_sys_add_u64(reinterpret_cast<uint64_t*>(sig), (uint64_t)sent[r]);
  }
}

// Bounded wait until everything this PE expects has arrived (word s counts rows from PE s).
__global__ void k_wait_arrivals(MoePlanDev pl, int parity, int which_sig, const int* __restrict__ expected, unsigned long long timeout_ns,
                                int* err) {
  int s = threadIdx.x;
  if (s >= pl.P) return;
  const unsigned long long* sig = pl.arrive_sig + (size_t)parity * 4 * pl.P + (size_t)which_sig * pl.P + s;
  unsigned long long want = (unsigned long long)expected[s];
  unsigned long long t0 = ptx::globaltimer();
  while (ptx::ld_acquire_sys_u64(reinterpret_cast<const uint64_t*>(sig)) < want) {
    if (ptx::globaltimer() - t0 > timeout_ns) { atomicCAS(err, 0, 201 + which_sig); return; }
    __nanosleep(200);
  }
}

// combine_send: expert PE returns row (el, slot) to the entry buffer of the PE that sent it
__global__ void __launch_bounds__(256) k_combine_send(State st, MoePlanDev pl, const bf16* __restrict__ y, const int* __restrict__ meta,
                                                      int H, char* ybuf_sym, int parity, int which_sig) {
  __shared__ int sent[BSHMEM_MAX_PES];
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int Epr = pl.E / pl.P;
  if (threadIdx.x < BSHMEM_MAX_PES) sent[threadIdx.x] = 0;
  __syncthreads();
  const size_t row_bytes = (size_t)H * 2;
  const int total_rows = Epr * pl.cap;
  for (int rix = blockIdx.x * warps_per_block + (threadIdx.x >> 5); rix < total_rows; rix += gridDim.x * warps_per_block) {
    int el = rix / pl.cap, slot = rix - el * pl.cap;
    if (slot >= pl.recv_count[el]) continue;
    int m = meta[rix];
    int src_pe = m >> 26, entry = m & ((1 << 26) - 1);
    char* dst = dev::ptr(st, ybuf_sym, src_pe) + (size_t)entry * row_bytes;
    dev::copy_bytes<dev::WARP>(dst, reinterpret_cast<const char*>(y) + (size_t)rix * row_bytes, row_bytes);
    if (lane == 0) atomicAdd(&sent[src_pe], 1);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < pl.P && sent[threadIdx.x] > 0) {
    int r = threadIdx.x;
    unsigned long long* sig = dev::ptr(st, pl.arrive_sig, r) + (size_t)parity * 4 * pl.P + (size_t)which_sig * pl.P + pl.me;
    ptx::fence_acq_rel_sys();
    ptx::red_release_sys_add_u64(reinterpret_cast<uint64_t*>(sig), (uint64_t)sent[r]);
  }
}

// out[token] = sum_k w[entry] * ybuf[entry]   (entries over capacity contribute nothing)
// With `dlog` (backward pass only): out[token] += sum_k dlog[entry] * wr[expert of entry] — the gradient that reaches
// the layer input through the router logits, added here so that d_x is written once.
template <bool kWeighted>
__global__ void k_combine_reduce(MoePlanDev pl, const bf16* __restrict__ ybuf, const float* __restrict__ w, const int* __restrict__ topk_idx,
                                 const int* __restrict__ pos, int T, int topk, int H, bf16* __restrict__ out,
                                 const float* __restrict__ dlog = nullptr, const bf16* __restrict__ wr = nullptr) {
  const int token = blockIdx.x;
  if (token >= T) return;
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = 0; k < topk; ++k) {
      int i = token * topk + k;
      int e = topk_idx[i];
      if (pl.base_me[e] + pos[i] >= pl.cap) continue;
      float wk = kWeighted ? w[i] : 1.f;
      uint4 yv = ptx::ld_relaxed_v4(reinterpret_cast<const uint4*>(ybuf + (size_t)i * H) + v);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&yv);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float2 f = __bfloat1622float2(h[q]);
        acc[2 * q] += wk * f.x;
        acc[2 * q + 1] += wk * f.y;
      }
    }
    if (dlog != nullptr) {
      for (int k = 0; k < topk; ++k) {
        const int i = token * topk + k;
        const float g = dlog[i];
        uint4 wv = __ldg(reinterpret_cast<const uint4*>(wr + (size_t)topk_idx[i] * H) + v);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float2 f = __bfloat1622float2(h[q]);
          acc[2 * q] += g * f.x;
          acc[2 * q + 1] += g * f.y;
        }
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) oh[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    reinterpret_cast<uint4*>(out + (size_t)token * H)[v] = o;
  }
}

// d_w[entry] = <ybuf[entry], d_out[token]>   (gradient of the routing weight)
__global__ void k_router_weight_grad(MoePlanDev pl, const bf16* __restrict__ ybuf, const bf16* __restrict__ dout, const int* __restrict__ topk_idx,
                                     const int* __restrict__ pos, int n_entries, int topk, int H, float* __restrict__ dw) {
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (i >= n_entries) return;
  float acc = 0.f;
  if (pl.base_me[topk_idx[i]] + pos[i] < pl.cap) {
    const uint4* a = reinterpret_cast<const uint4*>(ybuf + (size_t)i * H);
    const uint4* b = reinterpret_cast<const uint4*>(dout + (size_t)(i / topk) * H);
    for (int v = lane; v < H / 8; v += 32) {
      uint4 av = ptx::ld_relaxed_v4(a + v), bv = b[v];
      const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&av);
      const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float2 x = __bfloat1622float2(ah[q]), y = __bfloat1622float2(bh[q]);
        acc += x.x * y.x + x.y * y.y;
      }
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) dw[i] = acc;
}

// Router backward.  The routing weights are a softmax over the chosen experts' logits (softmax over all experts,
// renormalised over the top-k), so only the chosen logits receive a gradient:
//   d_logit[entry k] = w_k * (d_w_k - sum_j w_j * d_w_j)
__global__ void k_router_dlogits(const float* __restrict__ w, const float* __restrict__ dw, int T, int topk, float* __restrict__ dlog) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float s = 0.f;
  for (int k = 0; k < topk; ++k) s += w[t * topk + k] * dw[t * topk + k];
  for (int k = 0; k < topk; ++k) dlog[t * topk + k] = w[t * topk + k] * (dw[t * topk + k] - s);
}

// d_Wr[e, :] += sum over the CTA's tokens routed to e of d_logit * x[token, :]   (fp32 accumulation, atomics across CTAs).
// A CTA takes kTok tokens and 2048 columns; its (token, k) entries are first bucketed by expert in shared memory, so
// the loads of the hit rows can be issued back to back.
constexpr int kDwrTok = 128;
__global__ void __launch_bounds__(256) k_router_dwr(const bf16* __restrict__ x, const int* __restrict__ topk_idx, const float* __restrict__ dlog,
                                                   int T, int H, int E, int topk, float* __restrict__ dwr) {
  __shared__ int cnt[64], start[65], fill[64];
  __shared__ int ent[kDwrTok * 8];
  const int t0 = blockIdx.x * kDwrTok;
  const int nt = min(kDwrTok, T - t0);
  const int n_ent = nt * topk;
  if (threadIdx.x < 64) { cnt[threadIdx.x] = 0; fill[threadIdx.x] = 0; }
  __syncthreads();
  for (int i = threadIdx.x; i < n_ent; i += blockDim.x) atomicAdd(&cnt[topk_idx[t0 * topk + i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int a = 0;
    for (int e = 0; e < E; ++e) { start[e] = a; a += cnt[e]; }
    start[E] = a;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_ent; i += blockDim.x) {
    const int e = topk_idx[t0 * topk + i];
    ent[start[e] + atomicAdd(&fill[e], 1)] = i;
  }
  __syncthreads();
  const int col = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (col >= H) return;
  for (int e = 0; e < E; ++e) {
    const int b = start[e], n = start[e + 1] - b;
    if (n == 0) continue;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int j0 = 0; j0 < n; j0 += 4) {
      uint4 xv[4];
      float g[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = ent[b + min(j0 + u, n - 1)];
        g[u] = j0 + u < n ? dlog[t0 * topk + i] : 0.f;
        xv[u] = *reinterpret_cast<const uint4*>(x + (size_t)(t0 + i / topk) * H + col);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&xv[u]);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float2 f = __bfloat1622float2(h[q]);
          acc[2 * q] += g[u] * f.x;
          acc[2 * q + 1] += g[u] * f.y;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(&dwr[(size_t)e * H + col + j], acc[j]);
  }
}

__global__ void k_f32_to_bf16(const float* __restrict__ in, bf16* __restrict__ out, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = __float2bfloat16_rn(in[i]);
}

// ---------------------------------------------------------------------------------------
// SwiGLU on the interleaved gate/up layout: every 64 columns = 32 gate followed by 32 up
// ---------------------------------------------------------------------------------------
__global__ void k_swiglu_fwd(const bf16* __restrict__ gu, const int* __restrict__ counts, int cap, int F, bf16* __restrict__ h) {
  const int row = blockIdx.x;
  const int el = row / cap;
  if (row - el * cap >= counts[el]) return;
  const bf16* g = gu + (size_t)row * 2 * F;
  bf16* o = h + (size_t)row * F;
  for (int c = threadIdx.x; c < F / 8; c += blockDim.x) {     // 8 outputs per thread
    int blk = (c * 8) / 32, in = (c * 8) % 32;
    uint4 gv = *reinterpret_cast<const uint4*>(g + blk * 64 + in);
    uint4 uv = *reinterpret_cast<const uint4*>(g + blk * 64 + 32 + in);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 gf = __bfloat1622float2(gh[q]), uf = __bfloat1622float2(uh[q]);
      oh[q] = __floats2bfloat162_rn(gf.x / (1.f + __expf(-gf.x)) * uf.x, gf.y / (1.f + __expf(-gf.y)) * uf.y);
    }
    *reinterpret_cast<uint4*>(o + c * 8) = ov;
  }
}

// d_gu (interleaved) from d_h and the saved pre-activations
__global__ void k_swiglu_bwd(const bf16* __restrict__ gu, const bf16* __restrict__ dh, const int* __restrict__ counts, int cap, int F,
                             bf16* __restrict__ dgu) {
  const int row = blockIdx.x;
  const int el = row / cap;
  if (row - el * cap >= counts[el]) return;
  const bf16* g = gu + (size_t)row * 2 * F;
  const bf16* d = dh + (size_t)row * F;
  bf16* o = dgu + (size_t)row * 2 * F;
  for (int c = threadIdx.x; c < F / 8; c += blockDim.x) {
    int blk = (c * 8) / 32, in = (c * 8) % 32;
    uint4 gv = *reinterpret_cast<const uint4*>(g + blk * 64 + in);
    uint4 uv = *reinterpret_cast<const uint4*>(g + blk * 64 + 32 + in);
    uint4 dv = *reinterpret_cast<const uint4*>(d + c * 8);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uv);
    const __nv_bfloat162* dhh = reinterpret_cast<const __nv_bfloat162*>(&dv);
    uint4 og, ou;
    __nv_bfloat162* ogh = reinterpret_cast<__nv_bfloat162*>(&og);
    __nv_bfloat162* ouh = reinterpret_cast<__nv_bfloat162*>(&ou);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 gf = __bfloat1622float2(gh[q]), uf = __bfloat1622float2(uh[q]), df = __bfloat1622float2(dhh[q]);
      float sx = 1.f / (1.f + __expf(-gf.x)), sy = 1.f / (1.f + __expf(-gf.y));
      float silx = gf.x * sx, sily = gf.y * sy;
      // d silu(g)/dg = s * (1 + g * (1 - s))
      ogh[q] = __floats2bfloat162_rn(df.x * uf.x * sx * (1.f + gf.x * (1.f - sx)), df.y * uf.y * sy * (1.f + gf.y * (1.f - sy)));
      ouh[q] = __floats2bfloat162_rn(df.x * silx, df.y * sily);
    }
    *reinterpret_cast<uint4*>(o + blk * 64 + in) = og;
    *reinterpret_cast<uint4*>(o + blk * 64 + 32 + in) = ou;
  }
}

// out[c][r] = in[r][c] for r < rows_valid (per expert region), zero for rows_valid <= r < ld_out:
// the zero padding makes the ragged K extent of the weight-gradient GEMMs harmless.
__global__ void k_transpose_pad(const bf16* __restrict__ in, const int* __restrict__ counts, int cap, int cols, bf16* __restrict__ out) {
  __shared__ bf16 tile[32][33];
  const int el = blockIdx.z;
  const int valid = counts[el];
  const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
  const bf16* src = in + (size_t)el * cap * cols;
  bf16* dst = out + (size_t)el * cols * cap;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int r = r0 + j, c = c0 + threadIdx.x;
    tile[j][threadIdx.x] = (r < valid && c < cols) ? src[(size_t)r * cols + c] : __float2bfloat16(0.f);
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int c = c0 + j, r = r0 + threadIdx.x;
    if (c < cols && r < cap) dst[(size_t)c * cap + r] = tile[threadIdx.x][j];
  }
}

thread_local std::string g_err;
#define RT_TRY(call) do { cudaError_t _e = (call); if (_e != cudaSuccess) { g_err = std::string(#call) + ": " + cudaGetErrorString(_e); return 7; } } while (0)

}  // namespace

extern "C" {

const char* bshmem_moe_last_error() { return g_err.c_str(); }

int bshmem_moe_router_topk(const void* x, const void* wr, int T, int H, int E, int topk, int* topk_idx, float* topk_w, float* probs,
                           void* stream) {
  if (E > 64 || topk > 8 || topk > E || H % 8) { g_err = "router: E <= 64, topk <= min(8, E), H % 8 == 0"; return 1; }
  int threads = 256, blocks = (T * 32 + threads - 1) / threads;
  k_router_topk<<<blocks, threads, 0, (cudaStream_t)stream>>>((const bf16*)x, (const bf16*)wr, T, H, E, topk, topk_idx, topk_w, probs);
  RT_TRY(cudaGetLastError());
  return 0;
}

int bshmem_moe_plan(const int* topk_idx, int n_entries, int E, int* pos, int* counts, void* stream) {
  k_plan<<<E, 1024, 0, (cudaStream_t)stream>>>(topk_idx, n_entries, pos, counts);
  RT_TRY(cudaGetLastError());
  return 0;
}

int bshmem_moe_offsets(const MoePlanDev* pl, const int* counts_all, int parity, void* stream) {
  k_offsets<<<1, 128, 0, (cudaStream_t)stream>>>(*pl, counts_all, parity);
  RT_TRY(cudaGetLastError());
  return 0;
}

// rows: [T, H] bf16 token rows (x, or d_out in the backward pass with scale = routing weights)
int bshmem_moe_dispatch(const bshmem_dev_state_t* st, const MoePlanDev* pl, const void* rows, const float* scale, const int* topk_idx,
                        const int* pos, int n_entries, int topk, int H, void* recv_sym, int* meta_sym, int parity, int which_sig, int ctas,
                        void* stream) {
  if (H % 8) { g_err = "dispatch: H % 8 != 0"; return 1; }
  if (ctas < 1) ctas = 1;
  if (scale)
    k_dispatch<true><<<ctas, 256, 0, (cudaStream_t)stream>>>(*st, *pl, (const bf16*)rows, scale, topk_idx, pos, n_entries, topk, H,
                                                             (char*)recv_sym, meta_sym, parity, which_sig);
  else
    k_dispatch<false><<<ctas, 256, 0, (cudaStream_t)stream>>>(*st, *pl, (const bf16*)rows, nullptr, topk_idx, pos, n_entries, topk, H,
                                                              (char*)recv_sym, meta_sym, parity, which_sig);
  RT_TRY(cudaGetLastError());
  return 0;
}

int bshmem_moe_wait_arrivals(const MoePlanDev* pl, int parity, int which_sig, const int* expected, int timeout_ms, int* err, void* stream) {
  k_wait_arrivals<<<1, 32, 0, (cudaStream_t)stream>>>(*pl, parity, which_sig, expected, (unsigned long long)timeout_ms * 1000000ull, err);
  RT_TRY(cudaGetLastError());
  return 0;
}

int bshmem_moe_combine_send(const bshmem_dev_state_t* st, const MoePlanDev* pl, const void* y, const int* meta, int H, void* ybuf_sym,
                            int parity, int which_sig, int ctas, void* stream) {
  if (ctas < 1) ctas = 1;
  k_combine_send<<<ctas, 256, 0, (cudaStream_t)stream>>>(*st, *pl, (const bf16*)y, meta, H, (char*)ybuf_sym, parity, which_sig);
  RT_TRY(cudaGetLastError());
  return 0;
}

int bshmem_moe_combine_reduce(const MoePlanDev* pl, const void* ybuf, const float* w, const int* topk_idx, const int* pos, int T, int topk,
                              int H, void* out, void* stream) {
  if (w) k_combine_reduce<true><<<T, 256, 0, (cudaStream_t)stream>>>(*pl, (const bf16*)ybuf, w, topk_idx, pos, T, topk, H, (bf16*)out);
  else k_combine_reduce<false><<<T, 256, 0, (cudaStream_t)stream>>>(*pl, (const bf16*)ybuf, nullptr, topk_idx, pos, T, topk, H, (bf16*)out);
  RT_TRY(cudaGetLastError());
  return 0;
}

// The same reduction for the backward pass's closing step, plus the router term (see k_combine_reduce).
int bshmem_moe_combine_reduce_router(const MoePlanDev* pl, const void* ybuf, const int* topk_idx, const int* pos, int T, int topk, int H,
                                     void* out, const float* dlog, const void* wr, void* stream) {
  k_combine_reduce<false><<<T, 256, 0, (cudaStream_t)stream>>>(*pl, (const bf16*)ybuf, nullptr, topk_idx, pos, T, topk, H, (bf16*)out, dlog,
                                                                (const bf16*)wr);
  RT_TRY(cudaGetLastError());
  return 0;
}

// Router backward: d_logits of the chosen experts [T * topk] from the routing weights and their gradient, then
// d_Wr [E, H] = d_logits^T · x (accumulated in the fp32 scratch `dwr_f32`, which this call clears first) as bf16.
int bshmem_moe_router_backward(const void* x, const int* topk_idx, const float* topk_w, const float* dtopk_w, int T, int H, int E, int topk,
                               float* dlog, float* dwr_f32, void* dwr, void* stream) {
  if (E > 64 || topk > 8 || H % 8) { g_err = "router backward: at most 64 experts, top-8, H % 8 == 0"; return 1; }
  cudaStream_t st = (cudaStream_t)stream;
  k_router_dlogits<<<(T + 255) / 256, 256, 0, st>>>(topk_w, dtopk_w, T, topk, dlog);
  RT_TRY(cudaGetLastError());
  RT_TRY(cudaMemsetAsync(dwr_f32, 0, sizeof(float) * (size_t)E * H, st));
  dim3 grid((T + kDwrTok - 1) / kDwrTok, (H + 2047) / 2048);
  k_router_dwr<<<grid, 256, 0, st>>>((const bf16*)x, topk_idx, dlog, T, H, E, topk, dwr_f32);
  RT_TRY(cudaGetLastError());
  k_f32_to_bf16<<<64, 256, 0, st>>>(dwr_f32, (bf16*)dwr, (size_t)E * H);
  RT_TRY(cudaGetLastError());
  return 0;
}

int bshmem_moe_router_weight_grad(const MoePlanDev* pl, const void* ybuf, const void* dout, const int* topk_idx, const int* pos, int n_entries,
                                  int topk, int H, float* dw, void* stream) {
  int threads = 256, blocks = (n_entries * 32 + threads - 1) / threads;
  k_router_weight_grad<<<blocks, threads, 0, (cudaStream_t)stream>>>(*pl, (const bf16*)ybuf, (const bf16*)dout, topk_idx, pos, n_entries, topk, H, dw);
  RT_TRY(cudaGetLastError());
  return 0;
}

int bshmem_moe_swiglu_fwd(const void* gu, const int* counts, int groups, int cap, int F, void* h, void* stream) {
  if (F % 32) { g_err = "swiglu: F % 32 != 0"; return 1; }
  k_swiglu_fwd<<<groups * cap, 256, 0, (cudaStream_t)stream>>>((const bf16*)gu, counts, cap, F, (bf16*)h);
  RT_TRY(cudaGetLastError());
  return 0;
}

int bshmem_moe_swiglu_bwd(const void* gu, const void* dh, const int* counts, int groups, int cap, int F, void* dgu, void* stream) {
  if (F % 32) { g_err = "swiglu: F % 32 != 0"; return 1; }
  k_swiglu_bwd<<<groups * cap, 256, 0, (cudaStream_t)stream>>>((const bf16*)gu, (const bf16*)dh, counts, cap, F, (bf16*)dgu);
  RT_TRY(cudaGetLastError());
  return 0;
}

// in: [groups][cap][cols] → out: [groups][cols][cap], rows beyond counts[g] become zero columns
int bshmem_moe_transpose_pad(const void* in, const int* counts, int groups, int cap, int cols, void* out, void* stream) {
  dim3 grid((cols + 31) / 32, (cap + 31) / 32, groups), block(32, 8);
  k_transpose_pad<<<grid, block, 0, (cudaStream_t)stream>>>((const bf16*)in, counts, cap, cols, (bf16*)out);
  RT_TRY(cudaGetLastError());
  return 0;
}

}  // extern "C"
