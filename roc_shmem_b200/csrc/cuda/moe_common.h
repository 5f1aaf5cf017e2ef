// moe_common.h — plan structure shared by the MoE kernels and the grouped expert GEMM.
#pragma once
#include <stdint.h>

// Everything a PE needs to know to move one call's tokens: filled by the `offsets` kernel from
// the gathered per-expert counts.  All arrays live in device memory; `arrive_sig` is symmetric.
typedef struct {
  int P, E, me, cap;               // PEs, experts, my PE, rows per expert buffer
  int* base_me;                    // [E]    first slot of my entries inside expert e's buffer
  int* src_start;                  // [E/P][P+1] prefix of rows per source PE inside my experts' buffers
  int* recv_count;                 // [E/P]  rows that arrive for my expert (clamped to cap)
  int* expect_from;                // [P]    rows PE s sends me (dispatch) / I must return to s
  int* send_to;                    // [P]    rows I send to PE s = rows that come back from s
  int* dropped;                    // [1]    rows over capacity (counted at the receiver)
  unsigned long long* arrive_sig;  // symmetric [2 parities][4 phases][P]: rows landed from PE s
} MoePlanDev;

enum { MOE_SIG_FWD_DISPATCH = 0, MOE_SIG_FWD_COMBINE = 1, MOE_SIG_BWD_DISPATCH = 2, MOE_SIG_BWD_COMBINE = 3 };
