// Segment-parallel scans: what the two scan kernels and the stitch kernel share.
//
// One chunk step of either scan is affine in the state: S' = M_c S + B_c (forward: M_c = gamma I - K^T diag(rs) W;
// adjoint: the same with the roles of k / w exchanged), so a segment of chunks has a summary (B, M) with
// S_out = M S_in + B.  A long sequence is cut into segments; a pre-scan computes every segment's summary in parallel
// (the offset walk from a zero state gives B, the transfer walk from the identity with the inhomogeneous operand
// zeroed gives M), a stitch chains the summaries in sequence order, and the real walk then runs all segments in
// parallel from their true start states (reference: miles_ext_kernels/cake/_impl/gdn/ops.py:405-531, 1191-1317,
// 1601-1613).
//
// Warm-up rule: when the summed gate of the `warm_chunks` chunks a state passes last on its way out of a segment is
// below `warm_log2` (log2 domain; -10 nats by default), whatever entered the segment is scaled below 2^warm_log2 on
// the way out: the offset walk then covers those chunks only and M is taken as zero.  Every party evaluates the
// same test on the same values, in the same order.
#pragma once

#include <stdint.h>

namespace mek {

struct ScanPlan {
  const int32_t* seg_flags;  // null: an ordinary walk.  Else a pre-scan over segments; per segment:
                             //   bit 0  inner: the walk starts from zero / the identity (else from `state_row`'s state)
                             //   bit 1  skip: no summary is needed (the sequence's last segment in walk order)
  const int32_t* state_row;  // pre-scan: per segment, the row of the boundary-state tensor a non-inner walk starts from
  float* summary;            // pre-scan: fp32 [segments][HV][2][128][128]: B, then M
  int warm_chunks;           // 0 switches the warm-up rule off
  float warm_log2;
  const int32_t* seq_order;  // any walk: which sequence the CTA with blockIdx.x = i takes (null: sequence i)
};

// The gate a state accumulates over chunks [first, last): the chunk-end values of the chunk-local cumulative gate.
__device__ __forceinline__ float gate_over_chunks(const float* g_cs, const int32_t* chunk_start,
                                                  const int32_t* chunk_len, int first, int last, int num_v_heads,
                                                  int hv) {
  float sum = 0.f;
  for (int c = first; c < last; ++c)
    sum += g_cs[int64_t(chunk_start[c] + chunk_len[c] - 1) * num_v_heads + hv];
  return sum;
}

// Forward scans leave a segment through its last chunks, adjoint scans through its first.
__device__ __forceinline__ bool warm_up_suffices(const ScanPlan& plan, const float* g_cs, const int32_t* chunk_start,
                                                 const int32_t* chunk_len, int c_begin, int c_end, int num_v_heads,
                                                 int hv, bool reverse) {
  if (plan.warm_chunks <= 0 || c_end - c_begin <= plan.warm_chunks) return false;
  const int first = reverse ? c_begin : c_end - plan.warm_chunks;
  return gate_over_chunks(g_cs, chunk_start, chunk_len, first, first + plan.warm_chunks, num_v_heads, hv) <
         plan.warm_log2;
}

}  // namespace mek
