// Stitch of a segment-parallel scan: chains the segments' summaries (B, M) of every (sequence, value head) in walk
// order and writes the state each segment's real walk starts from,
//     S_next = B                 after a segment that started from the sequence's boundary state, or whose gates let
//                                the warm-up rule apply (M taken as zero),
//     S_next = M S + B           otherwise (fp32 FMA, fixed order),
// forward from the sequence's initial state, or in reverse from its final adjoint state (reference:
// miles_ext_kernels/cake/_impl/gdn/ops.py:1601-1613).  CTAs per (sequence, value head, slice of the state's columns);
// the running state lives in shared memory.  The same chain composes the summary of a whole run of segments (context parallelism: a rank's
// (B, M)) and folds the ranks' summaries into the state that enters a rank.
#include "common.cuh"
#include "scan_plan.cuh"

namespace mek {

constexpr int kStitchCols = 32;  // columns of the state per CTA (grid.z = 128 / kStitchCols)

// mode bits: 1 = start from the identity instead of the boundary state; 2 = leave the offsets out (B := 0);
// 4 = every segment started from zero, the first too.  Modes 4 and 5 | 2 compose the summary of a whole run of
// segments (its B, then its M); mode 0 with rank summaries as the "segments" folds a chain of ranks.
// `final_pitch`: floats between the final states of consecutive (sequence, value head) pairs (16384: packed).
// `compose`: the grid's upper half of blockIdx.z runs mode 7 into final_out + 16384 while the lower half runs
// `mode`: the (B, M) pair of a run of segments in one launch, interleaved per head.
__global__ void __launch_bounds__(256) scan_stitch_kernel(
    const float* __restrict__ summary, const float* __restrict__ boundary, const float* __restrict__ g_cs,
    float* __restrict__ seg_state, float* __restrict__ final_out, const int32_t* __restrict__ chunk_start,
    const int32_t* __restrict__ chunk_len, const int32_t* __restrict__ seg_chunk_start,
    const int32_t* __restrict__ seq_seg_start, int num_v_heads, int reverse, int warm_chunks, float warm_log2,
    int mode, int64_t final_pitch, int compose) {
  extern __shared__ float s_state[];  // [128][kStitchCols]: this CTA's columns of the state
  const int n = blockIdx.x, hv = blockIdx.y, tid = threadIdx.x;
  constexpr int kSlices = 128 / kStitchCols;
  const int slice = int(blockIdx.z) % kSlices;
  if (compose != 0 && int(blockIdx.z) >= kSlices) {
    mode = 7;
    final_out += 16384;
  }
  const int seg_begin = seq_seg_start[n], seg_end = seq_seg_start[n + 1];
  const ScanPlan plan = {nullptr, nullptr, nullptr, warm_chunks, warm_log2};
  // the columns of a state are independent of one another (S' = M S + B column by column): blockIdx.z picks
  // kStitchCols of the 128, so that a call with few chains still fills the SMs.  A thread owns half of its row's slice.
  constexpr int kHalf = kStitchCols / 2, kVec = kHalf / 4;
  const int col0 = slice * kStitchCols;
  const int r = tid >> 1, c0 = (tid & 1) * kHalf;  // row; first column inside the slice

  // the state the walk starts from
  for (int i = tid; i < 128 * (kStitchCols / 4); i += 256) {
    const int row = i / (kStitchCols / 4), col = col0 + (i % (kStitchCols / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (mode & 1) {
      v = make_float4(row == col ? 1.f : 0.f, row == col + 1 ? 1.f : 0.f, row == col + 2 ? 1.f : 0.f,
                      row == col + 3 ? 1.f : 0.f);
    } else if (boundary != nullptr) {
      v = *reinterpret_cast<const float4*>(boundary + (int64_t(n) * num_v_heads + hv) * 16384 + row * 128 + col);
    }
    reinterpret_cast<float4*>(s_state)[i] = v;
  }
  __syncthreads();

  auto store_state = [&](float* out) {  // this CTA's columns of a [128][128] state
    for (int i = tid; i < 128 * (kStitchCols / 4); i += 256) {
      const int row = i / (kStitchCols / 4), col = col0 + (i % (kStitchCols / 4)) * 4;
      *reinterpret_cast<float4*>(out + row * 128 + col) = reinterpret_cast<float4*>(s_state)[i];
    }
  };
  const int count = seg_end - seg_begin;
  for (int step = 0; step < count; ++step) {
    const int s = reverse ? seg_end - 1 - step : seg_begin + step;
    if (seg_state != nullptr) store_state(seg_state + (int64_t(s) * num_v_heads + hv) * 16384);
    if (step + 1 == count && final_out == nullptr) break;
    const float* b_mat = summary + (int64_t(s) * num_v_heads + hv) * 2 * 16384;
    const float* m_mat = b_mat + 16384;
    const bool inner = (mode & 4) != 0 || step > 0;
    // the segment table is read only under the warm-up rule: a fold over rank summaries (warm_chunks = 0) numbers
    // its "segments" along the gathered chain, which can be longer than any local table
    const bool replace = !inner || (warm_chunks > 0 &&
                                    warm_up_suffices(plan, g_cs, chunk_start, chunk_len, seg_chunk_start[s],
                                                     seg_chunk_start[s + 1], num_v_heads, hv, reverse != 0));
    float acc[kHalf];
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (!(mode & 2)) b = reinterpret_cast<const float4*>(b_mat + r * 128 + col0 + c0)[j];
      acc[4 * j] = b.x, acc[4 * j + 1] = b.y, acc[4 * j + 2] = b.z, acc[4 * j + 3] = b.w;
    }
    if (!replace) {
      for (int k0 = 0; k0 < 128; k0 += 4) {
        const float4 m4 = *reinterpret_cast<const float4*>(m_mat + r * 128 + k0);
        const float mv[4] = {m4.x, m4.y, m4.z, m4.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float4* row = reinterpret_cast<const float4*>(s_state + (k0 + t) * kStitchCols + c0);
#pragma unroll
          for (int j = 0; j < kVec; ++j) {
            const float4 x = row[j];
            acc[4 * j] = fmaf(mv[t], x.x, acc[4 * j]);
            acc[4 * j + 1] = fmaf(mv[t], x.y, acc[4 * j + 1]);
            acc[4 * j + 2] = fmaf(mv[t], x.z, acc[4 * j + 2]);
            acc[4 * j + 3] = fmaf(mv[t], x.w, acc[4 * j + 3]);
          }
        }
      }
    }
    __syncthreads();  // every thread has read the old state
#pragma unroll
    for (int j = 0; j < kVec; ++j)
      reinterpret_cast<float4*>(s_state + r * kStitchCols + c0)[j] =
          make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
    __syncthreads();
  }
  if (final_out != nullptr) store_state(final_out + (int64_t(n) * num_v_heads + hv) * final_pitch);
}

}  // namespace mek

extern "C" int mek_gdn_scan_stitch(const MekGdnDims* seg_dims, int num_seqs, const int32_t* seq_seg_start,
                                   const float* summary, const float* boundary, const float* g_cs, float* seg_state,
                                   float* final_out, int reverse, int warm_chunks, float warm_log2, int mode,
                                   void* stream) {
  using namespace mek;
  if (seg_dims == nullptr || num_seqs <= 0 || seg_dims->num_v_heads <= 0 || !seq_seg_start || !summary ||
      (!seg_state && !final_out) || warm_chunks < 0 || mode < 0 || mode > 7)
    return fail(MEK_ERR_INVALID, "scan_stitch: a null pointer, bad extents or an unknown mode");
  if (warm_chunks > 0 && (!g_cs || !seg_dims->seq_chunk_start || !seg_dims->chunk_start || !seg_dims->chunk_len))
    return fail(MEK_ERR_INVALID, "scan_stitch: the warm-up rule needs the gates and the chunk tables");
  const size_t smem = 128 * kStitchCols * sizeof(float);
  if (int rc = want_smem(scan_stitch_kernel, smem, "scan_stitch")) return rc;
  scan_stitch_kernel<<<dim3(num_seqs, seg_dims->num_v_heads, 128 / kStitchCols), 256, smem,
                       static_cast<cudaStream_t>(stream)>>>(
      summary, boundary, g_cs, seg_state, final_out, seg_dims->chunk_start, seg_dims->chunk_len,
      seg_dims->seq_chunk_start, seq_seg_start, seg_dims->num_v_heads, reverse, warm_chunks, warm_log2, mode, 16384, 0);
  return launched("scan_stitch");
}

extern "C" int mek_gdn_scan_compose(const MekGdnDims* seg_dims, const int32_t* seq_seg_start, const float* summary,
                                    const float* g_cs, float* out, int reverse, int warm_chunks, float warm_log2,
                                    void* stream) {
  using namespace mek;
  if (seg_dims == nullptr || seg_dims->num_v_heads <= 0 || !seq_seg_start || !summary || !out || warm_chunks < 0)
    return fail(MEK_ERR_INVALID, "scan_compose: a null pointer or bad extents");
  if (warm_chunks > 0 && (!g_cs || !seg_dims->seq_chunk_start || !seg_dims->chunk_start || !seg_dims->chunk_len))
    return fail(MEK_ERR_INVALID, "scan_compose: the warm-up rule needs the gates and the chunk tables");
  const size_t smem = 128 * kStitchCols * sizeof(float);
  if (int rc = want_smem(scan_stitch_kernel, smem, "scan_compose")) return rc;
  scan_stitch_kernel<<<dim3(1, seg_dims->num_v_heads, 2 * (128 / kStitchCols)), 256, smem,
                       static_cast<cudaStream_t>(stream)>>>(
      summary, nullptr, g_cs, nullptr, out, seg_dims->chunk_start, seg_dims->chunk_len, seg_dims->seq_chunk_start,
      seq_seg_start, seg_dims->num_v_heads, reverse, warm_chunks, warm_log2, 4, 2 * 16384, 1);
  return launched("scan_compose");
}
