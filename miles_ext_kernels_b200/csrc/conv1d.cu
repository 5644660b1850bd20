// Packed causal depthwise conv1d (kernel size 4) + SiLU, forward and backward, sm_100a: the short convolution in
// front of the GDN / KDA op,
//     pre[t, c] = sum_{k<4} w[c, k] x[t - 3 + k, c]   (tokens before the document's first count as zero),
//     y = bf16(pre sigmoid(pre))
// (reference: miles_ext_kernels/cake/_impl/conv1d/ops.py:226-257; arithmetic and rounding points as in
// tests/cake/conv1d/test_conv1d_gpu.py:112-160).  HBM-bound: a warp walks a run of tokens for 256 channels (16 bytes
// per lane and token, 512 contiguous bytes per warp and token) with a sliding window in registers, so x is read once
// (plus a 3-token halo per run).
//
// Backward: dpre = dy silu'(p) with p the BF16-rounded preactivation ("bf16" policy, the rounding point of
// flash-linear-attention) or the unrounded one ("fp32" policy); dx[t] = sum_k w[c, k] dpre[t + 3 - k] inside the
// document; dw[c, k] = sum_t dpre[t] x[t - 3 + k].  The weight gradient is summed in a fixed order: per run in
// registers (FP32; under the fp32 policy FP32 over four tokens, then FP64), then over the runs in FP64 by a second launch.  The number of runs is
// a function of the token count alone: identical inputs give identical bits.
#include <type_traits>

#include "common.cuh"
#include "umma.cuh"

namespace mek {

constexpr int kConvTaps = 4;
constexpr int kConvMaxRuns = 128;

// Per token: how many earlier tokens of its document a tap may reach (0..3) in the low two bits, and how many later
// ones (0..3) in the next two.
__global__ void conv_reach_kernel(const int32_t* __restrict__ cu, int num_docs, int tokens, uint8_t* __restrict__ reach) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  int lo = 0, hi = num_docs;  // the document d with cu[d] <= t < cu[d + 1]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid;
  }
  // empty documents: several d share cu[d]; take the last one that starts at or before t
  while (lo + 1 < num_docs && cu[lo + 1] <= t) ++lo;
  const int before = min(t - cu[lo], 3), after = min(cu[lo + 1] - 1 - t, 3);
  reach[t] = uint8_t(max(before, 0) | (max(after, 0) << 2));
}

__device__ __forceinline__ void load8f(const __nv_bfloat16* p, float* v) {
  const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
  const float2 a = unpack_bf16(raw.x), b = unpack_bf16(raw.y), c = unpack_bf16(raw.z), d = unpack_bf16(raw.w);
  v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y, v[4] = c.x, v[5] = c.y, v[6] = d.x, v[7] = d.y;
}
__device__ __forceinline__ void unpack8(uint4 raw, float* v) {
  const float2 a = unpack_bf16(raw.x), b = unpack_bf16(raw.y), c = unpack_bf16(raw.z), d = unpack_bf16(raw.w);
  v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y, v[4] = c.x, v[5] = c.y, v[6] = d.x, v[7] = d.y;
}
__device__ __forceinline__ void store8f(__nv_bfloat16* p, const float* v) {
  *reinterpret_cast<uint4*>(p) =
      make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}
// w [C, 4] (fp32 or bf16) -> taps[k][j] of this lane's 8 channels
template <typename W, int CH = 8>
__device__ __forceinline__ void load_taps(const W* w, int c0, float taps[kConvTaps][CH]) {
#pragma unroll
  for (int j = 0; j < CH; ++j)
#pragma unroll
    for (int k = 0; k < kConvTaps; ++k) taps[k][j] = float(w[(c0 + j) * kConvTaps + k]);
}

// The FP32 preactivation in the order and with the roundings of the reference arithmetic -- oldest tap first, every
// product and every sum rounded on its own (no fused multiply-add) -- so that its BF16 rounding, at which the bf16
// policy evaluates SiLU', falls on the same side.
__device__ __forceinline__ float preactivation(float w0, float x3, float w1, float x2, float w2, float x1, float w3,
                                               float x0) {
  float pre = __fmul_rn(w0, x3);
  pre = __fadd_rn(pre, __fmul_rn(w1, x2));
  pre = __fadd_rn(pre, __fmul_rn(w2, x1));
  return __fadd_rn(pre, __fmul_rn(w3, x0));
}

__device__ __forceinline__ uint4 load_row(const __nv_bfloat16* base, int64_t t, int channels, int c0) {
  return __ldg(reinterpret_cast<const uint4*>(base + t * channels + c0));
}

// A thread's CH channels of one token: 16 bytes (CH = 8) or 8 bytes (CH = 4; half the registers per thread, so that
// two blocks fit an SM)
template <int CH>
struct ConvRow;
template <>
struct ConvRow<8> {
  typedef uint4 type;
  static __device__ __forceinline__ type load(const __nv_bfloat16* base, int64_t t, int channels, int c0) {
    return __ldg(reinterpret_cast<const uint4*>(base + t * channels + c0));
  }
  static __device__ __forceinline__ void unpack(type raw, float* v) { unpack8(raw, v); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) { store8f(p, v); }
};
template <>
struct ConvRow<4> {
  typedef uint2 type;
  static __device__ __forceinline__ type load(const __nv_bfloat16* base, int64_t t, int channels, int c0) {
    return __ldg(reinterpret_cast<const uint2*>(base + t * channels + c0));
  }
  static __device__ __forceinline__ void unpack(type raw, float* v) {
    const float2 a = unpack_bf16(raw.x), b = unpack_bf16(raw.y);
    v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
  }
};

// One token of the forward sweep.  kEdge = false: the token has three earlier tokens in its document (no selects).
template <bool kEdge, int CH>
__device__ __forceinline__ void conv_fwd_token(const float (&taps)[kConvTaps][CH], float (&win)[3][CH],
                                               typename ConvRow<CH>::type raw,
                                               int before, __nv_bfloat16* y_row) {
  float cur[CH], out[CH];
  ConvRow<CH>::unpack(raw, cur);
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const float x1 = !kEdge || before >= 1 ? win[2][j] : 0.f, x2 = !kEdge || before >= 2 ? win[1][j] : 0.f;
    const float x3 = !kEdge || before >= 3 ? win[0][j] : 0.f;
    // fused multiply-adds here (oldest tap first): y is rounded to BF16 and the backward, whose SiLU' must see the
    // reference's rounding of the preactivation, recomputes it in the reference's order
    const float pre = fmaf(taps[3][j], cur[j], fmaf(taps[2][j], x1, fmaf(taps[1][j], x2, taps[0][j] * x3)));
    out[j] = __fdividef(pre, 1.0f + __expf(-pre));
    win[0][j] = win[1][j], win[1][j] = win[2][j], win[2][j] = cur[j];
  }
  ConvRow<CH>::store(y_row, out);
}

// grid (runs, channel groups of 8 warps x 256); a warp owns tokens [run * run_len, + run_len) of 256 channels.  Tokens
// go in batches of four; the next batch's loads are issued before the current batch's arithmetic.
template <typename W, int CH>
__global__ void __launch_bounds__(256, CH == 4 ? 4 : 2) conv1d_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ x_prev,
                                                            const W* __restrict__ w, const uint8_t* __restrict__ reach,
                                                            __nv_bfloat16* __restrict__ y, int tokens, int channels,
                                                            int run_len) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = (blockIdx.y * 8 + warp) * (32 * CH) + lane * CH;
  if (c0 >= channels) return;
  const int t0 = blockIdx.x * run_len, t1 = min(t0 + run_len, tokens);
  if (t0 >= t1) return;
  float taps[kConvTaps][CH];
  load_taps<W, CH>(w, c0, taps);
  float win[3][CH];  // x[t - 3], x[t - 2], x[t - 1]
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const int t = t0 - 3 + i;  // rows before the first token come from the history rows, when there are any
    if (t >= 0) ConvRow<CH>::unpack(ConvRow<CH>::load(x, t, channels, c0), win[i]);
    else if (x_prev != nullptr) ConvRow<CH>::unpack(ConvRow<CH>::load(x_prev, t + 3, channels, c0), win[i]);
    else
#pragma unroll
      for (int j = 0; j < CH; ++j) win[i][j] = 0.f;
  }
  typename ConvRow<CH>::type raw[4], next[4];
  int before[4], next_before[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = min(t0 + i, t1 - 1);
    raw[i] = ConvRow<CH>::load(x, t, channels, c0);
    before[i] = reach[t] & 3;
  }
  for (int tb = t0; tb < t1; tb += 4) {
    if (tb + 4 < t1) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = min(tb + 4 + i, t1 - 1);
        next[i] = ConvRow<CH>::load(x, t, channels, c0);
        next_before[i] = reach[t] & 3;
      }
    }
    __nv_bfloat16* y_row = y + int64_t(tb) * channels + c0;
    if (tb + 3 < t1 && (before[0] & before[1] & before[2] & before[3]) == 3) {
#pragma unroll
      for (int i = 0; i < 4; ++i) conv_fwd_token<false, CH>(taps, win, raw[i], 3, y_row + int64_t(i) * channels);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (tb + i < t1) conv_fwd_token<true, CH>(taps, win, raw[i], before[i], y_row + int64_t(i) * channels);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) raw[i] = next[i], before[i] = next_before[i];
  }
}

// One step of the backward sweep: dpre of token u (needs x[u - 3 .. u]) and dx of token t = u - 3 (needs
// dpre[t .. t + 3]).  kEdge = false: u and t are the run's own tokens with three neighbours inside their documents on
// the side that matters, so nothing is selected or skipped.
template <bool kEdge, bool kRoundPre, int CH, typename Sum>
__device__ __forceinline__ void conv_bwd_token(const float (&taps)[kConvTaps][CH], float (&xw)[3][CH], float (&dp)[3][CH],
                                               Sum (&sum)[kConvTaps][CH], typename ConvRow<CH>::type raw_x,
                                               typename ConvRow<CH>::type raw_g, int before,
                                               int after, bool has_u, bool own_u, bool write_t,
                                               __nv_bfloat16* dx_row) {
  float cur[CH], d[CH];
  if (!kEdge || has_u) {
    float g[CH];
    ConvRow<CH>::unpack(raw_x, cur);
    ConvRow<CH>::unpack(raw_g, g);
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      const float x1 = !kEdge || before >= 1 ? xw[2][j] : 0.f, x2 = !kEdge || before >= 2 ? xw[1][j] : 0.f;
      const float x3 = !kEdge || before >= 3 ? xw[0][j] : 0.f;
      const float pre = preactivation(taps[0][j], x3, taps[1][j], x2, taps[2][j], x1, taps[3][j], cur[j]);
      const float p = kRoundPre ? __bfloat162float(__float2bfloat16_rn(pre)) : pre;
      const float sg = __fdividef(1.0f, 1.0f + __expf(-p));
      d[j] = g[j] * (sg * fmaf(p, 1.0f - sg, 1.0f));
      if (!kEdge || own_u) {  // the run's own tokens feed the weight gradient
        sum[3][j] += Sum(d[j]) * Sum(cur[j]);
        sum[2][j] += Sum(d[j]) * Sum(x1);
        sum[1][j] += Sum(d[j]) * Sum(x2);
        sum[0][j] += Sum(d[j]) * Sum(x3);
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < CH; ++j) cur[j] = 0.f, d[j] = 0.f;
  }
  if (!kEdge || write_t) {
    float out[CH];
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      float v = taps[3][j] * dp[0][j];
      v = fmaf(taps[2][j], !kEdge || after >= 1 ? dp[1][j] : 0.f, v);
      v = fmaf(taps[1][j], !kEdge || after >= 2 ? dp[2][j] : 0.f, v);
      v = fmaf(taps[0][j], !kEdge || after >= 3 ? d[j] : 0.f, v);
      out[j] = v;
    }
    ConvRow<CH>::store(dx_row, out);
  }
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    xw[0][j] = xw[1][j], xw[1][j] = xw[2][j], xw[2][j] = cur[j];
    dp[0][j] = dp[1][j], dp[1][j] = dp[2][j], dp[2][j] = d[j];
  }
}

// One sweep over tokens [t0 ... t1 + 3) in batches of four, the next batch's loads issued before the current batch's
// arithmetic.  The weight gradient's products are summed in FP32 inside a batch when Acc is FP64 (four terms), and the
// batch sums in Acc.
template <typename W, typename Acc, bool kRoundPre, int CH>
__global__ void __launch_bounds__(256, CH == 4 ? 2 : 1) conv1d_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                         const __nv_bfloat16* __restrict__ x_prev,
                                                         const __nv_bfloat16* __restrict__ x_next,
                                                         const W* __restrict__ w, const __nv_bfloat16* __restrict__ dy,
                                                         const __nv_bfloat16* __restrict__ dy_next,
                                                         const uint8_t* __restrict__ reach,
                                                         __nv_bfloat16* __restrict__ dx, Acc* __restrict__ dw_partial,
                                                         int tokens, int channels, int run_len) {
  constexpr bool kBatchSums = !std::is_same<Acc, float>::value;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = (blockIdx.y * 8 + warp) * (32 * CH) + lane * CH;
  if (c0 >= channels) return;
  const int t0 = blockIdx.x * run_len, t1 = min(t0 + run_len, tokens);
  if (t0 >= t1) return;
  float taps[kConvTaps][CH];
  load_taps<W, CH>(w, c0, taps);
  Acc acc[kConvTaps][CH];
#pragma unroll
  for (int k = 0; k < kConvTaps; ++k)
#pragma unroll
    for (int j = 0; j < CH; ++j) acc[k][j] = Acc(0);
  float xw[3][CH];   // x[u - 3], x[u - 2], x[u - 1]
  float dp[3][CH];   // dpre[u - 3], dpre[u - 2], dpre[u - 1]
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const int t = t0 - 3 + i;
    if (t >= 0) ConvRow<CH>::unpack(ConvRow<CH>::load(x, t, channels, c0), xw[i]);
    else if (x_prev != nullptr) ConvRow<CH>::unpack(ConvRow<CH>::load(x_prev, t + 3, channels, c0), xw[i]);
    else
#pragma unroll
      for (int j = 0; j < CH; ++j) xw[i][j] = 0.f;
#pragma unroll
    for (int j = 0; j < CH; ++j) dp[i][j] = 0.f;  // dpre before t0 is never used: dx starts at t0
  }
  // rows after the last token come from the continuation rows (x_next, dy_next: 3 rows each), when there are any
  const int u_end = x_next != nullptr ? t1 + 3 : min(t1 + 3, tokens);
  auto row_of = [&](const __nv_bfloat16* here, const __nv_bfloat16* after, int u) {
    return u < tokens ? ConvRow<CH>::load(here, u, channels, c0) : ConvRow<CH>::load(after, u - tokens, channels, c0);
  };
  typename ConvRow<CH>::type raw_x[4], raw_g[4], next_x[4], next_g[4];
  int reach_u[4], reach_t[4], next_u[4], next_t[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int u = min(t0 + i, u_end - 1);
    raw_x[i] = row_of(x, x_next, u);
    raw_g[i] = row_of(dy, dy_next, u);
    reach_u[i] = reach[u];
    reach_t[i] = reach[min(max(t0 + i - 3, 0), tokens - 1)];
  }
  for (int ub = t0; ub < t1 + 3; ub += 4) {
    if (ub + 4 < t1 + 3) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int u = min(ub + 4 + i, u_end - 1);
        next_x[i] = row_of(x, x_next, u);
        next_g[i] = row_of(dy, dy_next, u);
        next_u[i] = reach[u];
        next_t[i] = reach[min(ub + 1 + i, tokens - 1)];
      }
    }
    __nv_bfloat16* dx_row = dx + int64_t(ub - 3) * channels + c0;  // only dereferenced for tokens >= t0
    const int all_u = reach_u[0] & reach_u[1] & reach_u[2] & reach_u[3];
    const int all_t = reach_t[0] & reach_t[1] & reach_t[2] & reach_t[3];
    const bool inner = ub - 3 >= t0 && ub + 3 < t1 && (all_u & 3) == 3 && (all_t >> 2 & 3) == 3;
    if (kBatchSums) {
      float part[kConvTaps][CH];
#pragma unroll
      for (int k = 0; k < kConvTaps; ++k)
#pragma unroll
        for (int j = 0; j < CH; ++j) part[k][j] = 0.f;
      if (inner) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          conv_bwd_token<false, kRoundPre, CH>(taps, xw, dp, part, raw_x[i], raw_g[i], 3, 3, true, true, true,
                                           dx_row + int64_t(i) * channels);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int u = ub + i;
          if (u < t1 + 3)
            conv_bwd_token<true, kRoundPre, CH>(taps, xw, dp, part, raw_x[i], raw_g[i], reach_u[i] & 3,
                                            (reach_t[i] >> 2) & 3, u < u_end, u < t1, u - 3 >= t0,
                                            dx_row + int64_t(i) * channels);
        }
      }
#pragma unroll
      for (int k = 0; k < kConvTaps; ++k)
#pragma unroll
        for (int j = 0; j < CH; ++j) acc[k][j] += Acc(part[k][j]);
    } else {
      auto& sum = reinterpret_cast<float(&)[kConvTaps][CH]>(acc);
      if (inner) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          conv_bwd_token<false, kRoundPre, CH>(taps, xw, dp, sum, raw_x[i], raw_g[i], 3, 3, true, true, true,
                                           dx_row + int64_t(i) * channels);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int u = ub + i;
          if (u < t1 + 3)
            conv_bwd_token<true, kRoundPre, CH>(taps, xw, dp, sum, raw_x[i], raw_g[i], reach_u[i] & 3,
                                            (reach_t[i] >> 2) & 3, u < u_end, u < t1, u - 3 >= t0,
                                            dx_row + int64_t(i) * channels);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
      raw_x[i] = next_x[i], raw_g[i] = next_g[i], reach_u[i] = next_u[i], reach_t[i] = next_t[i];
  }
  if (dw_partial != nullptr) {
    Acc* out = dw_partial + (int64_t(blockIdx.x) * channels + c0) * kConvTaps;
#pragma unroll
    for (int j = 0; j < CH; ++j)
#pragma unroll
      for (int k = 0; k < kConvTaps; ++k) out[j * kConvTaps + k] = acc[k][j];
  }
}

template <typename Acc, typename W>
__global__ void conv1d_dw_kernel(const Acc* __restrict__ dw_partial, int runs, int64_t entries, W* __restrict__ dw) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= entries) return;
  double sum = 0.0;
  for (int r = 0; r < runs; ++r) sum += double(dw_partial[int64_t(r) * entries + i]);
  dw[i] = W(float(sum));
}

}  // namespace mek

namespace {

struct ConvPlan {
  int runs, run_len;
};
ConvPlan conv_plan(int tokens) {
  int runs = (tokens + 63) / 64;
  if (runs > mek::kConvMaxRuns) runs = mek::kConvMaxRuns;
  if (runs < 1) runs = 1;
  const int run_len = (tokens + runs - 1) / runs;
  return {(tokens + run_len - 1) / run_len, run_len};
}

int check_conv(const char* what, int tokens, int channels, int num_docs) {
  using namespace mek;
  if (tokens <= 0 || num_docs <= 0) return fail(MEK_ERR_INVALID, "%s: no tokens or no documents", what);
  if (channels <= 0 || channels % 8 != 0)
    return fail(MEK_ERR_INVALID, "%s: the channel count must be a positive multiple of 8, got %d", what, channels);
  return MEK_OK;
}

}  // namespace

extern "C" {

int mek_conv1d_runs(int tokens) { return tokens > 0 ? conv_plan(tokens).runs : 0; }

int mek_conv1d_reach(const int32_t* cu_seqlens, int num_docs, int tokens, uint8_t* reach, void* stream) {
  using namespace mek;
  if (!cu_seqlens || !reach || num_docs <= 0 || tokens <= 0)
    return fail(MEK_ERR_INVALID, "conv1d_reach: a null pointer, no documents or no tokens");
  conv_reach_kernel<<<(tokens + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(cu_seqlens, num_docs, tokens,
                                                                                        reach);
  return launched("conv1d_reach");
}

int mek_conv1d_fwd(const void* x, const void* x_prev, const void* weight, int weight_is_bf16, const uint8_t* reach,
                   void* y, int tokens, int channels, void* stream) {
  using namespace mek;
  if (!x || !weight || !reach || !y) return fail(MEK_ERR_INVALID, "conv1d_fwd: a null pointer");
  if (int rc = check_conv("conv1d_fwd", tokens, channels, 1)) return rc;
  const ConvPlan plan = conv_plan(tokens);
  constexpr int kFwdCh = 4;  // channels per thread
  const dim3 grid(plan.runs, (channels + 256 * kFwdCh - 1) / (256 * kFwdCh));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (weight_is_bf16)
    conv1d_fwd_kernel<__nv_bfloat16, kFwdCh><<<grid, 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(x_prev),
        static_cast<const __nv_bfloat16*>(weight), reach, static_cast<__nv_bfloat16*>(y), tokens, channels, plan.run_len);
  else
    conv1d_fwd_kernel<float, kFwdCh><<<grid, 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(x_prev),
        static_cast<const float*>(weight), reach, static_cast<__nv_bfloat16*>(y), tokens, channels, plan.run_len);
  return launched("conv1d_fwd");
}

int mek_conv1d_bwd(const void* x, const void* x_prev, const void* x_next, const void* weight, int weight_is_bf16,
                   const void* dy, const void* dy_next, const uint8_t* reach, void* dx, void* dw_partial, void* dw,
                   int fp32_policy, int tokens, int channels, void* stream) {
  using namespace mek;
  if (!x || !weight || !dy || !reach || !dx) return fail(MEK_ERR_INVALID, "conv1d_bwd: a null pointer");
  if ((dw == nullptr) != (dw_partial == nullptr))
    return fail(MEK_ERR_INVALID, "conv1d_bwd: dw and its partial sums go together");
  if ((x_next == nullptr) != (dy_next == nullptr))
    return fail(MEK_ERR_INVALID, "conv1d_bwd: the continuation rows of x and of dy go together");
  if (int rc = check_conv("conv1d_bwd", tokens, channels, 1)) return rc;
  const ConvPlan plan = conv_plan(tokens);
  constexpr int kBwdCh = 4;  // channels per thread of the backward kernel
  const dim3 grid(plan.runs, (channels + 256 * kBwdCh - 1) / (256 * kBwdCh));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* gp = static_cast<const __nv_bfloat16*>(dy);
  const __nv_bfloat16* xprev = static_cast<const __nv_bfloat16*>(x_prev);
  const __nv_bfloat16* xnext = static_cast<const __nv_bfloat16*>(x_next);
  const __nv_bfloat16* gnext = static_cast<const __nv_bfloat16*>(dy_next);
  __nv_bfloat16* dxp = static_cast<__nv_bfloat16*>(dx);
  const int64_t entries = int64_t(channels) * kConvTaps;
  const unsigned sum_grid = unsigned((entries + 255) / 256);
#define MEK_CONV_BWD(WT, ACC, ROUND)                                                                                 \
  conv1d_bwd_kernel<WT, ACC, ROUND, kBwdCh><<<grid, 256, 0, s>>>(xp, xprev, xnext, static_cast<const WT*>(weight), gp, gnext, \
                                                         reach, dxp, static_cast<ACC*>(dw_partial), tokens, channels, \
                                                         plan.run_len);                                              \
  if (int rc = launched("conv1d_bwd")) return rc;                                                                    \
  if (dw != nullptr) conv1d_dw_kernel<<<sum_grid, 256, 0, s>>>(static_cast<const ACC*>(dw_partial), plan.runs, entries, \
                                                               static_cast<WT*>(dw));
  if (fp32_policy) {
    if (weight_is_bf16) { MEK_CONV_BWD(__nv_bfloat16, double, false) } else { MEK_CONV_BWD(float, double, false) }
  } else {
    if (weight_is_bf16) { MEK_CONV_BWD(__nv_bfloat16, float, true) } else { MEK_CONV_BWD(float, float, true) }
  }
#undef MEK_CONV_BWD
  return launched("conv1d_bwd (weight gradient)");
}

}  // extern "C"
