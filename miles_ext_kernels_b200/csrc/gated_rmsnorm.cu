// SiLU-gated RMSNorm over rows of 128, forward and backward, sm_100a: the output norm of the GDN layer,
//     rstd = 1 / sqrt(mean(x^2) + eps),   y = bf16(((x rstd) w) silu(z))                               (FP32 inside)
// (reference: miles_ext_kernels/cake/_impl/gated_rmsnorm/ops.py:8-24; closed-form backward as in
// tests/cake/gated_rmsnorm/inputs.py:75-95).  HBM-bound row work: one warp per row, 8 bytes per lane and tensor, x
// and the gate z read where they lie (each with its own token and head stride: z is usually a column slice of the
// layer's input projection).
//
// The weight gradient sums a term per row.  Every reduction has a fixed order: a warp adds the terms of its rows in
// row order (FP32), a block adds its 8 warps in warp order (FP32), and a second launch adds the blocks' partial sums
// in block order in FP64.  The number of blocks is a function of the row count alone, so identical inputs give
// identical bits.
#include "common.cuh"
#include "umma.cuh"

namespace mek {

constexpr int kNormRowsPerBlock = 32;  // 8 warps x 2 half-warps x 2 rows in flight
constexpr int kNormMaxBlocks = 148 * 4;

struct RowView {
  const __nv_bfloat16* base;
  int64_t token_stride, head_stride;
  __device__ __forceinline__ const __nv_bfloat16* row(int64_t r, int heads) const {
    return base + (r / heads) * token_stride + (r % heads) * head_stride;
  }
};

// A half-warp owns a row: 16 lanes x 16 bytes.
__device__ __forceinline__ void load8(const __nv_bfloat16* p, int l16, float* v) {
  const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p) + l16);
  const float2 a = unpack_bf16(raw.x), b = unpack_bf16(raw.y), c = unpack_bf16(raw.z), d = unpack_bf16(raw.w);
  v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y, v[4] = c.x, v[5] = c.y, v[6] = d.x, v[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, int l16, const float* v) {
  reinterpret_cast<uint4*>(p)[l16] =
      make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}
__device__ __forceinline__ float half_warp_sum(float x) {
#pragma unroll
  for (int m = 8; m >= 1; m >>= 1) x += __shfl_xor_sync(0xffffffffu, x, m);
  return x;
}

__global__ void __launch_bounds__(256) gated_rmsnorm_fwd_kernel(RowView x, RowView z, const __nv_bfloat16* __restrict__ w,
                                                                __nv_bfloat16* __restrict__ y, int64_t rows, int heads,
                                                                float eps) {
  const int l16 = threadIdx.x & 15, half = threadIdx.x >> 4;  // 16 half-warps per block, 2 rows each
  const int64_t r0 = int64_t(blockIdx.x) * kNormRowsPerBlock + half * 2;
  float wv[8], xv[2][8], zv[2][8];
  load8(w, l16, wv);
#pragma unroll
  for (int i = 0; i < 2; ++i) {  // both rows' loads in flight before any arithmetic
    const int64_t r = r0 + i < rows ? r0 + i : rows - 1;
    load8(x.row(r, heads), l16, xv[i]);
    load8(z.row(r, heads), l16, zv[i]);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float ss = 0.f, out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) ss = fmaf(xv[i][j], xv[i][j], ss);
    const float rstd = rsqrtf(half_warp_sum(ss) * (1.0f / 128.0f) + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = ((xv[i][j] * rstd) * wv[j]) * __fdividef(zv[i][j], 1.0f + __expf(-zv[i][j]));
    if (r0 + i < rows) store8(y + (r0 + i) * 128, l16, out);
  }
}

// dx = rstd dn - x rstd^3 mean(dn x), dn = dy silu(z) w;  dz = dy n w s (1 + z (1 - s)), n = x rstd, s = sigmoid(z);
// dw += dy silu(z) n.  Block b takes the row groups b, b + gridDim.x, ...
__global__ void __launch_bounds__(256) gated_rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, RowView x, RowView z,
                                                                const __nv_bfloat16* __restrict__ w,
                                                                __nv_bfloat16* __restrict__ dx,
                                                                __nv_bfloat16* __restrict__ dz,
                                                                float* __restrict__ dw_partial, int64_t rows, int heads,
                                                                float eps) {
  __shared__ float s_dw[16][128];
  const int l16 = threadIdx.x & 15, half = threadIdx.x >> 4;
  float wv[8], acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  load8(w, l16, wv);
  for (int64_t group = blockIdx.x; group * kNormRowsPerBlock < rows; group += gridDim.x) {
    const int64_t r0 = group * kNormRowsPerBlock + half * 2;
    float xv[2][8], zv[2][8], gv[2][8];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int64_t r = r0 + i < rows ? r0 + i : rows - 1;
      load8(x.row(r, heads), l16, xv[i]);
      load8(z.row(r, heads), l16, zv[i]);
      load8(dy + r * 128, l16, gv[i]);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const bool live = r0 + i < rows;  // uniform over the half-warp
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(xv[i][j], xv[i][j], ss);
      const float rstd = rsqrtf(half_warp_sum(ss) * (1.0f / 128.0f) + eps);
      float dot = 0.f, dn[8], dzv[8], dxv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float s = __fdividef(1.0f, 1.0f + __expf(-zv[i][j]));
        const float a = gv[i][j] * (zv[i][j] * s);
        const float n = xv[i][j] * rstd;
        dn[j] = a * wv[j];
        dot = fmaf(dn[j], xv[i][j], dot);
        dzv[j] = gv[i][j] * n * wv[j] * s * (1.0f + zv[i][j] * (1.0f - s));
        if (live) acc[j] = fmaf(a, n, acc[j]);
      }
      const float mean = half_warp_sum(dot) * (1.0f / 128.0f);
      const float r3 = rstd * rstd * rstd;
#pragma unroll
      for (int j = 0; j < 8; ++j) dxv[j] = rstd * dn[j] - xv[i][j] * r3 * mean;
      if (live) {
        store8(dx + (r0 + i) * 128, l16, dxv);
        store8(dz + (r0 + i) * 128, l16, dzv);
      }
    }
  }
  if (dw_partial == nullptr) return;
#pragma unroll
  for (int j = 0; j < 8; ++j) s_dw[half][l16 * 8 + j] = acc[j];
  __syncthreads();
  if (threadIdx.x < 128) {
    float sum = 0.f;
#pragma unroll
    for (int hw = 0; hw < 16; ++hw) sum += s_dw[hw][threadIdx.x];
    dw_partial[int64_t(blockIdx.x) * 128 + threadIdx.x] = sum;
  }
}

__global__ void __launch_bounds__(128) gated_rmsnorm_dw_kernel(const float* __restrict__ dw_partial, int blocks,
                                                               __nv_bfloat16* __restrict__ dw) {
  double sum = 0.0;
  for (int b = 0; b < blocks; ++b) sum += double(dw_partial[int64_t(b) * 128 + threadIdx.x]);
  dw[threadIdx.x] = __float2bfloat16_rn(float(sum));
}

}  // namespace mek

namespace {

int norm_blocks(int64_t rows) {
  const int64_t groups = (rows + mek::kNormRowsPerBlock - 1) / mek::kNormRowsPerBlock;
  return int(groups < mek::kNormMaxBlocks ? groups : mek::kNormMaxBlocks);
}

int check_norm(const char* what, int64_t rows, int heads, int64_t xt, int64_t xh, int64_t zt, int64_t zh, const void* x,
               const void* z) {
  using namespace mek;
  if (rows <= 0 || heads <= 0 || rows % heads != 0)
    return fail(MEK_ERR_INVALID, "%s: rows=%lld must be a positive multiple of heads=%d", what, (long long)rows, heads);
  if ((xt | xh | zt | zh) % 8 != 0 || xh < 0 || zh < 0 || xt < 0 || zt < 0)
    return fail(MEK_ERR_INVALID, "%s: token and head strides must be non-negative multiples of 8 elements", what);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(z)) % 16 != 0)
    return fail(MEK_ERR_INVALID, "%s: x and z must be 16-byte aligned", what);
  return MEK_OK;
}

}  // namespace

extern "C" {

int mek_gated_rmsnorm_partial_rows(int64_t rows) { return rows > 0 ? norm_blocks(rows) : 0; }

int mek_gated_rmsnorm_fwd(const void* x, const void* z, const void* weight, void* y, int64_t rows, int heads,
                          int64_t x_token_stride, int64_t x_head_stride, int64_t z_token_stride, int64_t z_head_stride,
                          float eps, void* stream) {
  using namespace mek;
  if (!x || !z || !weight || !y) return fail(MEK_ERR_INVALID, "gated_rmsnorm_fwd: a null pointer");
  if (int rc = check_norm("gated_rmsnorm_fwd", rows, heads, x_token_stride, x_head_stride, z_token_stride,
                          z_head_stride, x, z))
    return rc;
  const RowView xv{static_cast<const __nv_bfloat16*>(x), x_token_stride, x_head_stride};
  const RowView zv{static_cast<const __nv_bfloat16*>(z), z_token_stride, z_head_stride};
  const unsigned grid = unsigned((rows + kNormRowsPerBlock - 1) / kNormRowsPerBlock);
  gated_rmsnorm_fwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      xv, zv, static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(y), rows, heads, eps);
  return launched("gated_rmsnorm_fwd");
}

int mek_gated_rmsnorm_bwd(const void* dy, const void* x, const void* z, const void* weight, void* dx, void* dz,
                          float* dw_partial, void* dw, int64_t rows, int heads, int64_t x_token_stride,
                          int64_t x_head_stride, int64_t z_token_stride, int64_t z_head_stride, float eps,
                          void* stream) {
  using namespace mek;
  if (!dy || !x || !z || !weight || !dx || !dz) return fail(MEK_ERR_INVALID, "gated_rmsnorm_bwd: a null pointer");
  if ((dw == nullptr) != (dw_partial == nullptr))
    return fail(MEK_ERR_INVALID, "gated_rmsnorm_bwd: dw and its partial sums go together");
  if (int rc = check_norm("gated_rmsnorm_bwd", rows, heads, x_token_stride, x_head_stride, z_token_stride,
                          z_head_stride, x, z))
    return rc;
  const RowView xv{static_cast<const __nv_bfloat16*>(x), x_token_stride, x_head_stride};
  const RowView zv{static_cast<const __nv_bfloat16*>(z), z_token_stride, z_head_stride};
  const int blocks = norm_blocks(rows);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  gated_rmsnorm_bwd_kernel<<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dy), xv, zv,
                                                  static_cast<const __nv_bfloat16*>(weight),
                                                  static_cast<__nv_bfloat16*>(dx), static_cast<__nv_bfloat16*>(dz),
                                                  dw_partial, rows, heads, eps);
  if (int rc = launched("gated_rmsnorm_bwd")) return rc;
  if (dw != nullptr) {
    gated_rmsnorm_dw_kernel<<<1, 128, 0, s>>>(dw_partial, blocks, static_cast<__nv_bfloat16*>(dw));
    return launched("gated_rmsnorm_bwd (weight gradient)");
  }
  return MEK_OK;
}

}  // extern "C"
