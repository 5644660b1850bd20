// KDA: the gated delta rule with a per-key-channel decay g [T, H, 128] (packed documents, zero initial state, one
// value head per key head), chunk 64, sm_100a.  Reference semantics: tests/cake/kda/_reference.py:13-15, 102-142 and
// the chunked form restated in oracle/kda_oracle.py.
//
// With G the chunk-local cumulative gate per channel (kept in the log2 domain) and G_L its value at the chunk's last
// token, three decayed copies of the operands carry every state-related decay, all with factors <= 1:
//     qg = q 2^G        kg = k 2^G        kr = k 2^{G_L - G}
// so the state scan, the output and the adjoint scan are the GDN kernels run on (kr, qg) with a per-channel chunk
// decay (mek_kda_fwd_h / mek_kda_fwd_o / mek_kda_bwd_dh).  What is new here:
//   kda_prep        G, qg, kg, kr and the chunk-end gate                                  [CUDA cores, coalesced]
//   kda_intra       Aqk_ij = scale sum_d q_id k_jd 2^{G_id - G_jd}, L_ij = beta_i sum_d k_id k_jd 2^{G_id - G_jd}
//                   pair by pair (each exponent is formed from a non-positive difference: finite for any gate),
//                   then A = (I + L)^-1, w = A (beta kg), u = A (beta v)                    [CUDA cores + tcgen05]
//   kda_tail_mma    the state-side gradient contractions of one (chunk, head)               [tcgen05]
//   kda_tail_pair   the pairwise decayed gradient contractions, dq, dk and the per-channel gate gradient with its
//                   in-chunk suffix sum                                                     [CUDA cores]
//   qk_grad_finish  fp32 dq / dk -> the L2 norm's pull-back (optional) -> bf16
#include "common.cuh"
#include "tiles.cuh"

namespace mek {

// ---------------------------------------------------------------------------------------------------------------
// prep: one block per (chunk, head), one thread per key channel
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) kda_prep_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const float* __restrict__ g,
    float* __restrict__ g2, __nv_bfloat16* __restrict__ qg, __nv_bfloat16* __restrict__ kg,
    __nv_bfloat16* __restrict__ kr, float* __restrict__ gl2, const int32_t* __restrict__ chunk_start,
    const int32_t* __restrict__ chunk_len, int num_heads) {
  const int c = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const int start = chunk_start[c], len = chunk_len[c];
  if (len <= 0) return;
  const int64_t stride = int64_t(num_heads) * kDim;
  const int64_t base = int64_t(start) * stride + h * kDim + d;
  float acc = 0.f;
  for (int i = 0; i < len; ++i) {
    const int64_t at = base + i * stride;
    acc += g[at];
    const float gi = acc * kLog2e, e = fast_exp2(gi);
    g2[at] = gi;
    qg[at] = __float2bfloat16_rn(__bfloat162float(q[at]) * e);
    kg[at] = __float2bfloat16_rn(__bfloat162float(k[at]) * e);
  }
  const float gl = acc * kLog2e;
  gl2[(int64_t(c) * num_heads + h) * kDim + d] = gl;
  for (int i = 0; i < len; ++i) {
    const int64_t at = base + i * stride;
    kr[at] = __float2bfloat16_rn(__bfloat162float(k[at]) * fast_exp2(gl - g2[at]));
  }
}

// ---------------------------------------------------------------------------------------------------------------
// intra: Aqk, A, w, u of one (chunk, head)
// ---------------------------------------------------------------------------------------------------------------
struct KdaIntraSmem {
  static constexpr int kRow = 129;                                  // fp32 row stride of the q / k / G copies
  static constexpr uint32_t kQ = 0;                                 // fp32 [64][129]; later the bf16 tiles below
  static constexpr uint32_t kK = kQ + 64 * kRow * 4;
  static constexpr uint32_t kG = kK + 64 * kRow * 4;
  // after the pair phase (the copies above are dead; about 100 KB in all, so that two CTAs share an SM):
  static constexpr uint32_t kA = 0;                                 // [64][64] bf16
  static constexpr uint32_t kKB = 8192;                             // [64][128] beta kg
  static constexpr uint32_t kVB = kKB + 16384;                      // [64][128] beta v
  static constexpr uint32_t kSqk = kVB + 16384;                     // fp32 [64][65]
  static constexpr uint32_t kSkk = kSqk + 64 * 65 * 4;
  static constexpr uint32_t kL = kSkk + 64 * 65 * 4;                // fp32 [64][68]
  static constexpr uint32_t kBeta = ((kG + 64 * kRow * 4 + 255) / 256) * 256;  // beta[64]
  static constexpr uint32_t kBytes = kBeta + 256;
  static_assert(kL + 64 * 68 * 4 <= kBeta, "the results of the pair phase fit the dead copies");
};

__global__ void __launch_bounds__(288, 2) kda_intra_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
    const __nv_bfloat16* __restrict__ kg, const float* __restrict__ g2, const float* __restrict__ beta,
    __nv_bfloat16* __restrict__ a_out, __nv_bfloat16* __restrict__ aqk_out, __nv_bfloat16* __restrict__ w_out,
    __nv_bfloat16* __restrict__ u_out, const int32_t* __restrict__ chunk_start, const int32_t* __restrict__ chunk_len,
    int num_heads, float scale, int32_t* __restrict__ status) {
  extern __shared__ uint8_t raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y;
  const int start = chunk_start[c], len = chunk_len[c];
  if (len <= 0) return;
  constexpr int kRow = KdaIntraSmem::kRow;
  float* sq = reinterpret_cast<float*>(sm + KdaIntraSmem::kQ);
  float* sk = reinterpret_cast<float*>(sm + KdaIntraSmem::kK);
  float* sg = reinterpret_cast<float*>(sm + KdaIntraSmem::kG);
  float* s_qk = reinterpret_cast<float*>(sm + KdaIntraSmem::kSqk);
  float* s_kk = reinterpret_cast<float*>(sm + KdaIntraSmem::kSkk);
  float* s_l = reinterpret_cast<float*>(sm + KdaIntraSmem::kL);
  float* s_beta = reinterpret_cast<float*>(sm + KdaIntraSmem::kBeta);
  const int64_t stride = int64_t(num_heads) * kDim;
  const int64_t tile = int64_t(c) * num_heads + h;

  if (tid == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 256);
  for (int i = tid; i < 64 * 16; i += 288) {  // 8 channels of one row per step, 16-byte loads
    const int r = i >> 4, d = (i & 15) * 8;
    const bool live = r < len;
    const int64_t at = int64_t(start + (live ? r : len - 1)) * stride + h * kDim + d;
    float qv[8], kv[8];
    unpack8(live ? ldg16(q + at) : make_uint4(0u, 0u, 0u, 0u), qv);
    unpack8(live ? ldg16(k + at) : make_uint4(0u, 0u, 0u, 0u), kv);
    // rows past the chunk's length keep the last gate: every pair exponent stays <= 0
    const float4 g_lo = __ldg(reinterpret_cast<const float4*>(g2 + at));
    const float4 g_hi = __ldg(reinterpret_cast<const float4*>(g2 + at + 4));
    const float gv[8] = {g_lo.x, g_lo.y, g_lo.z, g_lo.w, g_hi.x, g_hi.y, g_hi.z, g_hi.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      sq[r * kRow + d + j] = qv[j];
      sk[r * kRow + d + j] = kv[j];
      sg[r * kRow + d + j] = gv[j];
    }
  }
  if (tid < 64) s_beta[tid] = tid < len ? beta[int64_t(start + tid) * num_heads + h] : 0.f;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  // pair phase: a thread owns a 4 x 4 block (bi, bj), bj <= bi, of the lower triangle and one half of the channels:
  // threads 0..239 the 120 blocks below the diagonal, threads 256..287 (one warp) the 16 diagonal blocks.
  // Below the diagonal every pair of a block is valid and 2^{G_i - G_j} factors as 2^{G_i - G_{j0+3}} 2^{G_{j0+3} - G_j}
  // with both exponents <= 0: 7 exponentials per channel instead of 16.
  float aqk[4][4], akk[4][4];
  int i0 = 0, j0 = 0;
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) aqk[a][b] = akk[a][b] = 0.f;
  if (tid < 240) {
    const int t = tid >> 1, half = tid & 1;
    int bi = int((sqrtf(8.f * t + 1.f) + 1.f) * 0.5f);
    while (bi * (bi + 1) / 2 <= t) ++bi;
    while (bi * (bi - 1) / 2 > t) --bi;
    const int bj = t - bi * (bi - 1) / 2;
    i0 = 4 * bi, j0 = 4 * bj;
    for (int d = half * 64; d < half * 64 + 64; ++d) {
      float qe[4], ke[4], kj[4], gj[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        kj[a] = sk[(j0 + a) * kRow + d];
        gj[a] = sg[(j0 + a) * kRow + d];
      }
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float ea = fast_exp2(sg[(i0 + a) * kRow + d] - gj[3]);
        qe[a] = sq[(i0 + a) * kRow + d] * ea;
        ke[a] = sk[(i0 + a) * kRow + d] * ea;
      }
#pragma unroll
      for (int b = 0; b < 3; ++b) kj[b] *= fast_exp2(gj[3] - gj[b]);
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          aqk[a][b] = fmaf(qe[a], kj[b], aqk[a][b]);
          akk[a][b] = fmaf(ke[a], kj[b], akk[a][b]);
        }
    }
  } else if (tid >= 256) {
    const int bi = (tid - 256) >> 1, half = tid & 1;
    i0 = j0 = 4 * bi;
    for (int d = half * 64; d < half * 64 + 64; ++d) {
      float qi[4], ki[4], gi[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        qi[a] = sq[(i0 + a) * kRow + d];
        ki[a] = sk[(i0 + a) * kRow + d];
        gi[a] = sg[(i0 + a) * kRow + d];
      }
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b <= a; ++b) {  // the exponent of a valid pair is <= 0
          const float e = fast_exp2(gi[a] - gi[b]) * ki[b];
          aqk[a][b] = fmaf(qi[a], e, aqk[a][b]);
          akk[a][b] = fmaf(ki[a], e, akk[a][b]);
        }
    }
  }
  // the two channel halves of a block sit in neighbouring lanes: half 0 + half 1, then one of them writes -- after a
  // block barrier, because the results take the place of the q / k / G copies
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const float oq = __shfl_xor_sync(0xffffffffu, aqk[a][b], 1), ok_ = __shfl_xor_sync(0xffffffffu, akk[a][b], 1);
      aqk[a][b] = (tid & 1) ? oq + aqk[a][b] : aqk[a][b] + oq;
      akk[a][b] = (tid & 1) ? ok_ + akk[a][b] : akk[a][b] + ok_;
    }
  __syncthreads();
  if ((tid < 240 || tid >= 256) && (tid & 1) == 0) {
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        s_qk[(i0 + a) * 65 + j0 + b] = aqk[a][b];
        s_kk[(i0 + a) * 65 + j0 + b] = akk[a][b];
      }
  }
  __syncthreads();

  // Aqk rows -> global; L rows -> shared
  if (tid < 64) {
    const int i = tid;
    const float bi = s_beta[i];
    __nv_bfloat16* dst = aqk_out + tile * 4096 + i * 64;
#pragma unroll 2
    for (int jj = 0; jj < 8; ++jj) {
      float x[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int j = jj * 8 + e;
        x[e] = j <= i ? scale * s_qk[i * 65 + j] : 0.f;
        s_l[i * 68 + j] = j < i ? bi * s_kk[i * 65 + j] : 0.f;
      }
      reinterpret_cast<uint4*>(dst)[jj] = pack8(x);
    }
  }
  __syncthreads();

  // kb = bf16(beta kg), vb = bf16(beta v)
  for (int i = tid; i < 64 * 16; i += 288) {
    const int r = i >> 4, cc = i & 15;
    const float b = s_beta[r];
    float x[8];
    uint4 rawk = make_uint4(0u, 0u, 0u, 0u), rawv = rawk;
    if (r < len) {
      rawk = ldg16(kg + int64_t(start + r) * stride + h * kDim + cc * 8);
      rawv = ldg16(v + int64_t(start + r) * stride + h * kDim + cc * 8);
    }
    unpack8(rawk, x);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] *= b;
    set_tile_chunk(sm + KdaIntraSmem::kKB, 8192, r, cc, pack8(x));
    unpack8(rawv, x);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] *= b;
    set_tile_chunk(sm + KdaIntraSmem::kVB, 8192, r, cc, pack8(x));
  }
  // A = (I + L)^-1 : thread c solves (I + L) x = e_c by forward substitution (columns are independent)
  if (tid < 64) {
    float x[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      float acc0 = (i == tid) ? 1.f : 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
#pragma unroll
      for (int j = 0; j < i; j += 4) {
        const float4 l = *reinterpret_cast<const float4*>(s_l + i * 68 + j);
        acc0 = fmaf(-l.x, x[j], acc0);
        if (j + 1 < i) acc1 = fmaf(-l.y, x[j + 1], acc1);
        if (j + 2 < i) acc2 = fmaf(-l.z, x[j + 2], acc2);
        if (j + 3 < i) acc3 = fmaf(-l.w, x[j + 3], acc3);
      }
      x[i] = (acc0 + acc1) + (acc2 + acc3);
    }
    uint8_t* at = sm + KdaIntraSmem::kA;
#pragma unroll
    for (int i = 0; i < 64; ++i)
      *reinterpret_cast<__nv_bfloat16*>(at + sw128_offset(i, tid >> 3) + (tid & 7) * 2) = __float2bfloat16_rn(x[i]);
  }
  fence_async_smem();
  __syncthreads();
  tc_fence_after();

  const uint32_t sbase = smem_u32(sm);
  if (tid == 0) {
    const Operand a{sbase + KdaIntraSmem::kA, 8192};
    const Operand kb{sbase + KdaIntraSmem::kKB, 8192};
    const Operand vb{sbase + KdaIntraSmem::kVB, 8192};
    // alternating: the instructions of one product wait for one another
    umma_gemm_pair<64, 128>(tmem, a, false, kb, true, 64, false, false, tmem + 128, a, false, vb, true, 64, false, false);
    umma_commit(&bar);
  }
  if (tid < 128) store_tile<64, 64, 128>(sm + KdaIntraSmem::kA, 8192, a_out + tile * 4096, 64, 64, tid);
  bool ok = true;
  if (warp < 4) {
    ok = __all_sync(0xffffffffu, mbar_wait(&bar, 0));
    tc_fence_after();
    if (ok) {
      const int i = warp * 16 + (lane & 15);
      const bool live = lane < 16 && i < len;
      __nv_bfloat16* wd = w_out + int64_t(start + i) * stride + h * kDim;
      __nv_bfloat16* ud = u_out + int64_t(start + i) * stride + h * kDim;
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        float s[32];
        tmem_ld32(tmem_addr(tmem, warp, p * 32), s);
        tmem_ld_wait();
        __nv_bfloat16* dst = (p < 4 ? wd : ud) + (p & 3) * 32;
        if (live) {
#pragma unroll
          for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(dst)[j] = pack8(s + 8 * j);
        }
      }
    }
    if (!ok && tid == 0) atomicExch(status, kDevWaitTimeout | (6 << 8));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

// ---------------------------------------------------------------------------------------------------------------
// tail, tensor-core part: one CTA per (chunk, head)
// ---------------------------------------------------------------------------------------------------------------
struct KdaTailSmem {
  static constexpr uint32_t kH = 0;                    // [128][128] h; later DW at +0, KB at +16384
  static constexpr uint32_t kDH = 32768;               // [128][128] dh; later VB at +0
  static constexpr uint32_t kDO = 65536;               // [64][128] do
  static constexpr uint32_t kDOS = kDO + 16384;        // [64][128] bf16(scale do)
  static constexpr uint32_t kVN = kDOS + 16384;        // [64][128] v_new
  static constexpr uint32_t kDVN = kVN + 16384;        // [64][128] dv_new
  static constexpr uint32_t kKG = kDVN + 16384;        // [64][128] kg
  static constexpr uint32_t kV = kKG + 16384;          // [64][128] v
  static constexpr uint32_t kA = kV + 16384;           // [64][64] A
  static constexpr uint32_t kDA = kA + 8192;           // [64][64] dA
  static constexpr uint32_t kX = kDA + 8192;           // [64][64] X = A^T dA
  static constexpr uint32_t kScal = kX + 8192;         // beta[64], red[2][64]
  static constexpr uint32_t kBytes = kScal + 1024;
};

__global__ void __launch_bounds__(256) kda_tail_mma_kernel(
    const __nv_bfloat16* __restrict__ v, const __nv_bfloat16* __restrict__ kg, const float* __restrict__ beta,
    const __nv_bfloat16* __restrict__ a_in, const __nv_bfloat16* __restrict__ h_tape,
    const __nv_bfloat16* __restrict__ dh_tape, const __nv_bfloat16* __restrict__ v_new,
    const __nv_bfloat16* __restrict__ dv_new, const __nv_bfloat16* __restrict__ d_o, float* __restrict__ m1,
    float* __restrict__ m2, float* __restrict__ dqg, float* __restrict__ dkr, float* __restrict__ dkg,
    float* __restrict__ hdh, __nv_bfloat16* __restrict__ dv, float* __restrict__ dbeta_part,
    const int32_t* __restrict__ chunk_start, const int32_t* __restrict__ chunk_len, int num_heads, float scale,
    int32_t* __restrict__ status) {
  extern __shared__ uint8_t raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y;
  const int start = chunk_start[c], len = chunk_len[c];
  if (len <= 0) return;
  const int quad = warp & 3, ch = warp >> 2;
  const int row = quad * 16 + (lane & 15);
  const bool owner = lane < 16;
  const bool live = owner && row < len;
  float* s_beta = reinterpret_cast<float*>(sm + KdaTailSmem::kScal);
  float* s_red = s_beta + 64;
  Abort abort{&abort_flag};
  const int64_t stride = int64_t(num_heads) * kDim;
  const int64_t tile = int64_t(c) * num_heads + h;
  const int64_t rows = int64_t(start) * stride + h * kDim;

  if (tid == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
    abort_flag = 0;
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 512);
  load_tile<128, 128, 256>(sm + KdaTailSmem::kH, 16384, h_tape + tile * 16384, 128, 128, tid);
  load_tile<128, 128, 256>(sm + KdaTailSmem::kDH, 16384, dh_tape + tile * 16384, 128, 128, tid);
  load_tile<64, 128, 256>(sm + KdaTailSmem::kDO, 8192, d_o + rows, stride, len, tid);
  load_tile<64, 128, 256>(sm + KdaTailSmem::kVN, 8192, v_new + rows, stride, len, tid);
  load_tile<64, 128, 256>(sm + KdaTailSmem::kDVN, 8192, dv_new + rows, stride, len, tid);
  load_tile<64, 128, 256>(sm + KdaTailSmem::kKG, 8192, kg + rows, stride, len, tid);
  load_tile<64, 128, 256>(sm + KdaTailSmem::kV, 8192, v + rows, stride, len, tid);
  load_tile<64, 64, 256>(sm + KdaTailSmem::kA, 8192, a_in + tile * 4096, 64, 64, tid);
  if (tid < 64) s_beta[tid] = tid < len ? beta[int64_t(start + tid) * num_heads + h] : 0.f;
  __syncthreads();
  for (int i = tid; i < 64 * 16; i += 256) {  // bf16(scale do)
    const int r = i >> 4, cc = i & 15;
    float x[8];
    unpack8(tile_chunk(sm + KdaTailSmem::kDO, 8192, r, cc), x);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] *= scale;
    set_tile_chunk(sm + KdaTailSmem::kDOS, 8192, r, cc, pack8(x));
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t sbase = smem_u32(sm);
  const Operand op_h{sbase + KdaTailSmem::kH, 16384}, op_dh{sbase + KdaTailSmem::kDH, 16384};
  const Operand op_dw{sbase + KdaTailSmem::kH, 8192}, op_kb{sbase + KdaTailSmem::kH + 16384, 8192};
  const Operand op_vb{sbase + KdaTailSmem::kDH, 8192};
  const Operand op_do{sbase + KdaTailSmem::kDO, 8192}, op_dos{sbase + KdaTailSmem::kDOS, 8192};
  const Operand op_vn{sbase + KdaTailSmem::kVN, 8192}, op_dvn{sbase + KdaTailSmem::kDVN, 8192};
  const Operand op_a{sbase + KdaTailSmem::kA, 8192}, op_da{sbase + KdaTailSmem::kDA, 8192};
  const Operand op_x{sbase + KdaTailSmem::kX, 8192};
  constexpr uint32_t cAqk = 0, cDkr = 64, cDqg = 192, cDw = 320;

  uint32_t phase = 0;
  auto mma_wait = [&]() {
    if (!mbar_wait(&bar, phase)) abort.raise();
    phase ^= 1;
    tc_fence_after();
  };
  auto stage_sync = [&]() {
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  };

  // ---- phase 1: dAqk = do v_new^T ; dkr = v_new dh^T ; dqg = (scale do) h^T ; dw = -dv_new h^T --------------------
  if (tid == 0) {
    // in alternating pairs: the instructions of one product wait for one another
    umma_gemm_pair<64, 64, 128>(tmem + cAqk, op_do, false, op_vn, false, 128, false, false, tmem + cDkr, op_vn, false,
                                op_dh, false, 128, false, false);
    umma_gemm_pair<64, 128>(tmem + cDqg, op_dos, false, op_h, false, 128, false, false, tmem + cDw, op_dvn, false, op_h,
                            false, 128, false, /*neg=*/true);
    umma_commit(&bar);
  }
  if (tid < 128) {  // sum_v dh[k, v] h[k, v] per key channel
    float acc = 0.f;
#pragma unroll 4
    for (int cc = 0; cc < 16; ++cc) {
      float a[8], b[8];
      unpack8(tile_chunk(sm + KdaTailSmem::kH, 16384, tid, cc), a);
      unpack8(tile_chunk(sm + KdaTailSmem::kDH, 16384, tid, cc), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc = fmaf(a[j], b[j], acc);
    }
    hdh[tile * kDim + tid] = acc;
  }
  mma_wait();
  __syncthreads();  // every thread is past its reads of h / dh: their space takes dw, kb and vb
  const float beta_row = s_beta[row];
  {
    float s[32];
    tmem_ld32(tmem_addr(tmem, warp, cAqk + ch * 32), s);
    tmem_ld_wait();
    if (owner) {
      float* dst = m1 + tile * 4096 + row * 64 + ch * 32;
#pragma unroll
      for (int j = 0; j < 32; ++j) dst[j] = (ch * 32 + j <= row) ? scale * s[j] : 0.f;
    }
    float* dkr_row = dkr + rows + int64_t(row) * stride + ch * 64;
    float* dqg_row = dqg + rows + int64_t(row) * stride + ch * 64;
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      float a[32], b[32], w[32];
      tmem_ld32(tmem_addr(tmem, warp, cDkr + ch * 64 + p * 32), a);
      tmem_ld32(tmem_addr(tmem, warp, cDqg + ch * 64 + p * 32), b);
      tmem_ld32(tmem_addr(tmem, warp, cDw + ch * 64 + p * 32), w);
      tmem_ld_wait();
      if (live) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          reinterpret_cast<float4*>(dkr_row + p * 32)[j] = make_float4(a[4 * j], a[4 * j + 1], a[4 * j + 2], a[4 * j + 3]);
          reinterpret_cast<float4*>(dqg_row + p * 32)[j] = make_float4(b[4 * j], b[4 * j + 1], b[4 * j + 2], b[4 * j + 3]);
        }
      }
      if (owner) {
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
          set_tile_chunk(sm + KdaTailSmem::kH, 8192, row, ch * 8 + p * 4 + jj, pack8(w + jj * 8));
      }
    }
  }
  for (int i = tid; i < 64 * 16; i += 256) {  // kb = bf16(beta kg), vb = bf16(beta v)
    const int r = i >> 4, cc = i & 15;
    const float b = s_beta[r];
    float x[8];
    unpack8(tile_chunk(sm + KdaTailSmem::kKG, 8192, r, cc), x);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] *= b;
    set_tile_chunk(sm + KdaTailSmem::kH + 16384, 8192, r, cc, pack8(x));
    unpack8(tile_chunk(sm + KdaTailSmem::kV, 8192, r, cc), x);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] *= b;
    set_tile_chunk(sm + KdaTailSmem::kDH, 8192, r, cc, pack8(x));
  }
  stage_sync();

  // ---- phase 2: dkgb = A^T dw ; dvb = A^T dv_new ; dA = dw kb^T + dv_new vb^T -------------------------------------
  if (tid == 0) {
    umma_gemm_pair<64, 128>(tmem + 0, op_a, true, op_dw, true, 64, false, false, tmem + 128, op_a, true, op_dvn, true, 64,
                            false, false);
    umma_gemm<64, 64>(tmem + 256, op_dw, false, op_kb, false, 128, false);
    umma_gemm<64, 64>(tmem + 256, op_dvn, false, op_vb, false, 128, true);
    umma_commit(&bar);
  }
  mma_wait();
  {
    float dot = 0.f;
    float* dkg_row = dkg + rows + int64_t(row) * stride + ch * 64;
    __nv_bfloat16* dv_row = dv + rows + int64_t(row) * stride + ch * 64;
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      float a[32], b[32];
      tmem_ld32(tmem_addr(tmem, warp, 0 + ch * 64 + p * 32), a);
      tmem_ld32(tmem_addr(tmem, warp, 128 + ch * 64 + p * 32), b);
      tmem_ld_wait();
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        float kgv[8], vv[8], out[8], dk8[8];
        unpack8(tile_chunk(sm + KdaTailSmem::kKG, 8192, row, ch * 8 + p * 4 + jj), kgv);
        unpack8(tile_chunk(sm + KdaTailSmem::kV, 8192, row, ch * 8 + p * 4 + jj), vv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float x = a[jj * 8 + e], y = b[jj * 8 + e];
          dot = fmaf(x, kgv[e], dot);
          dot = fmaf(y, vv[e], dot);
          dk8[e] = beta_row * x;
          out[e] = beta_row * y;
        }
        if (live) {
          reinterpret_cast<float4*>(dkg_row + p * 32)[2 * jj] = make_float4(dk8[0], dk8[1], dk8[2], dk8[3]);
          reinterpret_cast<float4*>(dkg_row + p * 32)[2 * jj + 1] = make_float4(dk8[4], dk8[5], dk8[6], dk8[7]);
          reinterpret_cast<uint4*>(dv_row + p * 32)[jj] = pack8(out);
        }
      }
    }
    if (owner) s_red[ch * 64 + row] = dot;
    float s[32];
    tmem_ld32(tmem_addr(tmem, warp, 256 + ch * 32), s);
    tmem_ld_wait();
    if (owner) {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) set_tile_chunk(sm + KdaTailSmem::kDA, 8192, row, ch * 4 + jj, pack8(s + jj * 8));
    }
  }
  stage_sync();
  if (tid < len) dbeta_part[int64_t(start + tid) * num_heads + h] = s_red[tid] + s_red[64 + tid];

  // ---- phase 3: X = A^T dA ------------------------------------------------------------------------------------------
  if (tid == 0) {
    umma_gemm<64, 64>(tmem + 320, op_a, true, op_da, true, 64, false);
    umma_commit(&bar);
  }
  mma_wait();
  {
    float s[32];
    tmem_ld32(tmem_addr(tmem, warp, 320 + ch * 32), s);
    tmem_ld_wait();
    if (owner) {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) set_tile_chunk(sm + KdaTailSmem::kX, 8192, row, ch * 4 + jj, pack8(s + jj * 8));
    }
  }
  stage_sync();

  // ---- phase 4: Y = X A^T ; dL = bf16(-tril(Y, -1)) -----------------------------------------------------------------
  if (tid == 0) {
    umma_gemm<64, 64>(tmem + 384, op_x, false, op_a, false, 64, false);
    umma_commit(&bar);
  }
  mma_wait();
  {
    float s[32];
    tmem_ld32(tmem_addr(tmem, warp, 384 + ch * 32), s);
    tmem_ld_wait();
    if (owner) {
      float* dst = m2 + tile * 4096 + row * 64 + ch * 32;
#pragma unroll
      for (int j = 0; j < 32; ++j) dst[j] = (ch * 32 + j < row) ? round_bf16(-s[j]) : 0.f;
    }
  }
  if (abort.raised() && tid == 0) atomicExch(status, kDevWaitTimeout | (7 << 8));
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------------------------------------
// tail, pairwise part: one block per (chunk, head); thread (d, role) owns key channel d in one of two passes
// ---------------------------------------------------------------------------------------------------------------
// With E_ij = 2^{G_i - G_j} per channel (j <= i), M1 = scale tril(do v_new^T) and M2 = bf16(-tril(A^T dA A^T, -1)):
//   row pass     RQ_i = sum_{j<=i} M1_ij k_j E_ij,  RK_i = sum_{j<i} M2_ij k_j E_ij     -> dq, the row part of dk, dg
//   column pass  CC_j = sum_{i>=j} (M1_ij q_i + beta_i M2_ij k_i) E_ij                  -> the column part of dk, dg
// No pair costs an exponential: E runs along a row or a column as a product of the per-token factors
// R_i = 2^{G_i - G_{i-1}} <= 1 (E_{i,j-1} = E_ij R_j, E_{i+1,j} = E_ij R_{i+1}); all sums live in registers.  512
// threads: thread (d, role, half) owns channel d in the row pass (role 0) or the column pass (role 1) for the even
// (half 0) or odd (half 1) blocks of four rows / columns, so sixteen warps hide each other's latencies.
struct KdaPairSmem {
  static constexpr uint32_t kQ = 0;                  // fp32 [64][128] q
  static constexpr uint32_t kK = 32768;              // fp32 [64][128] k
  static constexpr uint32_t kR = 2 * 32768;          // fp32 [64][128] R
  static constexpr uint32_t kCC = 3 * 32768;         // fp32 [64][128] column-pass sums
  static constexpr uint32_t kM1 = 4 * 32768;         // fp32 [64][64] M1
  static constexpr uint32_t kM2 = kM1 + 16384;       // fp32 [64][64] M2
  static constexpr uint32_t kM1T = kM2 + 16384;      // fp32 [64][68] M1^T
  static constexpr uint32_t kM2T = kM1T + 17408;     // fp32 [64][68] (beta_i M2_ij)^T
  static constexpr uint32_t kBeta = kM2T + 17408;    // beta[64], db[64][4]
  static constexpr uint32_t kBytes = kBeta + 256 + 1024;
};

__global__ void __launch_bounds__(512) kda_tail_pair_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const float* __restrict__ g2,
    const float* __restrict__ beta, const float* __restrict__ m1, const float* __restrict__ m2,
    const float* __restrict__ dqg, const float* __restrict__ dkr, const float* __restrict__ dkg,
    const float* __restrict__ hdh, const float* __restrict__ dbeta_part, float* __restrict__ dq, float* __restrict__ dk,
    float* __restrict__ dg, float* __restrict__ dbeta, const int32_t* __restrict__ chunk_start,
    const int32_t* __restrict__ chunk_len, int num_heads) {
  extern __shared__ uint8_t raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 127) & ~uintptr_t(127));
  const int tid = threadIdx.x, d = tid & 127, role = (tid >> 7) & 1, half = tid >> 8, warp = (tid >> 5) & 3;
  const int lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y;
  const int start = chunk_start[c], len = chunk_len[c];
  if (len <= 0) return;
  float* sQ = reinterpret_cast<float*>(sm + KdaPairSmem::kQ);
  float* sK = reinterpret_cast<float*>(sm + KdaPairSmem::kK);
  float* sR = reinterpret_cast<float*>(sm + KdaPairSmem::kR);
  float* sCC = reinterpret_cast<float*>(sm + KdaPairSmem::kCC);
  float* sM1 = reinterpret_cast<float*>(sm + KdaPairSmem::kM1);
  float* sM2 = reinterpret_cast<float*>(sm + KdaPairSmem::kM2);
  float* sM1T = reinterpret_cast<float*>(sm + KdaPairSmem::kM1T);
  float* sM2T = reinterpret_cast<float*>(sm + KdaPairSmem::kM2T);
  float* s_beta = reinterpret_cast<float*>(sm + KdaPairSmem::kBeta);
  float* s_db = s_beta + 64;
  const int64_t stride = int64_t(num_heads) * kDim;
  const int64_t tile = int64_t(c) * num_heads + h;
  const int64_t col = int64_t(start) * stride + h * kDim + d;

  if (tid < 64) s_beta[tid] = tid < len ? beta[int64_t(start + tid) * num_heads + h] : 0.f;
#pragma unroll 8
  for (int i = tid >> 7; i < 64; i += 4) {  // rows past the chunk's length: q = k = 0, R = 1
    const bool live = i < len;
    const int64_t at = col + int64_t(live ? i : 0) * stride;
    sQ[i * 128 + d] = live ? __bfloat162float(q[at]) : 0.f;
    sK[i * 128 + d] = live ? __bfloat162float(k[at]) : 0.f;
    sR[i * 128 + d] = (live && i > 0) ? fast_exp2(g2[at] - g2[at - stride]) : 1.f;
  }
  __syncthreads();  // beta is in place for the transposed copy of M2
#pragma unroll 8
  for (int i = tid; i < 4096; i += 512) {  // M and its transpose (rows of 68 floats: 16-byte aligned, few conflicts)
    const float a = m1[tile * 4096 + i], b = m2[tile * 4096 + i];
    const int ii = i >> 6, jj = i & 63;
    sM1[i] = a;
    sM2[i] = b;
    sM1T[jj * 68 + ii] = a;
    sM2T[jj * 68 + ii] = s_beta[ii] * b;
  }
  __syncthreads();

  float chunk_end = 0.f;
  if (role == 0) {
    // ---- row pass: four rows at a time.  For j below the block, E_{i0+r, j} = E_{i0, j} E_{i0+r, i0}: the four rows
    // share k_j E_{i0, j} and take their own factor (<= 1) once at the end; the 4 x 4 diagonal block is done apart.
    const float gl = g2[col + int64_t(len - 1) * stride];
    for (int i0 = 4 * half; i0 < len; i0 += 8) {
      float rq[4] = {0.f, 0.f, 0.f, 0.f}, rk[4] = {0.f, 0.f, 0.f, 0.f};
      float gi4[4], xq4[4], xr4[4], xg4[4];  // the rows' global operands, in flight while the sums run
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int64_t at = col + int64_t(i0 + r < len ? i0 + r : len - 1) * stride;
        gi4[r] = g2[at], xq4[r] = dqg[at], xr4[r] = dkr[at], xg4[r] = dkg[at];
      }
      float e = sR[i0 * 128 + d];  // E_{i0, i0 - 1}
      for (int j0 = i0 - 4; j0 >= 0; j0 -= 4) {
        float av[4][4], bv[4][4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float4 a = *reinterpret_cast<const float4*>(sM1 + (i0 + r) * 64 + j0);
          const float4 b = *reinterpret_cast<const float4*>(sM2 + (i0 + r) * 64 + j0);
          av[r][0] = a.x, av[r][1] = a.y, av[r][2] = a.z, av[r][3] = a.w;
          bv[r][0] = b.x, bv[r][1] = b.y, bv[r][2] = b.z, bv[r][3] = b.w;
        }
#pragma unroll
        for (int t = 3; t >= 0; --t) {
          const float kj = sK[(j0 + t) * 128 + d] * e;
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            rq[r] = fmaf(av[r][t], kj, rq[r]);
            rk[r] = fmaf(bv[r][t], kj, rk[r]);
          }
          e *= sR[(j0 + t) * 128 + d];
        }
      }
      float r4[4], k4[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) r4[r] = sR[(i0 + r) * 128 + d], k4[r] = sK[(i0 + r) * 128 + d];
      {
        float f = 1.f;
#pragma unroll
        for (int r = 1; r < 4; ++r) {
          f *= r4[r];  // E_{i0 + r, i0}
          rq[r] *= f;
          rk[r] *= f;
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {  // the diagonal block: pairs (i0 + r, i0 + t), t <= r
        const float4 a = *reinterpret_cast<const float4*>(sM1 + (i0 + r) * 64 + i0);
        const float4 b = *reinterpret_cast<const float4*>(sM2 + (i0 + r) * 64 + i0);  // zero on the diagonal
        const float at4[4] = {a.x, a.y, a.z, a.w}, bt4[4] = {b.x, b.y, b.z, b.w};
        float ee = 1.f;
#pragma unroll
        for (int t = r; t >= 0; --t) {
          const float kj = k4[t] * ee;
          rq[r] = fmaf(at4[t], kj, rq[r]);
          rk[r] = fmaf(bt4[t], kj, rk[r]);
          ee *= r4[t];
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int i = i0 + r;
        float db = 0.f;
        if (i < len) {
          const float qi = sQ[i * 128 + d], ki = k4[r], bi = s_beta[i];
          const int64_t at = col + i * stride;
          const float gi = gi4[r];
          const float eg = fast_exp2(gi), er = fast_exp2(gl - gi);
          const float qgr = round_bf16(qi * eg), kgr = round_bf16(ki * eg), krr = round_bf16(ki * er);
          const float xq = xq4[r], xr = xr4[r], xg = xg4[r];
          dq[at] = fmaf(xq, eg, rq[r]);
          dk[at] = fmaf(bi, rk[r], fmaf(xr, er, xg * eg));                             // + the column part below
          dg[at] = qi * rq[r] + ki * bi * rk[r] + xq * qgr + xg * kgr - xr * krr;      // likewise
          chunk_end = fmaf(xr, krr, chunk_end);
          db = ki * rk[r];  // dbeta_i += sum_d k_id RK_id
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) db += __shfl_xor_sync(0xffffffffu, db, m);
        if (lane == 0 && i < len) s_db[i * 4 + warp] = db;
      }
    }
    if (half == 0) chunk_end = fmaf(fast_exp2(gl), hdh[tile * kDim + d], chunk_end);
  } else {
    // ---- column pass: four columns at a time.  For i below the block, E_{i, j0+c} = E_{i, j0+3} E_{j0+3, j0+c}.
    for (int j0 = 4 * half; j0 < len; j0 += 8) {
      float cc[4] = {0.f, 0.f, 0.f, 0.f};
      float e = 1.f;
      for (int i0 = j0 + 4; i0 < len; i0 += 4) {  // rows at or past the chunk's length hold q = k = 0 and R = 1
        float av[4][4], bv[4][4];
#pragma unroll
        for (int cidx = 0; cidx < 4; ++cidx) {
          const float4 a = *reinterpret_cast<const float4*>(sM1T + (j0 + cidx) * 68 + i0);
          const float4 b = *reinterpret_cast<const float4*>(sM2T + (j0 + cidx) * 68 + i0);
          av[cidx][0] = a.x, av[cidx][1] = a.y, av[cidx][2] = a.z, av[cidx][3] = a.w;
          bv[cidx][0] = b.x, bv[cidx][1] = b.y, bv[cidx][2] = b.z, bv[cidx][3] = b.w;
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          e *= sR[(i0 + t) * 128 + d];  // E_{i0 + t, j0 + 3}
          const float tq = sQ[(i0 + t) * 128 + d] * e, tk = sK[(i0 + t) * 128 + d] * e;
#pragma unroll
          for (int cidx = 0; cidx < 4; ++cidx) cc[cidx] = fmaf(av[cidx][t], tq, fmaf(bv[cidx][t], tk, cc[cidx]));
        }
      }
      float r4[4], k4[4], q4[4];
#pragma unroll
      for (int r = 0; r < 4; ++r)
        r4[r] = sR[(j0 + r) * 128 + d], k4[r] = sK[(j0 + r) * 128 + d], q4[r] = sQ[(j0 + r) * 128 + d];
      {
        float f = 1.f;
#pragma unroll
        for (int cidx = 2; cidx >= 0; --cidx) {
          f *= r4[cidx + 1];  // E_{j0 + 3, j0 + cidx}
          cc[cidx] *= f;
        }
      }
#pragma unroll
      for (int cidx = 0; cidx < 4; ++cidx) {  // the diagonal block: pairs (j0 + r, j0 + cidx), r >= cidx
        const float4 a = *reinterpret_cast<const float4*>(sM1T + (j0 + cidx) * 68 + j0);
        const float4 b = *reinterpret_cast<const float4*>(sM2T + (j0 + cidx) * 68 + j0);
        const float at4[4] = {a.x, a.y, a.z, a.w}, bt4[4] = {b.x, b.y, b.z, b.w};
        float ee = 1.f;
#pragma unroll
        for (int r = cidx; r < 4; ++r) {
          if (r > cidx) ee *= r4[r];
          cc[cidx] = fmaf(fmaf(at4[r], q4[r], bt4[r] * k4[r]), ee, cc[cidx]);
        }
        sCC[(j0 + cidx) * 128 + d] = cc[cidx];
      }
    }
  }
  float* s_end = sR;  // after the passes: the chunk-end term per channel (two halves) in R's space ...
  float* s_dg = sQ;   // ... and the per-row gate gradients in q's space
  __syncthreads();
  if (role == 0) s_end[half * 128 + d] = chunk_end;
  __syncthreads();
  // every thread: the column parts join the row parts (which the row pass left in dk and dg) -- elementwise, so the
  // global reads overlap; the block barriers above order the row pass's global writes before these reads
#pragma unroll 8
  for (int i = tid >> 7; i < len; i += 4) {
    const int64_t at = col + i * stride;
    const float cc = sCC[i * 128 + d];
    dk[at] += cc;
    float dgi = dg[at] - sK[i * 128 + d] * cc;
    if (i == len - 1) dgi += s_end[d] + s_end[128 + d];
    s_dg[i * 128 + d] = dgi;
  }
  __syncthreads();
  if (tid < 128) {  // the in-chunk suffix sum, one channel per thread
    float running = 0.f;
    for (int i = len - 1; i >= 0; --i) {
      running += s_dg[i * 128 + d];
      dg[col + i * stride] = running;
    }
  } else if (tid < 256 && d < len) {
    const int64_t at = int64_t(start + d) * num_heads + h;
    dbeta[at] = dbeta_part[at] + ((s_db[d * 4] + s_db[d * 4 + 1]) + (s_db[d * 4 + 2] + s_db[d * 4 + 3]));
  }
}

// One warp per row of 128: out = bf16(x) or, with the norm's saved r, bf16(r (x - y (x . y))), y = raw r.
__global__ void __launch_bounds__(256) qk_grad_finish_kernel(const float* __restrict__ x,
                                                             const __nv_bfloat16* __restrict__ raw_rows,
                                                             const float* __restrict__ rstd,
                                                             __nv_bfloat16* __restrict__ out, int64_t rows) {
  const int64_t row = int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float4 xv = reinterpret_cast<const float4*>(x + row * kDim)[lane];
  if (rstd != nullptr) {
    const float r = rstd[row];
    const uint2 rawv = __ldg(reinterpret_cast<const uint2*>(raw_rows + row * kDim) + lane);
    const float2 a = unpack_bf16(rawv.x), b = unpack_bf16(rawv.y);
    const float y0 = a.x * r, y1 = a.y * r, y2 = b.x * r, y3 = b.y * r;
    float dot = xv.x * y0 + xv.y * y1 + xv.z * y2 + xv.w * y3;
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, m);
    xv = make_float4(r * (xv.x - y0 * dot), r * (xv.y - y1 * dot), r * (xv.z - y2 * dot), r * (xv.w - y3 * dot));
  }
  uint2 o;
  o.x = pack_bf16(xv.x, xv.y);
  o.y = pack_bf16(xv.z, xv.w);
  reinterpret_cast<uint2*>(out + row * kDim)[lane] = o;
}

}  // namespace mek

namespace {

int check_kda(const MekGdnDims* d, const char* what) {
  using namespace mek;
  if (d == nullptr) return fail(MEK_ERR_INVALID, "%s: dims is null", what);
  if (d->total_tokens <= 0 || d->num_chunks <= 0 || d->num_seqs <= 0)
    return fail(MEK_ERR_INVALID, "%s: no tokens", what);
  if (d->num_qk_heads != d->num_v_heads || d->num_v_heads < 1 || d->num_v_heads > 64)
    return fail(MEK_ERR_INVALID, "%s: KDA serves 1 to 64 heads with one value head per key head, got H=%d HV=%d", what,
                d->num_qk_heads, d->num_v_heads);
  if (d->head_dim != 128) return fail(MEK_ERR_UNSUPPORTED, "%s: head dims must be 128, not %d", what, d->head_dim);
  return MEK_OK;
}

typedef const __nv_bfloat16* In;
typedef __nv_bfloat16* Out;

}  // namespace

extern "C" {

int mek_kda_prep(const MekGdnDims* d, const void* q, const void* k, const float* g, float* g2, void* qg, void* kg,
                 void* kr, float* gl2, void* stream) {
  using namespace mek;
  if (int rc = check_kda(d, "kda_prep")) return rc;
  kda_prep_kernel<<<dim3(d->num_chunks, d->num_v_heads), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      In(q), In(k), g, g2, Out(qg), Out(kg), Out(kr), gl2, d->chunk_start, d->chunk_len, d->num_v_heads);
  return launched("kda_prep");
}

int mek_kda_intra(const MekGdnDims* d, const void* q, const void* k, const void* v, const void* kg, const float* g2,
                  const float* beta, void* a_out, void* aqk_out, void* w_out, void* u_out, int32_t* status,
                  void* stream) {
  using namespace mek;
  if (int rc = check_kda(d, "kda_intra")) return rc;
  const size_t smem = KdaIntraSmem::kBytes + 1024;
  if (int rc = want_smem(kda_intra_kernel, smem, "kda_intra")) return rc;
  kda_intra_kernel<<<dim3(d->num_chunks, d->num_v_heads), 288, smem, static_cast<cudaStream_t>(stream)>>>(
      In(q), In(k), In(v), In(kg), g2, beta, Out(a_out), Out(aqk_out), Out(w_out), Out(u_out), d->chunk_start,
      d->chunk_len, d->num_v_heads, d->scale, status);
  return launched("kda_intra");
}

int mek_kda_bwd_tail(const MekGdnDims* d, const void* q, const void* k, const void* v, const void* kg, const float* g2,
                     const float* beta, const void* a, const void* h_tape, const void* dh_tape, const void* v_new,
                     const void* dv_new, const void* d_o, float* m1, float* m2, float* dqg, float* dkr, float* dkg,
                     float* hdh, float* dbeta_part, float* dq32, float* dk32, void* dv, float* dg, float* dbeta,
                     int32_t* status, void* stream) {
  using namespace mek;
  if (int rc = check_kda(d, "kda_bwd_tail")) return rc;
  const size_t smem_a = KdaTailSmem::kBytes + 1024, smem_b = KdaPairSmem::kBytes + 128;
  if (int rc = want_smem(kda_tail_mma_kernel, smem_a, "kda_bwd_tail")) return rc;
  if (int rc = want_smem(kda_tail_pair_kernel, smem_b, "kda_bwd_tail")) return rc;
  const dim3 grid(d->num_chunks, d->num_v_heads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  kda_tail_mma_kernel<<<grid, 256, smem_a, s>>>(In(v), In(kg), beta, In(a), In(h_tape), In(dh_tape), In(v_new),
                                                In(dv_new), In(d_o), m1, m2, dqg, dkr, dkg, hdh, Out(dv), dbeta_part,
                                                d->chunk_start, d->chunk_len, d->num_v_heads, d->scale, status);
  if (int rc = launched("kda_bwd_tail (tensor-core part)")) return rc;
  kda_tail_pair_kernel<<<grid, 512, smem_b, s>>>(In(q), In(k), g2, beta, m1, m2, dqg, dkr, dkg, hdh, dbeta_part, dq32,
                                                 dk32, dg, dbeta, d->chunk_start, d->chunk_len, d->num_v_heads);
  return launched("kda_bwd_tail (pairwise part)");
}

int mek_qk_grad_finish(const float* x, const void* raw_rows, const float* rstd, void* out, int64_t rows,
                       void* stream) {
  using namespace mek;
  if (rows <= 0 || !x || !out) return fail(MEK_ERR_INVALID, "qk_grad_finish: rows=%lld or a null pointer", (long long)rows);
  if (rstd != nullptr && raw_rows == nullptr)
    return fail(MEK_ERR_INVALID, "qk_grad_finish: the norm's pull-back needs the raw rows");
  qk_grad_finish_kernel<<<unsigned((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      x, In(raw_rows), rstd, Out(out), rows);
  return launched("qk_grad_finish");
}

}  // extern "C"
