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
//   kda_intra       Aqk_ij = scale sum_d q_id k_jd 2^{G_id - G_jd}, L_ij = beta_i sum_d k_id k_jd 2^{G_id - G_jd}:
//                   blocks of 16 rows; below the block diagonal one tensor-core product of operands scaled against
//                   the gate at the block's first row, on it pair by pair (every exponent is formed from a
//                   non-positive difference: finite for any gate); then A = (I + L)^-1, w = A (beta kg),
//                   u = A (beta v)                                                          [tcgen05 + CUDA cores]
//   kda_tail_mma    the state-side gradient contractions, persistent over the (chunk, head) items, computed
//                   transposed (channel = accumulator row) so that its fp32 results leave in whole lines      [tcgen05]
//   kda_tail_pair   the decayed gradient contractions (the same split: tensor core below the block diagonal,
//                   running products on it), dq, dk and the per-channel gate gradient with its in-chunk suffix
//                   sum                                                                     [tcgen05 + CUDA cores]
//   qk_grad_finish  fp32 dq / dk -> the L2 norm's pull-back (optional) -> bf16
#include "common.cuh"
#include "tiles.cuh"
#include "tma.cuh"

namespace mek {

// ---------------------------------------------------------------------------------------------------------------
// prep: one block per (chunk, head), one thread per pair of key channels
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(64) kda_prep_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const float* __restrict__ g,
    float* __restrict__ g2, __nv_bfloat16* __restrict__ qg, __nv_bfloat16* __restrict__ kg,
    __nv_bfloat16* __restrict__ kr, float* __restrict__ gl2, const int32_t* __restrict__ chunk_start,
    const int32_t* __restrict__ chunk_len, int num_heads) {
  // a thread owns two neighbouring key channels: 4-byte bf16 pairs and 8-byte gate pairs (whole lines per warp)
  const int c = blockIdx.x, h = blockIdx.y, d = 2 * threadIdx.x;
  const int start = chunk_start[c], len = chunk_len[c];
  if (len <= 0) return;
  const int64_t stride = int64_t(num_heads) * kDim;
  const int64_t base = int64_t(start) * stride + h * kDim + d;
  auto pair_at = [](const __nv_bfloat16* p) { return unpack_bf16(*reinterpret_cast<const uint32_t*>(p)); };
  auto put_pair = [](__nv_bfloat16* p, float x, float y) { *reinterpret_cast<uint32_t*>(p) = pack_bf16(x, y); };
  // tokens in batches of eight: a batch's loads are all issued before the running sum needs the first of them
  float acc0 = 0.f, acc1 = 0.f;
  for (int i0 = 0; i0 < len; i0 += 8) {
    float2 gv[8], qv[8], kv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool in = i0 + j < len;
      const int64_t at = base + (in ? i0 + j : i0) * stride;
      gv[j] = in ? *reinterpret_cast<const float2*>(g + at) : make_float2(0.f, 0.f);
      qv[j] = pair_at(q + at);
      kv[j] = pair_at(k + at);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (i0 + j < len) {
        const int64_t at = base + (i0 + j) * stride;
        acc0 += gv[j].x, acc1 += gv[j].y;
        const float g0 = acc0 * kLog2e, g1 = acc1 * kLog2e, e0 = fast_exp2(g0), e1 = fast_exp2(g1);
        *reinterpret_cast<float2*>(g2 + at) = make_float2(g0, g1);
        put_pair(qg + at, qv[j].x * e0, qv[j].y * e1);
        put_pair(kg + at, kv[j].x * e0, kv[j].y * e1);
      }
    }
  }
  const float gl0 = acc0 * kLog2e, gl1 = acc1 * kLog2e;
  *reinterpret_cast<float2*>(gl2 + (int64_t(c) * num_heads + h) * kDim + d) = make_float2(gl0, gl1);
  for (int i0 = 0; i0 < len; i0 += 8) {
    float2 gv[8], kv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t at = base + (i0 + j < len ? i0 + j : i0) * stride;
      gv[j] = *reinterpret_cast<const float2*>(g2 + at);
      kv[j] = pair_at(k + at);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (i0 + j < len)
        put_pair(kr + base + (i0 + j) * stride, kv[j].x * fast_exp2(gl0 - gv[j].x), kv[j].y * fast_exp2(gl1 - gv[j].y));
  }
}

// ---------------------------------------------------------------------------------------------------------------
// intra: Aqk, A, w, u of one (chunk, head)
// ---------------------------------------------------------------------------------------------------------------
// The two pairwise matrices  S_qk[i][j] = sum_d q_id k_jd 2^{G_id - G_jd}  and  S_kk (k in place of q), j <= i, are
// split by blocks of 16 rows.  With R the first row of i's block and j in an EARLIER block,
//     2^{G_i - G_j} = 2^{G_i - G_R} 2^{G_R - G_j}          (both exponents <= 0 per channel: G falls along the chunk)
// so the blocks below the block diagonal are ONE tensor-core product of bounded bf16 operands,
//     [q~ ; k~'] [128 x 128]  x  stack^T [128 x 96],   q~_i = q_i 2^{G_i - G_R},  k~'_i = k_i 2^{G_i - G_R},
//     stack = [k_j 2^{G_16 - G_j}, j < 16 ; k_j 2^{G_32 - G_j}, j < 32 ; k_j 2^{G_48 - G_j}, j < 48]
// (row block I of the result reads its own 16 I columns of the stack); only the four 16 x 16 blocks on the diagonal
// are summed pair by pair on CUDA cores, every exponent formed from a non-positive difference.  Finite for any gate:
// a factor that underflows belongs to a pair whose true weight underflows too.
struct KdaIntraSmem {
  static constexpr int kGRow = 132;                                 // fp32 row stride of the G copy
  static constexpr uint32_t kQK = 0;          // [128][128] bf16: rows 0..63 q -> q~, 64..127 k -> k~'; 2 blocks of 16 KiB
  static constexpr uint32_t kStack = 32768;   // [96][128] bf16: 2 blocks of 12 KiB
  static constexpr uint32_t kG = kStack + 24576;                    // fp32 [64][132]
  static constexpr uint32_t kVB = kG + 64 * kGRow * 4;              // [64][128] beta v
  static constexpr uint32_t kBeta = kVB + 16384;                    // beta[64]
  static constexpr uint32_t kBytes = kBeta + 256;
  // after the block product (the operands above are dead):
  static constexpr uint32_t kA = kQK;                               // [64][64] bf16
  static constexpr uint32_t kKB = kQK + 8192;                       // [64][128] beta kg
  static constexpr uint32_t kL = kStack;                            // fp32 [64][64], the TF32 operand layout (16 KiB)
  static constexpr uint32_t kSqk = kG;                              // fp32 [64][65]
  static constexpr uint32_t kSkk = kSqk + 64 * 65 * 4;
  static_assert(kKB + 16384 <= kStack && 64 * 64 * 4 <= 24576 && 2 * 64 * 65 * 4 <= 64 * kGRow * 4, "overlays fit");
};

// element (row, d) of a bf16 tile made of 64-column swizzled blocks `block_stride` bytes apart
__device__ __forceinline__ float tile_elem(const uint8_t* tile, uint32_t block_stride, int row, int d) {
  const uint8_t* at = tile + (d >> 6) * block_stride + sw128_offset(row, (d & 63) >> 3) + (d & 7) * 2;
  return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(at));
}

struct KdaIntraMaps {
  CUtensorMap q, k;  // rows [tokens, H * 128], box 64 x 64
};

constexpr int kIntraThreads = 320;  // 40 sub-blocks of the block diagonal x 8 channel slices

__global__ void __launch_bounds__(kIntraThreads, 2) kda_intra_kernel(
    const __grid_constant__ KdaIntraMaps maps, const __nv_bfloat16* __restrict__ v,
    const __nv_bfloat16* __restrict__ kg, const float* __restrict__ g2, const float* __restrict__ beta,
    __nv_bfloat16* __restrict__ a_out, __nv_bfloat16* __restrict__ aqk_out, __nv_bfloat16* __restrict__ w_out,
    __nv_bfloat16* __restrict__ u_out, const int32_t* __restrict__ chunk_start, const int32_t* __restrict__ chunk_len,
    int num_heads, float scale, int32_t* __restrict__ status) {
  extern __shared__ uint8_t raw[];
  __shared__ uint64_t bar, bar_load;
  __shared__ uint32_t tmem_slot;
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y;
  const int start = chunk_start[c], len = chunk_len[c];
  if (len <= 0) return;
  constexpr int kGRow = KdaIntraSmem::kGRow;
  uint8_t* qk_tile = sm + KdaIntraSmem::kQK;      // rows 0..63 q, rows 64..127 k
  uint8_t* stack = sm + KdaIntraSmem::kStack;
  float* sg = reinterpret_cast<float*>(sm + KdaIntraSmem::kG);
  float* s_qk = reinterpret_cast<float*>(sm + KdaIntraSmem::kSqk);
  float* s_kk = reinterpret_cast<float*>(sm + KdaIntraSmem::kSkk);
  float* s_l = reinterpret_cast<float*>(sm + KdaIntraSmem::kL);
  float* s_beta = reinterpret_cast<float*>(sm + KdaIntraSmem::kBeta);
  const int64_t stride = int64_t(num_heads) * kDim;
  const int64_t tile = int64_t(c) * num_heads + h;
  const uint32_t sbase = smem_u32(sm);

  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_init(&bar_load, 1);
    fence_mbar_init();
    // q and k rows by TMA into the stacked operand: block b of q at b * 16 KiB, of k 8 KiB behind it
    mbar_arrive_expect(&bar_load, 2 * 16384);
    tma_load_box(sbase + KdaIntraSmem::kQK, &maps.q, h * kDim, start, &bar_load);
    tma_load_box(sbase + KdaIntraSmem::kQK + 16384, &maps.q, h * kDim + 64, start, &bar_load);
    tma_load_box(sbase + KdaIntraSmem::kQK + 8192, &maps.k, h * kDim, start, &bar_load);
    tma_load_box(sbase + KdaIntraSmem::kQK + 24576, &maps.k, h * kDim + 64, start, &bar_load);
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 256);
  for (int i = tid; i < 64 * 32; i += kIntraThreads) {  // the gates: rows past the chunk's length keep the last gate
    const int r = i >> 5, d = (i & 31) * 4;              // (every pair exponent stays <= 0)
    const int64_t at = int64_t(start + (r < len ? r : len - 1)) * stride + h * kDim + d;
    *reinterpret_cast<float4*>(sg + r * kGRow + d) = __ldg(reinterpret_cast<const float4*>(g2 + at));
  }
  if (tid < 64) s_beta[tid] = tid < len ? beta[int64_t(start + tid) * num_heads + h] : 0.f;
  __syncthreads();  // the barrier's initialisation is visible to every waiter
  bool ok = __all_sync(0xffffffffu, mbar_wait(&bar_load, 0));
  if (len < kChunk) {  // a ragged chunk's boxes reach into the next sequence: clear those rows of q and k
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int i = tid; i < (64 - len) * 32; i += kIntraThreads) {
      const int r = len + (i >> 5), part = i & 31;  // 8 chunks of q and of k in each of the two blocks
      const int blk = part >> 4, which = (part >> 3) & 1, cc = part & 7;
      *reinterpret_cast<uint4*>(qk_tile + blk * 16384 + which * 8192 + r * 128 + cc * 16) = zero;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  // ---- the four 16 x 16 diagonal blocks, pair by pair: thread (4 x 4 sub-block, eighth of the channels) ----------
  // sub-blocks (bi, bj), bj <= bi, of a 16-block: 10 of them, 40 in all, times 8 channel slices = every thread.  A
  // thread takes four runs of 4 channels (8-byte loads of the swizzled rows).  Off the sub-diagonal every pair is
  // valid and 2^{G_i - G_j} factors as 2^{G_i - G_{j0+3}} 2^{G_{j0+3} - G_j} with both exponents <= 0.
  float aqk[4][4], akk[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) aqk[a][b] = akk[a][b] = 0.f;
  int i0 = 0, j0 = 0;
  {
    // warps 0..3 take the 16 sub-blocks on the diagonal, warps 4..9 the 24 below it: no warp runs both branches
    const int s = tid >> 3, slice = tid & 7;
    const int big = s < 16 ? s >> 2 : (s - 16) / 6, t = s < 16 ? 0 : (s - 16) % 6;
    const int bi = s < 16 ? (s & 3) : (t < 1 ? 1 : (t < 3 ? 2 : 3));
    const int bj = s < 16 ? bi : t - bi * (bi - 1) / 2;
    i0 = 16 * big + 4 * bi, j0 = 16 * big + 4 * bj;
    // 4 channels d .. d + 3 of tile row `row`: half of a 16-byte chunk
    auto four = [&](int row, int d, float* out) {
      const uint2 w = *reinterpret_cast<const uint2*>(qk_tile + (d >> 6) * 16384 + sw128_offset(row, (d & 63) >> 3) +
                                                      (d & 4) * 2);
      const float2 lo = unpack_bf16(w.x), hi = unpack_bf16(w.y);
      out[0] = lo.x, out[1] = lo.y, out[2] = hi.x, out[3] = hi.y;
    };
    auto gates = [&](int row, int d, float* out) {
      const float4 x = *reinterpret_cast<const float4*>(sg + row * kGRow + d);
      out[0] = x.x, out[1] = x.y, out[2] = x.z, out[3] = x.w;
    };
#pragma unroll 1
    for (int n = 0; n < 4; ++n) {
      const int d = (n * 8 + slice) * 4;
      if (bi != bj) {
        float kj[4][4], g3[4];
        gates(j0 + 3, d, g3);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          float gj[4];
          four(64 + j0 + b, d, kj[b]);
          if (b < 3) {
            gates(j0 + b, d, gj);
#pragma unroll
            for (int e = 0; e < 4; ++e) kj[b][e] *= fast_exp2(g3[e] - gj[e]);
          }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          float qa[4], ka[4], ga[4];
          four(i0 + a, d, qa);
          four(64 + i0 + a, d, ka);
          gates(i0 + a, d, ga);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float ea = fast_exp2(ga[e] - g3[e]);
            qa[e] *= ea, ka[e] *= ea;
          }
#pragma unroll
          for (int b = 0; b < 4; ++b)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              aqk[a][b] = fmaf(qa[e], kj[b][e], aqk[a][b]);
              akk[a][b] = fmaf(ka[e], kj[b][e], akk[a][b]);
            }
        }
      } else {
        float qi[4][4], ki[4][4], gi[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          four(i0 + a, d, qi[a]);
          four(64 + i0 + a, d, ki[a]);
          gates(i0 + a, d, gi[a]);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b <= a; ++b)
#pragma unroll
            for (int e = 0; e < 4; ++e) {  // the exponent of a valid pair is <= 0
              const float w = fast_exp2(gi[a][e] - gi[b][e]) * ki[b][e];
              aqk[a][b] = fmaf(qi[a][e], w, aqk[a][b]);
              akk[a][b] = fmaf(ki[a][e], w, akk[a][b]);
            }
      }
    }
  }
  // the eight channel slices of a sub-block sit in neighbouring lanes: a fixed-order butterfly sum
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      float x = aqk[a][b], y = akk[a][b];
#pragma unroll
      for (int m = 1; m <= 4; m <<= 1) {
        x += __shfl_xor_sync(0xffffffffu, x, m);
        y += __shfl_xor_sync(0xffffffffu, y, m);
      }
      aqk[a][b] = x, akk[a][b] = y;
    }

  // ---- the stack: row r holds k_j 2^{G_R - G_j} for (R, j) = (16, r), (32, r - 16), (48, r - 48) ------------------
  for (int i = tid; i < 96 * 16; i += kIntraThreads) {
    const int r = i >> 4, cc = i & 15;
    const int ref = r < 16 ? 16 : (r < 48 ? 32 : 48);
    const int j = r < 16 ? r : (r < 48 ? r - 16 : r - 48);
    float x[8];
    unpack8(*reinterpret_cast<const uint4*>(qk_tile + (cc >> 3) * 16384 + sw128_offset(64 + j, cc & 7)), x);
    const float* gr = sg + ref * kGRow + cc * 8;
    const float* gj = sg + j * kGRow + cc * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] *= fast_exp2(gr[e] - gj[e]);
    *reinterpret_cast<uint4*>(stack + (cc >> 3) * 12288 + sw128_offset(r, cc & 7)) = pack8(x);
  }
  __syncthreads();  // the stack and the diagonal sums have read the raw rows: they become q~ and k~' in place
  for (int i = tid; i < 64 * 16; i += kIntraThreads) {
    const int r = i >> 4, cc = i & 15;
    const float* gi = sg + r * kGRow + cc * 8;
    const float* gr = sg + (r & ~15) * kGRow + cc * 8;
    float f[8], x[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = fast_exp2(gi[e] - gr[e]);
    uint8_t* qa = qk_tile + (cc >> 3) * 16384 + sw128_offset(r, cc & 7);
    uint8_t* ka = qk_tile + (cc >> 3) * 16384 + sw128_offset(64 + r, cc & 7);
    unpack8(*reinterpret_cast<const uint4*>(qa), x);
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] *= f[e];
    *reinterpret_cast<uint4*>(qa) = pack8(x);
    unpack8(*reinterpret_cast<const uint4*>(ka), x);
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] *= f[e];
    *reinterpret_cast<uint4*>(ka) = pack8(x);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  // ---- the blocks below the block diagonal: [q~ ; k~'] stack^T, M = 128, N = 96, K = 128 --------------------------
  if (tid == 0) {
    const Operand op_a{sbase + KdaIntraSmem::kQK, 16384}, op_b{sbase + KdaIntraSmem::kStack, 12288};
    umma_gemm<128, 96>(tmem, op_a, false, op_b, false, 128, false);
    umma_commit(&bar);
  }
  ok = __all_sync(0xffffffffu, mbar_wait(&bar, 0)) && ok;
  tc_fence_after();
  // every thread is past the operands: S_qk and S_kk take the gates' space, rows i of warps 0..1 / 2..3
  if (warp < 4) {
    const int i = (warp & 1) * 32 + lane;
    float* dst = (warp < 2 ? s_qk : s_kk) + i * 65;
    const int blk = i >> 4;
    // row block 1 reads columns 0..15 of the product, block 2 columns 16..47, block 3 columns 48..95 (j = 0 .. 16 blk - 1)
#pragma unroll
    for (int p = 0; p < 3; ++p) {
      float s[32];
      tmem_ld32(tmem_addr(tmem, warp, p * 32), s);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const int col = p * 32 + e;
        const int owner = col < 16 ? 1 : (col < 48 ? 2 : 3);
        const int j = col < 16 ? col : (col < 48 ? col - 16 : col - 48);
        if (blk == owner) dst[j] = s[e];
      }
    }
  }
  if ((tid & 7) == 0) {  // the diagonal blocks' sums (entries above the diagonal are zero)
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        s_qk[(i0 + a) * 65 + j0 + b] = aqk[a][b];
        s_kk[(i0 + a) * 65 + j0 + b] = akk[a][b];
      }
  }
  tc_fence_before();
  __syncthreads();

  // Aqk rows -> global; L rows -> shared (a thread per run of 8 columns)
  for (int t = tid; t < 64 * 8; t += kIntraThreads) {
    const int i = t >> 3, jj = t & 7;
    const float bi = s_beta[i];
    float x[8], l8[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int j = jj * 8 + e;
      x[e] = j <= i ? scale * s_qk[i * 65 + j] : 0.f;
      l8[e] = j < i ? bi * s_kk[i * 65 + j] : 0.f;
    }
    // four consecutive columns are contiguous in the operand layout
    *reinterpret_cast<float4*>(s_l + wy_l_index(i, jj * 8)) = make_float4(l8[0], l8[1], l8[2], l8[3]);
    *reinterpret_cast<float4*>(s_l + wy_l_index(i, jj * 8 + 4)) = make_float4(l8[4], l8[5], l8[6], l8[7]);
    reinterpret_cast<uint4*>(aqk_out + tile * 4096 + i * 64)[jj] = pack8(x);
  }
  __syncthreads();

  // kb = bf16(beta kg), vb = bf16(beta v): by the warps that do not solve, while the first two do
  for (int i = tid - 64; i >= 0 && i < 64 * 16; i += kIntraThreads - 64) {
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
  // A = (I + L)^-1 by blocks of 32, as in gdn_wy_kernel: with I + L = [[M11, 0], [L21, M22]],
  //     A = [[X11, 0], [X21, X22]],  X11 = M11^-1, X22 = M22^-1 (fp32 forward substitution, 64 threads, 496 FMAs each)
  //     X21 = -X22 (L21 X11)  (two tensor-core products with TF32 operands; A is rounded to bf16 afterwards)
  // The products' operands take the quarters of L that are dead by then: L11 -> B1 = X11^T, the never-used upper
  // right -> X22 (rows 32..63 of A2, whose rows 0..31 are whatever lies in L21: a result row depends on its own
  // operand row only, and rows 0..31 of the results are not read), L22 -> B2 = T^T.
  float* s_b1 = s_l;
  float* s_a2 = s_l + 1024;
  float* s_b2 = s_l + 3072;
  uint8_t* a_tile = sm + KdaIntraSmem::kA;
  if (tid < 64) {
    const int b = tid >> 5, c = tid & 31, base = 32 * b;
    float x[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float acc0 = (i == c) ? 1.f : 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
#pragma unroll
      for (int j = 0; j < i; j += 4) {
        const float4 l = *reinterpret_cast<const float4*>(s_l + wy_l_index(base + i, base + j));
        acc0 = fmaf(-l.x, x[j], acc0);
        if (j + 1 < i) acc1 = fmaf(-l.y, x[j + 1], acc1);
        if (j + 2 < i) acc2 = fmaf(-l.z, x[j + 2], acc2);
        if (j + 3 < i) acc3 = fmaf(-l.w, x[j + 3], acc3);
      }
      x[i] = (acc0 + acc1) + (acc2 + acc3);
    }
    asm volatile("bar.sync 1, 64;" ::: "memory");  // every solving thread has read L11 / L22: their space is rewritten
    const int col = base + c;
#pragma unroll
    for (int i = 0; i < 32; ++i)
      *reinterpret_cast<__nv_bfloat16*>(a_tile + sw128_offset(base + i, col >> 3) + (col & 7) * 2) =
          __float2bfloat16_rn(x[i]);
    if (b == 0) {  // row c of B1 = column c of X11
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        *reinterpret_cast<float4*>(s_b1 + f32_block_index(c, i)) = make_float4(x[i], x[i + 1], x[i + 2], x[i + 3]);
    } else {  // column c of X22 in the rows 32..63 of A2
#pragma unroll
      for (int i = 0; i < 32; ++i) s_a2[f32_block_index(32 + i, c)] = x[i];
    }
  } else {
    // the upper right block of A is zero
    for (int i = tid - 64; i < 32 * 4; i += kIntraThreads - 64)
      set_tile_chunk(a_tile, 8192, i >> 2, 4 + (i & 3), make_uint4(0u, 0u, 0u, 0u));
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  {
    const uint32_t l_addr = sbase + KdaIntraSmem::kL;
    const uint32_t b1_addr = l_addr, a2_addr = l_addr + 4096, b2_addr = l_addr + 12288;
    constexpr uint32_t kColT = 128, kColX = 160;  // free until the w / u products
    if (tid == 0) {  // T' = L[:, 0:32] X11 (rows 32..63 are T = L21 X11)
      const uint32_t idesc = umma_idesc_tf32(64, 32);
      for (uint32_t k0 = 0; k0 < 32; k0 += 8)
        umma_tf32(tmem + kColT, umma_desc_sw128(l_addr + k0 * 4, 16u, kSbo), umma_desc_sw128(b1_addr + k0 * 4, 16u, kSbo),
                  idesc, k0 > 0 ? 1u : 0u);
      umma_commit(&bar);
    }
    if (warp < 4) {
      ok = __all_sync(0xffffffffu, mbar_wait(&bar, 1)) && ok;
      tc_fence_after();
      float tt[32];
      tmem_ld32(tmem_addr(tmem, warp, kColT), tt);
      tmem_ld_wait();
      if (warp >= 2 && lane < 16) {  // row i = 16 warp + lane of T' -> column i - 32 of B2 = T^T
        const int kk = 16 * warp + lane - 32;
#pragma unroll
        for (int n = 0; n < 32; ++n) s_b2[f32_block_index(n, kk)] = tt[n];
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0) {  // X' = -A2 T (rows 32..63 are X21)
      const uint32_t idesc = umma_idesc_tf32(64, 32, /*neg_a=*/true);
      for (uint32_t k0 = 0; k0 < 32; k0 += 8)
        umma_tf32(tmem + kColX, umma_desc_sw128(a2_addr + k0 * 4, 16u, kSbo), umma_desc_sw128(b2_addr + k0 * 4, 16u, kSbo),
                  idesc, k0 > 0 ? 1u : 0u);
      umma_commit(&bar);
    }
    if (warp < 4) {
      ok = __all_sync(0xffffffffu, mbar_wait(&bar, 0)) && ok;
      tc_fence_after();
      float xv[32];
      tmem_ld32(tmem_addr(tmem, warp, kColX), xv);
      tmem_ld_wait();
      if (warp >= 2 && lane < 16) {
        const int i = 16 * warp + lane;
#pragma unroll
        for (int j = 0; j < 4; ++j) set_tile_chunk(a_tile, 8192, i, j, pack8(xv + 8 * j));
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }

  if (tid == 0) {
    const Operand a{sbase + KdaIntraSmem::kA, 8192};
    const Operand kb{sbase + KdaIntraSmem::kKB, 8192};
    const Operand vb{sbase + KdaIntraSmem::kVB, 8192};
    // alternating: the instructions of one product wait for one another
    umma_gemm_pair<64, 128>(tmem, a, false, kb, true, 64, false, false, tmem + 128, a, false, vb, true, 64, false, false);
    umma_commit(&bar);
  }
  if (tid < 128) store_tile<64, 64, 128>(sm + KdaIntraSmem::kA, 8192, a_out + tile * 4096, 64, 64, tid);
  if (warp < 4) {
    ok = __all_sync(0xffffffffu, mbar_wait(&bar, 1)) && ok;
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
// tail, tensor-core part: persistent, one CTA per SM walks the (chunk, head) items
// ---------------------------------------------------------------------------------------------------------------
// Everything the decayed part reads per key channel (dqg, dkr, dkg, hdh) is computed TRANSPOSED, channel = accumulator
// row = tensor-memory lane = thread, so that a warp writes 32 consecutive channels of one token: whole 128-byte
// lines.  The factors beta and scale are applied to the fp32 results instead of to bf16 operands:
//   phase 1  dqg^T = h do^T        dkr^T = dh v_new^T      dw^T = -h dv_new^T      (128 x 64, K = 128)
//            dAqk  = do v_new^T    (64 x 64)               dvb^T = dv_new^T A      (128 x 64, K = 64)
//   phase 2  dkgb^T = dw^T A       (128 x 64, K = 64)      dAu = dw kg^T + dv_new v^T   (64 x 64; dA = dAu diag(beta))
//   phase 3  Xu = A^T dAu          -> dbeta = diag(Xu) (= sum_d dkgb kg + sum_v dvb v), X = bf16(Xu diag(beta))
//   phase 4  Y = X A^T             -> M2 = bf16(-tril(Y, -1))
// The next item's tiles arrive by TMA while the current one computes: the state tiles, do and v_new are free as soon
// as phase 1's products are done, dv_new and A are double-buffered, kg and v follow when phase 2's products are done.
struct KdaTailSmem {
  static constexpr uint32_t kH = 0;                    // [128][128] h
  static constexpr uint32_t kDH = 32768;               // [128][128] dh
  static constexpr uint32_t kDO = 65536;               // [64][128] do
  static constexpr uint32_t kVN = kDO + 16384;         // [64][128] v_new
  static constexpr uint32_t kDVN = kVN + 16384;        // 2 x [64][128] dv_new
  static constexpr uint32_t kKG = kDVN + 2 * 16384;    // [64][128] kg
  static constexpr uint32_t kV = kKG + 16384;          // [64][128] v
  static constexpr uint32_t kA = kV + 16384;           // 2 x [64][64] A
  static constexpr uint32_t kDW = kA + 2 * 8192;       // [128 channels][64 tokens] dw^T
  static constexpr uint32_t kDA = kDW + 16384;         // [64][64] dAu
  static constexpr uint32_t kX = kDA + 8192;           // [64][64] X
  static constexpr uint32_t kScal = kX + 8192;         // beta[2][64]
  static constexpr uint32_t kBytes = kScal + 512;
};

struct KdaTailMaps {
  CUtensorMap d_o, v_new, dv_new, kg, v;  // rows [tokens, H * 128], box 64 x 64
  CUtensorMap h, dh;                      // tiles [num_tiles * 128, 128], box 64 x 128
  CUtensorMap a;                          // tiles [num_tiles * 64, 64], box 64 x 64
};

constexpr int kKdaTailThreads = 256;

__global__ void __launch_bounds__(kKdaTailThreads) kda_tail_mma_kernel(
    const __grid_constant__ KdaTailMaps maps, const float* __restrict__ beta, float* __restrict__ m1,
    float* __restrict__ m2, float* __restrict__ dqg, float* __restrict__ dkr, float* __restrict__ dkg,
    float* __restrict__ hdh, __nv_bfloat16* __restrict__ dv, float* __restrict__ dbeta_part,
    const int32_t* __restrict__ chunk_start, const int32_t* __restrict__ chunk_len, int num_chunks, int num_heads,
    float scale, int32_t* __restrict__ status) {
  extern __shared__ uint8_t raw[];
  __shared__ uint64_t bar;        // tensor-core commits
  __shared__ uint64_t bar_one;    // h, dh, do, v_new, dv_new, A of an item
  __shared__ uint64_t bar_two;    // kg, v of an item
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool issuer = tid == 0, loader = tid == 32;
  const int quad = warp & 3, wg = warp >> 2;
  // 128-row accumulators: this thread's row (a key or value channel) and its 32 of the 64 columns (tokens)
  const int chan = quad * 32 + lane, tok0 = wg * 32;
  // 64-row accumulators (lanes 0..15 of a quadrant), read in the 16-lane fragment shape: the rows fr, fr + 8 at
  // the columns fc + 8 n + {0, 1}, n = 0..3
  const int fr = quad * 16 + (lane >> 2), fq = lane & 3, fc = wg * 32 + fq * 2;
  float* s_beta = reinterpret_cast<float*>(sm + KdaTailSmem::kScal);  // [2][64]
  Abort abort{&abort_flag};
  const int64_t stride = int64_t(num_heads) * kDim;
  const int num_items = num_chunks * num_heads;
  const uint32_t sbase = smem_u32(sm);

  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_init(&bar_one, 1);
    mbar_init(&bar_two, 1);
    fence_mbar_init();
    abort_flag = 0;
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  // an item is live when it exists and its chunk is not a pad chunk of a device-built table (pads come last)
  auto item_live = [&](int it) { return it < num_items && chunk_len[it / num_heads] > 0; };
  auto load_one = [&](int it, int buf) {  // loader thread
    const int c = it / num_heads, hd = it % num_heads, start = chunk_start[c];
    mbar_arrive_expect(&bar_one, 2 * 32768 + 3 * 16384 + 8192);
    tma_load_tile128(sbase + KdaTailSmem::kH, 16384, &maps.h, 0, it * 128, &bar_one);
    tma_load_tile128(sbase + KdaTailSmem::kDH, 16384, &maps.dh, 0, it * 128, &bar_one);
    tma_load_tile128(sbase + KdaTailSmem::kDO, 8192, &maps.d_o, hd * kDim, start, &bar_one);
    tma_load_tile128(sbase + KdaTailSmem::kVN, 8192, &maps.v_new, hd * kDim, start, &bar_one);
    tma_load_tile128(sbase + KdaTailSmem::kDVN + buf * 16384, 8192, &maps.dv_new, hd * kDim, start, &bar_one);
    tma_load_box(sbase + KdaTailSmem::kA + buf * 8192, &maps.a, 0, it * 64, &bar_one);
  };
  auto load_two = [&](int it) {
    const int c = it / num_heads, hd = it % num_heads, start = chunk_start[c];
    mbar_arrive_expect(&bar_two, 2 * 16384);
    tma_load_tile128(sbase + KdaTailSmem::kKG, 8192, &maps.kg, hd * kDim, start, &bar_two);
    tma_load_tile128(sbase + KdaTailSmem::kV, 8192, &maps.v, hd * kDim, start, &bar_two);
  };
  auto load_beta = [&](int it, int buf) {  // every thread calls; the first 64 copy
    if (tid < 64) {
      const int c = it / num_heads, hd = it % num_heads, len = chunk_len[c];
      s_beta[buf * 64 + tid] = tid < len ? beta[int64_t(chunk_start[c] + tid) * num_heads + hd] : 0.f;
    }
  };

  int item = blockIdx.x;
  bool live = item_live(item);
  if (live) {
    if (loader) {
      load_one(item, 0);
      load_two(item);
    }
    load_beta(item, 0);
  }
  const Operand op_h{sbase + KdaTailSmem::kH, 16384}, op_dh{sbase + KdaTailSmem::kDH, 16384};
  const Operand op_do{sbase + KdaTailSmem::kDO, 8192}, op_vn{sbase + KdaTailSmem::kVN, 8192};
  const Operand op_kg{sbase + KdaTailSmem::kKG, 8192}, op_v{sbase + KdaTailSmem::kV, 8192};
  const Operand op_dw{sbase + KdaTailSmem::kDW, 16384}, op_da{sbase + KdaTailSmem::kDA, 8192};
  const Operand op_x{sbase + KdaTailSmem::kX, 8192};
  // tensor-memory columns
  constexpr uint32_t cDqg = 0, cDkr = 64, cDw = 128, cDvb = 192, cAqk = 256, cDkg = 320, cDa = 384, cX = 448, cDa2 = 256, cY = 256;

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

  int parity = 0;
  for (; live; item += gridDim.x, parity ^= 1) {
    const int c = item / num_heads, hd = item % num_heads;
    const int start = chunk_start[c], len = chunk_len[c];
    const int next = item + gridDim.x;
    const bool has_next = item_live(next);
    const int64_t rows = int64_t(start) * stride + hd * kDim;
    const int64_t tile = item;
    const float* beta_s = s_beta + parity * 64;
    uint8_t* dvn_tile = sm + KdaTailSmem::kDVN + parity * 16384;
    const Operand op_dvn{sbase + KdaTailSmem::kDVN + parity * 16384, 8192};
    const Operand op_a{sbase + KdaTailSmem::kA + parity * 8192, 8192};

    if (!mbar_wait(&bar_one, parity)) abort.raise();
    if (len < kChunk) {  // a ragged chunk's boxes reach into the next sequence: clear those rows
      clear_tile_rows<kKdaTailThreads>(sm + KdaTailSmem::kDO, len, tid);
      clear_tile_rows<kKdaTailThreads>(sm + KdaTailSmem::kVN, len, tid);
      clear_tile_rows<kKdaTailThreads>(dvn_tile, len, tid);
    }
    stage_sync();
    if (abort.raised()) break;
    if (has_next) load_beta(next, parity ^ 1);

    // ---- phase 1 -------------------------------------------------------------------------------------------------
    if (issuer) {
      umma_gemm_pair<128, 64>(tmem + cDqg, op_h, false, op_do, false, 128, false, false, tmem + cDkr, op_dh, false,
                              op_vn, false, 128, false, false);
      umma_gemm_pair<128, 64, 64>(tmem + cDw, op_h, false, op_dvn, false, 128, false, /*neg=*/true, tmem + cDvb, op_dvn,
                                  true, op_a, true, 64, false, false);
      umma_gemm<64, 64>(tmem + cAqk, op_do, false, op_vn, false, 128, false);
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
    __syncthreads();  // the products and every thread's reads of h / dh are done: the next item's tiles may land
    if (has_next && loader) load_one(next, parity ^ 1);
    {
      // dqg, dkr: 32 tokens of this thread's channel; a warp writes 32 consecutive channels of a token
      float a[32], b[32];
      tmem_ld32(tmem_addr(tmem, warp, cDqg + tok0), a);
      tmem_ld32(tmem_addr(tmem, warp, cDkr + tok0), b);
      tmem_ld_wait();
      float* dqg_col = dqg + rows + chan;
      float* dkr_col = dkr + rows + chan;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (tok0 + j < len) {
          dqg_col[int64_t(tok0 + j) * stride] = scale * a[j];
          dkr_col[int64_t(tok0 + j) * stride] = b[j];
        }
      }
      // dw^T -> its tile (row = channel); dvb^T -> dv = bf16(beta dvb)
      tmem_ld32(tmem_addr(tmem, warp, cDw + tok0), a);
      tmem_ld32(tmem_addr(tmem, warp, cDvb + tok0), b);
      tmem_ld_wait();
#pragma unroll
      for (int jj = 0; jj < 4; ++jj)
        *reinterpret_cast<uint4*>(sm + KdaTailSmem::kDW + sw128_offset(chan, wg * 4 + jj)) = pack8(a + jj * 8);
      __nv_bfloat16* dv_col = dv + rows + chan;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (tok0 + j < len) dv_col[int64_t(tok0 + j) * stride] = __float2bfloat16_rn(beta_s[tok0 + j] * b[j]);
      // M1 = scale tril(dAqk)
      float s[16];
      tmem_ld_frag16(tmem_addr(tmem, warp, cAqk + wg * 32), s);
      tmem_ld_frag16(tmem_addr(tmem, warp, cAqk + wg * 32 + 16), s + 8);
      tmem_ld_wait();
      float* m1_tile = m1 + tile * 4096;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int col = fc + 8 * n;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int r = fr + 8 * hh;
          const float x0 = col <= r ? scale * s[4 * n + 2 * hh] : 0.f, x1 = col + 1 <= r ? scale * s[4 * n + 2 * hh + 1] : 0.f;
          *reinterpret_cast<float2*>(m1_tile + r * 64 + col) = make_float2(x0, x1);
        }
      }
    }
    if (!mbar_wait(&bar_two, parity)) abort.raise();
    if (len < kChunk) {
      clear_tile_rows<kKdaTailThreads>(sm + KdaTailSmem::kKG, len, tid);
      clear_tile_rows<kKdaTailThreads>(sm + KdaTailSmem::kV, len, tid);
    }
    stage_sync();

    // ---- phase 2 -------------------------------------------------------------------------------------------------
    if (issuer) {
      // dAu as two chains into two accumulators (the epilogue adds them): one chain's instructions wait for one another
      umma_gemm_pair<64, 64>(tmem + cDa, op_dw, true, op_kg, false, 128, false, false, tmem + cDa2, op_dvn, false, op_v,
                             false, 128, false, false);
      umma_gemm<128, 64>(tmem + cDkg, op_dw, false, op_a, true, 64, false);
      umma_commit(&bar);
    }
    mma_wait();
    {
      float a[32];
      tmem_ld32(tmem_addr(tmem, warp, cDkg + tok0), a);
      float s[16], s2[16];
      tmem_ld_frag16(tmem_addr(tmem, warp, cDa + wg * 32), s);
      tmem_ld_frag16(tmem_addr(tmem, warp, cDa + wg * 32 + 16), s + 8);
      tmem_ld_frag16(tmem_addr(tmem, warp, cDa2 + wg * 32), s2);
      tmem_ld_frag16(tmem_addr(tmem, warp, cDa2 + wg * 32 + 16), s2 + 8);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) s[j] += s2[j];
      float* dkg_col = dkg + rows + chan;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (tok0 + j < len) dkg_col[int64_t(tok0 + j) * stride] = beta_s[tok0 + j] * a[j];
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int col = fc + 8 * n;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int r = fr + 8 * hh;
          *reinterpret_cast<uint32_t*>(sm + KdaTailSmem::kDA + sw128_offset(r, col >> 3) + (col & 7) * 2) =
              pack_bf16(s[4 * n + 2 * hh], s[4 * n + 2 * hh + 1]);
        }
      }
    }
    stage_sync();
    if (has_next && loader) load_two(next);  // kg and v are done with

    // ---- phase 3: Xu = A^T dAu -------------------------------------------------------------------------------------
    if (issuer) {
      umma_gemm<64, 64>(tmem + cX, op_a, true, op_da, true, 64, false);
      umma_commit(&bar);
    }
    mma_wait();
    {
      float s[16];
      tmem_ld_frag16(tmem_addr(tmem, warp, cX + wg * 32), s);
      tmem_ld_frag16(tmem_addr(tmem, warp, cX + wg * 32 + 16), s + 8);
      tmem_ld_wait();
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int col = fc + 8 * n;
        const float b0 = beta_s[col], b1 = beta_s[col + 1];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int r = fr + 8 * hh;
          const float x0 = s[4 * n + 2 * hh], x1 = s[4 * n + 2 * hh + 1];
          if (col == r && r < len) dbeta_part[int64_t(start + r) * num_heads + hd] = x0;
          if (col + 1 == r && r < len) dbeta_part[int64_t(start + r) * num_heads + hd] = x1;
          *reinterpret_cast<uint32_t*>(sm + KdaTailSmem::kX + sw128_offset(r, col >> 3) + (col & 7) * 2) =
              pack_bf16(b0 * x0, b1 * x1);
        }
      }
    }
    stage_sync();

    // ---- phase 4: Y = X A^T ; M2 = bf16(-tril(Y, -1)) --------------------------------------------------------------
    if (issuer) {
      umma_gemm<64, 64>(tmem + cY, op_x, false, op_a, false, 64, false);
      umma_commit(&bar);
    }
    mma_wait();
    {
      float s[16];
      tmem_ld_frag16(tmem_addr(tmem, warp, cY + wg * 32), s);
      tmem_ld_frag16(tmem_addr(tmem, warp, cY + wg * 32 + 16), s + 8);
      tmem_ld_wait();
      float* m2_tile = m2 + tile * 4096;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int col = fc + 8 * n;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int r = fr + 8 * hh;
          const float x0 = col < r ? round_bf16(-s[4 * n + 2 * hh]) : 0.f;
          const float x1 = col + 1 < r ? round_bf16(-s[4 * n + 2 * hh + 1]) : 0.f;
          *reinterpret_cast<float2*>(m2_tile + r * 64 + col) = make_float2(x0, x1);
        }
      }
    }
    live = has_next;
    // the next item's phase 1 overwrites the accumulators this epilogue has just read, and its beta row replaces the
    // one two items back: every thread must be past both
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  if (abort.raised()) {  // copies of the next item may still be in flight: give them time to land before the CTA ends
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 100000ull) {
    }
  }
  if (abort.raised() && tid == 0) atomicExch(status, kDevWaitTimeout | (7 << 8));
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------------------------------------
// tail, decayed part: one block per (chunk, head); thread (d, quarter) owns key channel d
// ---------------------------------------------------------------------------------------------------------------
// With E_ij = 2^{G_i - G_j} per channel (j <= i), M1 = scale tril(do v_new^T) and M2 = bf16(-tril(A^T dA A^T, -1)):
//   row pass     RQ_i = sum_{j<=i} M1_ij k_j E_ij,  RK_i = sum_{j<i} M2_ij k_j E_ij     -> dq, the row part of dk, dg
//   column pass  CC_j = sum_{i>=j} (M1_ij q_i + beta_i M2_ij k_i) E_ij                  -> the column part of dk, dg
// Both are split by blocks of 16 rows, like the forward's pairwise matrices.  With R the first row of i's block and
// j in an earlier block, E_ij = 2^{G_i - G_R} 2^{G_R - G_j} (both exponents <= 0), so everything below the block
// diagonal is tensor-core work on bounded bf16 operands (q~, k~', the stack: see kda_intra_kernel), computed
// TRANSPOSED so that a thread finds its channel's sums in its own tensor-memory lane:
//   DR^T [128 d x 128] = stack^T AR^T     AR row i (M1) / 64 + i (M2): the row's entries against its own block's
//                                         part of the stack, zero elsewhere -> RQ_i = 2^{G_i - G_R} DR^T[d][i], RK alike
//   PI^T [128 d x 64 j] = q~_I^T M1[I, :] + k~'_I^T (beta M2)[I, :]   (I = 1, 2, 3; entries of earlier blocks only)
//                                         -> CC_j = sum_{I > block(j)} 2^{G_{16 I} - G_j} PI^T[d][j]
// The four 16 x 16 blocks on the diagonal are summed on CUDA cores, without an exponential per pair: E runs along a
// row or a column as a product of the per-token factors R_i = 2^{G_i - G_{i-1}} <= 1; these sums run while the
// tensor core works.  512 threads: thread (d, quarter) owns channel d for the groups of four rows AND of four columns
// 4 quarter + 16 n: the row part and the column part of a (token, channel) pair meet in one thread.
struct KdaPairSmem {
  static constexpr uint32_t kG = 0;                    // fp32 [64][128] G (log2); after the passes: per-row dg
  static constexpr uint32_t kR = 32768;                // fp32 [64][128] R; after the passes: the chunk-end terms
  static constexpr uint32_t kRaw = 2 * 32768;          // bf16 [64][128] q, then k (raw rows, swizzled)
  static constexpr uint32_t kCvt = 3 * 32768;          // bf16 [64][128] q~, then k~'
  static constexpr uint32_t kStack = 4 * 32768;        // bf16 [96][128], 2 blocks of 12 KiB
  static constexpr uint32_t kAR = kStack + 24576;      // bf16 [128][96] K-major, 2 blocks of 16 KiB; later CC fp32 [64][128]
  static constexpr uint32_t kX1 = kAR + 32768;         // bf16 [64][64] M1, entries of earlier blocks
  static constexpr uint32_t kX2 = kX1 + 8192;          // bf16 [64][64] beta M2, entries of earlier blocks
  static constexpr uint32_t kMd = kX2 + 8192;          // fp32 [2][4][16][20]: the diagonal blocks of M1, M2
  static constexpr uint32_t kBeta = kMd + 2 * 4 * 16 * 20 * 4;   // beta[64], db[64][4]
  static constexpr uint32_t kBytes = kBeta + 256 + 1024;
};

struct KdaPairMaps {
  CUtensorMap q, k;  // rows [tokens, H * 128], box 64 x 64
};

__global__ void __launch_bounds__(512) kda_tail_pair_kernel(
    const __grid_constant__ KdaPairMaps maps, const float* __restrict__ g2,
    const float* __restrict__ beta, const float* __restrict__ m1, const float* __restrict__ m2,
    const float* __restrict__ dqg, const float* __restrict__ dkr, const float* __restrict__ dkg,
    const float* __restrict__ hdh, const float* __restrict__ dbeta_part, float* __restrict__ dq, float* __restrict__ dk,
    float* __restrict__ dg, float* __restrict__ dbeta, const int32_t* __restrict__ chunk_start,
    const int32_t* __restrict__ chunk_len, int num_heads, int32_t* __restrict__ status) {
  extern __shared__ uint8_t raw[];
  __shared__ uint64_t bar, bar_load;
  __shared__ uint32_t tmem_slot;
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, d = tid & 127, quarter = tid >> 7, warp4 = (tid >> 5) & 3;
  const int warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y;
  const int start = chunk_start[c], len = chunk_len[c];
  if (len <= 0) return;
  float* sG = reinterpret_cast<float*>(sm + KdaPairSmem::kG);
  float* sR = reinterpret_cast<float*>(sm + KdaPairSmem::kR);
  uint8_t* q_raw = sm + KdaPairSmem::kRaw;
  uint8_t* k_raw = q_raw + 16384;
  uint8_t* q_cvt = sm + KdaPairSmem::kCvt;
  uint8_t* k_cvt = q_cvt + 16384;
  uint8_t* stack = sm + KdaPairSmem::kStack;
  uint8_t* ar = sm + KdaPairSmem::kAR;
  uint8_t* x1 = sm + KdaPairSmem::kX1;
  uint8_t* x2 = sm + KdaPairSmem::kX2;
  float* sM1d = reinterpret_cast<float*>(sm + KdaPairSmem::kMd);   // [4][16][20]
  float* sM2d = sM1d + 4 * 16 * 20;
  float* s_beta = reinterpret_cast<float*>(sm + KdaPairSmem::kBeta);
  float* s_db = s_beta + 64;
  const int64_t stride = int64_t(num_heads) * kDim;
  const int64_t tile = int64_t(c) * num_heads + h;
  const int64_t col = int64_t(start) * stride + h * kDim + d;
  const uint32_t sbase = smem_u32(sm);
  // element [i][d] of a swizzled bf16 tile for this thread's channel: the channel's part of the address is fixed
  const uint32_t d_base = uint32_t(d >> 6) * 8192u + uint32_t(d & 7) * 2u, d_chunk = uint32_t(d & 63) >> 3;
  auto rq_at = [&](const uint8_t* t, int i) {
    return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(
        t + d_base + uint32_t(i) * 128u + ((d_chunk ^ (uint32_t(i) & 7u)) << 4)));
  };

  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_init(&bar_load, 1);
    fence_mbar_init();
    mbar_arrive_expect(&bar_load, 2 * 16384);
    tma_load_tile128(sbase + KdaPairSmem::kRaw, 8192, &maps.q, h * kDim, start, &bar_load);
    tma_load_tile128(sbase + KdaPairSmem::kRaw + 16384, 8192, &maps.k, h * kDim, start, &bar_load);
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 512);
  if (tid < 64) s_beta[tid] = tid < len ? beta[int64_t(start + tid) * num_heads + h] : 0.f;
  // Every global read of the prologue is issued before the first of them is used: the gates, and the entries of M1
  // and M2 for the products' operands -- AR (rows against their own block's part of the stack), X1 / X2 (the entries
  // of earlier blocks) -- and for the fp32 diagonal blocks.
  float gate[16];
#pragma unroll
  for (int n = 0; n < 16; ++n) {  // rows past the chunk's length keep the last gate (R = 1 there)
    const int i = (tid >> 7) + 4 * n;
    gate[n] = g2[col + int64_t(i < len ? i : len - 1) * stride];
  }
  float4 ar_lo[3], ar_hi[3];
#pragma unroll
  for (int it = 0; it < 3; ++it) {
    const int t = tid + 512 * it;
    const int n = t / 12, cc = t % 12;            // row of AR, 16-byte chunk of its 96 columns
    const int i = n & 63, colb = cc * 8;
    const int owner = colb < 16 ? 1 : (colb < 48 ? 2 : 3);
    const int j = colb < 16 ? colb : (colb < 48 ? colb - 16 : colb - 48);
    ar_lo[it] = ar_hi[it] = make_float4(0.f, 0.f, 0.f, 0.f);
    if ((i >> 4) == owner) {
      const float* src = (n < 64 ? m1 : m2) + tile * 4096 + i * 64 + j;
      ar_lo[it] = __ldg(reinterpret_cast<const float4*>(src));
      ar_hi[it] = __ldg(reinterpret_cast<const float4*>(src) + 1);
    }
  }
  const int xi = tid >> 3, xc = tid & 7;
  const float* s1 = m1 + tile * 4096 + xi * 64 + xc * 8;
  const float* s2 = m2 + tile * 4096 + xi * 64 + xc * 8;
  const float4 a0 = __ldg(reinterpret_cast<const float4*>(s1)), a1 = __ldg(reinterpret_cast<const float4*>(s1) + 1);
  const float4 b0 = __ldg(reinterpret_cast<const float4*>(s2)), b1 = __ldg(reinterpret_cast<const float4*>(s2) + 1);
#pragma unroll
  for (int n = 0; n < 16; ++n) sG[((tid >> 7) + 4 * n) * 128 + d] = gate[n];
#pragma unroll
  for (int it = 0; it < 3; ++it) {
    const int t = tid + 512 * it;
    const int n = t / 12, cc = t % 12;
    const float x[8] = {ar_lo[it].x, ar_lo[it].y, ar_lo[it].z, ar_lo[it].w, ar_hi[it].x, ar_hi[it].y, ar_hi[it].z, ar_hi[it].w};
    *reinterpret_cast<uint4*>(ar + (cc >> 3) * 16384 + sw128_offset(n, cc & 7)) = pack8(x);
  }
  {
    const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    const bool earlier = (xc >> 1) < (xi >> 4);     // the 8 columns lie in a block before the row's
    float xa[8], xb[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) xa[e] = earlier ? av[e] : 0.f, xb[e] = earlier ? bv[e] : 0.f;
    *reinterpret_cast<uint4*>(x1 + sw128_offset(xi, xc)) = pack8(xa);
    *reinterpret_cast<uint4*>(x2 + sw128_offset(xi, xc)) = pack8(xb);
    if ((xc >> 1) == (xi >> 4)) {                   // ... or in the row's own block: the fp32 diagonal blocks
      const int at = ((xi >> 4) * 16 + (xi & 15)) * 20 + (xc & 1) * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) sM1d[at + e] = av[e], sM2d[at + e] = bv[e];
    }
  }
  __syncthreads();  // beta, the gates and the barriers' initialisation are in place
#pragma unroll
  for (int n = 0; n < 16; ++n) {
    const int i = (tid >> 7) + 4 * n;
    sR[i * 128 + d] = (i < len && i > 0) ? fast_exp2(sG[i * 128 + d] - sG[(i - 1) * 128 + d]) : 1.f;
  }
  bool ok = __all_sync(0xffffffffu, mbar_wait(&bar_load, 0));
  if (len < kChunk) {  // a ragged chunk's boxes reach into the next sequence: clear those rows
    clear_tile_rows<512>(q_raw, len, tid);
    clear_tile_rows<512>(k_raw, len, tid);
  }
  __syncthreads();
  // the stack (row r holds k_j 2^{G_R - G_j} for (R, j) = (16, r), (32, r - 16), (48, r - 48)) and q~, k~'
  for (int t = tid; t < 96 * 16; t += 512) {
    const int r = t >> 4, cc = t & 15;
    const int ref = r < 16 ? 16 : (r < 48 ? 32 : 48);
    const int j = r < 16 ? r : (r < 48 ? r - 16 : r - 48);
    float x[8];
    unpack8(tile_chunk(k_raw, 8192, j, cc), x);
    const float* gr = sG + ref * 128 + cc * 8;
    const float* gj = sG + j * 128 + cc * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] *= fast_exp2(gr[e] - gj[e]);
    *reinterpret_cast<uint4*>(stack + (cc >> 3) * 12288 + sw128_offset(r, cc & 7)) = pack8(x);
  }
  for (int t = tid; t < 64 * 16; t += 512) {
    const int r = t >> 4, cc = t & 15;
    const float* gi = sG + r * 128 + cc * 8;
    const float* gr = sG + (r & ~15) * 128 + cc * 8;
    float f[8], x[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = fast_exp2(gi[e] - gr[e]);
    unpack8(tile_chunk(q_raw, 8192, r, cc), x);
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] *= f[e];
    set_tile_chunk(q_cvt, 8192, r, cc, pack8(x));
    unpack8(tile_chunk(k_raw, 8192, r, cc), x);
    const float br = s_beta[r];
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] *= f[e] * br;
    set_tile_chunk(k_cvt, 8192, r, cc, pack8(x));
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  constexpr uint32_t kColDR = 0, kColP = 128;  // tensor-memory columns: DR^T, then P1^T, P2^T, P3^T (64 each)
  if (tid == 0) {
    const Operand op_stack{sbase + KdaPairSmem::kStack, 12288}, op_ar{sbase + KdaPairSmem::kAR, 16384};
    const Operand op_q{sbase + KdaPairSmem::kCvt, 8192}, op_k{sbase + KdaPairSmem::kCvt + 16384, 8192};
    const Operand op_x1{sbase + KdaPairSmem::kX1, 8192}, op_x2{sbase + KdaPairSmem::kX2, 8192};
    umma_gemm<128, 128>(tmem + kColDR, op_stack, true, op_ar, false, 96, false);
#pragma unroll
    for (int blk = 1; blk < 4; ++blk) {
      umma_gemm<128, 64>(tmem + kColP + 64 * (blk - 1), operand_at(op_q, 16 * blk), true, operand_at(op_x1, 16 * blk),
                         true, 16, false);
      umma_gemm<128, 64>(tmem + kColP + 64 * (blk - 1), operand_at(op_k, 16 * blk), true, operand_at(op_x2, 16 * blk),
                         true, 16, true);
    }
    umma_commit(&bar);
  }
  bool products_seen = false;
  auto wait_products = [&]() {  // a whole warp at a time (a warp shares its quarter, and so its trip counts)
    if (!products_seen) {
      ok = __all_sync(0xffffffffu, mbar_wait(&bar, 0)) && ok;
      tc_fence_after();
      products_seen = true;
    }
  };
  const uint32_t my_lane = tmem + (uint32_t(warp4 * 32) << 16);  // this thread's channel is its tensor-memory lane

  // What a thread carries out of its pass, per row / column of its eight groups of four: the row pass dk's row part
  // and the gate gradient's row part, the column pass CC and the gate gradient's column part.  The gate gradient is
  // a sum of terms that cancel along the chunk (sum_i q_i RQ_i = sum_j k_j CK_j term by term), so both passes form
  // their tensor-core parts from the SAME rounded factors (q~, beta k~', the stack, bf16 M): the terms still cancel
  // to fp32 accuracy, which exact factors on one side and rounded ones on the other would not.
  // Every thread runs both passes for the groups of four rows / columns 4 quarter + 16 n, n = 0..3: it ends up
  // holding the row part and the column part of the same 16 (token, channel) pairs.
  float keep_a[16], keep_b[16], keep_c[16], keep_k[16], keep_db[16];
#pragma unroll
  for (int n = 0; n < 16; ++n) keep_a[n] = keep_b[n] = keep_c[n] = keep_k[n] = keep_db[n] = 0.f;
  float chunk_end = 0.f;
  {
    // ---- row pass: four rows at a time.  For j below the group (inside the 16-block), E_{i0+r, j} = E_{i0, j}
    // E_{i0+r, i0}: the four rows share k_j E_{i0, j} and take their own factor (<= 1) once at the end; the 4 x 4
    // diagonal block is done apart; the earlier blocks come from the tensor core.
    const float gl = sG[(len - 1) * 128 + d];
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int i0 = 4 * quarter + 16 * n;
      if (i0 < len) {  // uniform over the warp
        const int big = i0 >> 4, bs = i0 & ~15;
        const float* m1d = sM1d + big * 16 * 20;
        const float* m2d = sM2d + big * 16 * 20;
        float rq[4] = {0.f, 0.f, 0.f, 0.f}, rk[4] = {0.f, 0.f, 0.f, 0.f};
        float xq4[4], xr4[4], xg4[4];  // the rows' global operands, in flight while the sums run
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int64_t at = col + int64_t(i0 + r < len ? i0 + r : len - 1) * stride;
          xq4[r] = dqg[at], xr4[r] = dkr[at], xg4[r] = dkg[at];
        }
        float e = sR[i0 * 128 + d];  // E_{i0, i0 - 1}
        for (int j0 = i0 - 4; j0 >= bs; j0 -= 4) {
          float av[4][4], bv[4][4];
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const float4 a = *reinterpret_cast<const float4*>(m1d + (i0 + r - bs) * 20 + j0 - bs);
            const float4 b = *reinterpret_cast<const float4*>(m2d + (i0 + r - bs) * 20 + j0 - bs);
            av[r][0] = a.x, av[r][1] = a.y, av[r][2] = a.z, av[r][3] = a.w;
            bv[r][0] = b.x, bv[r][1] = b.y, bv[r][2] = b.z, bv[r][3] = b.w;
          }
#pragma unroll
          for (int t = 3; t >= 0; --t) {
            const float kj = rq_at(k_raw, j0 + t) * e;
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
        for (int r = 0; r < 4; ++r) r4[r] = sR[(i0 + r) * 128 + d], k4[r] = rq_at(k_raw, i0 + r);
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
        for (int r = 0; r < 4; ++r) {  // the diagonal 4 x 4 block: pairs (i0 + r, i0 + t), t <= r (M2 is zero on the diagonal)
          const float4 a = *reinterpret_cast<const float4*>(m1d + (i0 + r - bs) * 20 + i0 - bs);
          const float4 b = *reinterpret_cast<const float4*>(m2d + (i0 + r - bs) * 20 + i0 - bs);
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
        // the earlier blocks: this channel's lane of DR^T, columns i0 .. i0 + 3 (M1) and 64 + i0 .. (M2)
        wait_products();
        float offq[4], offk[4];
        tmem_ld4(my_lane + kColDR + i0, offq);
        tmem_ld4(my_lane + kColDR + 64 + i0, offk);
        tmem_ld_wait();
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int i = i0 + r;
          if (i < len) {
            const float gi = sG[i * 128 + d];
            const float down = fast_exp2(gi - sG[bs * 128 + d]);  // 2^{G_i - G_R}
            const float rqt = fmaf(down, offq[r], rq[r]), rkt = fmaf(down, offk[r], rk[r]);
            const float qi = rq_at(q_raw, i), ki = k4[r], bi = s_beta[i];
            const int64_t at = col + i * stride;
            const float eg = fast_exp2(gi), er = fast_exp2(gl - gi);
            const float qgr = round_bf16(qi * eg), kgr = round_bf16(ki * eg), krr = round_bf16(ki * er);
            const float xq = xq4[r], xr = xr4[r], xg = xg4[r];
            dq[at] = fmaf(xq, eg, rqt);
            keep_a[4 * n + r] = fmaf(bi, rkt, fmaf(xr, er, xg * eg));                // dk without its column part
            // the gate gradient's row part: the tensor-core sums against the rounded factors they were formed from
            keep_b[4 * n + r] = fmaf(rq_at(q_cvt, i), offq[r], fmaf(rq_at(k_cvt, i), offk[r], qi * rq[r] + ki * bi * rk[r])) +
                                xq * qgr + xg * kgr - xr * krr;
            chunk_end = fmaf(xr, krr, chunk_end);
            keep_db[4 * n + r] = ki * rkt;  // dbeta_i += sum_d k_id RK_id
          }
        }
      }
    }
    if (quarter == 0) chunk_end = fmaf(fast_exp2(gl), hdh[tile * kDim + d], chunk_end);
  }
  {
    // ---- column pass: four columns at a time.  For i below the group (inside the 16-block), E_{i, j0+c} =
    // E_{i, j0+3} E_{j0+3, j0+c}; the later blocks come from the tensor core.
    wait_products();
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int j0 = 4 * quarter + 16 * n;
      if (j0 < len) {
        const int big = j0 >> 4, bs = j0 & ~15;
        const int be = len < bs + 16 ? len : bs + 16;
        const float* m1d = sM1d + big * 16 * 20;
        const float* m2d = sM2d + big * 16 * 20;
        float cc[4] = {0.f, 0.f, 0.f, 0.f};
        float e = 1.f;
        for (int i0 = j0 + 4; i0 < be; i0 += 4) {  // rows at or past the chunk's length hold q = k = 0 and R = 1
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            e *= sR[(i0 + t) * 128 + d];  // E_{i0 + t, j0 + 3}
            const float tq = rq_at(q_raw, i0 + t) * e, tk = rq_at(k_raw, i0 + t) * e * s_beta[i0 + t];
            const float4 a = *reinterpret_cast<const float4*>(m1d + (i0 + t - bs) * 20 + j0 - bs);
            const float4 b = *reinterpret_cast<const float4*>(m2d + (i0 + t - bs) * 20 + j0 - bs);
            cc[0] = fmaf(a.x, tq, fmaf(b.x, tk, cc[0]));
            cc[1] = fmaf(a.y, tq, fmaf(b.y, tk, cc[1]));
            cc[2] = fmaf(a.z, tq, fmaf(b.z, tk, cc[2]));
            cc[3] = fmaf(a.w, tq, fmaf(b.w, tk, cc[3]));
          }
        }
        float r4[4], k4[4], q4[4], b4[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          r4[r] = sR[(j0 + r) * 128 + d], k4[r] = rq_at(k_raw, j0 + r), q4[r] = rq_at(q_raw, j0 + r);
          b4[r] = s_beta[j0 + r];
        }
        {
          float f = 1.f;
#pragma unroll
          for (int cidx = 2; cidx >= 0; --cidx) {
            f *= r4[cidx + 1];  // E_{j0 + 3, j0 + cidx}
            cc[cidx] *= f;
          }
        }
#pragma unroll
        for (int cidx = 0; cidx < 4; ++cidx) {  // the diagonal 4 x 4 block: pairs (j0 + r, j0 + cidx), r >= cidx
          float ee = 1.f;
#pragma unroll
          for (int r = cidx; r < 4; ++r) {
            if (r > cidx) ee *= r4[r];
            cc[cidx] = fmaf(fmaf(m1d[(j0 + r - bs) * 20 + j0 + cidx - bs], q4[r],
                                 m2d[(j0 + r - bs) * 20 + j0 + cidx - bs] * b4[r] * k4[r]), ee, cc[cidx]);
          }
        }
        float kcc[4];
#pragma unroll
        for (int cidx = 0; cidx < 4; ++cidx) kcc[cidx] = k4[cidx] * cc[cidx];
        // the later blocks: sum over I > block(j) of 2^{G_{16 I} - G_j} PI^T[d][j]; for the gate gradient the same
        // sums against the stack's own (rounded) k_j 2^{G_{16 I} - G_j}
        for (int blk = big + 1; blk < 4; ++blk) {
          float p[4];
          tmem_ld4(my_lane + kColP + 64 * (blk - 1) + j0, p);
          tmem_ld_wait();
          const float gref = sG[(16 * blk) * 128 + d];
          const int base_row = blk == 1 ? 0 : (blk == 2 ? 16 : 48);
#pragma unroll
          for (int cidx = 0; cidx < 4; ++cidx) {
            cc[cidx] = fmaf(fast_exp2(gref - sG[(j0 + cidx) * 128 + d]), p[cidx], cc[cidx]);
            const float kst = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(
                stack + (d >> 6) * 12288 + sw128_offset(base_row + j0 + cidx, (d & 63) >> 3) + (d & 7) * 2));
            kcc[cidx] = fmaf(kst, p[cidx], kcc[cidx]);
          }
        }
#pragma unroll
        for (int cidx = 0; cidx < 4; ++cidx) keep_c[4 * n + cidx] = cc[cidx], keep_k[4 * n + cidx] = kcc[cidx];
      }
    }
  }
  wait_products();
  // dbeta's row part: sum over the channels of k_id RK_id.  The 16 rows' partials of the warp's 32 channels are summed
  // by a butterfly that halves the rows a lane carries at every step (16 shuffles instead of 80); then one partial
  // per warp of the quarter.
  {
#pragma unroll
    for (int width = 8, m = 16; width >= 1; width >>= 1, m >>= 1) {
      const bool up = (lane & m) != 0;  // this lane keeps the upper half of the rows it still carries
#pragma unroll
      for (int j = 0; j < width; ++j) {
        const float mine = up ? keep_db[j + width] : keep_db[j], send = up ? keep_db[j] : keep_db[j + width];
        keep_db[j] = mine + __shfl_xor_sync(0xffffffffu, send, m);
      }
    }
    keep_db[0] += __shfl_xor_sync(0xffffffffu, keep_db[0], 1);
    // lane bits 4..1 spell which of the 16 rows the lane holds: bit 4 the upper eight, bit 3 the upper four, ...
    const int which = (lane >> 1) & 15, i = 4 * quarter + 16 * (which >> 2) + (which & 3);
    if ((lane & 1) == 0 && i < len) s_db[i * 4 + warp4] = keep_db[0];
  }
  __syncthreads();  // both passes are done with the gates and the factors: their space takes the sums below
  float* s_end = sG;               // the chunk-end term per channel, one partial per quarter  [4][128]
  float* s_tot = sG + 4 * 128;     // the gate gradient summed over each group of four rows     [16][128]
  s_end[quarter * 128 + d] = chunk_end;
  __syncthreads();
  // dk and the gate gradient of this thread's 16 (token, channel) pairs; the in-chunk suffix sum of the gate gradient
  // by groups: every thread sums its groups, publishes the totals and adds the totals of the later groups
  float dgv[16];
#pragma unroll
  for (int n = 0; n < 4; ++n) {
    float total = 0.f;
#pragma unroll
    for (int r = 3; r >= 0; --r) {
      const int i = 4 * quarter + 16 * n + r;
      float dgi = 0.f;
      if (i < len) {
        dk[col + i * stride] = keep_a[4 * n + r] + keep_c[4 * n + r];
        dgi = keep_b[4 * n + r] - keep_k[4 * n + r];
        if (i == len - 1) dgi += (s_end[d] + s_end[128 + d]) + (s_end[256 + d] + s_end[384 + d]);
      }
      total += dgi;
      dgv[4 * n + r] = total;  // the suffix sum inside the group
    }
    s_tot[(quarter + 4 * n) * 128 + d] = total;
  }
  __syncthreads();
#pragma unroll
  for (int n = 0; n < 4; ++n) {
    const int group = quarter + 4 * n;
    float later = 0.f;
    for (int g = 15; g > group; --g) later += s_tot[g * 128 + d];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = 4 * quarter + 16 * n + r;
      if (i < len) dg[col + i * stride] = dgv[4 * n + r] + later;
    }
  }
  if (tid < len) {
    const int64_t at = int64_t(start + tid) * num_heads + h;
    dbeta[at] = dbeta_part[at] + ((s_db[tid * 4] + s_db[tid * 4 + 1]) + (s_db[tid * 4 + 2] + s_db[tid * 4 + 3]));
  }
  if (!ok && tid == 0) atomicExch(status, kDevWaitTimeout | (8 << 8));
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
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
  kda_prep_kernel<<<dim3(d->num_chunks, d->num_v_heads), 64, 0, static_cast<cudaStream_t>(stream)>>>(
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
  KdaIntraMaps maps;
  if (int rc = make_rows_map(&maps.q, q, d->total_tokens, d->num_v_heads, "kda_intra")) return rc;
  if (int rc = make_rows_map(&maps.k, k, d->total_tokens, d->num_v_heads, "kda_intra")) return rc;
  kda_intra_kernel<<<dim3(d->num_chunks, d->num_v_heads), kIntraThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      maps, In(v), In(kg), g2, beta, Out(a_out), Out(aqk_out), Out(w_out), Out(u_out), d->chunk_start,
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
  const size_t smem_a = KdaTailSmem::kBytes + 1024, smem_b = KdaPairSmem::kBytes + 1024;
  KdaPairMaps maps;
  if (int rc = make_rows_map(&maps.q, q, d->total_tokens, d->num_v_heads, "kda_bwd_tail")) return rc;
  if (int rc = make_rows_map(&maps.k, k, d->total_tokens, d->num_v_heads, "kda_bwd_tail")) return rc;
  KdaTailMaps tail_maps;
  const int64_t tiles = int64_t(d->num_chunks) * d->num_v_heads;
  if (tiles * 128 > int64_t(INT32_MAX)) return fail(MEK_ERR_UNSUPPORTED, "kda_bwd_tail: %lld state tiles", (long long)tiles);
  struct {
    CUtensorMap* map;
    const void* base;
  } const row_maps[] = {{&tail_maps.d_o, d_o}, {&tail_maps.v_new, v_new}, {&tail_maps.dv_new, dv_new},
                        {&tail_maps.kg, kg},   {&tail_maps.v, v}};
  for (const auto& m : row_maps)
    if (int rc = make_rows_map(m.map, m.base, d->total_tokens, d->num_v_heads, "kda_bwd_tail")) return rc;
  if (int rc = make_tiles_map(&tail_maps.h, h_tape, tiles, 128, 128, "kda_bwd_tail")) return rc;
  if (int rc = make_tiles_map(&tail_maps.dh, dh_tape, tiles, 128, 128, "kda_bwd_tail")) return rc;
  if (int rc = make_tiles_map(&tail_maps.a, a, tiles, 64, 64, "kda_bwd_tail")) return rc;
  if (int rc = want_smem(kda_tail_mma_kernel, smem_a, "kda_bwd_tail")) return rc;
  if (int rc = want_smem(kda_tail_pair_kernel, smem_b, "kda_bwd_tail")) return rc;
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) {
    cudaGetLastError();
    return fail(MEK_ERR_CUDA, "kda_bwd_tail: cannot query the SM count");
  }
  const dim3 grid(d->num_chunks, d->num_v_heads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  kda_tail_mma_kernel<<<tiles < sms ? int(tiles) : sms, kKdaTailThreads, smem_a, s>>>(
      tail_maps, beta, m1, m2, dqg, dkr, dkg, hdh, Out(dv), dbeta_part, d->chunk_start, d->chunk_len, d->num_chunks,
      d->num_v_heads, d->scale, status);
  if (int rc = launched("kda_bwd_tail (tensor-core part)")) return rc;
  kda_tail_pair_kernel<<<grid, 512, smem_b, s>>>(maps, g2, beta, m1, m2, dqg, dkr, dkg, hdh, dbeta_part, dq32, dk32, dg,
                                                 dbeta, d->chunk_start, d->chunk_len, d->num_v_heads, status);
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
