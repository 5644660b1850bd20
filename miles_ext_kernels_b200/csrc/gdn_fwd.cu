// Forward kernels of the chunked gated delta rule (chunk 64, K = V = 128), sm_100a.
//
//   prep      per-row L2 norm of q / k (optional) and the chunk-local cumulative gate in the log2 domain
//   wy        per (chunk, value head): Aqk = tril(scale q k^T 2^{G_i-G_j}),  A = (I + tril(beta_i 2^{G_i-G_j} k_i.k_j, -1))^-1,
//             w = A bf16(beta 2^G k),  u = A bf16(beta v)                      [tcgen05, TMEM accumulators]
//   fwd_h     per (sequence, value head), serial over chunks: h_tape = bf16(h); v_new = u - w h_tape;
//             h = gamma h + k^T bf16(rowscale v_new)                           [tcgen05, fp32 state in registers]
//   fwd_o     per (chunk, value head): o = bf16(qscale (q h_tape) + Aqk v_new)  [tcgen05]
//
// The stages and their rounding points follow the reference's dataflow (reference:
// miles_ext_kernels/cake/_impl/gdn/ops.py:1320-1450 launch order; semantics
// miles_ext_kernels/cake/_vendor/cake_gdn_det_train_kcp/cake_fake_backend.py:173-279, 418-430).
//
// Shared-memory operand tiles use the swizzled block layout of umma.cuh; one tile serves as a K-major operand
// (contraction over the feature axis) and as an MN-major operand (contraction over the token axis).
#include "common.cuh"
#include "scan_plan.cuh"
#include "tiles.cuh"
#include "tma.cuh"

namespace mek {

// ---------------------------------------------------------------------------------------------------------------
// prep
// ---------------------------------------------------------------------------------------------------------------
// Half a warp per row of 128 bf16 (16-byte loads), two rows per half warp with both loads issued up front:
// y = bf16(x r), r = 1 / sqrt(sum x^2 + 1e-6), r saved.  Row (token, head) of x sits at token * pitch + head * 128
// (x may be a column slice of a packed row); y and rstd are dense.
__global__ void __launch_bounds__(256) l2norm_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                                     float* __restrict__ rstd, int64_t rows, int heads, int64_t pitch) {
  const int part = threadIdx.x & 15;  // 16-byte piece of the row
  const int64_t row0 = int64_t(blockIdx.x) * 32 + (threadIdx.x >> 4);
  uint4 raw[2];
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    const int64_t row = row0 + 16 * n;
    raw[n] = make_uint4(0u, 0u, 0u, 0u);
    if (row < rows) raw[n] = ldg16(x + (row / heads) * pitch + (row % heads) * kDim + part * 8);
  }
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    const int64_t row = row0 + 16 * n;
    float v[8];
    unpack8(raw[n], v);
    // the same order of additions as a lane of the earlier one-warp-per-row form took: pairs, then a butterfly
    float ss = (v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]) + (v[4] * v[4] + v[5] * v[5] + v[6] * v[6] + v[7] * v[7]);
#pragma unroll
    for (int m = 8; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
    const float r = 1.0f / sqrtf(ss + 1e-6f);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= r;
    if (row < rows) {
      *reinterpret_cast<uint4*>(y + row * kDim + part * 8) = pack8(v);
      if (part == 0) rstd[row] = r;
    }
  }
}

// One block per chunk, one thread per value head: g_cs[t, hv] = log2(e) * sum_{s <= t, same chunk} g[s, hv].
__global__ void gate_cumsum_kernel(const float* __restrict__ g, float* __restrict__ g_cs,
                                   const int32_t* __restrict__ chunk_start, const int32_t* __restrict__ chunk_len,
                                   int num_v_heads) {
  const int c = blockIdx.x;
  const int start = chunk_start[c], len = chunk_len[c];
  for (int hv = threadIdx.x; hv < num_v_heads; hv += blockDim.x) {
    float acc = 0.f;
    for (int i0 = 0; i0 < len; i0 += 8) {  // a batch's loads are issued before the running sum needs the first
      float gv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) gv[j] = i0 + j < len ? g[int64_t(start + i0 + j) * num_v_heads + hv] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (i0 + j < len) {
          acc += gv[j];
          g_cs[int64_t(start + i0 + j) * num_v_heads + hv] = acc * kLog2e;
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// wy
// ---------------------------------------------------------------------------------------------------------------
struct WySmem {
  static constexpr uint32_t kQ = 0;                // [64][128] q; after the first products: fp32 L [64][64], swizzled,
                                                   // whose dead quarters take the TF32 operands; at the end A (bf16)
  static constexpr uint32_t kK = 16384;            // [64][128] k -> beta 2^G k (in place)
  static constexpr uint32_t kV = 32768;            // [64][128] v -> beta v (in place)
  static constexpr uint32_t kScal = kV + 16384;    // beta[64], g2[64]
  static constexpr uint32_t kBytes = kScal + 512;
};

// Four CTAs per SM (50 KB of shared memory each) hide each other's global-load and solve latencies; tensor memory:
// 128 columns each.
struct WyMaps {
  CUtensorMap q, k, v;      // rows, box 64 x 64
  CUtensorMap w_out, u_out;  // rows, box 64 x 64 (stores)
};

__global__ void __launch_bounds__(128) gdn_wy_kernel(
    const __grid_constant__ WyMaps maps, const float* __restrict__ beta, const float* __restrict__ g_cs, __nv_bfloat16* __restrict__ a_out,
    __nv_bfloat16* __restrict__ aqk_out, __nv_bfloat16* __restrict__ w_out, __nv_bfloat16* __restrict__ u_out,
    const int32_t* __restrict__ chunk_start, const int32_t* __restrict__ chunk_len, int num_qk_heads, int num_v_heads,
    float scale, int32_t* __restrict__ status) {
  extern __shared__ uint8_t raw[];
  __shared__ uint64_t bar, bar_load;
  __shared__ uint32_t tmem_slot;
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, hv = blockIdx.y, hq = hv / (num_v_heads / num_qk_heads);
  const int start = chunk_start[c], len = chunk_len[c];
  if (len <= 0) return;  // a pad chunk of a device-built table
  float* s_beta = reinterpret_cast<float*>(sm + WySmem::kScal);
  float* s_g2 = s_beta + 64;
  float* s_l = reinterpret_cast<float*>(sm + WySmem::kQ);
  constexpr uint32_t kUpper = 16u << 16;  // an M = 64 accumulator in lanes 16..31 of each quadrant

  const int64_t v_stride = int64_t(num_v_heads) * kDim;
  const uint32_t sbase = smem_u32(sm);
  if (tid == 0) {  // all three tiles in flight at once (TMA), the scalars by plain loads meanwhile
    mbar_init(&bar, 1);
    mbar_init(&bar_load, 1);
    fence_mbar_init();
    mbar_arrive_expect(&bar_load, 3 * 16384);
    tma_load_tile128(sbase + WySmem::kQ, 8192, &maps.q, hq * kDim, start, &bar_load);
    tma_load_tile128(sbase + WySmem::kK, 8192, &maps.k, hq * kDim, start, &bar_load);
    tma_load_tile128(sbase + WySmem::kV, 8192, &maps.v, hv * kDim, start, &bar_load);
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 128);
  if (tid < 64) {
    const int i = tid < len ? tid : len - 1;
    s_beta[tid] = tid < len ? beta[int64_t(start + i) * num_v_heads + hv] : 0.f;
    s_g2[tid] = g_cs[int64_t(start + i) * num_v_heads + hv];
  }
  __syncthreads();  // the barrier's initialisation is visible to every waiter
  bool ok = __all_sync(0xffffffffu, mbar_wait(&bar_load, 0));
  if (len < kChunk) {  // a ragged chunk's boxes reach into the next sequence: clear those rows
    clear_tile_rows<128>(sm + WySmem::kQ, len, tid);
    clear_tile_rows<128>(sm + WySmem::kK, len, tid);
    clear_tile_rows<128>(sm + WySmem::kV, len, tid);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  // q k^T -> lanes 0..15, k k^T -> lanes 16..31 of the same 64 columns
  if (tid == 0) {
    const Operand op_q{sbase + WySmem::kQ, 8192}, op_k{sbase + WySmem::kK, 8192};
    umma_gemm_pair<64, 64>(tmem, op_q, false, op_k, false, 128, false, false, tmem + kUpper, op_k, false, op_k, false,
                           128, false, false);  // alternating: one product's instructions wait for one another
    umma_commit(&bar);
  }
  ok = __all_sync(0xffffffffu, mbar_wait(&bar, 0)) && ok;
  tc_fence_after();
  __syncthreads();  // every thread sees the products done: the q tile's space now takes L

  if (ok) {
    // lanes 0..15: Aqk row i -> global; lanes 16..31: L row i -> shared.  Both are the product's entry times the
    // decay 2^{G_i - G_col} and a row factor (scale / beta_i), Aqk with its diagonal and L without: one instruction
    // stream for both lane halves up to the stores.
    const int i = warp * 16 + (lane & 15);
    const bool upper = lane >= 16;
    const float gi = s_g2[i], factor = upper ? s_beta[i] : scale;
    const int last = upper ? i - 1 : i;  // the last column that is kept
    __nv_bfloat16* dst = aqk_out + (int64_t(c) * num_v_heads + hv) * 4096 + i * 64;
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      float s[32];
      tmem_ld32(tmem_addr(tmem, warp, p * 32), s);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int col = p * 32 + j;
        s[j] = col <= last ? factor * s[j] * fast_exp2(gi - s_g2[col]) : 0.f;
      }
      if (!upper) {
#pragma unroll
        for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(dst + p * 32)[j] = pack8(s + 8 * j);
      } else {
        // four consecutive columns are contiguous in the operand layout: 16-byte stores
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(s_l + wy_l_index(i, p * 32 + j)) = make_float4(s[j], s[j + 1], s[j + 2], s[j + 3]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();

  // A = (I + L)^-1 by blocks of 32: with I + L = [[M11, 0], [L21, M22]],
  //     A = [[X11, 0], [X21, X22]],  X11 = M11^-1, X22 = M22^-1 (fp32 forward substitution, 64 threads, 496 FMAs each)
  //     X21 = -X22 (L21 X11)  (two tensor-core products with TF32 operands; A is rounded to bf16 afterwards)
  // The products' operands take the quarters of L that are dead by then (L as two blocks of 32 columns, rows 0..31 /
  // 32..63 of each a quarter of 4 KiB):
  //     L11 -> B1 = X11^T [32 x 32]      L21 (stays: rows 32..63 of the first product's A operand, the block itself)
  //     upper right (never used) -> X22  L22 -> B2 = T^T [32 x 32]
  // A2 = [*; X22] [64 x 32] starts at L21, so that its rows 32..63 are the upper right quarter; its rows 0..31 (and the
  // first product's: B1 by then) are whatever lies there -- a row of the result depends on its own operand row only,
  // and the results' rows 0..31 are not read.
  float* s_b1 = s_l;
  float* s_a2 = s_l + 1024;
  float* s_b2 = s_l + 3072;
  // Warps 0..1 solve in registers while warps 2..3 turn k and v into the last products' operands, kb = bf16(beta 2^G k)
  // and vb = bf16(beta v), in place.  The solving threads keep their columns of X11 / X22 in registers until A can be
  // written (its tile takes L's space once the products are done).
  float x[32];
  if (tid < 64) {
    const int b = tid >> 5, c = tid & 31, base = 32 * b;
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
    if (b == 0) {  // row c of B1 = column c of X11
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        *reinterpret_cast<float4*>(s_b1 + f32_block_index(c, i)) = make_float4(x[i], x[i + 1], x[i + 2], x[i + 3]);
    } else {  // column c of X22 in the rows 32..63 of A2
#pragma unroll
      for (int i = 0; i < 32; ++i) s_a2[f32_block_index(32 + i, c)] = x[i];
    }
  } else {
    const int t = tid - 64;
    for (int i = t; i < 64 * 16; i += 64) {
      const int r = i >> 4, cc = i & 15;
      const float b = s_beta[r], sc = b * fast_exp2(s_g2[r]);
      float y[8];
      unpack8(tile_chunk(sm + WySmem::kK, 8192, r, cc), y);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] *= sc;
      set_tile_chunk(sm + WySmem::kK, 8192, r, cc, pack8(y));
      unpack8(tile_chunk(sm + WySmem::kV, 8192, r, cc), y);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] *= b;
      set_tile_chunk(sm + WySmem::kV, 8192, r, cc, pack8(y));
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t l_addr = sbase + WySmem::kQ;
  const uint32_t b1_addr = l_addr, a2_addr = l_addr + 4096, b2_addr = l_addr + 12288;
  uint8_t* a_tile = sm + WySmem::kQ;  // written when the second product is done
  constexpr uint32_t kColT = 64, kColX = 96;  // free until the w / u products
  if (tid == 0) {  // T' = L[:, 0:32] X11 (rows 32..63 are T = L21 X11)
    const uint32_t idesc = umma_idesc_tf32(64, 32);
    for (uint32_t k0 = 0; k0 < 32; k0 += 8)
      umma_tf32(tmem + kColT, umma_desc_sw128(l_addr + k0 * 4, 16u, kSbo), umma_desc_sw128(b1_addr + k0 * 4, 16u, kSbo),
                idesc, k0 > 0 ? 1u : 0u);
    umma_commit(&bar);
  }
  ok = mbar_wait(&bar, 1) && ok;
  tc_fence_after();
  {
    float t[32];
    tmem_ld32(tmem_addr(tmem, warp, kColT), t);
    tmem_ld_wait();
    if (warp >= 2 && lane < 16) {  // row i = 16 warp + lane of T' -> column i - 32 of B2 = T^T
      const int kk = 16 * warp + lane - 32;
#pragma unroll
      for (int n = 0; n < 32; ++n) s_b2[f32_block_index(n, kk)] = t[n];
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (tid == 0) {  // X' = -A2 T (rows 32..63 are X21)
    const uint32_t idesc = umma_idesc_tf32(64, 32, /*neg_a=*/true);
    for (uint32_t k0 = 0; k0 < 32; k0 += 8)
      umma_tf32(tmem + kColX, umma_desc_sw128(a2_addr + k0 * 4, 16u, kSbo),
                umma_desc_sw128(b2_addr + k0 * 4, 16u, kSbo), idesc, k0 > 0 ? 1u : 0u);
    umma_commit(&bar);
  }
  ok = mbar_wait(&bar, 0) && ok;
  tc_fence_after();
  {
    // both products are done: A (bf16) takes the first half of L's space -- the diagonal blocks from the solving
    // threads' registers, X21 from the product, zeros above
    float xv[32];
    tmem_ld32(tmem_addr(tmem, warp, kColX), xv);
    tmem_ld_wait();
    if (warp >= 2) {
      if (lane < 16) {
        const int i = 16 * warp + lane;
#pragma unroll
        for (int j = 0; j < 4; ++j) set_tile_chunk(a_tile, 8192, i, j, pack8(xv + 8 * j));
      } else {  // the upper right block of A is zero: the 16 rows 16 (warp - 2) .. + 15
        const int i = 16 * (warp - 2) + lane - 16;
#pragma unroll
        for (int j = 0; j < 4; ++j) set_tile_chunk(a_tile, 8192, i, 4 + j, make_uint4(0u, 0u, 0u, 0u));
      }
    } else {
      const int b = tid >> 5, base = 32 * b, col = base + (tid & 31);
#pragma unroll
      for (int i = 0; i < 32; ++i)
        *reinterpret_cast<__nv_bfloat16*>(a_tile + sw128_offset(base + i, col >> 3) + (col & 7) * 2) =
            __float2bfloat16_rn(x[i]);
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  // w = A kb -> lanes 0..15, u = A vb -> lanes 16..31 of columns 0..127
  if (tid == 0) {
    const Operand a{sbase + WySmem::kQ, 8192};
    const Operand kb{sbase + WySmem::kK, 8192};
    const Operand vb{sbase + WySmem::kV, 8192};
    umma_gemm_pair<64, 128>(tmem, a, false, kb, true, 64, false, false, tmem + kUpper, a, false, vb, true, 64, false,
                            false);
    umma_commit(&bar);
  }
  // A -> global while the MMAs run
  store_tile<64, 64, 128>(sm + WySmem::kQ, 8192, a_out + (int64_t(c) * num_v_heads + hv) * 4096, 64, 64, tid);
  ok = mbar_wait(&bar, 1) && ok;  // the fourth commit on this barrier
  tc_fence_after();
  __syncthreads();  // every thread has stored its part of A: the tile's space is staged over below

  ok = __all_sync(0xffffffffu, ok);
  // w and u leave through shared memory (the dead q / k tiles' space) and one TMA store each: a thread's row piece
  // written straight to global memory would touch a different 128-byte line in every lane.  A ragged chunk's rows are
  // stored by hand (a 64-row box would run into the next sequence).
  const bool by_box = len == kChunk;
  if (ok) {
    const int i = warp * 16 + (lane & 15);
    const bool live = i < len;
    __nv_bfloat16* dst = (lane < 16 ? w_out : u_out) + int64_t(start + i) * v_stride + hv * kDim;
    uint8_t* stage = sm + (lane < 16 ? WySmem::kQ : WySmem::kK);
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      float s[32];
      tmem_ld32(tmem_addr(tmem, warp, p * 32), s);
      tmem_ld_wait();
      if (by_box) {
#pragma unroll
        for (int j = 0; j < 4; ++j) set_tile_chunk(stage, 8192, i, p * 4 + j, pack8(s + 8 * j));
      } else if (live) {
#pragma unroll
        for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(dst + p * 32)[j] = pack8(s + 8 * j);
      }
    }
  }
  if (by_box) {
    fence_async_smem();
    __syncthreads();
    if (tid == 0 && ok) {
      tma_store_tile128(&maps.w_out, hv * kDim, start, sbase + WySmem::kQ, 8192);
      tma_store_tile128(&maps.u_out, hv * kDim, start, sbase + WySmem::kK, 8192);
      tma_store_commit();
      tma_store_wait_read();  // the tiles must outlive the copies' reads; this thread keeps the CTA alive until then
    }
  }
  if (!ok && tid == 0) atomicExch(status, kDevWaitTimeout | (1 << 8));
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 128);
}

// ---------------------------------------------------------------------------------------------------------------
// fwd_h : the state recurrence
// ---------------------------------------------------------------------------------------------------------------
// One CTA per (sequence, value head), warp-specialised: two epilogue warpgroups (256 threads), one MMA-issuing warp
// and one copy warp.  The fp32 state h [K, V] lives in the epilogue threads' registers: thread (k, half) holds row k
// of one half of the V columns (warpgroup 0: columns 0..63, warpgroup 1: 64..127).  Per chunk:
//   A  epilogue   h_tape = bf16(h) -> shared (MN-major B operand)                 -> "state tile ready"
//      issuer     D1 = w h_tape (M=64,N=128,K=128) [+ q h_tape for the fused output]
//      copy warp  h_tape tile -> the tape (TMA store); next chunk's w / k / u (/ q / Aqk) tiles (TMA loads)
//   B  epilogue   v_new = u - D1 -> shared; vs = bf16(rowscale v_new) -> shared   -> "v tiles ready"
//      issuer     D2 = k^T vs (M=128,N=128,K=64) [+ Aqk v_new for the fused output]
//      copy warp  v_new tile -> the tape, the previous chunk's output tile -> o (TMA stores; a ragged chunk's rows
//                 are stored by the epilogue threads)
//   C  epilogue   h = gamma h + D2.
// The roles meet on mbarriers only (no block barrier inside the walk): the epilogue threads never wait for an
// instruction to be issued or for a store to leave, only for the two products on the step's dependency chain.
struct FwdHSmem {
  static constexpr uint32_t kStage = 4 * 16384 + 8192;   // w, k, u, q tiles and Aqk of one chunk
  static constexpr uint32_t kW = 0, kK = 16384, kU = 32768, kQ = 49152, kAqk = 65536;
  static constexpr uint32_t kH = 2 * kStage;      // [128 k][128 v] bf16(h), 2 blocks of 16 KiB (one per V half)
  static constexpr uint32_t kVS = kH + 32768;     // [64][128] bf16(rowscale v_new)
  static constexpr uint32_t kVN = kVS + 16384;    // [64][128] v_new (the tape's source; the fused output's operand)
  static constexpr uint32_t kG = kVN + 16384;     // gates[2][128]: GDN g2 per token [64]; KDA chunk-end gate per channel
  static constexpr uint32_t kO = kG + 1024;      // [64][128] the fused output of the previous chunk (its store's source)
  static constexpr uint32_t kBytes = kO + 16384;
};

// With `o` != nullptr the walk also writes the op's output, chunk by chunk (the reference's fused `fwd_ho`):
//   o = bf16(qscale (q h_tape) + Aqk v_new)
// Both products read what the step already holds in shared memory (h_tape, v_new) and run on the tensor core behind
// the step's own products; their epilogue runs one step later, while the epilogue threads wait for the next step's
// products, on a second set of tensor-memory columns -- the chain of dependent steps does not get longer and h is not
// read back.
// `gl2` != nullptr selects the per-channel-decay variant (KDA): `k` then holds k 2^{G_L - G} (the decay to the chunk
// end is folded into the operand, so rowscale = 1) and the state decays per key channel: row k by 2^{gl2[c, hv, k]}.
struct FwdHMaps {
  CUtensorMap k, w, u, q;  // rows, box 64 x 64 (q: the fused output only)
  CUtensorMap aqk;         // tiles [num_tiles * 64, 64], box 64 x 64 (the fused output only)
  CUtensorMap h_out;       // tiles [num_tiles * 128, 128], box 64 x 128: the state tape (stores)
  CUtensorMap v_new_out;   // rows, box 64 x 64: the corrected values' tape (stores)
  CUtensorMap o_out;       // rows, box 64 x 64: the op's output (stores; the fused output only)
};

constexpr int kScanEpilogueThreads = 256;            // warps 0..7
constexpr int kScanIssuer = kScanEpilogueThreads;    // warp 8, lane 0: every tcgen05.mma of the walk
constexpr int kScanMover = kScanEpilogueThreads + 32;  // warp 9, lane 0: every TMA load and store
constexpr int kScanThreads = kScanEpilogueThreads + 64;

__global__ void __launch_bounds__(kScanThreads) gdn_fwd_h_kernel(
    const __grid_constant__ FwdHMaps maps, const float* __restrict__ g_cs, const float* __restrict__ h0,
    __nv_bfloat16* __restrict__ v_new, float* __restrict__ final_state, const int32_t* __restrict__ chunk_start,
    const int32_t* __restrict__ chunk_len, const int32_t* __restrict__ seq_chunk_start, int num_qk_heads,
    int num_v_heads, const float* __restrict__ gl2, const ScanPlan plan, __nv_bfloat16* __restrict__ o, float scale,
    int32_t* __restrict__ status) {
  extern __shared__ uint8_t raw[];
  // bar_h: the state tile (and this chunk's operand tiles) are ready -- every epilogue thread arrives
  // bar_vs: the v tiles are ready -- every epilogue thread arrives
  // bar_d1 / bar_d2 / bar_o: commits of the step's two products and of the fused output's products
  // bar_free_h / bar_free_vn: the copy warp's store of this step has read the state tile / the v_new tile
  // bar_seen: the copy warp is past this step's wait for a free stage
  // bar_out / bar_free_o: the previous chunk's output tile is complete -- every epilogue thread arrives / its store has
  // read the tile
  __shared__ uint64_t bar_load[2], bar_h, bar_vs, bar_d1, bar_d2, bar_o, bar_free_h, bar_free_vn, bar_out, bar_free_o, bar_seen;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool kda = gl2 != nullptr;
  const int quad = warp & 3, half = (warp >> 2) & 1;   // tensor-memory lane quadrant; V half of this warpgroup
  const int krow = quad * 32 + lane;                   // row of h this (epilogue) thread holds
  // grid (heads, sequences): the heads of one sequence are neighbours in launch order, so that with `seq_order`
  // (longest first) every long walk starts before any short one
  const int n = plan.seq_order != nullptr ? plan.seq_order[blockIdx.y] : int(blockIdx.y);
  const int hv = blockIdx.x, hq = hv / (num_v_heads / num_qk_heads);
  float* s_g2 = reinterpret_cast<float*>(sm + FwdHSmem::kG);
  Abort abort{&abort_flag};

  // pre-scan of a segment-parallel plan: blockIdx.z = 0 is the offset walk (B), 1 the transfer walk (M: from the
  // identity, with u = 0); neither writes the tapes.  Decided before anything is allocated: the whole CTA leaves.
  const bool prescan = plan.seg_flags != nullptr;
  const bool transfer = prescan && blockIdx.z == 1;
  int c_first = seq_chunk_start[n];
  const int c_last = seq_chunk_start[n + 1];
  int state_row = n;
  if (prescan) {
    const int flags = plan.seg_flags[n];
    const bool inner = (flags & 1) != 0;
    if ((flags & 2) != 0 || (transfer && !inner) || c_first >= c_last) return;
    state_row = inner ? -1 : plan.state_row[n];
    if (inner && warm_up_suffices(plan, g_cs, chunk_start, chunk_len, c_first, c_last, num_v_heads, hv, false)) {
      if (transfer) return;  // M is taken as zero
      c_first = c_last - plan.warm_chunks;
    }
  }

  const bool fused = o != nullptr && !prescan;
  const bool tapes = !prescan;  // the walk writes h_tape and v_new
  if (tid == 0) {
    mbar_init(&bar_load[0], 1);
    mbar_init(&bar_load[1], 1);
    mbar_init(&bar_h, kScanEpilogueThreads);
    mbar_init(&bar_vs, kScanEpilogueThreads);
    mbar_init(&bar_d1, 1);
    mbar_init(&bar_d2, 1);
    mbar_init(&bar_o, 1);
    mbar_init(&bar_free_h, 1);
    mbar_init(&bar_free_vn, 1);
    mbar_init(&bar_out, kScanEpilogueThreads);
    mbar_init(&bar_free_o, 1);
    mbar_init(&bar_seen, 1);
    fence_mbar_init();
    abort_flag = 0;
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 512);
  const uint32_t sbase = smem_u32(sm);
  const int64_t v_stride = int64_t(num_v_heads) * kDim;
  const int c_begin = c_first, c_end = c_last;
  tc_fence_before();
  __syncthreads();  // the barriers' initialisation and the tensor-memory base are visible to every role
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const Operand op_h{sbase + FwdHSmem::kH, 16384}, op_vs{sbase + FwdHSmem::kVS, 8192};
  const Operand op_vn{sbase + FwdHSmem::kVN, 8192};
  // tensor-memory columns: D1 0..127 (lanes 0..15 of each quadrant), D2 128..255, the fused output's two accumulators
  // (q h_tape at +0, Aqk v_new at +64, both lane split: logical columns 64..127 in lanes 16..31) in one of two sets
  // at 256 and 384
  constexpr uint32_t kColO = 256;
  constexpr uint32_t kUpper = 16u << 16;

  if (tid == kScanIssuer) {
    // ---- every product of the walk, in the order of the step's dependency chain ----------------------------------
    for (int c = c_begin; c < c_end; ++c) {
      const uint32_t step = uint32_t(c - c_begin), par = step & 1u;
      const uint32_t sst = sbase + par * FwdHSmem::kStage;
      const Operand op_w{sst + FwdHSmem::kW, 8192}, op_k{sst + FwdHSmem::kK, 8192};
      if (!abort.wait(&bar_h, par)) break;
      tc_fence_after();
      // D1 = w h_tape as one chain of N = 128 instructions into the columns 0..127 of lanes 0..15 (a chain of eight
      // dependent instructions is shorter than sixteen alternating between two lane halves)
      umma_gemm<64, 128>(tmem, op_w, false, op_h, true, 128, false);
      umma_commit(&bar_d1);
      if (fused) {  // q h_tape behind it; the state update's commit covers it (commits are cumulative)
        const Operand op_q{sst + FwdHSmem::kQ, 8192};
        const uint32_t set = tmem + kColO + par * 128;
        umma_gemm_pair<64, 64>(set, op_q, false, op_h, true, 128, false, false, set + kUpper, op_q, false,
                               operand_at(op_h, 0, 1), true, 128, false, false);
      }
      if (!abort.wait(&bar_vs, par)) break;
      tc_fence_after();
      umma_gemm<128, 128>(tmem + 128, op_k, true, op_vs, true, 64, false);
      umma_commit(&bar_d2);
      if (fused) {  // Aqk v_new, behind the state update's product
        const Operand op_a{sst + FwdHSmem::kAqk, 8192};
        const uint32_t set = tmem + kColO + par * 128 + 64;
        umma_gemm_pair<64, 64>(set, op_a, false, op_vn, true, 64, false, false, set + kUpper, op_a, false,
                               operand_at(op_vn, 0, 1), true, 64, false, false);
        umma_commit(&bar_o);
      }
    }
  } else if (tid == kScanMover) {
    // ---- every copy of the walk: operand tiles in, tapes out ------------------------------------------------------
    auto load = [&](int c, uint32_t stage) {
      const uint32_t base = sbase + stage * FwdHSmem::kStage;
      const int start = chunk_start[c];
      mbar_arrive_expect(&bar_load[stage], fused ? 4 * 16384 + 8192 : 3 * 16384);
      tma_load_tile128(base + FwdHSmem::kW, 8192, &maps.w, hv * kDim, start, &bar_load[stage]);
      tma_load_tile128(base + FwdHSmem::kK, 8192, &maps.k, hq * kDim, start, &bar_load[stage]);
      tma_load_tile128(base + FwdHSmem::kU, 8192, &maps.u, hv * kDim, start, &bar_load[stage]);
      if (fused) {
        tma_load_tile128(base + FwdHSmem::kQ, 8192, &maps.q, hq * kDim, start, &bar_load[stage]);
        tma_load_box(base + FwdHSmem::kAqk, &maps.aqk, 0, int((int64_t(c) * num_v_heads + hv) * 64),
                     &bar_load[stage]);
      }
    };
    if (c_begin < c_end) load(c_begin, 0);
    for (int c = c_begin; c < c_end; ++c) {
      const uint32_t step = uint32_t(c - c_begin), par = step & 1u;
      if (c + 1 < c_end) {
        // the other stage's last readers were the previous chunk's products (and its epilogue, which ended before
        // they were issued)
        if (c > c_begin && !abort.wait(fused ? &bar_o : &bar_d2, par ^ 1u)) break;
        load(c + 1, par ^ 1u);
      }
      // "This thread is past its wait for a free stage": the epilogue threads wait for it before they release the
      // step's second group of products, so the barrier waited on above cannot complete twice before this thread has
      // looked at it (a wait by parity would then miss the phase for good); and this thread in turn waits for the
      // epilogue's release (bar_vs) before its next step, so neither barrier runs ahead of its waiter.
      mbar_arrive(&bar_seen);
      if (tapes) {
        if (!abort.wait(&bar_h, par)) break;
        tma_store_tile128(&maps.h_out, 0, int((int64_t(c) * num_v_heads + hv) * 128), sbase + FwdHSmem::kH, 16384);
        tma_store_commit();
        tma_store_wait_read();
        mbar_arrive(&bar_free_h);
      }
      if (!abort.wait(&bar_vs, par)) break;
      if (tapes) {
        if (chunk_len[c] == kChunk) {  // a ragged chunk's rows are stored by the epilogue threads
          tma_store_tile128(&maps.v_new_out, hv * kDim, chunk_start[c], sbase + FwdHSmem::kVN, 8192);
          tma_store_commit();
          tma_store_wait_read();
        }
        mbar_arrive(&bar_free_vn);
        if (fused && c > c_begin) {  // the previous chunk's output: complete once its second part is written
          if (!abort.wait(&bar_out, par ^ 1u)) break;
          if (chunk_len[c - 1] == kChunk) {  // a ragged chunk's rows are stored by the epilogue threads
            tma_store_tile128(&maps.o_out, hv * kDim, chunk_start[c - 1], sbase + FwdHSmem::kO, 8192);
            tma_store_commit();
            tma_store_wait_read();
          }
          mbar_arrive(&bar_free_o);
        }
      }
    }
    tma_store_wait_all();
  } else if (tid < kScanEpilogueThreads) {
    // ---- the state and the epilogues ---------------------------------------------------------------------------------
    // the gates of chunk c by cp.async (the tiles come from the copy warp)
    auto prefetch_gates = [&](int c, int stage, int start, int len) {
      const int t = tid - 64;
      if (kda) {
        if (t >= 0 && t < 128) cp_async4(smem_u32(s_g2 + stage * 128 + t), gl2 + (int64_t(c) * num_v_heads + hv) * kDim + t);
      } else if (t >= 0 && t < 64) {
        cp_async4(smem_u32(s_g2 + stage * 128 + t), g_cs + int64_t(start + (t < len ? t : len - 1)) * num_v_heads + hv);
      }
      cp_async_commit();
    };
    int start = 0, len = 0;
    if (c_begin < c_end) {
      start = chunk_start[c_begin], len = chunk_len[c_begin];
      prefetch_gates(c_begin, 0, start, len);
    }

    // fp32 state: 64 columns of row krow
    float h[64];
    if (transfer) {
#pragma unroll
      for (int j = 0; j < 64; ++j) h[j] = (krow == half * 64 + j) ? 1.f : 0.f;
    } else if (h0 != nullptr && state_row >= 0) {
      const float4* src = reinterpret_cast<const float4*>(
          h0 + ((int64_t(state_row) * num_v_heads + hv) * kDim + krow) * kDim + half * 64);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float4 t = __ldg(src + j);
        h[4 * j] = t.x, h[4 * j + 1] = t.y, h[4 * j + 2] = t.z, h[4 * j + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 64; ++j) h[j] = 0.f;
    }
    // this thread's piece of a [64 x 128] lane-split accumulator: row out_row, logical columns out_col .. + 32
    const int out_row = quad * 16 + (lane & 15), out_col = (lane >> 4) * 64 + half * 32;

    // the fused output of the previous chunk: its products were committed on bar_o a step ago
    uint32_t phase_o = 0;
    struct Rows {
      int start, len;
      float qs;
    } cur = {0, 0, 0.f}, prev = {0, 0, 0.f};  // of the chunk the walk is at / of the one before it
    // in two parts (16 of this thread's 32 columns each), one per wait of the step: a part is about as long as the
    // wait it fills
    // Inside the walk a full chunk's output goes to a shared tile that the copy warp stores as one box (a thread's
    // own stores would touch a line per lane); a ragged chunk's rows, and the walk's last chunk, go out by hand.
    bool alive = true;
    uint32_t tiles_out = 0;  // output tiles handed to the copy warp so far
    auto write_output = [&](int c_prev, int part, const Rows& rows, bool in_walk) {
      if (part == 0) {
        if (!abort.wait(&bar_o, phase_o)) alive = false;
        phase_o ^= 1;
        tc_fence_after();
        // the store of the tile before this one has read it
        if (alive && in_walk && tiles_out > 0 && !abort.wait(&bar_free_o, (tiles_out - 1) & 1u)) alive = false;
      }
      if (!alive) return;
      const uint32_t set = kColO + uint32_t((c_prev - c_begin) & 1) * 128;
      float a[16], b[16];
      tmem_ld16(tmem_addr(tmem, warp, set + half * 32 + part * 16), a);
      tmem_ld16(tmem_addr(tmem, warp, set + 64 + half * 32 + part * 16), b);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) a[j] = fmaf(rows.qs, a[j], b[j]);
      if (in_walk && rows.len == kChunk) {
        set_tile_chunk(sm + FwdHSmem::kO, 8192, out_row, (out_col >> 3) + part * 2, pack8(a));
        set_tile_chunk(sm + FwdHSmem::kO, 8192, out_row, (out_col >> 3) + part * 2 + 1, pack8(a + 8));
      } else if (out_row < rows.len) {
        __nv_bfloat16* dst = o + int64_t(rows.start + out_row) * v_stride + hv * kDim + out_col + part * 16;
        reinterpret_cast<uint4*>(dst)[0] = pack8(a);
        reinterpret_cast<uint4*>(dst)[1] = pack8(a + 8);
      }
      if (in_walk && part == 1) {
        fence_async_smem();
        mbar_arrive(&bar_out);
        ++tiles_out;
      }
    };

    for (int c = c_begin; c < c_end && alive; ++c) {
      const uint32_t step = uint32_t(c - c_begin), par = step & 1u;
      const int stage = int(par);
      // the next chunk's extent: requested now, needed when its gates are (nothing on the step's path waits for it)
      int next_start = 0, next_len = 0;
      if (c + 1 < c_end) next_start = chunk_start[c + 1], next_len = chunk_len[c + 1];
      uint8_t* st = sm + stage * FwdHSmem::kStage;
      // A. h_tape = bf16(h): this thread's half row -> shared (block `half`)
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) set_tile_chunk(sm + FwdHSmem::kH, 16384, krow, half * 8 + cc, pack8(h + 8 * cc));
      cp_async_wait_all();  // this chunk's gates have landed (issued one step ago) ...
      if (!abort.wait(&bar_load[stage], (step >> 1) & 1u)) break;  // ... and so have its tiles
      if (len < kChunk) {  // a ragged chunk's boxes reach into the next sequence: clear those rows
        clear_tile_rows<kScanEpilogueThreads>(st + FwdHSmem::kW, len, tid);
        clear_tile_rows<kScanEpilogueThreads>(st + FwdHSmem::kK, len, tid);
        clear_tile_rows<kScanEpilogueThreads>(st + FwdHSmem::kU, len, tid);
        if (fused) clear_tile_rows<kScanEpilogueThreads>(st + FwdHSmem::kQ, len, tid);
      }
      if (transfer) clear_tile_rows<kScanEpilogueThreads>(st + FwdHSmem::kU, 0, tid);  // the homogeneous recurrence: u = 0
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&bar_h);
      // while the first product runs: the previous chunk's output, the next chunk's gates
      if (fused && step > 0) write_output(c - 1, 0, cur, true);  // `cur` still describes chunk c - 1 here
      if (c + 1 < c_end) prefetch_gates(c + 1, stage ^ 1, next_start, next_len);
      // every epilogue thread's writes of this step (cleared rows, gates) are visible past the barrier they all
      // arrived on
      if (!alive || !abort.wait(&bar_h, par)) break;
      // what B needs besides the product, read while the product runs: this thread's piece of u and the gates' factors
      const float* g2 = s_g2 + stage * 128;
      const float g_last = kda ? g2[krow] : g2[len - 1];  // KDA: this thread's key channel
      // row i = 16 quad + lane % 16; logical V columns (lane / 16) * 64 + half * 32 .. + 32
      const int i = quad * 16 + (lane & 15);
      const int lcol = (lane >> 4) * 64 + half * 32;
      const bool live = i < len;
      const bool by_hand = tapes && len < kChunk;  // a ragged chunk: no 64-row box may be stored
      const float rs = live ? (kda ? 1.f : fast_exp2(g_last - g2[i])) : 0.f;
      const float qs_next = kda ? scale : scale * fast_exp2(g2[i]);
      const float gamma = fast_exp2(g_last);
      uint4 uraw[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) uraw[jj] = tile_chunk(st + FwdHSmem::kU, 8192, i, (lcol >> 3) + jj);
      // B. v_new = u - D1; vs = bf16(rowscale v_new)  (the previous step's tape store has read the v_new tile)
      if (tapes && step > 0 && !abort.wait(&bar_free_vn, par ^ 1u)) break;
      // The copy warp is past its wait for a free stage.  Asked before the arrival that releases the step's second
      // group of products: the barrier that the copy warp waits on therefore cannot complete twice behind its back.
      if (!abort.wait(&bar_seen, par)) break;
      if (!abort.wait(&bar_d1, par)) break;
      tc_fence_after();
      {
        __nv_bfloat16* vrow = v_new + int64_t(start + i) * v_stride + hv * kDim + lcol;
        float d[32];
        tmem_ld32_halves(tmem_addr(tmem, warp, half * 32), d);
        tmem_ld_wait();
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          float uv[8], vs[8];
          unpack8(uraw[jj], uv);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            uv[e] = live ? uv[e] - d[jj * 8 + e] : 0.f;
            vs[e] = rs * uv[e];
          }
          const uint4 packed = pack8(uv);
          if (by_hand && live) reinterpret_cast<uint4*>(vrow)[jj] = packed;
          set_tile_chunk(sm + FwdHSmem::kVS, 8192, i, (lcol >> 3) + jj, pack8(vs));
          if (tapes) set_tile_chunk(sm + FwdHSmem::kVN, 8192, i, (lcol >> 3) + jj, packed);
        }
        if (fused) {  // what the output's epilogue needs one step from now
          prev = cur;
          cur = {start, len, qs_next};
        }
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&bar_vs);
      if (fused && step > 0) write_output(c - 1, 1, prev, true);
      // this step's tape store has read the state tile (long ago: asked here, off the path to the next step's A)
      if (tapes && !abort.wait(&bar_free_h, par)) break;
      if (!abort.wait(&bar_d2, par)) break;
      tc_fence_after();

      // C. h = gamma h + D2
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        float d[32];
        tmem_ld32(tmem_addr(tmem, warp, 128 + half * 64 + p * 32), d);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) h[p * 32 + j] = fmaf(gamma, h[p * 32 + j], d[j]);
      }
      tc_fence_before();
      start = next_start, len = next_len;
    }
    if (fused && c_end > c_begin && alive && !abort.raised()) {
      write_output(c_end - 1, 0, cur, false);
      write_output(c_end - 1, 1, cur, false);
    }
    cp_async_wait_all();

    float* out_state = prescan ? plan.summary + ((int64_t(n) * num_v_heads + hv) * 2 + (transfer ? 1 : 0)) * kDim * kDim
                               : (final_state ? final_state + (int64_t(n) * num_v_heads + hv) * kDim * kDim : nullptr);
    if (out_state != nullptr && alive && !abort.raised()) {
      float4* dst = reinterpret_cast<float4*>(out_state + krow * kDim + half * 64);
#pragma unroll
      for (int j = 0; j < 16; ++j) dst[j] = make_float4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
    }
  }
  if (abort.raised()) {  // copies may still be in flight: give them time to land before the CTA's memory goes
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 100000ull) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (abort.raised() && tid == 0) atomicExch(status, kDevWaitTimeout | (2 << 8));
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------------------------------------------
// fwd_o
// ---------------------------------------------------------------------------------------------------------------
struct FwdOSmem {
  static constexpr uint32_t kQ = 0;               // [64][128] q
  static constexpr uint32_t kVN = 16384;          // [64][128] v_new
  static constexpr uint32_t kH = 32768;           // [128][128] h_tape
  static constexpr uint32_t kAqk = kH + 32768;    // [64][64]
  static constexpr uint32_t kG = kAqk + 8192;
  static constexpr uint32_t kBytes = kG + 256;
};

struct FwdOMaps {
  CUtensorMap q, v_new;  // rows, box 64 x 64
  CUtensorMap h;         // tiles [num_tiles * 128, 128], box 64 x 128
  CUtensorMap aqk;       // tiles [num_tiles * 64, 64], box 64 x 64
};

__global__ void __launch_bounds__(128) gdn_fwd_o_kernel(
    const __grid_constant__ FwdOMaps maps, const float* __restrict__ g_cs, __nv_bfloat16* __restrict__ o,
    const int32_t* __restrict__ chunk_start, const int32_t* __restrict__ chunk_len, int num_qk_heads, int num_v_heads,
    float scale, int32_t* __restrict__ status) {
  extern __shared__ uint8_t raw[];
  __shared__ uint64_t bar, bar_load;
  __shared__ uint32_t tmem_slot;
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, hv = blockIdx.y, hq = hv / (num_v_heads / num_qk_heads);
  const int start = chunk_start[c], len = chunk_len[c];
  if (len <= 0) return;  // a pad chunk of a device-built table
  float* s_g2 = reinterpret_cast<float*>(sm + FwdOSmem::kG);

  const int64_t v_stride = int64_t(num_v_heads) * kDim;
  const int64_t tile = int64_t(c) * num_v_heads + hv;
  const uint32_t sbase = smem_u32(sm);
  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_init(&bar_load, 1);
    fence_mbar_init();
    mbar_arrive_expect(&bar_load, 2 * 16384 + 32768 + 8192);
    tma_load_tile128(sbase + FwdOSmem::kQ, 8192, &maps.q, hq * kDim, start, &bar_load);
    tma_load_tile128(sbase + FwdOSmem::kVN, 8192, &maps.v_new, hv * kDim, start, &bar_load);
    tma_load_tile128(sbase + FwdOSmem::kH, 16384, &maps.h, 0, int(tile * 128), &bar_load);
    tma_load_box(sbase + FwdOSmem::kAqk, &maps.aqk, 0, int(tile * 64), &bar_load);
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 128);
  // g_cs == nullptr: the per-channel-decay variant, whose q operand already holds q 2^G (qscale = scale)
  if (tid < 64) s_g2[tid] = g_cs ? g_cs[int64_t(start + (tid < len ? tid : len - 1)) * num_v_heads + hv] : 0.f;
  __syncthreads();  // the barrier's initialisation is visible to every waiter
  const bool landed = __all_sync(0xffffffffu, mbar_wait(&bar_load, 0));
  if (len < kChunk) {  // a ragged chunk's boxes reach into the next sequence: clear those rows
    clear_tile_rows<128>(sm + FwdOSmem::kQ, len, tid);
    clear_tile_rows<128>(sm + FwdOSmem::kVN, len, tid);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  if (tid == 0) {
    const Operand op_q{sbase + FwdOSmem::kQ, 8192}, op_vn{sbase + FwdOSmem::kVN, 8192};
    const Operand op_h{sbase + FwdOSmem::kH, 16384}, op_a{sbase + FwdOSmem::kAqk, 8192};
    // both [64 x 128] products as two N = 64 halves: V columns 0..63 -> lanes 0..15, 64..127 -> lanes 16..31
    umma_gemm<64, 64>(tmem, op_q, false, op_h, true, 128, false);
    umma_gemm<64, 64>(tmem + (16u << 16), op_q, false, operand_at(op_h, 0, 1), true, 128, false);
    umma_gemm<64, 64>(tmem + 64, op_a, false, op_vn, true, 64, false);
    umma_gemm<64, 64>(tmem + 64 + (16u << 16), op_a, false, operand_at(op_vn, 0, 1), true, 64, false);
    umma_commit(&bar);
  }
  const bool ok = __all_sync(0xffffffffu, mbar_wait(&bar, 0)) && landed;
  tc_fence_after();
  if (ok) {
    const int i = warp * 16 + (lane & 15);
    const bool live = i < len;
    const float qs = scale * fast_exp2(s_g2[i]);
    __nv_bfloat16* dst = o + int64_t(start + i) * v_stride + hv * kDim + (lane >> 4) * 64;
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      float a[32], b[32];
      tmem_ld32(tmem_addr(tmem, warp, p * 32), a);
      tmem_ld32(tmem_addr(tmem, warp, 64 + p * 32), b);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) a[j] = fmaf(qs, a[j], b[j]);
      if (live) {
#pragma unroll
        for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(dst + p * 32)[j] = pack8(a + 8 * j);
      }
    }
  }
  if (!ok && tid == 0) atomicExch(status, kDevWaitTimeout | (3 << 8));
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 128);
}

}  // namespace mek

// ---------------------------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------------------------
namespace {

int check_dims(const MekGdnDims* d, const char* what) {
  using namespace mek;
  if (d == nullptr) return fail(MEK_ERR_INVALID, "%s: dims is null", what);
  if (d->total_tokens <= 0 || d->num_chunks <= 0 || d->num_seqs <= 0)
    return fail(MEK_ERR_INVALID, "%s: no tokens (total_tokens=%lld, num_chunks=%d, num_seqs=%d)", what,
                (long long)d->total_tokens, d->num_chunks, d->num_seqs);
  if (d->num_qk_heads <= 0 || d->num_v_heads <= 0 || d->num_v_heads % d->num_qk_heads != 0)
    return fail(MEK_ERR_INVALID, "%s: the value heads (HV=%d) must be a positive multiple of the q / k heads (H=%d)",
                what, d->num_v_heads, d->num_qk_heads);
  if (d->head_dim != 128) return fail(MEK_ERR_UNSUPPORTED, "%s: head dims must be 128, not %d", what, d->head_dim);
  if (d->num_v_heads > 65535 || d->num_seqs > 65535)
    return fail(MEK_ERR_INVALID, "%s: more than 65535 value heads or sequences", what);
  if (!d->chunk_start || !d->chunk_len || !d->seq_chunk_start)
    return fail(MEK_ERR_INVALID, "%s: a chunk table pointer is null", what);
  return MEK_OK;
}

}  // namespace

extern "C" {

int mek_gdn_l2norm(const void* x, void* y, float* rstd, int64_t rows, int heads, int64_t x_pitch, void* stream) {
  using namespace mek;
  if (rows <= 0 || heads <= 0 || !x || !y || !rstd)
    return fail(MEK_ERR_INVALID, "l2norm: rows=%lld, heads=%d or a null pointer", (long long)rows, heads);
  const int64_t pitch = x_pitch != 0 ? x_pitch : int64_t(heads) * kDim;
  if (pitch < int64_t(heads) * kDim || pitch % 8 != 0 || reinterpret_cast<uintptr_t>(x) % 16 != 0)
    return fail(MEK_ERR_INVALID, "l2norm: x_pitch %lld does not hold %d heads of 128 in 16-byte pieces", (long long)x_pitch,
                heads);
  l2norm_kernel<<<unsigned((rows + 31) / 32), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), rstd, rows, heads, pitch);
  return launched("l2norm");
}

int mek_gdn_gate_cumsum(const MekGdnDims* d, const float* g, float* g_cs, void* stream) {
  using namespace mek;
  if (int rc = check_dims(d, "gate_cumsum")) return rc;
  const int threads = d->num_v_heads <= 32 ? 32 : (d->num_v_heads <= 64 ? 64 : 128);
  gate_cumsum_kernel<<<d->num_chunks, threads, 0, static_cast<cudaStream_t>(stream)>>>(g, g_cs, d->chunk_start,
                                                                                    d->chunk_len, d->num_v_heads);
  return launched("gate_cumsum");
}

int mek_gdn_wy_fwd(const MekGdnDims* d, const void* q, const void* k, const void* v, const float* beta,
                   const float* g_cs, void* a_out, void* aqk_out, void* w_out, void* u_out, int32_t* status,
                   void* stream) {
  using namespace mek;
  if (int rc = check_dims(d, "wy_fwd")) return rc;
  const size_t smem = WySmem::kBytes + 1024;
  if (int rc = want_smem(gdn_wy_kernel, smem, "wy_fwd")) return rc;
  WyMaps maps;
  if (int rc = make_rows_map(&maps.q, q, d->total_tokens, d->num_qk_heads, "wy_fwd", d->qk_pitch)) return rc;
  if (int rc = make_rows_map(&maps.k, k, d->total_tokens, d->num_qk_heads, "wy_fwd", d->qk_pitch)) return rc;
  if (int rc = make_rows_map(&maps.v, v, d->total_tokens, d->num_v_heads, "wy_fwd", d->v_pitch)) return rc;
  if (int rc = make_rows_map(&maps.w_out, w_out, d->total_tokens, d->num_v_heads, "wy_fwd")) return rc;
  if (int rc = make_rows_map(&maps.u_out, u_out, d->total_tokens, d->num_v_heads, "wy_fwd")) return rc;
  gdn_wy_kernel<<<dim3(d->num_chunks, d->num_v_heads), 128, smem, static_cast<cudaStream_t>(stream)>>>(
      maps, beta, g_cs, static_cast<__nv_bfloat16*>(a_out), static_cast<__nv_bfloat16*>(aqk_out),
      static_cast<__nv_bfloat16*>(w_out), static_cast<__nv_bfloat16*>(u_out), d->chunk_start, d->chunk_len,
      d->num_qk_heads, d->num_v_heads, d->scale, status);
  return launched("wy_fwd");
}

namespace {
struct FusedOutput {
  const void* q;
  const void* aqk;
  void* o;
};

int launch_fwd_h(const MekGdnDims* d, const void* k, const void* w, const void* u, const float* g_cs, const float* h0,
                 void* h_tape, void* v_new, float* final_state, const float* gl2, const mek::ScanPlan& plan,
                 const FusedOutput& fused, int32_t* status, void* stream, const char* what) {
  using namespace mek;
  const size_t smem = FwdHSmem::kBytes + 1024;
  if (int rc = want_smem(gdn_fwd_h_kernel, smem, what)) return rc;
  FwdHMaps maps;
  if (int rc = make_rows_map(&maps.k, k, d->total_tokens, d->num_qk_heads, what, d->qk_pitch)) return rc;
  if (int rc = make_rows_map(&maps.w, w, d->total_tokens, d->num_v_heads, what)) return rc;
  if (int rc = make_rows_map(&maps.u, u, d->total_tokens, d->num_v_heads, what)) return rc;
  if (fused.o != nullptr) {
    if (int rc = make_rows_map(&maps.q, fused.q, d->total_tokens, d->num_qk_heads, what, d->qk_pitch)) return rc;
    if (int rc = make_tiles_map(&maps.aqk, fused.aqk, int64_t(d->num_chunks) * d->num_v_heads, 64, 64, what))
      return rc;
    if (int rc = make_rows_map(&maps.o_out, fused.o, d->total_tokens, d->num_v_heads, what)) return rc;
  } else {
    maps.q = maps.k;  // never read
    maps.aqk = maps.k;
    maps.o_out = maps.k;
  }
  if (plan.seg_flags == nullptr) {  // an ordinary walk writes the two tapes
    if (!h_tape || !v_new) return fail(MEK_ERR_INVALID, "%s: h_tape or v_new is null", what);
    if (int rc = make_tiles_map(&maps.h_out, h_tape, int64_t(d->num_chunks) * d->num_v_heads, 128, 128, what)) return rc;
    if (int rc = make_rows_map(&maps.v_new_out, v_new, d->total_tokens, d->num_v_heads, what)) return rc;
  } else {
    maps.h_out = maps.k;  // a pre-scan writes no tape
    maps.v_new_out = maps.k;
  }
  if (d->num_seqs > 65535)
    return fail(MEK_ERR_UNSUPPORTED, "%s: at most 65,535 sequences (or scan segments) per call, got %d", what,
                d->num_seqs);
  const dim3 grid(d->num_v_heads, d->num_seqs, plan.seg_flags != nullptr ? 2 : 1);
  ScanPlan ordered = plan;
  ordered.seq_order = d->seq_order;
  gdn_fwd_h_kernel<<<grid, kScanThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      maps, g_cs, h0, static_cast<__nv_bfloat16*>(v_new), final_state,
      d->chunk_start, d->chunk_len, d->seq_chunk_start, d->num_qk_heads, d->num_v_heads, gl2, ordered,
      static_cast<__nv_bfloat16*>(fused.o), d->scale, status);
  return launched(what);
}
const mek::ScanPlan kNoPlan = {nullptr, nullptr, nullptr, 0, 0.f};
const FusedOutput kNoOutput = {nullptr, nullptr, nullptr};
}  // namespace

int mek_gdn_fwd_h(const MekGdnDims* d, const void* k, const void* w, const void* u, const float* g_cs, const float* h0,
                  void* h_tape, void* v_new, float* final_state, int32_t* status, void* stream) {
  if (int rc = check_dims(d, "fwd_h")) return rc;
  return launch_fwd_h(d, k, w, u, g_cs, h0, h_tape, v_new, final_state, nullptr, kNoPlan, kNoOutput, status, stream,
                      "fwd_h");
}

int mek_gdn_fwd_ho(const MekGdnDims* d, const void* q, const void* k, const void* w, const void* u, const void* aqk,
                   const float* g_cs, const float* h0, void* h_tape, void* v_new, void* o, float* final_state,
                   int32_t* status, void* stream) {
  using namespace mek;
  if (int rc = check_dims(d, "fwd_ho")) return rc;
  if (!q || !aqk || !o) return fail(MEK_ERR_INVALID, "fwd_ho: q, aqk or o is null");
  const FusedOutput fused = {q, aqk, o};
  return launch_fwd_h(d, k, w, u, g_cs, h0, h_tape, v_new, final_state, nullptr, kNoPlan, fused, status, stream,
                      "fwd_ho");
}

int mek_gdn_fwd_h_prescan(const MekGdnDims* d, const void* k, const void* w, const void* u, const float* g_cs,
                          const float* boundary, const int32_t* seg_flags, const int32_t* state_row, int warm_chunks,
                          float warm_log2, float* summary, int32_t* status, void* stream) {
  using namespace mek;
  if (int rc = check_dims(d, "fwd_h_prescan")) return rc;
  if (!seg_flags || !state_row || !summary || warm_chunks < 0)
    return fail(MEK_ERR_INVALID, "fwd_h_prescan: a null table or summary, or negative warm_chunks");
  const ScanPlan plan = {seg_flags, state_row, summary, warm_chunks, warm_log2};
  return launch_fwd_h(d, k, w, u, g_cs, boundary, nullptr, nullptr, nullptr, nullptr, plan, kNoOutput, status, stream,
                      "fwd_h_prescan");
}

int mek_kda_fwd_h(const MekGdnDims* d, const void* kr, const void* w, const void* u, const float* gl2, const float* h0,
                  void* h_tape, void* v_new, float* final_state, int32_t* status, void* stream) {
  using namespace mek;
  if (int rc = check_dims(d, "kda_fwd_h")) return rc;
  if (d->num_qk_heads != d->num_v_heads) return fail(MEK_ERR_INVALID, "kda_fwd_h: KDA has one value head per key head");
  if (gl2 == nullptr) return fail(MEK_ERR_INVALID, "kda_fwd_h: gl2 is null");
  return launch_fwd_h(d, kr, w, u, nullptr, h0, h_tape, v_new, final_state, gl2, kNoPlan, kNoOutput, status, stream,
                      "kda_fwd_h");
}

// The per-channel-decay variant's pre-scan over the segments of a plan (no warm-up rule: it reads scalar gates).
int mek_kda_fwd_h_prescan(const MekGdnDims* d, const void* kr, const void* w, const void* u, const float* gl2,
                          const float* boundary, const int32_t* seg_flags, const int32_t* state_row, float* summary,
                          int32_t* status, void* stream) {
  using namespace mek;
  if (int rc = check_dims(d, "kda_fwd_h_prescan")) return rc;
  if (d->num_qk_heads != d->num_v_heads)
    return fail(MEK_ERR_INVALID, "kda_fwd_h_prescan: KDA has one value head per key head");
  if (!gl2 || !seg_flags || !state_row || !summary)
    return fail(MEK_ERR_INVALID, "kda_fwd_h_prescan: gl2, a table or the summary is null");
  const ScanPlan plan = {seg_flags, state_row, summary, 0, 0.f};
  return launch_fwd_h(d, kr, w, u, nullptr, boundary, nullptr, nullptr, nullptr, gl2, plan, kNoOutput, status, stream,
                      "kda_fwd_h_prescan");
}

int mek_gdn_fwd_o(const MekGdnDims* d, const void* q, const void* aqk, const void* v_new, const void* h_tape,
                  const float* g_cs, void* o, int32_t* status, void* stream) {
  using namespace mek;
  if (int rc = check_dims(d, "fwd_o")) return rc;
  const size_t smem = FwdOSmem::kBytes + 1024;
  if (int rc = want_smem(gdn_fwd_o_kernel, smem, "fwd_o")) return rc;
  const int64_t tiles = int64_t(d->num_chunks) * d->num_v_heads;
  FwdOMaps maps;
  if (int rc = make_rows_map(&maps.q, q, d->total_tokens, d->num_qk_heads, "fwd_o", d->qk_pitch)) return rc;
  if (int rc = make_rows_map(&maps.v_new, v_new, d->total_tokens, d->num_v_heads, "fwd_o")) return rc;
  if (int rc = make_tiles_map(&maps.h, h_tape, tiles, 128, 128, "fwd_o")) return rc;
  if (int rc = make_tiles_map(&maps.aqk, aqk, tiles, 64, 64, "fwd_o")) return rc;
  gdn_fwd_o_kernel<<<dim3(d->num_chunks, d->num_v_heads), 128, smem, static_cast<cudaStream_t>(stream)>>>(
      maps, g_cs, static_cast<__nv_bfloat16*>(o), d->chunk_start, d->chunk_len, d->num_qk_heads, d->num_v_heads,
      d->scale, status);
  return launched("fwd_o");
}

int mek_kda_fwd_o(const MekGdnDims* d, const void* qg, const void* aqk, const void* v_new, const void* h_tape, void* o,
                  int32_t* status, void* stream) {
  return mek_gdn_fwd_o(d, qg, aqk, v_new, h_tape, nullptr, o, status, stream);
}

}  // extern "C"
