// Gradient tail of the chunked gated delta rule, sm_100a: one CTA per (chunk, key head) walks the value heads of
// the key head's group and writes dq, dk (one rounding of the fp32 group sum, after the L2 norm's pull-back when the
// op normalised), dv, dbeta and dg (in-chunk suffix sum included).  It fuses what the reference runs as three
// launches -- dqkwg, wy_bwd, finalize (reference: miles_ext_kernels/cake/_impl/gdn/ops.py:1642-1727) -- so the
// per-value-head partials dq_hv, dk_hv, dw, dk2, dg1, dg2 never reach global memory.
//
// Arithmetic per (chunk, value head) follows the reference's program #8 and #9 (reference:
// miles_ext_kernels/cake/_vendor/cake_gdn_det_train_kcp/cake_fake_backend.py:458-587, 630-640):
//   dAqk = tril(do v_new^T); dS = bf16(scale dAqk D);           D_ij = 2^{G_i - G_j}, j <= i
//   dq  += dS k + do_g h^T;  dk += dS^T q + rowscale (v_new dh^T)
//   dw   = bf16(-dv_new h^T); dkb = A^T dw; dvb = A^T dv_new;  dv = bf16(beta dvb)
//   dk  += beta 2^G dkb;  dL = bf16(-tril(A^T dA A^T, -1)) with dA = dw kb^T + dv_new vb^T, evaluated as
//          A^T dA A^T = dkb (A kb)^T + dvb (A vb)^T = bf16(dkb) w^T + bf16(dvb) u^T   (w, u: the forward's tapes)
//   dk  += bf16(beta dL D) k + bf16(beta dL D)^T k
//   dbeta, dg: row sums of the products above; the chunk-end term gamma sum(dh h) + sum(dkh k) lands on the chunk's
//   last token before the suffix sum.
// Every reduction has a fixed order; no atomics.
#include "common.cuh"
#include "tiles.cuh"
#include "tma.cuh"

namespace mek {

struct TailSmem {
  static constexpr uint32_t kQK = 0;                   // 2 x {[64][128] q, [64][128] k}: one buffer per (chunk, key head)
  static constexpr uint32_t kQKStride = 32768;
  static constexpr uint32_t kH = 2 * kQKStride;        // [128][128] h_tape; after phase A: dw at +0, dv at +16384
  static constexpr uint32_t kDH = kH + 32768;          // [128][128] dh_tape
  static constexpr uint32_t kDO = kDH + 32768;         // [64][128] do; after phase A: u
  static constexpr uint32_t kVN = kDO + 16384;         // [64][128] v_new; after phase A: w
  static constexpr uint32_t kDVN = kVN + 16384;        // [64][128] dv_new; after phase A: bf16(dkb)
  static constexpr uint32_t kV = kDVN + 16384;         // [64][128] v; after phase A: bf16(dvb)
  static constexpr uint32_t kA = kV + 16384;           // [64][64] A
  static constexpr uint32_t kAqk = kA + 8192;          // [64][64] Aqk
  static constexpr uint32_t kB8 = kAqk + 8192;         // [64][64] dS, then bf16(beta dL D)
  static constexpr uint32_t kScal = kB8 + 8192;        // floats: beta[2][64], g2[2][64], cs[2][4][64], red[8][64],
                                                       //         red2[8][64], warp[16 + 1], rs[2][4][64]
  static constexpr uint32_t kBytes = kScal + (2 * 64 * 2 + 2 * 4 * 64 + 16 * 64 + 32 + 2 * 4 * 64) * 4;
};

// Threads: kTailGroups warpgroups.  Warps w, w + 4, ... share the accumulator rows 16 (w % 4) .. + 15; a thread owns
// kTailW columns of its row in every 128-wide accumulator.  The 64-wide ones (dAqk, Y, k k^T: lanes 0..15 of a
// quadrant) are read in the 16-lane fragment shape instead, so that all 32 threads of a warp share their elements.
constexpr int kTailThreads = 512;
constexpr int kTailGroups = kTailThreads / 128;  // warpgroups
constexpr int kTailW = 64 / kTailGroups;         // columns of a thread's piece
constexpr int kTailJ = kTailW / 8;               // ... in 16-byte chunks of a tile row
constexpr int kTailPieces = 2 * kTailGroups;     // column pieces of a 128-wide row

__device__ __forceinline__ void tail_tmem_ld(uint32_t taddr, float* v) {
  if constexpr (kTailW == 32) tmem_ld32(taddr, v);
  else tmem_ld16(taddr, v);
}
// the pieces' partial sums of one row, added in a fixed pairwise order
__device__ __forceinline__ float tail_row_sum(const float* pieces, int row) {
  float level[kTailPieces];
#pragma unroll
  for (int i = 0; i < kTailPieces; ++i) level[i] = pieces[i * 64 + row];
#pragma unroll
  for (int n = kTailPieces; n > 1; n >>= 1)
#pragma unroll
    for (int i = 0; i < n / 2; ++i) level[i] = level[2 * i] + level[2 * i + 1];
  return level[0];
}

// Tensor-memory columns.  A [64 x 128] accumulator takes 64 columns: its logical columns 0..63 sit in lanes 0..15 of
// each quadrant and 64..127 in lanes 16..31 (two N = 64 instructions), so every lane of a warp owns a row piece.
// [64 x 64] accumulators (Ta, Tb) are not split: lanes 0..15 only.
constexpr uint32_t kColDQ = 0, kColDK = 64, kColT0 = 128, kColT1 = 192, kColT2 = 256, kColT3 = 320, kColTa = 384,
                   kColTb = 448;
constexpr uint32_t kUpperLanes = 16u << 16;

template <int N>
__device__ __forceinline__ void cp_async_wait_pending() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// One persistent CTA per SM walks (chunk, key head) pairs; inside a pair it walks the value heads of the group.
// Per value head, three waited tensor-core phases:
//   A  (needs only loaded tiles)  dAqk = do v_new^T, dkh = v_new dh^T, dq2 = do h^T, dw = -dv_new h^T, dvb = A^T dv_new
//   B  (needs dS, dw)             dq += dS k, dk += dS^T q, dkb = A^T dw
//   C  (needs dkb, dvb)           Y = bf16(dkb) w^T + bf16(dvb) u^T, KK = k k^T
// and a fourth that nobody waits for until the pair ends: dk += bf16(beta dL D) k + bf16(beta dL D)^T k.
// While one value head computes, the next one's tiles arrive by TMA in the buffers the current one has finished
// with (q / k of the next pair are double-buffered); one elected thread issues every copy, and the copies of an item
// complete on one mbarrier in three instalments (Aqk; the states and A; the row tiles).
struct TailMaps {
  CUtensorMap q, k;                      // rows [tokens, H * 128], box 64 x 64
  CUtensorMap v, d_o, v_new, dv_new, w, u;  // rows [tokens, HV * 128], box 64 x 64
  CUtensorMap h, dh;                     // tiles [num_tiles * 128, 128], box 64 x 128
  CUtensorMap a, aqk;                    // tiles [num_tiles * 64, 64], box 64 x 64
  CUtensorMap dv_out;                    // rows [tokens, HV * 128] of the gradient, box 64 x 64, written
};

__global__ void __launch_bounds__(kTailThreads) gdn_bwd_tail_kernel(
    const __grid_constant__ TailMaps maps, const float* __restrict__ beta, const float* __restrict__ g_cs,
    const __nv_bfloat16* __restrict__ q_raw, const __nv_bfloat16* __restrict__ k_raw,
    const float* __restrict__ rstd_q, const float* __restrict__ rstd_k, __nv_bfloat16* __restrict__ dq,
    __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv, float* __restrict__ dbeta, float* __restrict__ dg,
    const int32_t* __restrict__ chunk_start, const int32_t* __restrict__ chunk_len, int num_chunks, int num_qk_heads,
    int num_v_heads, float scale, int64_t raw_pitch, int64_t dqk_pitch, int64_t dv_pitch,
    int32_t* __restrict__ status) {
  extern __shared__ uint8_t raw[];
  __shared__ uint64_t bar;         // tensor-core commits
  __shared__ uint64_t bar2;        // ... of the second issuing thread
  __shared__ uint64_t bar_first;   // the first product of phase A alone (dAqk): its epilogue starts under the others
  __shared__ uint64_t bar_item;    // the item's tiles: three instalments, one arrival each
  __shared__ uint64_t bar_uw;      // the item's u and w
  __shared__ uint64_t bar_qk[2];   // q and k of a pair, one barrier per buffer
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool loader = tid == 64;   // the thread that issues every copy
  const int group = num_v_heads / num_qk_heads;
  const int num_pairs = num_chunks * num_qk_heads;
  // accumulator rows: warps w, w + 4, ... share the rows 16 (w % 4) .. + 15.  A 128-wide accumulator is split
  // 2 x kTailGroups ways: the lane half picks logical columns 0..63 / 64..127, the warpgroup the kTailW-column piece
  // inside that half.  A 64-wide accumulator lives in lanes 0..15 only and is split by the warpgroup.
  const int quad = warp & 3, ch = warp >> 2, lh = lane >> 4;
  const int row = quad * 16 + (lane & 15);
  const bool owner = lane < 16;            // holds a piece of the 64-wide accumulators
  const int cq = lh * kTailGroups + ch;    // which piece of a 128-wide accumulator
  const int lcol = lh * 64 + ch * kTailW;  // its first logical column
  const int lchunk = lcol >> 3;        // ... as a 16-byte chunk index of a tile row
  // A 64-wide accumulator (lanes 0..15 of each quadrant) is read by the whole warp: the warp (quad, ch) takes its 16
  // rows x 16 columns, a thread the rows fr and fr + 8 at the columns fc + 8 i + {0, 1}.
  const int fr = quad * 16 + (lane >> 2), fq = lane & 3, fc = ch * 16 + fq * 2;

  float* s_beta = reinterpret_cast<float*>(sm + TailSmem::kScal);  // [2][64]
  float* s_g2 = s_beta + 128;                                      // [2][64]
  float* s_cs = s_g2 + 128;                                        // [2][4][64] partial column sums per quadrant
  float* s_red = s_cs + 512;                                       // [kTailPieces][64]
  float* s_red2 = s_red + 512;                                     // [kTailPieces][64]
  float* s_warp = s_red2 + 512;                                    // [warps + 1]
  float* s_rs = s_warp + 32;                                       // [2][4][64] partial row sums per column piece
  Abort abort{&abort_flag};

  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_init(&bar2, 1);
    mbar_init(&bar_first, 1);
    mbar_init(&bar_item, 3);
    mbar_init(&bar_uw, 1);
    mbar_init(&bar_qk[0], 1);
    mbar_init(&bar_qk[1], 1);
    fence_mbar_init();
    abort_flag = 0;
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 512);
  const uint32_t sbase = smem_u32(sm);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  // a pair is live when it exists and its chunk is not a pad chunk of a device-built table (pads come last)
  auto pair_live = [&](int p) { return p < num_pairs && chunk_len[p / num_qk_heads] > 0; };
  // ---- asynchronous loads (issued by the loader thread only; scalars by cp.async from the first 64 threads) -----
  auto load_qk = [&](int p, int buf) {
    const int c = p / num_qk_heads, hq = p % num_qk_heads;
    const uint32_t base = sbase + TailSmem::kQK + buf * TailSmem::kQKStride;
    mbar_arrive_expect(&bar_qk[buf], 2 * 16384);
    tma_load_tile128(base, 8192, &maps.q, hq * kDim, chunk_start[c], &bar_qk[buf]);
    tma_load_tile128(base + 16384, 8192, &maps.k, hq * kDim, chunk_start[c], &bar_qk[buf]);
  };
  struct Item {
    int c, hv, start, len;
    int64_t tile;
  };
  auto item_of = [&](int p, int gi) {
    Item it;
    it.c = p / num_qk_heads;
    it.hv = (p % num_qk_heads) * group + gi;
    it.start = chunk_start[it.c];
    it.len = chunk_len[it.c];
    it.tile = int64_t(it.c) * num_v_heads + it.hv;
    return it;
  };
  auto load_scalars = [&](const Item& it, int buf) {  // every thread calls; the first 64 copy
    if (tid < 64) {
      const int64_t at = int64_t(it.start + (tid < it.len ? tid : it.len - 1)) * num_v_heads + it.hv;
      cp_async4(smem_u32(s_beta + buf * 64 + tid), beta + at);
      cp_async4(smem_u32(s_g2 + buf * 64 + tid), g_cs + at);
    }
    cp_async_commit();
  };
  auto load_rows = [&](uint32_t where, const CUtensorMap* map, const Item& it, uint64_t* on) {
    tma_load_tile128(sbase + where, 8192, map, it.hv * kDim, it.start, on);
  };
  // the three instalments of an item
  auto load_aqk = [&](const Item& it) {
    mbar_arrive_expect(&bar_item, 8192);
    tma_load_box(sbase + TailSmem::kAqk, &maps.aqk, 0, int(it.tile * 64), &bar_item);
  };
  auto load_states = [&](const Item& it) {
    mbar_arrive_expect(&bar_item, 2 * 32768 + 8192);
    tma_load_tile128(sbase + TailSmem::kH, 16384, &maps.h, 0, int(it.tile * 128), &bar_item);
    tma_load_tile128(sbase + TailSmem::kDH, 16384, &maps.dh, 0, int(it.tile * 128), &bar_item);
    tma_load_box(sbase + TailSmem::kA, &maps.a, 0, int(it.tile * 64), &bar_item);
  };
  auto load_row_tiles = [&](const Item& it) {
    mbar_arrive_expect(&bar_item, 4 * 16384);
    load_rows(TailSmem::kDO, &maps.d_o, it, &bar_item);
    load_rows(TailSmem::kVN, &maps.v_new, it, &bar_item);
    load_rows(TailSmem::kDVN, &maps.dv_new, it, &bar_item);
    load_rows(TailSmem::kV, &maps.v, it, &bar_item);
  };
  auto load_uw = [&](const Item& it) {
    mbar_arrive_expect(&bar_uw, 2 * 16384);
    load_rows(TailSmem::kDO, &maps.u, it, &bar_uw);
    load_rows(TailSmem::kVN, &maps.w, it, &bar_uw);
  };

  int pair = blockIdx.x;
  // The chunk-table reads of an item (global memory, two dependent loads) are issued one item ahead and carried in
  // registers: `ahead` is the item the walk takes next, `pair_ahead_live` whether the next pair exists.
  Item ahead = {0, 0, 0, 0, 0};
  bool this_pair_live = pair_live(pair);
  if (this_pair_live) {  // prologue: everything of the first item
    const Item it = item_of(pair, 0);
    ahead = it;
    if (loader) {
      load_qk(pair, 0);
      load_aqk(it);
      load_states(it);
      load_row_tiles(it);
    }
    load_scalars(it, 0);
  }
  const uint32_t tmem = tmem_slot;
  const Operand op_h{sbase + TailSmem::kH, 16384}, op_dh{sbase + TailSmem::kDH, 16384};
  const Operand op_dw{sbase + TailSmem::kH, 8192};
  const Operand op_do{sbase + TailSmem::kDO, 8192}, op_vn{sbase + TailSmem::kVN, 8192};
  const Operand op_u{sbase + TailSmem::kDO, 8192}, op_w{sbase + TailSmem::kVN, 8192};
  const Operand op_dvn{sbase + TailSmem::kDVN, 8192}, op_dkb{sbase + TailSmem::kDVN, 8192};
  const Operand op_dvb{sbase + TailSmem::kV, 8192};
  const Operand op_a{sbase + TailSmem::kA, 8192}, op_b8{sbase + TailSmem::kB8, 8192};

  uint32_t phase = 0;
  auto mma_wait = [&]() {
    if (!mbar_wait(&bar, phase)) abort.raise();
    phase ^= 1;
    tc_fence_after();
  };
  // Two threads of different warps issue each phase's products (independent accumulators): one thread's
  // instructions go out every ~52 cycles, the tensor core takes ~40 for these shapes.
  uint32_t phase2 = 0;
  auto mma_wait2 = [&]() {
    if (!mbar_wait(&bar2, phase2)) abort.raise();
    phase2 ^= 1;
    mma_wait();
  };
  const bool issuer = tid == 0, issuer2 = tid == 32;
  auto stage_sync = [&]() {
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  };
  // D[64 x 128] (+)= A B as two chains of N = 64 instructions, alternating: logical columns 0..63 -> lanes 0..15,
  // 64..127 -> lanes 16..31
  auto gemm128 = [&](uint32_t col, const Operand& a, bool a_mn, const Operand& b, bool b_mn, uint32_t kdim,
                     bool accumulate, bool neg_a = false) {
    const Operand b_hi = b_mn ? operand_at(b, 0, 1) : operand_at(b, 64, 0);
    umma_gemm_pair<64, 64>(tmem + col, a, a_mn, b, b_mn, kdim, accumulate, neg_a, tmem + col + kUpperLanes, a, a_mn,
                           b_hi, b_mn, kdim, accumulate, neg_a);
  };
  // Row and column sums of a [64 x 64] matrix held as fragments.  rows[0], rows[1]: this thread's part of the rows
  // fr, fr + 8 -> the piece's row sums (four lanes share a row); cols[4]: its part of four columns, both rows added
  // -> the quadrant's column sums (eight lanes share a column).  Fixed order.
  auto publish_fragment_rows = [&](float lo, float hi, float* where) {
    lo += __shfl_xor_sync(0xffffffffu, lo, 1);
    hi += __shfl_xor_sync(0xffffffffu, hi, 1);
    lo += __shfl_xor_sync(0xffffffffu, lo, 2);
    hi += __shfl_xor_sync(0xffffffffu, hi, 2);
    if (fq == 0) {
      where[ch * 64 + fr] = lo;
      where[ch * 64 + fr + 8] = hi;
    }
  };
  auto publish_fragment_columns = [&](float* cols, float* where) {
#pragma unroll
    for (int m = 4; m <= 16; m <<= 1)
#pragma unroll
      for (int j = 0; j < 4; ++j) cols[j] += __shfl_xor_sync(0xffffffffu, cols[j], m);
    if (lane < 4) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        where[quad * 64 + fc + 8 * i] = cols[2 * i];
        where[quad * 64 + fc + 8 * i + 1] = cols[2 * i + 1];
      }
    }
  };
  auto four = [](const float* p, int row) { return (p[row] + p[64 + row]) + (p[128 + row] + p[192 + row]); };

  // scaled terms of this thread's (row, column piece) that cannot accumulate in tensor memory, summed over the
  // group: dq gets qscale (do h^T); dk gets rowscale (v_new dh^T) and beta 2^G dkb
  float dq_reg[kTailW], dk_reg[kTailW];
  int item_parity = 0, qk_buf = 0, pairs_done = 0;
  bool aborted = false;
  bool next_pair_live = pair_live(pair + int(gridDim.x)), pair_after_live = false;
  for (; this_pair_live && !aborted; pair += gridDim.x, qk_buf ^= 1, ++pairs_done, this_pair_live = next_pair_live,
                                      next_pair_live = pair_after_live) {
    const int hq = pair % num_qk_heads;
    const uint32_t qk_base = sbase + TailSmem::kQK + qk_buf * TailSmem::kQKStride;
    uint8_t* q_tile = sm + TailSmem::kQK + qk_buf * TailSmem::kQKStride;
    uint8_t* k_tile = q_tile + 16384;
    const Operand op_q{qk_base, 8192}, op_k{qk_base + 16384, 8192};
    const int next_pair = pair + gridDim.x;
    const bool has_next_pair = next_pair_live;
    pair_after_live = pair_live(next_pair + int(gridDim.x));  // read now, needed when this pair is done
#pragma unroll
    for (int j = 0; j < kTailW; ++j) dq_reg[j] = dk_reg[j] = 0.f;

    for (int gi = 0; gi < group; ++gi, item_parity ^= 1) {
      const Item it = ahead;
      const int start = it.start, len = it.len, hv = it.hv;
      const bool live = row < len;
      const bool last_of_pair = gi + 1 == group;
      const bool has_next = !last_of_pair || has_next_pair;
      const Item nx = has_next ? (last_of_pair ? item_of(next_pair, 0) : item_of(pair, gi + 1)) : it;
      ahead = nx;
      const float* beta_s = s_beta + item_parity * 64;
      const float* g2 = s_g2 + item_parity * 64;

      // this item's tiles (issued while the previous item computed) have landed
      cp_async_wait_pending<0>();
      if (!mbar_wait(&bar_item, item_parity)) abort.raise();
      if (gi == 0 && !mbar_wait(&bar_qk[qk_buf], (pairs_done >> 1) & 1)) abort.raise();
      if (len < kChunk) {  // a ragged chunk's boxes reach into the next sequence: clear those rows
        clear_tile_rows<kTailThreads>(sm + TailSmem::kDO, len, tid);
        clear_tile_rows<kTailThreads>(sm + TailSmem::kVN, len, tid);
        clear_tile_rows<kTailThreads>(sm + TailSmem::kDVN, len, tid);
        clear_tile_rows<kTailThreads>(sm + TailSmem::kV, len, tid);
        if (gi == 0) {
          clear_tile_rows<kTailThreads>(q_tile, len, tid);
          clear_tile_rows<kTailThreads>(k_tile, len, tid);
        }
      }
      stage_sync();
      if (abort.raised()) {
        aborted = true;
        break;
      }
      // the other q / k buffer is free: the previous pair is done
      if (last_of_pair && has_next_pair && loader) load_qk(next_pair, qk_buf ^ 1);
      // Into L2 ahead of their copies into shared memory, whose buffers are free only a phase before they are read:
      // this item's u and w, the next item's states and row tiles.
      if (loader) {
        tma_prefetch_tile128(&maps.u, hv * kDim, start);
        tma_prefetch_tile128(&maps.w, hv * kDim, start);
        if (has_next) {
          tma_prefetch_tile128(&maps.h, 0, int(nx.tile * 128));
          tma_prefetch_tile128(&maps.dh, 0, int(nx.tile * 128));
          tma_prefetch_tile128(&maps.d_o, nx.hv * kDim, nx.start);
          tma_prefetch_tile128(&maps.v_new, nx.hv * kDim, nx.start);
          tma_prefetch_tile128(&maps.dv_new, nx.hv * kDim, nx.start);
          tma_prefetch_tile128(&maps.v, nx.hv * kDim, nx.start);
        }
      }

      // ---- phase A: everything that needs only loaded tiles -------------------------------------------------------
      if (issuer) {
        umma_gemm<64, 64>(tmem + kColTa, op_do, false, op_vn, false, 128, false);   // dAqk = do v_new^T
        umma_commit(&bar_first);
        gemm128(kColT0, op_vn, false, op_dh, false, 128, false);                    // dkh  = v_new dh^T
        gemm128(kColT3, op_a, true, op_dvn, true, 64, false);                       // dvb  = A^T dv_new
        umma_commit(&bar);
      }
      if (issuer2) {
        gemm128(kColT2, op_do, false, op_h, false, 128, false);                     // dq2  = do h^T
        gemm128(kColT1, op_dvn, false, op_h, false, 128, false, /*neg_a=*/true);    // dw   = -dv_new h^T
        umma_commit(&bar2);
      }
      // meanwhile: sum(dh . h) over the whole state tile
      float hdh = 0.f;
      for (int i = tid; i < 128 * 16; i += kTailThreads) {
        float a[8], b[8];
        unpack8(tile_chunk(sm + TailSmem::kH, 16384, i >> 4, i & 15), a);
        unpack8(tile_chunk(sm + TailSmem::kDH, 16384, i >> 4, i & 15), b);
#pragma unroll
        for (int j = 0; j < 8; ++j) hdh = fmaf(a[j], b[j], hdh);
      }
      const float gi_row = g2[row], beta_row = beta_s[row];
      const float g_last = g2[len - 1];
      const float rs_row = fast_exp2(g_last - gi_row);
      const float eg = fast_exp2(gi_row), qs_row = scale * eg, sk = beta_row * eg;
      float dG = 0.f, dB = 0.f, gdot = 0.f;
      // dAqk is done before the other products: its epilogue (reads Aqk, writes the dS tile; neither is an operand of
      // this phase) runs under them.  (Measured: starting the dkh / dq2 epilogue early the same way, or dkb's under
      // the dq / dk products, gains nothing or loses.)
      if (!mbar_wait(&bar_first, item_parity)) abort.raise();
      tc_fence_after();
      {
        // dAqk: dS = bf16(scale dAqk D) to its tile, P = dAqk . Aqk to the gate gradient (row sums - column sums)
        float s[8];
        tmem_ld_frag16(tmem_addr(tmem, warp, kColTa + ch * 16), s);
        const float g_lo = g2[fr], g_hi = g2[fr + 8];
        tmem_ld_wait();
        float rows[2] = {0.f, 0.f}, cols[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int col = fc + 8 * i;
          const float2 gc = *reinterpret_cast<const float2*>(g2 + col);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int r = fr + 8 * h;
            const float g_r = h ? g_hi : g_lo;
            const uint32_t at = sw128_offset(r, ch * 2 + i) + fq * 4;
            const float2 aq = unpack_bf16(*reinterpret_cast<const uint32_t*>(sm + TailSmem::kAqk + at));
            const float d0 = col <= r ? s[4 * i + 2 * h] : 0.f, d1 = col + 1 <= r ? s[4 * i + 2 * h + 1] : 0.f;
            const float ds0 = col <= r ? scale * d0 * fast_exp2(g_r - gc.x) : 0.f;
            const float ds1 = col + 1 <= r ? scale * d1 * fast_exp2(g_r - gc.y) : 0.f;
            *reinterpret_cast<uint32_t*>(sm + TailSmem::kB8 + at) = pack_bf16(ds0, ds1);
            const float p0 = d0 * aq.x, p1 = d1 * aq.y;
            rows[h] += p0 + p1;
            cols[2 * i] += p0;
            cols[2 * i + 1] += p1;
          }
        }
        publish_fragment_rows(rows[0], rows[1], s_rs);
        publish_fragment_columns(cols, s_cs);
      }
      mma_wait2();
      __syncthreads();  // every thread is past its reads of h / dh: epilogue A overwrites operand buffers
      {
        // dw -> its tile (the h region), phase B's operand; the phase's other results wait for a product to run under
        float wv[kTailW];
        tail_tmem_ld(tmem_addr(tmem, warp, kColT1 + ch * kTailW), wv);
        tmem_ld_wait();
#pragma unroll
        for (int jj = 0; jj < kTailJ; ++jj)
          set_tile_chunk(sm + TailSmem::kH, 8192, row, lchunk + jj, pack8(wv + jj * 8));
      }
      stage_sync();
      // do and v_new are done with: this value head's u and w take their buffers; then the next item's Aqk
      if (loader) {
        load_uw(it);
        if (has_next) load_aqk(nx);
      }
      if (has_next) load_scalars(nx, item_parity ^ 1);

      // ---- phase B: dq += dS k ; dk += dS^T q ; dkb = A^T dw ---------------------------------------------------------
      if (issuer) {
        gemm128(kColDQ, op_b8, false, op_k, true, 64, gi > 0);
        gemm128(kColDK, op_b8, true, op_q, true, 64, gi > 0);
        umma_commit(&bar);
      }
      if (issuer2) {
        gemm128(kColT1, op_a, true, op_dw, true, 64, false);  // dkb takes dw's columns; dkh, dq2 and dvb stay
        umma_commit(&bar2);
      }
      {
        // under phase B's products: dvb -> dv, dbeta, and its tile (the v buffer, read first), phase C's operand
        float y[kTailW];
        tail_tmem_ld(tmem_addr(tmem, warp, kColT3 + ch * kTailW), y);
        tmem_ld_wait();
        float dot_v = 0.f;
        uint4 vraw[kTailJ];
#pragma unroll
        for (int jj = 0; jj < kTailJ; ++jj) vraw[jj] = tile_chunk(sm + TailSmem::kV, 8192, row, lchunk + jj);
        __syncwarp();
#pragma unroll
        for (int jj = 0; jj < kTailJ; ++jj) {
          float vv[8], out[8];
          unpack8(vraw[jj], vv);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            dot_v = fmaf(y[jj * 8 + e], vv[e], dot_v);
            out[e] = y[jj * 8 + e] * beta_row;
          }
          set_tile_chunk(sm + TailSmem::kH + 16384, 8192, row, lchunk + jj, pack8(out));
        }
        dB += dot_v;
        // every thread reads only its own (row, chunk) cells of the v tile and rewrites exactly those with dvb
#pragma unroll
        for (int jj = 0; jj < kTailJ; ++jj) set_tile_chunk(sm + TailSmem::kV, 8192, row, lchunk + jj, pack8(y + jj * 8));
      }
      // dAqk's sums are read here, before the block barrier behind which phase C's epilogue rewrites them; they join
      // the gate gradient in the order they always did, after dkh's and dq2's
      const float aqk_sums = (owner && ch == 0) ? four(s_rs, row) - four(s_cs, row) : 0.f;
      mma_wait2();
      {
        // dkb -> its tile, phase C's operand; its sums wait until phase C's products run
        float dkb[kTailW];
        tail_tmem_ld(tmem_addr(tmem, warp, kColT1 + ch * kTailW), dkb);
        tmem_ld_wait();
#pragma unroll
        for (int jj = 0; jj < kTailJ; ++jj)
          set_tile_chunk(sm + TailSmem::kDVN, 8192, row, lchunk + jj, pack8(dkb + jj * 8));  // dv_new is done with
      }
      if (!mbar_wait(&bar_uw, item_parity)) abort.raise();  // u and w have landed
      if (len < kChunk) {
        clear_tile_rows<kTailThreads>(sm + TailSmem::kDO, len, tid);
        clear_tile_rows<kTailThreads>(sm + TailSmem::kVN, len, tid);
      }
      stage_sync();
      // dv leaves from its tile (the upper half of the h region) by one bulk store; a ragged chunk's rows by hand
      if (len < kChunk) {
        store_tile<64, 128, kTailThreads>(sm + TailSmem::kH + 16384, 8192, dv + int64_t(start) * dv_pitch + hv * kDim,
                                          dv_pitch, len, tid);
        __syncthreads();  // the tile is read: the next item's states may land on it
      }
      if (loader) {
        if (len == kChunk) {
          tma_store_tile128(&maps.dv_out, hv * kDim, start, sbase + TailSmem::kH + 16384, 8192);
          tma_store_commit();
        }
        if (has_next) {  // h / dh (and the dw tile) and A are done with, once the dv tile has been read
          tma_store_wait_read();
          load_states(nx);
        }
      }

      // ---- phase C: Y = bf16(dkb) w^T + bf16(dvb) u^T ; KK = k k^T ---------------------------------------------------
      if (issuer) {
        // Y as two chains into two accumulators (T3 is free by now: dvb was read under phase B); the epilogue adds them
        umma_gemm_pair<64, 64>(tmem + kColTa, op_dkb, false, op_w, false, 128, false, false, tmem + kColT3, op_dvb,
                               false, op_u, false, 128, false, false);
        umma_commit(&bar);
      }
      if (issuer2) {
        if (gi == 0) umma_gemm<64, 64>(tmem + kColTb, op_k, false, op_k, false, 128, false);  // KK: once per pair
        umma_commit(&bar2);
      }
      // Under phase C's products (which write other columns): what of phase A's and B's results no product reads.
      {
        // dkh and dq2 pieces: the scaled terms go to the register accumulators, their row dots to the gate gradient
        float a[kTailW], b[kTailW];
        tail_tmem_ld(tmem_addr(tmem, warp, kColT0 + ch * kTailW), a);
        tail_tmem_ld(tmem_addr(tmem, warp, kColT2 + ch * kTailW), b);
        tmem_ld_wait();
        float dot_k = 0.f, dot_q = 0.f;
#pragma unroll
        for (int jj = 0; jj < kTailJ; ++jj) {
          float kk[8], qq[8];
          unpack8(tile_chunk(k_tile, 8192, row, lchunk + jj), kk);
          unpack8(tile_chunk(q_tile, 8192, row, lchunk + jj), qq);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float x = rs_row * a[jj * 8 + e], y = qs_row * b[jj * 8 + e];
            dot_k = fmaf(x, kk[e], dot_k);
            dot_q = fmaf(y, qq[e], dot_q);
            dk_reg[jj * 8 + e] += x;
            dq_reg[jj * 8 + e] += y;
          }
        }
        dG += dot_q - dot_k;
        gdot += dot_k;
      }
      if (owner && ch == 0) dG += aqk_sums;
      {
        // dkb's part of dk and of the beta / gate gradients
        float dkb[kTailW];
        tail_tmem_ld(tmem_addr(tmem, warp, kColT1 + ch * kTailW), dkb);
        tmem_ld_wait();
        float dot_k = 0.f, dot_kb = 0.f;
#pragma unroll
        for (int jj = 0; jj < kTailJ; ++jj) {
          float kk[8];
          unpack8(tile_chunk(k_tile, 8192, row, lchunk + jj), kk);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float x = dkb[jj * 8 + e];
            dot_k = fmaf(x, kk[e], dot_k);
            dot_kb = fmaf(x, round_bf16(kk[e] * sk), dot_kb);  // kb = bf16(beta 2^G k), the forward's operand
            dk_reg[jj * 8 + e] = fmaf(sk, x, dk_reg[jj * 8 + e]);
          }
        }
        dB += eg * dot_k;
        dG += dot_kb;
      }
      mma_wait2();
      {
        // dL = bf16(-tril(Y, -1)); bf16(beta dL D) to its tile; dL D . KK to the beta gradient (row sums) and
        // beta dL D . KK to the gate gradient (row sums - column sums)
        float s[8], s2[8], kk[8];
        tmem_ld_frag16(tmem_addr(tmem, warp, kColTa + ch * 16), s);
        tmem_ld_frag16(tmem_addr(tmem, warp, kColT3 + ch * 16), s2);
        tmem_ld_frag16(tmem_addr(tmem, warp, kColTb + ch * 16), kk);
        const float g_lo = g2[fr], g_hi = g2[fr + 8], b_lo = beta_s[fr], b_hi = beta_s[fr + 8];
        tmem_ld_wait();
        float rows[2] = {0.f, 0.f}, dots[2] = {0.f, 0.f}, cols[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int col = fc + 8 * i;
          const float2 gc = *reinterpret_cast<const float2*>(g2 + col);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int r = fr + 8 * h, e = 4 * i + 2 * h;
            const float g_r = h ? g_hi : g_lo, b_r = h ? b_hi : b_lo;
            const bool in0 = col < r, in1 = col + 1 < r;
            const float dld0 = in0 ? round_bf16(-(s[e] + s2[e])) * fast_exp2(g_r - gc.x) : 0.f;
            const float dld1 = in1 ? round_bf16(-(s[e + 1] + s2[e + 1])) * fast_exp2(g_r - gc.y) : 0.f;
            const float k0 = in0 ? kk[e] : 0.f, k1 = in1 ? kk[e + 1] : 0.f;
            dots[h] = fmaf(dld1, k1, fmaf(dld0, k0, dots[h]));
            const float out0 = b_r * dld0, out1 = b_r * dld1;
            *reinterpret_cast<uint32_t*>(sm + TailSmem::kB8 + sw128_offset(r, ch * 2 + i) + fq * 4) =
                pack_bf16(out0, out1);
            const float p0 = out0 * k0, p1 = out1 * k1;  // dL . L
            rows[h] += p0 + p1;
            cols[2 * i] += p0;
            cols[2 * i + 1] += p1;
          }
        }
        publish_fragment_rows(rows[0], rows[1], s_rs);  // phase B has read dAqk's
        publish_fragment_rows(dots[0], dots[1], s_rs + 256);
        publish_fragment_columns(cols, s_cs + 256);
      }
      stage_sync();
      if (has_next && loader) load_row_tiles(nx);  // w, u, bf16(dkb), bf16(dvb) are done with

      // ---- phase D: dk += bf16(beta dL D) k + bf16(beta dL D)^T k ------------------------------------------------
      if (owner && ch == 0) {
        dG += four(s_rs, row) - four(s_cs + 256, row);
        dB += four(s_rs + 256, row);
      }
      // gate and beta gradients of this value head: combine the column quarters, add the chunk-end term, suffix sum
      float part = fmaf(fast_exp2(g_last), hdh, gdot);
#pragma unroll
      for (int m = 16; m >= 1; m >>= 1) part += __shfl_xor_sync(0xffffffffu, part, m);
      if (lane == 0) s_warp[warp] = part;
      s_red[cq * 64 + row] = dG;
      s_red2[cq * 64 + row] = dB;
      // Everybody's partial sums are out: the warps 2 and 3 wait for them and finish the sums; nobody else waits (the
      // thread that issues phase D least of all: its instructions take it several hundred cycles).
      const bool reducer = warp == 2 || warp == 3;
      if (reducer) asm volatile("bar.sync 1, %0;" ::"n"(kTailThreads) : "memory");
      else asm volatile("bar.arrive 1, %0;" ::"n"(kTailThreads) : "memory");
      if (issuer) {
        gemm128(kColDK, op_b8, false, op_k, true, 64, true);
        gemm128(kColDK, op_b8, true, op_k, true, 64, true);
        if (last_of_pair) umma_commit(&bar);  // otherwise the next item's first commit covers these too
      }
      if (reducer) {
        // the in-chunk suffix sum of the gate gradient as two warp scans joined by the upper total
        const int r = tid - 64;
        float suffix = 0.f;
        if (r < len) {
          suffix = tail_row_sum(s_red, r);
          if (r == len - 1) {
            float gamma_dot = 0.f;
#pragma unroll
            for (int wv = 0; wv < kTailThreads / 32; ++wv) gamma_dot += s_warp[wv];
            suffix += gamma_dot;
          }
        }
#pragma unroll
        for (int m = 1; m < 32; m <<= 1) {
          const float other = __shfl_down_sync(0xffffffffu, suffix, m);
          if (lane + m < 32) suffix += other;
        }
        if (r == 32) s_warp[kTailThreads / 32] = suffix;  // the total of rows 32..63
        asm volatile("bar.sync 2, 64;" ::: "memory");
        if (r < len) {
          if (r < 32) suffix += s_warp[kTailThreads / 32];
          dg[int64_t(start + r) * num_v_heads + hv] = suffix;
          dbeta[int64_t(start + r) * num_v_heads + hv] = tail_row_sum(s_red2, r);
        }
      }

      if (last_of_pair) {
        // ---- the group's dq, dk: fp32 sums, the norm's pull-back, one rounding ----------------------------------
        mma_wait();
        // this thread's columns of its row: in the raw operands and in the outputs (token pitches may differ:
        // either may be a column slice of a packed row)
        const int64_t out_at = int64_t(start + row) * dqk_pitch + hq * kDim + lcol;
        // acc: this thread's columns of the fp32 group sum.  With the op's L2 norm: dx = r (D - y (D . y)) with the
        // saved r and y = the unit row as the forward used it (the bf16 tile this pair's products read: no second
        // read of the raw rows, whose row-per-thread pieces would touch a line per lane); the dot product spans the
        // row's column pieces.
        auto finish = [&](float* acc, const uint8_t* unit_rows, const float* rstd, __nv_bfloat16* out) {
          if (rstd != nullptr) {
            const float r = live ? rstd[int64_t(start + row) * num_qk_heads + hq] : 0.f;
            float y[kTailW];
            float dot = 0.f;
#pragma unroll
            for (int jj = 0; jj < kTailJ; ++jj) {
              unpack8(tile_chunk(unit_rows, 8192, row, lchunk + jj), y + jj * 8);
#pragma unroll
              for (int e = 0; e < 8; ++e) dot = fmaf(acc[jj * 8 + e], y[jj * 8 + e], dot);
            }
            __syncthreads();  // the previous reduction has read s_red
            s_red[cq * 64 + row] = dot;
            __syncthreads();
            dot = tail_row_sum(s_red, row);
#pragma unroll
            for (int j = 0; j < kTailW; ++j) acc[j] = r * (acc[j] - y[j] * dot);
          }
          if (live) {
#pragma unroll
            for (int jj = 0; jj < kTailJ; ++jj) reinterpret_cast<uint4*>(out + out_at)[jj] = pack8(acc + jj * 8);
          }
        };
        {
          float b[kTailW];
          tail_tmem_ld(tmem_addr(tmem, warp, kColDQ + ch * kTailW), b);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < kTailW; ++j) dq_reg[j] += b[j];
        }
        finish(dq_reg, q_tile, rstd_q, dq);
        {
          float b[kTailW];
          tail_tmem_ld(tmem_addr(tmem, warp, kColDK + ch * kTailW), b);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < kTailW; ++j) dk_reg[j] += b[j];
        }
        finish(dk_reg, k_tile, rstd_k, dk);
      }
    }
  }
  cp_async_wait_pending<0>();
  if (loader) tma_store_wait_all();
  if (abort.raised()) {  // copies of the next item may still be in flight: give them time to land before the CTA ends
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 100000ull) {
    }
  }
  if (abort.raised() && tid == 0) atomicExch(status, kDevWaitTimeout | (5 << 8));
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace mek

extern "C" int mek_gdn_bwd_tail(const MekGdnDims* d, const void* q, const void* k, const void* v, const float* beta,
                                const float* g_cs, const void* a, const void* aqk, const void* w, const void* u,
                                const void* h_tape, const void* dh_tape, const void* v_new, const void* dv_new,
                                const void* d_o, const void* q_raw, const void* k_raw, const float* rstd_q,
                                const float* rstd_k, void* dq, void* dk, void* dv, float* dbeta, float* dg,
                                int32_t* status, void* stream) {
  using namespace mek;
  if (d == nullptr || d->num_chunks <= 0 || d->num_v_heads <= 0 || d->num_qk_heads <= 0 ||
      d->num_v_heads % d->num_qk_heads != 0)
    return fail(MEK_ERR_INVALID, "bwd_tail: bad extents");
  if (d->head_dim != 128) return fail(MEK_ERR_UNSUPPORTED, "bwd_tail: head dims must be 128, not %d", d->head_dim);
  if ((rstd_q == nullptr) != (rstd_k == nullptr) || (rstd_q != nullptr && (q_raw == nullptr || k_raw == nullptr)))
    return fail(MEK_ERR_INVALID, "bwd_tail: the norm's pull-back needs q_raw, k_raw, rstd_q and rstd_k together");
  typedef const __nv_bfloat16* In;
  typedef __nv_bfloat16* Out;
  const size_t smem = TailSmem::kBytes + 1024;
  if (int rc = want_smem(gdn_bwd_tail_kernel, smem, "bwd_tail")) return rc;
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) {
    cudaGetLastError();
    return fail(MEK_ERR_CUDA, "bwd_tail: cannot query the SM count");
  }
  const uint64_t tokens = uint64_t(d->total_tokens), tiles = uint64_t(d->num_chunks) * d->num_v_heads;
  const uint64_t qk_cols = uint64_t(d->num_qk_heads) * kDim, v_cols = uint64_t(d->num_v_heads) * kDim;
  TailMaps maps;
  struct {
    CUtensorMap* map;
    const void* base;
    uint64_t rows, cols;
    uint32_t box_rows;
    uint64_t pitch;
  } const wanted[] = {
      {&maps.q, q, tokens, qk_cols, 64, uint64_t(d->qk_pitch)}, {&maps.k, k, tokens, qk_cols, 64, uint64_t(d->qk_pitch)},
      {&maps.v, v, tokens, v_cols, 64, uint64_t(d->v_pitch)},   {&maps.d_o, d_o, tokens, v_cols, 64, 0},
      {&maps.v_new, v_new, tokens, v_cols, 64, 0},              {&maps.dv_new, dv_new, tokens, v_cols, 64, 0},
      {&maps.w, w, tokens, v_cols, 64, 0},                      {&maps.u, u, tokens, v_cols, 64, 0},
      {&maps.h, h_tape, tiles * 128, 128, 128, 0},              {&maps.dh, dh_tape, tiles * 128, 128, 128, 0},
      {&maps.a, a, tiles * 64, 64, 64, 0},                      {&maps.aqk, aqk, tiles * 64, 64, 64, 0},
      {&maps.dv_out, dv, tokens, v_cols, 64, uint64_t(d->dv_pitch)},
  };
  for (const auto& m : wanted)
    if (int rc = make_tile_map(m.map, m.base, m.rows, m.cols, m.box_rows, "bwd_tail", m.pitch)) return rc;
  const int64_t raw_pitch = d->raw_pitch != 0 ? d->raw_pitch : int64_t(qk_cols);
  const int64_t dqk_pitch = d->dqk_pitch != 0 ? d->dqk_pitch : int64_t(qk_cols);
  const int64_t dv_pitch = d->dv_pitch != 0 ? d->dv_pitch : int64_t(v_cols);
  if (raw_pitch < int64_t(qk_cols) || dqk_pitch < int64_t(qk_cols) || dv_pitch < int64_t(v_cols) ||
      (raw_pitch | dqk_pitch | dv_pitch) % 8 != 0)
    return fail(MEK_ERR_INVALID, "bwd_tail: a token pitch is smaller than its row or not a multiple of 8 elements");
  const int pairs = d->num_chunks * d->num_qk_heads;
  gdn_bwd_tail_kernel<<<pairs < sms ? pairs : sms, kTailThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      maps, beta, g_cs, In(q_raw), In(k_raw), rstd_q, rstd_k, Out(dq), Out(dk), Out(dv), dbeta, dg, d->chunk_start,
      d->chunk_len, d->num_chunks, d->num_qk_heads, d->num_v_heads, d->scale, raw_pitch, dqk_pitch, dv_pitch, status);
  return launched("bwd_tail");
}
