// Adjoint state scan of the chunked gated delta rule (reverse over chunks), sm_100a, with dv_local fused.
//
// Per (sequence, value head), from dh = dht (or 0), for each chunk from the last to the first:
//   dh_tape = bf16(dh)
//   dv_new  = bf16( bf16(Aqk^T do) + rowscale (k dh_tape) )            -> tape, and the W-side operand
//   dh      = gamma dh + q^T bf16(qscale do) - w^T dv_new
// after the first chunk dh is the gradient of the initial state.
//
// Reference semantics: miles_ext_kernels/cake/_vendor/cake_gdn_det_train_kcp/cake_fake_backend.py:313-349 (adjoint
// walk) and :433-448 (do_g, dv_intra); reference launches: miles_ext_kernels/cake/_impl/gdn/ops.py:1519-1640.
#include "common.cuh"
#include "scan_plan.cuh"
#include "tiles.cuh"
#include "tma.cuh"

namespace mek {

// One CTA per (sequence, value head), warp-specialised like the forward scan: two epilogue warpgroups (thread
// (k, half) holds row k of one half of the V columns of the fp32 adjoint state), two MMA-issuing threads and one
// copy warp; the roles meet on mbarriers only.  The step's first two products are independent chains of N = 128
// instructions into two accumulators, one chain per issuing thread, so the wait for them is as long as the longer
// chain; the third product is issued by the first thread alone.  Per chunk, last to first:
//   A  epilogue   dh_tape = bf16(dh) -> shared                                            -> "state tile ready"
//      issuers    D1 = k dh_tape, D1b = Aqk^T do
//      epilogue   meanwhile: do_g = bf16(qscale do) -> its own tile
//      copy warp  dh_tape tile -> the tape (TMA store); the tiles of the chunk walked next (TMA loads)
//   B  epilogue   dv_new = bf16(bf16(D1b) + rowscale D1) -> shared                          -> "dv tile ready"
//      issuer     D2 = q^T do_g - w^T dv_new
//      copy warp  dv_new tile -> the tape (TMA store; a ragged chunk's rows are stored by the epilogue threads)
//   C  epilogue   dh = gamma dh + D2.
struct BwdDhSmem {
  static constexpr uint32_t kStage = 4 * 16384 + 8192;  // k, q, w, do tiles and Aqk of one chunk
  static constexpr uint32_t kK = 0;                 // [64][128] k        K-major A of k dh
  static constexpr uint32_t kQ = 16384;             // [64][128] q        MN-major A of q^T do_g
  static constexpr uint32_t kW = 2 * 16384;         // [64][128] w        MN-major A of w^T dv_new (negated)
  static constexpr uint32_t kDO = 3 * 16384;        // [64][128] do
  static constexpr uint32_t kAqk = 4 * 16384;       // [64][64]
  static constexpr uint32_t kDV = 2 * kStage;       // [64][128] dv_new
  static constexpr uint32_t kDH = kDV + 16384;      // [128][128] bf16(dh), 2 blocks of 16 KiB (one per V half)
  static constexpr uint32_t kG = kDH + 32768;       // gates[2][128]
  static constexpr uint32_t kDOG = kG + 1024;       // [64][128] bf16(qscale do)
  static constexpr uint32_t kBytes = kDOG + 16384;
};

struct BwdDhMaps {
  CUtensorMap q, k, w, d_o;  // rows, box 64 x 64
  CUtensorMap aqk;           // tiles [num_tiles * 64, 64], box 64 x 64
  CUtensorMap dh_out;        // tiles [num_tiles * 128, 128], box 64 x 128: the adjoint state tape (stores)
  CUtensorMap dv_out;        // rows, box 64 x 64: the dv_new tape (stores)
};

constexpr int kAdjEpilogueThreads = 256;             // warps 0..7
constexpr int kAdjIssuer = kAdjEpilogueThreads;       // warp 8, lane 0: D1 and D2
constexpr int kAdjMover = kAdjEpilogueThreads + 32;   // warp 9, lane 0: every TMA load and store
constexpr int kAdjIssuer2 = kAdjEpilogueThreads + 64;  // warp 10, lane 0: D1b
constexpr int kAdjThreads = kAdjEpilogueThreads + 96;

__global__ void __launch_bounds__(kAdjThreads) gdn_bwd_dh_kernel(
    const __grid_constant__ BwdDhMaps maps, const float* __restrict__ g_cs,
    const float* __restrict__ dht, __nv_bfloat16* __restrict__ dv_new,
    float* __restrict__ dh0, const int32_t* __restrict__ chunk_start, const int32_t* __restrict__ chunk_len,
    const int32_t* __restrict__ seq_chunk_start, int num_qk_heads, int num_v_heads, float scale,
    const float* __restrict__ gl2, const ScanPlan plan, int32_t* __restrict__ status) {
  extern __shared__ uint8_t raw[];
  // bar_h: the state tile and this chunk's operand tiles are ready; bar_vs: the dv_new tile and do_g are ready (every
  // epilogue thread arrives on each); bar_d1 / bar_d2: the commits of the step's two groups of products;
  // bar_seen: the copy warp is past this step's wait for a free stage
  // bar_free_h / bar_free_dv: the copy warp's store of this step has read the state tile / the dv_new tile
  __shared__ uint64_t bar_load[2], bar_h, bar_vs, bar_d1, bar_d2, bar_free_h, bar_free_dv, bar_seen;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // gl2 != nullptr: the per-channel-decay variant (KDA): k holds k 2^{G_L - G}, q holds q 2^G, rowscale = 1,
  // qscale = scale, and the adjoint state decays per key channel
  const bool kda = gl2 != nullptr;
  const int quad = warp & 3, half = (warp >> 2) & 1;
  const int krow = quad * 32 + lane;
  // grid (heads, sequences): the heads of one sequence are neighbours in launch order, so that with `seq_order`
  // (longest first) every long walk starts before any short one
  const int n = plan.seq_order != nullptr ? plan.seq_order[blockIdx.y] : int(blockIdx.y);
  const int hv = blockIdx.x, hq = hv / (num_v_heads / num_qk_heads);
  float* s_g2 = reinterpret_cast<float*>(sm + BwdDhSmem::kG);
  Abort abort{&abort_flag};

  // pre-scan of a segment-parallel plan: blockIdx.z = 0 is the offset walk, 1 the transfer walk (from the identity,
  // with do = 0); neither writes the tapes.  The adjoint leaves a segment through its first chunks.
  const bool prescan = plan.seg_flags != nullptr;
  const bool transfer = prescan && blockIdx.z == 1;
  const int c_first = seq_chunk_start[n];
  int c_last = seq_chunk_start[n + 1];
  int state_row = n;
  if (prescan) {
    const int flags = plan.seg_flags[n];
    const bool inner = (flags & 1) != 0;
    if ((flags & 2) != 0 || (transfer && !inner) || c_first >= c_last) return;
    state_row = inner ? -1 : plan.state_row[n];
    if (inner && warm_up_suffices(plan, g_cs, chunk_start, chunk_len, c_first, c_last, num_v_heads, hv, true)) {
      if (transfer) return;  // M is taken as zero
      c_last = c_first + plan.warm_chunks;
    }
  }

  const bool tapes = !prescan;  // the walk writes dh_tape and dv_new
  if (tid == 0) {
    mbar_init(&bar_load[0], 1);
    mbar_init(&bar_load[1], 1);
    mbar_init(&bar_h, kAdjEpilogueThreads);
    mbar_init(&bar_vs, kAdjEpilogueThreads);
    mbar_init(&bar_d1, 2);  // one commit from each issuing thread
    mbar_init(&bar_d2, 1);
    mbar_init(&bar_free_h, 1);
    mbar_init(&bar_seen, 1);
    mbar_init(&bar_free_dv, 1);
    fence_mbar_init();
    abort_flag = 0;
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 512);
  const uint32_t sbase = smem_u32(sm);
  const int64_t v_stride = int64_t(num_v_heads) * kDim;
  tc_fence_before();
  __syncthreads();  // the barriers' initialisation and the tensor-memory base are visible to every role
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  // tensor-memory columns: D1 and D1b [64 x 128] in lanes 0..15 of each quadrant, D2 [128 x 128] in every lane
  constexpr uint32_t kD1 = 0, kD1b = 128, kD2 = 256;
  const int c_begin = c_first, c_end = c_last;
  const Operand op_dv{sbase + BwdDhSmem::kDV, 8192}, op_dh{sbase + BwdDhSmem::kDH, 16384};
  const Operand op_dog{sbase + BwdDhSmem::kDOG, 8192};

  if (tid == kAdjIssuer) {
    for (int c = c_end - 1; c >= c_begin; --c) {
      const uint32_t par = uint32_t(c_end - 1 - c) & 1u;
      const uint32_t sst = sbase + par * BwdDhSmem::kStage;
      const Operand op_k{sst + BwdDhSmem::kK, 8192}, op_q{sst + BwdDhSmem::kQ, 8192};
      const Operand op_w{sst + BwdDhSmem::kW, 8192};
      if (!abort.wait(&bar_h, par)) break;
      tc_fence_after();
      // The two [64 x 128] products of the step's first group go out as one chain of N = 128 instructions each, this
      // thread's and the second issuing thread's: two chains side by side end sooner than one thread's alternation,
      // and an N = 128 instruction reads a third less from shared memory than two of N = 64.
      umma_gemm<64, 128>(tmem + kD1, op_k, false, op_dh, true, 128, false);   // k dh_tape
      umma_commit(&bar_d1);
      if (!abort.wait(&bar_vs, par)) break;
      tc_fence_after();
      // one accumulator for both (two accumulators with alternating instructions and a sum in the epilogue measured
      // slower: the second tensor-memory load costs more than the shorter chain saves)
      umma_gemm<128, 128>(tmem + kD2, op_q, true, op_dog, true, 64, false);                 // q^T do_g
      umma_gemm<128, 128>(tmem + kD2, op_w, true, op_dv, true, 64, true, /*neg_a=*/true);   // - w^T dv_new
      umma_commit(&bar_d2);
    }
  } else if (tid == kAdjIssuer2) {
    for (int c = c_end - 1; c >= c_begin; --c) {
      const uint32_t par = uint32_t(c_end - 1 - c) & 1u;
      const uint32_t sst = sbase + par * BwdDhSmem::kStage;
      const Operand op_do{sst + BwdDhSmem::kDO, 8192}, op_aqk{sst + BwdDhSmem::kAqk, 8192};
      if (!abort.wait(&bar_h, par)) break;
      tc_fence_after();
      umma_gemm<64, 128>(tmem + kD1b, op_aqk, true, op_do, true, 64, false);   // Aqk^T do
      umma_commit(&bar_d1);  // these products end before the step's second group is issued: its commit frees the stage
    }
  } else if (tid == kAdjMover) {
    auto load = [&](int c, uint32_t stage) {
      const uint32_t base = sbase + stage * BwdDhSmem::kStage;
      const int start = chunk_start[c];
      mbar_arrive_expect(&bar_load[stage], 4 * 16384 + 8192);
      tma_load_tile128(base + BwdDhSmem::kK, 8192, &maps.k, hq * kDim, start, &bar_load[stage]);
      tma_load_tile128(base + BwdDhSmem::kQ, 8192, &maps.q, hq * kDim, start, &bar_load[stage]);
      tma_load_tile128(base + BwdDhSmem::kW, 8192, &maps.w, hv * kDim, start, &bar_load[stage]);
      tma_load_tile128(base + BwdDhSmem::kDO, 8192, &maps.d_o, hv * kDim, start, &bar_load[stage]);
      tma_load_box(base + BwdDhSmem::kAqk, &maps.aqk, 0, int((int64_t(c) * num_v_heads + hv) * 64), &bar_load[stage]);
    };
    if (c_begin < c_end) load(c_end - 1, 0);
    for (int c = c_end - 1; c >= c_begin; --c) {
      const uint32_t step = uint32_t(c_end - 1 - c), par = step & 1u;
      if (c > c_begin) {
        // the other stage's last readers were the previous step's products (its epilogue ended before them)
        if (step > 0 && !abort.wait(&bar_d2, par ^ 1u)) break;
        load(c - 1, par ^ 1u);
      }
      // "This thread is past its wait for a free stage": the epilogue threads wait for it before they release the
      // step's second group of products, so the barrier waited on above cannot complete twice before this thread has
      // looked at it (a wait by parity would then miss the phase for good); and this thread in turn waits for the
      // epilogue's release (bar_vs) before its next step, so neither barrier runs ahead of its waiter.
      mbar_arrive(&bar_seen);
      if (tapes) {
        if (!abort.wait(&bar_h, par)) break;
        tma_store_tile128(&maps.dh_out, 0, int((int64_t(c) * num_v_heads + hv) * 128), sbase + BwdDhSmem::kDH, 16384);
        tma_store_commit();
        tma_store_wait_read();
        mbar_arrive(&bar_free_h);
      }
      if (!abort.wait(&bar_vs, par)) break;
      if (tapes) {
        if (chunk_len[c] == kChunk) {  // a ragged chunk's rows are stored by the epilogue threads
          tma_store_tile128(&maps.dv_out, hv * kDim, chunk_start[c], sbase + BwdDhSmem::kDV, 8192);
          tma_store_commit();
          tma_store_wait_read();
        }
        mbar_arrive(&bar_free_dv);
      }
    }
    tma_store_wait_all();
  } else if (tid < kAdjEpilogueThreads) {
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
      start = chunk_start[c_end - 1], len = chunk_len[c_end - 1];
      prefetch_gates(c_end - 1, 0, start, len);
    }

    // fp32 adjoint state: 64 columns of row krow
    float dh[64];
    if (transfer) {
#pragma unroll
      for (int j = 0; j < 64; ++j) dh[j] = (krow == half * 64 + j) ? 1.f : 0.f;
    } else if (dht != nullptr && state_row >= 0) {
      const float4* src = reinterpret_cast<const float4*>(
          dht + ((int64_t(state_row) * num_v_heads + hv) * kDim + krow) * kDim + half * 64);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float4 t = __ldg(src + j);
        dh[4 * j] = t.x, dh[4 * j + 1] = t.y, dh[4 * j + 2] = t.z, dh[4 * j + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 64; ++j) dh[j] = 0.f;
    }

    bool alive = true;
    for (int c = c_end - 1; c >= c_begin; --c) {
      const uint32_t step = uint32_t(c_end - 1 - c), par = step & 1u;
      const int stage = int(par);
      // the next chunk's extent: requested now, needed when its gates are (nothing on the step's path waits for it)
      int next_start = 0, next_len = 0;
      if (c > c_begin) next_start = chunk_start[c - 1], next_len = chunk_len[c - 1];
      uint8_t* st = sm + stage * BwdDhSmem::kStage;
      // A. dh_tape = bf16(dh): this thread's half row -> shared (block `half`)
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) set_tile_chunk(sm + BwdDhSmem::kDH, 16384, krow, half * 8 + cc, pack8(dh + 8 * cc));
      cp_async_wait_all();  // this chunk's gates have landed (issued one step ago) ...
      if (!abort.wait(&bar_load[stage], (step >> 1) & 1u)) { alive = false; break; }  // ... and so have its tiles
      if (len < kChunk) {  // a ragged chunk's boxes reach into the next sequence: clear those rows
        clear_tile_rows<kAdjEpilogueThreads>(st + BwdDhSmem::kK, len, tid);
        clear_tile_rows<kAdjEpilogueThreads>(st + BwdDhSmem::kQ, len, tid);
        clear_tile_rows<kAdjEpilogueThreads>(st + BwdDhSmem::kW, len, tid);
        clear_tile_rows<kAdjEpilogueThreads>(st + BwdDhSmem::kDO, len, tid);
      }
      if (transfer) clear_tile_rows<kAdjEpilogueThreads>(st + BwdDhSmem::kDO, 0, tid);  // the homogeneous recurrence: do = 0
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&bar_h);
      if (c > c_begin) prefetch_gates(c - 1, stage ^ 1, next_start, next_len);
      // every epilogue thread's writes of this step (cleared rows, gates) are visible past the barrier they all
      // arrived on
      if (!abort.wait(&bar_h, par)) { alive = false; break; }
      const float* g2 = s_g2 + stage * 128;
      // While the first products run: do_g = bf16(qscale do) into its own tile (the products read do itself), and
      // the gates' factors of this thread's rows.
      for (int i = tid; i < 64 * 16; i += kAdjEpilogueThreads) {
        const int r = i >> 4, cc = i & 15;
        const float qs = kda ? scale : scale * fast_exp2(g2[r]);
        float x[8];
        unpack8(tile_chunk(st + BwdDhSmem::kDO, 8192, r, cc), x);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] *= qs;
        set_tile_chunk(sm + BwdDhSmem::kDOG, 8192, r, cc, pack8(x));
      }
      const float g_last = kda ? g2[krow] : g2[len - 1];
      const int i = quad * 16 + (lane & 15);
      const int lcol = (lane >> 4) * 64 + half * 32;
      const bool live = i < len;
      const bool by_hand = tapes && len < kChunk;  // a ragged chunk: no 64-row box may be stored
      const float rs = live ? (kda ? 1.f : fast_exp2(g_last - g2[i])) : 0.f;
      const float gamma = fast_exp2(g_last);
      // the previous step's tape store has read the dv_new tile
      if (tapes && step > 0 && !abort.wait(&bar_free_dv, par ^ 1u)) { alive = false; break; }
      // The copy warp is past its wait for a free stage.  Asked before the arrival that releases the step's second
      // group of products: the barrier that the copy warp waits on therefore cannot complete twice behind its back.
      if (!abort.wait(&bar_seen, par)) { alive = false; break; }
      if (!abort.wait(&bar_d1, par)) { alive = false; break; }
      tc_fence_after();

      // B. dv_new
      {
        __nv_bfloat16* drow = dv_new + int64_t(start + i) * v_stride + hv * kDim + lcol;
        float a[32], b[32];
        tmem_ld32_halves(tmem_addr(tmem, warp, kD1 + half * 32), a);
        tmem_ld32_halves(tmem_addr(tmem, warp, kD1b + half * 32), b);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) a[j] = live ? fmaf(rs, a[j], round_bf16(b[j])) : 0.f;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const uint4 packed = pack8(a + 8 * jj);
          if (by_hand && live) reinterpret_cast<uint4*>(drow)[jj] = packed;
          set_tile_chunk(sm + BwdDhSmem::kDV, 8192, i, (lcol >> 3) + jj, packed);
        }
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&bar_vs);
      // this step's tape store has read the state tile (long ago: asked here, off the path to the next step's A)
      if (tapes && !abort.wait(&bar_free_h, par)) { alive = false; break; }
      if (!abort.wait(&bar_d2, par)) { alive = false; break; }
      tc_fence_after();

      // C. dh = gamma dh + D2
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        float d[32];
        tmem_ld32(tmem_addr(tmem, warp, kD2 + half * 64 + p * 32), d);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) dh[p * 32 + j] = fmaf(gamma, dh[p * 32 + j], d[j]);
      }
      tc_fence_before();
      start = next_start, len = next_len;
    }
    cp_async_wait_all();

    float* out_state = prescan ? plan.summary + ((int64_t(n) * num_v_heads + hv) * 2 + (transfer ? 1 : 0)) * kDim * kDim
                               : (dh0 ? dh0 + (int64_t(n) * num_v_heads + hv) * kDim * kDim : nullptr);
    if (out_state != nullptr && alive && !abort.raised()) {
      float4* dst = reinterpret_cast<float4*>(out_state + krow * kDim + half * 64);
#pragma unroll
      for (int j = 0; j < 16; ++j) dst[j] = make_float4(dh[4 * j], dh[4 * j + 1], dh[4 * j + 2], dh[4 * j + 3]);
    }
  }
  if (abort.raised()) {  // copies may still be in flight: give them time to land before the CTA's memory goes
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 100000ull) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (abort.raised() && tid == 0) atomicExch(status, kDevWaitTimeout | (4 << 8));
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace mek

namespace {
int launch_bwd_dh(const MekGdnDims* d, const void* q, const void* k, const void* w, const void* d_o, const void* aqk,
                  const float* g_cs, const float* dht, void* dh_tape, void* dv_new, float* dh0, const float* gl2,
                  const mek::ScanPlan& plan, int32_t* status, void* stream, const char* what) {
  using namespace mek;
  const size_t smem = BwdDhSmem::kBytes + 1024;
  if (int rc = want_smem(gdn_bwd_dh_kernel, smem, what)) return rc;
  BwdDhMaps maps;
  if (int rc = make_rows_map(&maps.q, q, d->total_tokens, d->num_qk_heads, what, d->qk_pitch)) return rc;
  if (int rc = make_rows_map(&maps.k, k, d->total_tokens, d->num_qk_heads, what, d->qk_pitch)) return rc;
  if (int rc = make_rows_map(&maps.w, w, d->total_tokens, d->num_v_heads, what)) return rc;
  if (int rc = make_rows_map(&maps.d_o, d_o, d->total_tokens, d->num_v_heads, what)) return rc;
  if (int rc = make_tiles_map(&maps.aqk, aqk, int64_t(d->num_chunks) * d->num_v_heads, 64, 64, what)) return rc;
  if (plan.seg_flags == nullptr) {  // an ordinary walk writes the two tapes
    if (!dh_tape || !dv_new) return fail(MEK_ERR_INVALID, "%s: dh_tape or dv_new is null", what);
    if (int rc = make_tiles_map(&maps.dh_out, dh_tape, int64_t(d->num_chunks) * d->num_v_heads, 128, 128, what)) return rc;
    if (int rc = make_rows_map(&maps.dv_out, dv_new, d->total_tokens, d->num_v_heads, what)) return rc;
  } else {
    maps.dh_out = maps.k;  // a pre-scan writes no tape
    maps.dv_out = maps.k;
  }
  if (d->num_seqs > 65535)
    return fail(MEK_ERR_UNSUPPORTED, "%s: at most 65,535 sequences (or scan segments) per call, got %d", what,
                d->num_seqs);
  const dim3 grid(d->num_v_heads, d->num_seqs, plan.seg_flags != nullptr ? 2 : 1);
  ScanPlan ordered = plan;
  ordered.seq_order = d->seq_order;
  gdn_bwd_dh_kernel<<<grid, kAdjThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      maps, g_cs, dht, static_cast<__nv_bfloat16*>(dv_new), dh0, d->chunk_start,
      d->chunk_len, d->seq_chunk_start, d->num_qk_heads, d->num_v_heads, d->scale, gl2, ordered, status);
  return launched(what);
}
const mek::ScanPlan kNoPlan = {nullptr, nullptr, nullptr, 0, 0.f};

int check_bwd_dh(const MekGdnDims* d, const char* what) {
  using namespace mek;
  if (d == nullptr || d->num_seqs <= 0 || d->num_v_heads <= 0 || d->num_qk_heads <= 0 || d->num_chunks <= 0 ||
      d->total_tokens <= 0 || d->num_v_heads % d->num_qk_heads != 0)
    return fail(MEK_ERR_INVALID, "%s: bad extents", what);
  if (d->head_dim != 128) return fail(MEK_ERR_UNSUPPORTED, "%s: head dims must be 128, not %d", what, d->head_dim);
  return MEK_OK;
}
}  // namespace

extern "C" int mek_gdn_bwd_dh(const MekGdnDims* d, const void* q, const void* k, const void* w, const void* d_o,
                              const void* aqk, const float* g_cs, const float* dht, void* dh_tape, void* dv_new,
                              float* dh0, int32_t* status, void* stream) {
  if (int rc = check_bwd_dh(d, "bwd_dh")) return rc;
  return launch_bwd_dh(d, q, k, w, d_o, aqk, g_cs, dht, dh_tape, dv_new, dh0, nullptr, kNoPlan, status, stream,
                       "bwd_dh");
}

extern "C" int mek_gdn_bwd_dh_prescan(const MekGdnDims* d, const void* q, const void* k, const void* w,
                                      const void* d_o, const void* aqk, const float* g_cs, const float* boundary,
                                      const int32_t* seg_flags, const int32_t* state_row, int warm_chunks,
                                      float warm_log2, float* summary, int32_t* status, void* stream) {
  using namespace mek;
  if (int rc = check_bwd_dh(d, "bwd_dh_prescan")) return rc;
  if (!seg_flags || !state_row || !summary || warm_chunks < 0)
    return fail(MEK_ERR_INVALID, "bwd_dh_prescan: a null table or summary, or negative warm_chunks");
  const ScanPlan plan = {seg_flags, state_row, summary, warm_chunks, warm_log2};
  return launch_bwd_dh(d, q, k, w, d_o, aqk, g_cs, boundary, nullptr, nullptr, nullptr, nullptr, plan, status, stream,
                       "bwd_dh_prescan");
}

extern "C" int mek_kda_bwd_dh(const MekGdnDims* d, const void* qg, const void* kr, const void* w, const void* d_o,
                              const void* aqk, const float* gl2, const float* dht, void* dh_tape, void* dv_new,
                              float* dh0, int32_t* status, void* stream) {
  using namespace mek;
  if (int rc = check_bwd_dh(d, "kda_bwd_dh")) return rc;
  if (d->num_qk_heads != d->num_v_heads)
    return fail(MEK_ERR_INVALID, "kda_bwd_dh: KDA has one value head per key head");
  if (gl2 == nullptr) return fail(MEK_ERR_INVALID, "kda_bwd_dh: gl2 is null");
  return launch_bwd_dh(d, qg, kr, w, d_o, aqk, nullptr, dht, dh_tape, dv_new, dh0, gl2, kNoPlan, status, stream,
                       "kda_bwd_dh");
}

// The per-channel-decay variant's pre-scan over the segments of a plan (no warm-up rule: it reads scalar gates).
extern "C" int mek_kda_bwd_dh_prescan(const MekGdnDims* d, const void* qg, const void* kr, const void* w,
                                      const void* d_o, const void* aqk, const float* gl2, const float* boundary,
                                      const int32_t* seg_flags, const int32_t* state_row, float* summary,
                                      int32_t* status, void* stream) {
  using namespace mek;
  if (int rc = check_bwd_dh(d, "kda_bwd_dh_prescan")) return rc;
  if (d->num_qk_heads != d->num_v_heads)
    return fail(MEK_ERR_INVALID, "kda_bwd_dh_prescan: KDA has one value head per key head");
  if (!gl2 || !seg_flags || !state_row || !summary)
    return fail(MEK_ERR_INVALID, "kda_bwd_dh_prescan: gl2, a table or the summary is null");
  const ScanPlan plan = {seg_flags, state_row, summary, 0, 0.f};
  return launch_bwd_dh(d, qg, kr, w, d_o, aqk, nullptr, boundary, nullptr, nullptr, nullptr, gl2, plan, status, stream,
                       "kda_bwd_dh_prescan");
}
