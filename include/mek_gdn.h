/* C ABI of libmek_b200: the sm_100a kernels of the chunked gated delta rule (GDN) and its per-channel-decay
 * variant (KDA), forward and backward.
 *
 * Conventions (all entry points):
 *   - plain C types only: device pointers, extents, a CUDA stream handle passed as void* (cudaStream_t);
 *   - every call enqueues work on `stream` and returns without synchronising;
 *   - the return value is MEK_OK or an MEK_ERR_* code; mek_last_error() gives the text of the last failure on the
 *     calling thread.  The Python layer maps MEK_ERR_UNSUPPORTED -> NotImplementedError, MEK_ERR_INVALID ->
 *     ValueError, MEK_ERR_CUDA -> RuntimeError, as the reference's typed tvm-ffi exceptions do
 *     (reference: tools/templates/cake_host_shim.h:52-114);
 *   - kernels with bounded waits write a nonzero word to `status` (device int32) instead of hanging; the caller
 *     reads it after synchronising the stream.
 *
 * The reference exports, per generated library, a tvm-ffi typed function run(tensors..., scalars..., grid_x, grid_y,
 * grid_z) and build_cuda_version() (reference: tools/templates/cake_host_shim.h:62-64).  The entry points below
 * take their place: one per stage of the path, with raw pointers instead of DLPack tensors.
 */
#ifndef MEK_GDN_H_
#define MEK_GDN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  MEK_OK = 0,
  MEK_ERR_INVALID = 1,     /* bad extent / pointer / alignment: ValueError */
  MEK_ERR_UNSUPPORTED = 2, /* feature, dtype, head dimension or architecture not served: NotImplementedError */
  MEK_ERR_CUDA = 3         /* a CUDA runtime call failed: RuntimeError */
};

/* CUDART_VERSION the library was compiled against.
 * Replaces build_cuda_version() of every reference library (reference: miles_ext_kernels/cake/_runtime/loader.py:336-348). */
int mek_build_cuda_version(void);

/* Text of the last error on the calling thread ("" if none). */
const char* mek_last_error(void);

/* Compute capability gate: MEK_OK when `device` is sm_100 (B200), else MEK_ERR_UNSUPPORTED.
 * Replaces loader.device_arch's gate (reference: miles_ext_kernels/cake/_runtime/loader.py:477-491). */
int mek_check_device(int device);

/* Self-test of the tensor-core building block: D[128 lanes x ncols] = sum over `nk` instructions of A_k * B_k with
 * the operand images copied verbatim into shared memory and the descriptors given by the caller.  It lets the test
 * suite pin the shared-memory operand layouts (K-major and MN-major, 128-byte swizzle) against a CPU matmul.
 *   a_img/b_img   device bytes copied to 1024-byte aligned shared buffers (a_bytes, b_bytes <= 65536 each)
 *   a_desc/b_desc descriptor templates with a zero start address; a_off/b_off [nk] (device int32) byte offsets added
 *                 to the buffer's start per instruction
 *   idesc         instruction descriptor
 *   d_lane        first tensor-memory lane of the accumulator: 0, or 16 (an M = 64 accumulator may sit in the upper
 *                 half of each 32-lane quadrant, sharing its columns with another M = 64 accumulator)
 *   tf32          0: kind::f16 (bf16 operands, K = 16 per instruction); 1: kind::tf32 (fp32 words, K = 8)
 *   out           device float [128 * ncols], row = tensor-memory lane
 *   status        device int32, 0 = fine
 * With nk = 0 nothing is issued: the kernel's wait runs into its one-second limit, status becomes 1 and the kernel
 * returns normally (tensor memory freed) -- how the tests exercise the bounded waits without faulting the GPU.
 * No counterpart in the reference (its kernels are generated and tested end to end). */
int mek_selftest_umma(const void* a_img, int a_bytes, const void* b_img, int b_bytes, uint64_t a_desc, uint64_t b_desc,
                      const int32_t* a_off, const int32_t* b_off, int nk, uint32_t idesc, int ncols, int d_lane,
                      int tf32, float* out, int32_t* status, void* stream);

/* Self-test of the tile loads: one box (64 bf16 columns x box_rows rows, 128-byte swizzle) of the row-major bf16
 * matrix src [rows, cols] whose first element is (x, y) is copied by the copy engine (TMA) into shared memory and
 * from there, byte for byte, to out [box_rows * 128 bytes].  The tests compare it with the operand layout the
 * tensor-core self-test pins, including boxes that hang over the matrix's last row (zero-filled).
 *   box_rows 8..128, a multiple of 8; x a multiple of 8 elements; cols a multiple of 64
 * No counterpart in the reference. */
int mek_selftest_tma(const void* src, int64_t rows, int64_t cols, int box_rows, int x, int y, void* out,
                     int32_t* status, void* stream);
/* Cycles the tensor core takes for `count` products of shape (M, N, kdim) issued by 1 or 2 threads, or by one thread alternating between two accumulators (operands of
 * zeros; M in {64, 128}, N in {64, 128, 256}): the measurement behind the kernels' choice of instruction shapes. */
int mek_selftest_umma_rate(int m, int n, int a_mn, int b_mn, int kdim, int count, int issuers, int interleave,
                           long long* cycles, int32_t* status, void* stream);

/* Extents and chunk tables of one call.  Tokens are packed: [total_tokens, heads, 128]; a batch of B equal-length
 * sequences is B sequences of one packed row.  Chunks hold at most 64 tokens and never straddle a sequence.
 * Replaces the reference's ChunkMeta int32 tables (reference: miles_ext_kernels/cake/_impl/gdn/ops.py:157-174). */
typedef struct MekGdnDims {
  int64_t total_tokens;
  int32_t num_qk_heads;           /* H */
  int32_t num_v_heads;            /* HV, a multiple of H; value head hv reads q / k head hv / (HV / H) */
  int32_t head_dim;               /* 128 */
  int32_t num_seqs;               /* N */
  int32_t num_chunks;             /* NC */
  float scale;                    /* multiplies q k^T and q h */
  const int32_t* chunk_start;     /* device [NC]: first token of the chunk */
  const int32_t* chunk_len;       /* device [NC]: 1..64 */
  const int32_t* chunk_seq;       /* device [NC]: the chunk's sequence */
  const int32_t* seq_chunk_start; /* device [N + 1]: first chunk of each sequence */
  /* Token strides, in elements, of operands that may be column slices of a wider packed row (q, k, v as views of
   * one [T, (2 H + HV) * 128] row, gradients written into the packed gradient row); 0 = dense (heads * 128).  Inside
   * a token the heads stay contiguous.  Multiples of 8 elements (the copy engine's 16-byte rule). */
  int64_t qk_pitch;               /* of the q and k operands of an entry point */
  int64_t v_pitch;                /* of v */
  int64_t raw_pitch;              /* of q_raw and k_raw (gradient tail) */
  int64_t dqk_pitch;              /* of the dq and dk outputs */
  int64_t dv_pitch;               /* of the dv output */
  /* Optional, device [N]: the order in which the scans' CTAs take the sequences (a permutation; longest first
   * balances a packed batch of uneven documents over the SMs).  NULL: as numbered.  Results do not depend on it. */
  const int32_t* seq_order;
} MekGdnDims;

/* Chunk tables from a device cu_seqlens (int32, or int64 when offsets_are_int64) [num_seqs + 1], in one launch and
 * without a host round trip: chunk_start, chunk_len, chunk_seq int32 [bound] and seq_chunk_start int32 [num_seqs + 1],
 * bound >= ceil(total_tokens / 64) + num_seqs.  Entries past the real chunk count are pad chunks (length 0), which
 * every kernel skips.  Replaces the reference's device-side `meta` launch (reference:
 * miles_ext_kernels/cake/_impl/gdn/ops.py:311-376, 1808-1858). */
int mek_gdn_chunk_meta(const void* cu_seqlens, int offsets_are_int64, int num_seqs, int bound, int32_t* chunk_start,
                       int32_t* chunk_len, int32_t* chunk_seq, int32_t* seq_chunk_start, void* stream);

/* y = bf16(x r), r = 1 / sqrt(sum x^2 + 1e-6) per row of 128 bf16; rstd[row] = r.  Row (token, head) of x sits at
 * token * x_pitch + head * 128 (x_pitch = 0: dense, heads * 128); y and rstd are dense.
 * Replaces the `prep` stage's q / k normalisation (reference: miles_ext_kernels/cake/_impl/gdn/ops.py:1361-1380). */
int mek_gdn_l2norm(const void* x, void* y, float* rstd, int64_t rows, int heads, int64_t x_pitch, void* stream);

/* g_cs[t, hv] = log2(e) * chunk-local inclusive cumulative sum of g (fp32 [T, HV]).
 * Replaces the `prep` stage's gate cumsum (reference: ops.py:1361-1380). */
int mek_gdn_gate_cumsum(const MekGdnDims* dims, const float* g, float* g_cs, void* stream);

/* WY / UT transform per (chunk, value head): a_out, aqk_out bf16 [NC, HV, 64, 64]; w_out, u_out bf16 [T, HV, 128].
 * q, k bf16 [T, H, 128] (already normalised), v bf16 [T, HV, 128], beta fp32 [T, HV].
 * Replaces `_launch_wy` (reference: ops.py:1154-1188); Aqk follows the KCP prep program
 * (reference: _vendor/cake_gdn_det_train_kcp/cake_fake_backend.py:173-222). */
int mek_gdn_wy_fwd(const MekGdnDims* dims, const void* q, const void* k, const void* v, const float* beta,
                   const float* g_cs, void* a_out, void* aqk_out, void* w_out, void* u_out, int32_t* status,
                   void* stream);

/* State recurrence per (sequence, value head): h_tape bf16 [NC, HV, 128, 128] (state at the start of each chunk),
 * v_new bf16 [T, HV, 128], final_state fp32 [N, HV, 128, 128] or NULL; h0 fp32 [N, HV, 128, 128] or NULL.
 * Replaces `_launch_fwd_h` (reference: ops.py:1191-1317). */
int mek_gdn_fwd_h(const MekGdnDims* dims, const void* k, const void* w, const void* u, const float* g_cs,
                  const float* h0, void* h_tape, void* v_new, float* final_state, int32_t* status, void* stream);

/* The state scan with the output fused in (the reference's `fwd_ho`): mek_gdn_fwd_h that also writes
 * o bf16 [T, HV, 128] = bf16(scale 2^G (q h_tape) + Aqk v_new) chunk by chunk from the h_tape and v_new the step
 * holds in shared memory; h_tape and v_new are still written for the backward.  On segment dims it is the real walk
 * of a segmented plan.  Replaces the `fwd_h` + `fwd_o` launches (reference:
 * miles_ext_kernels/cake/_impl/gdn/ops.py:1191-1317, 1425-1440; cake_chain.py:1868-1973 of the det package). */
int mek_gdn_fwd_ho(const MekGdnDims* dims, const void* q, const void* k, const void* w, const void* u, const void* aqk,
                   const float* g_cs, const float* h0, void* h_tape, void* v_new, void* o, float* final_state,
                   int32_t* status, void* stream);

/* Output per (chunk, value head): o bf16 [T, HV, 128] = bf16(scale 2^G (q h_tape) + Aqk v_new).
 * Replaces the `fwd_o` launch (reference: ops.py:1425-1440). */
int mek_gdn_fwd_o(const MekGdnDims* dims, const void* q, const void* aqk, const void* v_new, const void* h_tape,
                  const float* g_cs, void* o, int32_t* status, void* stream);

/* Adjoint state scan per (sequence, value head), reverse over chunks, with dv_local fused:
 * dh_tape bf16 [NC, HV, 128, 128] (adjoint state at the end of each chunk), dv_new bf16 [T, HV, 128],
 * dh0 fp32 [N, HV, 128, 128] or NULL; dht fp32 [N, HV, 128, 128] or NULL; d_o bf16 [T, HV, 128].
 * Replaces the `dv_local` and `dhu` launches (reference: miles_ext_kernels/cake/_impl/gdn/ops.py:1519-1640). */
int mek_gdn_bwd_dh(const MekGdnDims* dims, const void* q, const void* k, const void* w, const void* d_o,
                   const void* aqk, const float* g_cs, const float* dht, void* dh_tape, void* dv_new, float* dh0,
                   int32_t* status, void* stream);

/* Segment-parallel scans (long sequences, fewer chains than SMs).  The sequences are cut into segments of whole
 * chunks; `seg_dims` is the call's MekGdnDims with num_seqs = the number of segments and seq_chunk_start = the
 * segments' chunk ranges [segments + 1].  One chunk step is affine in the state, so a segment has a summary (B, M)
 * with S_out = M S_in + B:
 *   *_prescan   per segment and value head the offset walk (from zero, or from row state_row[s] of `boundary` when
 *               the segment is the first its sequence's walk meets) -> B, and the transfer walk (from the identity,
 *               inhomogeneous operand zeroed) -> M; summary fp32 [segments, HV, 2, 128, 128]; no tape is written.
 *               seg_flags[s]: bit 0 = the walk starts from zero (a transfer walk exists), bit 1 = no summary needed.
 *   scan_stitch per (sequence, value head) chains the summaries in walk order from the sequence's boundary state
 *               (`boundary` fp32 [N, HV, 128, 128] or NULL) and writes the state every segment's real walk starts
 *               from: seg_state fp32 [segments, HV, 128, 128] (or NULL); seq_seg_start int32 [N + 1]; reverse = 1
 *               for the adjoint scan; final_out fp32 [N, HV, 128, 128] (or NULL): the state after the last segment.
 *               mode bits: 1 start from the identity, 2 leave the offsets out, 4 every segment started from zero
 *               (modes 4 and 7 compose the (B, M) of a run of segments: a rank's summary under context parallelism;
 *               mode 0 with warm_chunks = 0 over the ranks' summaries folds the chain of ranks before a rank).
 * The real walk is mek_gdn_fwd_h / mek_gdn_bwd_dh on seg_dims with h0 / dht = seg_state.
 * Warm-up rule: when the summed gate of the warm_chunks chunks through which a state leaves a segment is below
 * warm_log2 (log2 domain), the offset walk covers those chunks only and M is taken as zero (warm_chunks = 0: never).
 * Replaces the reference's pre-scan / split-scan launches and stitch (reference:
 * miles_ext_kernels/cake/_impl/gdn/ops.py:405-531, 1191-1317, 1551-1640). */
int mek_gdn_fwd_h_prescan(const MekGdnDims* seg_dims, const void* k, const void* w, const void* u, const float* g_cs,
                          const float* boundary, const int32_t* seg_flags, const int32_t* state_row, int warm_chunks,
                          float warm_log2, float* summary, int32_t* status, void* stream);
int mek_gdn_bwd_dh_prescan(const MekGdnDims* seg_dims, const void* q, const void* k, const void* w, const void* d_o,
                           const void* aqk, const float* g_cs, const float* boundary, const int32_t* seg_flags,
                           const int32_t* state_row, int warm_chunks, float warm_log2, float* summary,
                           int32_t* status, void* stream);
int mek_gdn_scan_stitch(const MekGdnDims* seg_dims, int num_seqs, const int32_t* seq_seg_start, const float* summary,
                        const float* boundary, const float* g_cs, float* seg_state, float* final_out, int reverse,
                        int warm_chunks, float warm_log2, int mode, void* stream);
/* The summary (B, M) of ONE run of segments (seq_seg_start [2]) composed from the segments' summaries, every segment
 * taken from zero / the identity, in one launch: out fp32 [HV, 2, 128, 128] (B, then M, per head) -- what a rank
 * publishes of its slice under context parallelism (reference: the fragment summaries of
 * miles_ext_kernels/cake/_impl/gdn/kcp.py:71-226). */
int mek_gdn_scan_compose(const MekGdnDims* seg_dims, const int32_t* seq_seg_start, const float* summary,
                         const float* g_cs, float* out, int reverse, int warm_chunks, float warm_log2, void* stream);

/* Gradient tail per (chunk, key head): dq, dk bf16 [T, H, 128] (fp32 sum over the key head's value heads, the L2
 * norm's pull-back r (D - y (D . y)) when rstd_q / rstd_k are given, one rounding), dv bf16 [T, HV, 128], dbeta and
 * dg fp32 [T, HV] (dg includes the in-chunk suffix sum).  q, k are the normalised rows the forward used; the
 * pull-back takes y from them (the bf16 unit rows the products read), so q_raw / k_raw -- which must accompany the
 * rstd pointers, as in the reference's signature -- are not read.
 * Replaces the `dqkwg`, `wy_bwd` and `finalize` launches (reference: ops.py:1642-1727). */
int mek_gdn_bwd_tail(const MekGdnDims* dims, const void* q, const void* k, const void* v, const float* beta,
                     const float* g_cs, const void* a, const void* aqk, const void* w, const void* u,
                     const void* h_tape, const void* dh_tape, const void* v_new, const void* dv_new, const void* d_o,
                     const void* q_raw, const void* k_raw, const float* rstd_q, const float* rstd_k, void* dq,
                     void* dk, void* dv, float* dbeta, float* dg, int32_t* status, void* stream);

/* Forward of the gated delta rule without any device allocation: o bf16 [T, HV, 128] and, when final_state is not
 * NULL, the fp32 final state [N, HV, 128, 128], from q, k (normalised), v, beta, the raw gate g and an optional h0.
 * The intermediates of the forward stages live in a fixed device array inside the library instead of
 * caller-allocated tensors, for hosts that may not allocate once their memory plan is set.  Limits:
 * total_tokens * num_v_heads <= 8192 and num_chunks * num_v_heads <= 256 (MEK_ERR_INVALID beyond).  The first call on
 * a device looks up the array's address and should come before any stream capture; calls that overlap on one GPU
 * share the array and race.  The array used is the current device's, so the caller's current device must be the one
 * that owns the operands and the stream (MEK_ERR_INVALID otherwise); no required pointer may be NULL.  Same results as mek_gdn_gate_cumsum + mek_gdn_wy_fwd + mek_gdn_fwd_h + mek_gdn_fwd_o.
 * This entry point has no counterpart in the reference. */
int mek_gdn_forward_static(const MekGdnDims* dims, const void* q, const void* k, const void* v, const float* beta,
                           const float* g, const float* h0, void* o, float* final_state, int32_t* status,
                           void* stream);

/* ---- KDA: the per-key-channel-decay variant (packed documents, zero initial state, HV = H <= 64) -----------------
 * Replaces the reference's KDA programs (reference: miles_ext_kernels/cake/_impl/kda/ops.py:142-234 entry points;
 * the generated kernels of cake/_vendor/cake_kda_det_train are not used). */

/* g2 fp32 [T, H, 128] = log2(e) * chunk-local cumulative gate; qg = bf16(q 2^g2), kg = bf16(k 2^g2),
 * kr = bf16(k 2^{G_L - g2}) bf16 [T, H, 128]; gl2 fp32 [NC, H, 128] = g2 at each chunk's last token. */
int mek_kda_prep(const MekGdnDims* dims, const void* q, const void* k, const float* g, float* g2, void* qg, void* kg,
                 void* kr, float* gl2, void* stream);

/* a_out, aqk_out bf16 [NC, H, 64, 64]; w_out, u_out bf16 [T, H, 128] (the WY transform with per-channel decays). */
int mek_kda_intra(const MekGdnDims* dims, const void* q, const void* k, const void* v, const void* kg, const float* g2,
                  const float* beta, void* a_out, void* aqk_out, void* w_out, void* u_out, int32_t* status,
                  void* stream);

/* The GDN scan / output / adjoint-scan kernels on the decayed operands (kr, qg) with a per-channel chunk decay.
 * h0 / final_state and dht / dh0: fp32 [N, H, 128, 128] per document, or null (zero initial state, nothing kept):
 * the states that cross rank boundaries under context parallelism (reference:
 * miles_ext_kernels/cake/_impl/kda/kcp.py:126-214). */
int mek_kda_fwd_h(const MekGdnDims* dims, const void* kr, const void* w, const void* u, const float* gl2,
                  const float* h0, void* h_tape, void* v_new, float* final_state, int32_t* status, void* stream);
int mek_kda_fwd_o(const MekGdnDims* dims, const void* qg, const void* aqk, const void* v_new, const void* h_tape,
                  void* o, int32_t* status, void* stream);
int mek_kda_bwd_dh(const MekGdnDims* dims, const void* qg, const void* kr, const void* w, const void* d_o,
                   const void* aqk, const float* gl2, const float* dht, void* dh_tape, void* dv_new, float* dh0,
                   int32_t* status, void* stream);
/* Their pre-scans over the segments of a scan plan (dims describe the segments as sequences; the tables and the
 * summary as in mek_gdn_fwd_h_prescan; no warm-up rule): with mek_gdn_scan_stitch and a walk over the segments from
 * their stitched start states, a long sequence's scan runs in parallel pieces (reference: the scan plans of
 * miles_ext_kernels/cake/_impl/gdn/ops.py:405-531, which the reference applies to GDN only). */
int mek_kda_fwd_h_prescan(const MekGdnDims* dims, const void* kr, const void* w, const void* u, const float* gl2,
                          const float* boundary, const int32_t* seg_flags, const int32_t* state_row, float* summary,
                          int32_t* status, void* stream);
int mek_kda_bwd_dh_prescan(const MekGdnDims* dims, const void* qg, const void* kr, const void* w, const void* d_o,
                           const void* aqk, const float* gl2, const float* boundary, const int32_t* seg_flags,
                           const int32_t* state_row, float* summary, int32_t* status, void* stream);

/* Gradient tail: dq32, dk32 fp32 [T, H, 128] (before the norm's pull-back and the rounding), dv bf16 [T, H, 128],
 * dg fp32 [T, H, 128] (in-chunk suffix sum included), dbeta fp32 [T, H].  Scratch the caller provides: m1, m2 fp32
 * [NC, H, 64, 64]; dqg, dkr, dkg fp32 [T, H, 128]; hdh fp32 [NC, H, 128]; dbeta_part fp32 [T, H]. */
int mek_kda_bwd_tail(const MekGdnDims* dims, const void* q, const void* k, const void* v, const void* kg,
                     const float* g2, const float* beta, const void* a, const void* h_tape, const void* dh_tape,
                     const void* v_new, const void* dv_new, const void* d_o, float* m1, float* m2, float* dqg,
                     float* dkr, float* dkg, float* hdh, float* dbeta_part, float* dq32, float* dk32, void* dv,
                     float* dg, float* dbeta, int32_t* status, void* stream);

/* out bf16 = x fp32 per row of 128, through the L2 norm's pull-back r (x - y (x . y)), y = raw r, when rstd is given. */
int mek_qk_grad_finish(const float* x, const void* raw_rows, const float* rstd, void* out, int64_t rows, void* stream);

/* ------------------------------------------------------------------------------------------------------------------
 * SiLU-gated RMSNorm over rows of 128 (the GDN layer's output norm), forward and backward:
 *     rstd = 1 / sqrt(mean(x^2) + eps),   y = bf16(((x rstd) weight) silu(z))
 * x, z bf16: row (token, head) at token * token_stride + head * head_stride elements (strides multiples of 8, bases
 * 16-byte aligned; z is usually a column slice of the layer's input projection); weight bf16 [128]; y, dy, dx, dz dense
 * bf16 [rows, 128]; rows = tokens * heads.  The weight gradient (bf16 [128], or NULL with dw_partial NULL) is summed
 * in a fixed order: per block in FP32 into dw_partial fp32 [mek_gated_rmsnorm_partial_rows(rows), 128], then over the
 * blocks in FP64.  Replaces the reference's `cake_rmsnorm_silu_gate_det_train` package (reference:
 * miles_ext_kernels/cake/_impl/gated_rmsnorm/ops.py:126-148). */
int mek_gated_rmsnorm_partial_rows(int64_t rows);
int mek_gated_rmsnorm_fwd(const void* x, const void* z, const void* weight, void* y, int64_t rows, int heads,
                          int64_t x_token_stride, int64_t x_head_stride, int64_t z_token_stride, int64_t z_head_stride,
                          float eps, void* stream);
int mek_gated_rmsnorm_bwd(const void* dy, const void* x, const void* z, const void* weight, void* dx, void* dz,
                          float* dw_partial, void* dw, int64_t rows, int heads, int64_t x_token_stride,
                          int64_t x_head_stride, int64_t z_token_stride, int64_t z_head_stride, float eps,
                          void* stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Packed causal depthwise conv1d (kernel size 4) + SiLU, the short convolution in front of the GDN / KDA op:
 *     pre[t, c] = sum_{k<4} w[c, k] x[t - 3 + k, c] (inside t's document),   y = bf16(pre sigmoid(pre))
 * x, y, dy, dx bf16 [tokens, channels] dense (channels a multiple of 8); weight [channels, 4] fp32, or bf16 when
 * weight_is_bf16; reach uint8 [tokens] from mek_conv1d_reach (cu_seqlens int32 [num_docs + 1] on the device).
 * Backward: SiLU' at the BF16-rounded preactivation, or at the unrounded one with FP64 weight-gradient sums when
 * fp32_policy; dw in the weight's dtype (or NULL with dw_partial NULL); dw_partial holds
 * mek_conv1d_runs(tokens) * channels * 4 floats (doubles under fp32_policy), summed in a fixed order.
 * Context parallelism (reference: ops.py:267-340): a rank whose first document began on the rank before passes that
 * rank's last 3 rows as x_prev [3, channels] and a cu_seqlens whose first entry is minus the number of those rows
 * that belong to the document; a rank whose last document goes on passes the next rank's first 3 rows of x and dy
 * as x_next, dy_next, a cu_seqlens whose last entry is tokens plus the number of rows that belong to the document,
 * and a reach table of tokens + 3 entries.  NULL: nothing on that side.  y, dx and the weight-gradient sums cover
 * the rank's own tokens only.
 * Replaces the reference's `cake_causal_conv1d_det_train` package (reference:
 * miles_ext_kernels/cake/_impl/conv1d/ops.py:226-257). */
int mek_conv1d_runs(int tokens);
int mek_conv1d_reach(const int32_t* cu_seqlens, int num_docs, int tokens, uint8_t* reach, void* stream);
int mek_conv1d_fwd(const void* x, const void* x_prev, const void* weight, int weight_is_bf16, const uint8_t* reach,
                   void* y, int tokens, int channels, void* stream);
int mek_conv1d_bwd(const void* x, const void* x_prev, const void* x_next, const void* weight, int weight_is_bf16,
                   const void* dy, const void* dy_next, const uint8_t* reach, void* dx, void* dw_partial, void* dw,
                   int fp32_policy, int tokens, int channels, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* MEK_GDN_H_ */
