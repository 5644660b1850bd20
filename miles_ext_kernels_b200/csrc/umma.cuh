// Blackwell (sm_100a) primitives shared by the gated-delta-rule kernels: tensor-memory allocation, shared-memory
// matrix descriptors, tcgen05.mma issue/commit, bounded mbarrier waits, tensor-memory loads, and the 128-byte
// swizzled tile layout every operand tile uses.
//
// Tile layout. An operand tile of R rows x 64 bf16 columns ("block") occupies R x 128 bytes; the 16-byte chunk c of
// row r sits at byte  r*128 + ((c ^ (r & 7)) << 4)  (the SWIZZLE_128B pattern of TMA and of the UMMA descriptors).
// A 128-column tile is two such blocks, `block_stride` bytes apart.  One block serves two roles without a copy:
//   * K-major operand  (contraction along the 64 contiguous columns): descriptor SBO = 1024 B (8 rows), k-step of
//     16 columns = +32 B on the start address;
//   * MN-major operand (contraction along the rows): descriptor SBO = 1024 B (8 rows of the contraction),
//     LBO = block_stride (next 64 columns of the M/N extent), k-step of 16 rows = +2048 B.
// Blocks start on 1024-byte boundaries.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mek {

// ---------------------------------------------------------------------------------------------------------------
// small PTX wrappers
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Generic-proxy writes to shared memory become visible to the async proxy (tcgen05.mma operand reads, TMA).
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Time limit of every wait in these kernels: one second of wall clock (%globaltimer), far beyond any legitimate MMA
// latency.  A wait that runs out returns false; the kernel then records an error status and leaves through its
// normal exit (tensor memory freed), so the context stays usable.
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > kWaitLimitNs) return false;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// tensor memory
// ---------------------------------------------------------------------------------------------------------------
// One warp allocates `ncols` (power of two, 32..512) columns; the base address lands in *slot (shared memory).
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Thread `lane` of warp w reads 32 consecutive fp32 columns of tensor-memory lane 32*(w%4)+lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// 16 lanes x 32 columns, twice (shape 16x32bx2): thread t < 16 reads lane t of the warp's quadrant at the columns
// [taddr, taddr + 32), thread t >= 16 reads lane t - 16 at the columns [taddr + 64, taddr + 96): a 64 x 128 accumulator
// that sits in lanes 0..15 only, read as (row, column half) by the whole warp.
__device__ __forceinline__ void tmem_ld32_halves(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.16x32bx2.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32], 64;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// The same for 4 consecutive columns.
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr)
               : "memory");
}

// 16 lanes x 16 columns shared by the whole warp (shape 16x256b, twice): thread t receives the rows t / 4 and
// t / 4 + 8 of the lanes the address names, at the columns 8 i + 2 (t % 4) + {0, 1}, i = 0, 1:
//   v[4 i + 0], v[4 i + 1]  row t / 4;   v[4 i + 2], v[4 i + 3]  row t / 4 + 8.
__device__ __forceinline__ void tmem_ld_frag16(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The tensor-memory address of (lane quadrant of this warp, column): bits 31..16 lane, 15..0 column.
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t warp, uint32_t col) {
  return base + (((warp & 3u) * 32u) << 16) + col;
}

// ---------------------------------------------------------------------------------------------------------------
// descriptors
// ---------------------------------------------------------------------------------------------------------------
// Instruction descriptor of tcgen05.mma.kind::f16 with bf16 operands and an fp32 accumulator.
//   bits 4..5 accumulator format (1 = f32); 7..9 A format (1 = bf16); 10..12 B format (1 = bf16); 13 negate A;
//   14 negate B; 15 A major (1 = MN); 16 B major (1 = MN); 17..22 N >> 3; 24..28 M >> 4.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, bool a_mn_major, bool b_mn_major, bool neg_a = false) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(neg_a) << 13) | (uint32_t(a_mn_major) << 15) |
         (uint32_t(b_mn_major) << 16) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// Shared-memory matrix descriptor, SWIZZLE_128B: bits 0..13 start address >> 4; 16..29 leading byte offset >> 4;
// 32..45 stride byte offset >> 4; 46..47 descriptor version (1 on sm_100); 61..63 layout type (2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((saddr >> 4) & 0x3FFFu);
  d |= uint64_t((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}

// D[tmem] (+)= A * B, one instruction (K = 16 bf16).  Issued by ONE thread.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same with TF32 operands (fp32 words in shared memory, 10 mantissa bits used), K = 8 per instruction.
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Instruction descriptor of tcgen05.mma.kind::tf32 (operand format code 2), fp32 accumulator, both operands K-major
// unless said otherwise.
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int m, int n, bool neg_a = false) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(neg_a) << 13) | (uint32_t(n >> 3) << 17) |
         (uint32_t(m >> 4) << 24);
}

// Arrive on `bar` once every tcgen05.mma issued so far by this thread has completed (implies
// tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// swizzled tiles
// ---------------------------------------------------------------------------------------------------------------
constexpr uint32_t kBlockCols = 64;     // bf16 columns of one swizzled block (128 bytes)
constexpr uint32_t kSbo = 1024;         // 8 rows x 128 bytes

// Byte offset of the 16-byte chunk `chunk` (0..7) of row `row` inside a block.
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

// An operand view of a tile made of SWIZZLE_128B blocks.
struct Operand {
  uint32_t saddr;         // shared address of block 0 (1024-byte aligned)
  uint32_t block_stride;  // bytes between consecutive 64-column blocks
};

// K-major use: contraction index = tile column.  `k0` = first contraction column (multiple of 16).
__device__ __forceinline__ uint64_t desc_kmajor(const Operand& t, uint32_t k0) {
  const uint32_t addr = t.saddr + (k0 / kBlockCols) * t.block_stride + (k0 % kBlockCols) * 2u;
  return umma_desc_sw128(addr, 16u, kSbo);
}

// MN-major use: contraction index = tile row.  `k0` = first contraction row (multiple of 16).  The M/N extent
// starts at column 0 of block 0 and continues in the next blocks.
__device__ __forceinline__ uint64_t desc_mnmajor(const Operand& t, uint32_t k0) {
  const uint32_t addr = t.saddr + k0 * 128u;
  return umma_desc_sw128(addr, t.block_stride, kSbo);
}

// The operand that starts `rows` rows (multiple of 8) below / `blocks` 64-column blocks to the right of `t`.
__device__ __forceinline__ Operand operand_at(const Operand& t, uint32_t rows, uint32_t blocks = 0) {
  return Operand{t.saddr + rows * 128u + blocks * t.block_stride, t.block_stride};
}

// D[M x N] (+)= A * B over a contraction of `kdim` (multiple of 16).  a_mn/b_mn pick the operand role of each tile.
// Issued by ONE thread; `accumulate` says whether the first instruction adds to what tensor memory holds.
//
// The issuing thread is on the critical path of its whole CTA (its warp joins the epilogue late), so the loop does
// no descriptor arithmetic: the first step's descriptors are built once and the later ones differ only in the 14-bit
// start-address field, by a constant (K-major: +32 bytes per step, and at every fourth step on to the next
// 64-column block; MN-major: +2048 bytes per step).  Shared addresses stay below 256 KiB, so the field never carries.
template <int M, int N>
__device__ __forceinline__ void umma_gemm(uint32_t tmem_d, const Operand& a, bool a_mn, const Operand& b, bool b_mn,
                                          uint32_t kdim, bool accumulate, bool neg_a = false) {
  const uint32_t idesc = umma_idesc(M, N, a_mn, b_mn, neg_a);
  uint64_t da = a_mn ? desc_mnmajor(a, 0) : desc_kmajor(a, 0);
  uint64_t db = b_mn ? desc_mnmajor(b, 0) : desc_kmajor(b, 0);
  const uint32_t a_step = a_mn ? 128u : 2u, b_step = b_mn ? 128u : 2u;  // in 16-byte units
  const uint32_t a_jump = a_mn ? 128u : (a.block_stride >> 4) - 6u;     // K-major: from column 48 to the next block
  const uint32_t b_jump = b_mn ? 128u : (b.block_stride >> 4) - 6u;
  const uint32_t steps = kdim >> 4;
#pragma unroll
  for (uint32_t k = 0; k < 8; ++k) {
    if (k < steps) {
      umma_f16(tmem_d, da, db, idesc, (accumulate || k > 0) ? 1u : 0u);
      da += (k & 3u) == 3u ? a_jump : a_step;
      db += (k & 3u) == 3u ? b_jump : b_step;
    }
  }
}

// Two products into two accumulators with their instructions alternating.  Consecutive instructions into ONE
// accumulator wait for one another (~82 cycles each on a B200, whatever the shape up to N = 128); two chains keep the
// tensor core busy (~47 cycles per M = 64, N = 64 instruction from one thread, ~41 from two threads).  The
// contraction lengths may differ; the longer product's tail goes out alone.
template <int M, int N, int N1 = N>
__device__ __forceinline__ void umma_gemm_pair(uint32_t d0, const Operand& a0, bool a0_mn, const Operand& b0,
                                               bool b0_mn, uint32_t kdim0, bool acc0, bool neg0, uint32_t d1,
                                               const Operand& a1, bool a1_mn, const Operand& b1, bool b1_mn,
                                               uint32_t kdim1, bool acc1, bool neg1) {
  const uint32_t idesc0 = umma_idesc(M, N, a0_mn, b0_mn, neg0), idesc1 = umma_idesc(M, N1, a1_mn, b1_mn, neg1);
  uint64_t da0 = a0_mn ? desc_mnmajor(a0, 0) : desc_kmajor(a0, 0), db0 = b0_mn ? desc_mnmajor(b0, 0) : desc_kmajor(b0, 0);
  uint64_t da1 = a1_mn ? desc_mnmajor(a1, 0) : desc_kmajor(a1, 0), db1 = b1_mn ? desc_mnmajor(b1, 0) : desc_kmajor(b1, 0);
  const uint32_t a0_step = a0_mn ? 128u : 2u, b0_step = b0_mn ? 128u : 2u;
  const uint32_t a1_step = a1_mn ? 128u : 2u, b1_step = b1_mn ? 128u : 2u;
  const uint32_t a0_jump = a0_mn ? 128u : (a0.block_stride >> 4) - 6u, b0_jump = b0_mn ? 128u : (b0.block_stride >> 4) - 6u;
  const uint32_t a1_jump = a1_mn ? 128u : (a1.block_stride >> 4) - 6u, b1_jump = b1_mn ? 128u : (b1.block_stride >> 4) - 6u;
  const uint32_t steps0 = kdim0 >> 4, steps1 = kdim1 >> 4;
#pragma unroll
  for (uint32_t k = 0; k < 8; ++k) {
    if (k < steps0) {
      umma_f16(d0, da0, db0, idesc0, (acc0 || k > 0) ? 1u : 0u);
      da0 += (k & 3u) == 3u ? a0_jump : a0_step;
      db0 += (k & 3u) == 3u ? b0_jump : b0_step;
    }
    if (k < steps1) {
      umma_f16(d1, da1, db1, idesc1, (acc1 || k > 0) ? 1u : 0u);
      da1 += (k & 3u) == 3u ? a1_jump : a1_step;
      db1 += (k & 3u) == 3u ? b1_jump : b1_step;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// bf16 packing
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float2 unpack_bf16(uint32_t w) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&w);
  return __bfloat1622float2(v);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace mek
