// Tile movers between global memory, registers and the swizzled shared-memory blocks of umma.cuh, and the
// per-thread views of M = 64 accumulators.
#pragma once

#include "umma.cuh"

namespace mek {

constexpr int kChunk = 64;    // tokens per chunk
constexpr int kDim = 128;     // head dimension (K = V)
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

// Cooperative load of `ROWS x COLS` bf16 from global (row stride in elements) into swizzled blocks starting at tile
// row `row0`.  Rows >= valid_rows are zero-filled.
template <int ROWS, int COLS, int NT>
__device__ __forceinline__ void load_tile(uint8_t* tile, uint32_t block_stride, const __nv_bfloat16* g,
                                          int64_t row_stride, int valid_rows, int tid, int row0 = 0) {
  constexpr int CPR = COLS / 8;
#pragma unroll 4
  for (int i = tid; i < ROWS * CPR; i += NT) {
    const int r = i / CPR, cc = i % CPR;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (r < valid_rows) val = ldg16(g + int64_t(r) * row_stride + cc * 8);
    *reinterpret_cast<uint4*>(tile + (cc >> 3) * block_stride + sw128_offset(row0 + r, cc & 7)) = val;
  }
}

// Cooperative store of a `ROWS x COLS` swizzled tile to global rows (row stride in elements); rows >= valid_rows
// are skipped.
template <int ROWS, int COLS, int NT>
__device__ __forceinline__ void store_tile(const uint8_t* tile, uint32_t block_stride, __nv_bfloat16* g,
                                           int64_t row_stride, int valid_rows, int tid) {
  constexpr int CPR = COLS / 8;
#pragma unroll 4
  for (int i = tid; i < ROWS * CPR; i += NT) {
    const int r = i / CPR, cc = i % CPR;
    if (r < valid_rows)
      *reinterpret_cast<uint4*>(g + int64_t(r) * row_stride + cc * 8) =
          *reinterpret_cast<const uint4*>(tile + (cc >> 3) * block_stride + sw128_offset(r, cc & 7));
  }
}

// ---------------------------------------------------------------------------------------------------------------
// asynchronous copies (cp.async): the next chunk's tiles land in shared memory while the current chunk computes
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Asynchronous version of load_tile: rows >= valid_rows are zero-filled (copy size 0).  `tile` is a shared address.
template <int ROWS, int COLS, int NT>
__device__ __forceinline__ void prefetch_tile(uint32_t tile, uint32_t block_stride, const __nv_bfloat16* g,
                                              int64_t row_stride, int valid_rows, int tid) {
  constexpr int CPR = COLS / 8;
#pragma unroll 4
  for (int i = tid; i < ROWS * CPR; i += NT) {
    const int r = i / CPR, cc = i % CPR;
    const bool valid = r < valid_rows;
    cp_async16(tile + (cc >> 3) * block_stride + sw128_offset(r, cc & 7),
               g + (valid ? int64_t(r) * row_stride : 0) + cc * 8, valid);
  }
}

// 8 consecutive bf16 (one 16-byte chunk) of row `row`, logical column chunk `cc` (0..COLS/8-1).
__device__ __forceinline__ uint4 tile_chunk(const uint8_t* tile, uint32_t block_stride, int row, int cc) {
  return *reinterpret_cast<const uint4*>(tile + (cc >> 3) * block_stride + sw128_offset(row, cc & 7));
}
__device__ __forceinline__ void set_tile_chunk(uint8_t* tile, uint32_t block_stride, int row, int cc, uint4 v) {
  *reinterpret_cast<uint4*>(tile + (cc >> 3) * block_stride + sw128_offset(row, cc & 7)) = v;
}

__device__ __forceinline__ uint4 pack8(const float* v) {
  return make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}
__device__ __forceinline__ void unpack8(uint4 w, float* v) {
  float2 a = unpack_bf16(w.x), b = unpack_bf16(w.y), c = unpack_bf16(w.z), d = unpack_bf16(w.w);
  v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y, v[4] = c.x, v[5] = c.y, v[6] = d.x, v[7] = d.y;
}

// bf16 rounding of a value kept in fp32 (the kernels' one rounding primitive, cvt.rn.bf16.f32).
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// fp32 L[i][j] as a K-major tf32 operand: two blocks of 32 columns (8 KiB each), 128 bytes per row, the 16-byte
// chunks of a row XOR-swizzled by the row (the layout of every operand tile, with 4-byte elements)
__device__ __forceinline__ int wy_l_index(int i, int j) {
  return (j >> 5) * 2048 + i * 32 + ((((j & 31) >> 2) ^ (i & 7)) << 2) + (j & 3);
}
// float index of element (row, k) of a one-block fp32 operand of 32 contraction columns
__device__ __forceinline__ int f32_block_index(int row, int k) { return row * 32 + (((k >> 2) ^ (row & 7)) << 2) + (k & 3); }

// A block-wide abort flag for bounded waits: a thread whose wait ran out raises it, every thread reads it right
// after the next __syncthreads and leaves its loop in step with the others.
struct Abort {
  volatile int* flag;
  __device__ __forceinline__ void raise() { *flag = 1; }
  __device__ __forceinline__ bool raised() const { return *flag != 0; }
  // A bounded wait that also gives up as soon as another thread of the block has raised the flag (warp-specialised
  // kernels, whose roles wait on one another through mbarriers: when one role gives up the others follow at once
  // instead of each running out its own second).  Returns false when the walk must stop.
  __device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity) const {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
      if (mbar_try_wait(bar, parity)) return true;
      if (*flag != 0) return false;
      if (global_timer_ns() - t0 > kWaitLimitNs) {
        *flag = 1;
        return false;
      }
    }
  }
};

}  // namespace mek
