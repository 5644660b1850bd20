// Tensor Memory Accelerator (TMA) tile loads for the gated-delta-rule kernels, sm_100a.
//
// Every operand tile of these kernels is a stack of 64-column bf16 blocks in the 128-byte swizzled layout of
// umma.cuh.  A 2-D tensor map with SWIZZLE_128B and a box of 64 columns x R rows writes exactly one such block, so
// one elected thread moves a whole tile with one or two instructions and the copy completes on an mbarrier
// (transaction bytes), with no per-thread address arithmetic and no generic-proxy stores.
//
// Two shapes of tensor are mapped:
//   rows   [tokens, heads * 128]  (q, k, v, dO, v_new, w, u ...): box 64 x 64 rows at (head * 128 + {0, 64}, token).
//          Rows past the tensor's end are zero-filled by the hardware; rows of a ragged chunk that belong to the
//          next sequence are NOT -- the kernels clear them after the copy has landed.
//   tiles  [num_tiles * R, C]     (state tapes 128 x 128, A / Aqk 64 x 64): box 64 x R at ({0, 64}, tile * R).
// The innermost coordinate is always a multiple of 64 elements (128 bytes), inside the 16-byte rule of the copy.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "umma.cuh"

namespace mek {

// ---------------------------------------------------------------------------------------------------------------
// host: tensor maps
// ---------------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's encoder, looked up once through the runtime (the library does not link against the driver).
inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) != cudaSuccess ||
        res != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      p = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// A bf16 matrix [rows, cols] (row stride = `pitch` elements, 0 = cols) read in boxes of 64 columns x box_rows rows.
inline int make_tile_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                         const char* what, uint64_t pitch = 0) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return fail(MEK_ERR_CUDA, "%s: the driver does not export cuTensorMapEncodeTiled", what);
  if (base == nullptr || (reinterpret_cast<uintptr_t>(base) & 15) != 0 || cols % 64 != 0 || rows == 0 ||
      box_rows == 0 || box_rows > 256)
    return fail(MEK_ERR_INVALID, "%s: a tensor map needs a 16-byte aligned base, columns in multiples of 64 and 1..256 "
                "box rows (rows=%llu cols=%llu box_rows=%u)", what, (unsigned long long)rows,
                (unsigned long long)cols, box_rows);
  if (pitch != 0 && (pitch < cols || pitch % 8 != 0))
    return fail(MEK_ERR_INVALID, "%s: a row pitch must be a multiple of 8 elements and at least the row's %llu columns, "
                "got %llu", what, (unsigned long long)cols, (unsigned long long)pitch);
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {(pitch != 0 ? pitch : cols) * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                             elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return fail(MEK_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed (%d)", what, int(rc));
  return MEK_OK;
}

// rows [tokens, heads * 128], read in boxes of 64 columns x 64 tokens
inline int make_rows_map(CUtensorMap* map, const void* base, int64_t tokens, int heads, const char* what,
                         int64_t pitch = 0) {
  return make_tile_map(map, base, uint64_t(tokens), uint64_t(heads) * 128, 64, what, uint64_t(pitch));
}
// tiles [num_tiles * rows, cols], read in boxes of 64 columns x `rows` rows
inline int make_tiles_map(CUtensorMap* map, const void* base, int64_t num_tiles, int rows, int cols, const char* what) {
  return make_tile_map(map, base, uint64_t(num_tiles) * rows, uint64_t(cols), uint32_t(rows), what);
}

// ---------------------------------------------------------------------------------------------------------------
// device
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// One arrival on the barrier that also announces `bytes` of copies which will complete on it.
__device__ __forceinline__ void mbar_arrive_expect(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// One box (64 columns x the map's box rows) whose first element is (x, y) -> shared memory at `dst` (1024-byte
// aligned); completes `box bytes` on the barrier.  x must be a multiple of 8 elements (16 bytes).
__device__ __forceinline__ void tma_load_box(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// A [R x 128] tile = two boxes, `block_stride` bytes apart in shared memory.
__device__ __forceinline__ void tma_load_tile128(uint32_t dst, uint32_t block_stride, const CUtensorMap* map, int x,
                                                 int y, uint64_t* bar) {
  tma_load_box(dst, map, x, y, bar);
  tma_load_box(dst + block_stride, map, x + 64, y, bar);
}

// The same tile, asked into L2 only: a later copy of it into shared memory finds it there.
__device__ __forceinline__ void tma_prefetch_tile128(const CUtensorMap* map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(map)),
               "r"(x), "r"(y)
               : "memory");
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(map)),
               "r"(x + 64), "r"(y)
               : "memory");
}

// One box (64 columns x the map's box rows) from shared memory at `src` (1024-byte aligned, the swizzled block
// layout) to the tensor at (x, y); joins the issuing thread's current bulk group.  Generic-proxy writes to the block
// must have been fenced (fence.proxy.async) by their writers before the issuing thread learns of them.
__device__ __forceinline__ void tma_store_box(const CUtensorMap* map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_tile128(const CUtensorMap* map, int x, int y, uint32_t src,
                                                  uint32_t block_stride) {
  tma_store_box(map, x, y, src);
  tma_store_box(map, x + 64, y, src + block_stride);
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until the bulk stores this thread committed have READ their shared-memory source (the source may be rewritten).
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Until they have completed (the data is in global memory).
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Clears the rows [first, 64) of a [64 x 128] tile (two 8 KiB blocks): the part of a ragged chunk's box that holds
// another sequence's tokens.  Every thread of the `NT` calling threads takes part.
template <int NT>
__device__ __forceinline__ void clear_tile_rows(uint8_t* tile, int first, int tid) {
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (int i = first * 8 + tid; i < 64 * 8; i += NT) {  // a row of a block is 8 chunks of 16 bytes, swizzled in place
    *reinterpret_cast<uint4*>(tile + i * 16) = zero;
    *reinterpret_cast<uint4*>(tile + 8192 + i * 16) = zero;
  }
}

}  // namespace mek
