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
 *   out           device float [128 * ncols], row = tensor-memory lane
 *   status        device int32, 0 = fine
 * No counterpart in the reference (its kernels are generated and tested end to end). */
int mek_selftest_umma(const void* a_img, int a_bytes, const void* b_img, int b_bytes, uint64_t a_desc, uint64_t b_desc,
                      const int32_t* a_off, const int32_t* b_off, int nk, uint32_t idesc, int ncols, float* out,
                      int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* MEK_GDN_H_ */
