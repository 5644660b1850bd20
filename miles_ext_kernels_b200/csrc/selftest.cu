// Self-test of the tcgen05 building block and the library-wide C-ABI helpers (version stamp, error text, device gate).
#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace mek {

char* error_buffer() {
  static thread_local char text[512] = {0};
  return text;
}

// Operand images are copied verbatim into shared memory; the caller's descriptors decide how the tensor core reads
// them.  128 threads: thread t dumps tensor-memory lane t.
__global__ void __launch_bounds__(128) selftest_umma_kernel(const uint4* a_img, int a_bytes, const uint4* b_img,
                                                            int b_bytes, uint64_t a_desc, uint64_t b_desc,
                                                            const int32_t* a_off, const int32_t* b_off, int nk,
                                                            uint32_t idesc, int ncols, int d_lane, int tf32,
                                                            float* out, int32_t* status) {
  extern __shared__ uint8_t raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  uint4* a_s = reinterpret_cast<uint4*>(base);
  uint4* b_s = reinterpret_cast<uint4*>(base + 65536);
  const uint32_t tid = threadIdx.x, warp = tid >> 5;

  for (int i = tid; i < a_bytes / 16; i += 128) a_s[i] = a_img[i];
  for (int i = tid; i < b_bytes / 16; i += 128) b_s[i] = b_img[i];
  if (tid == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 256);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  // nk == 0: nothing is issued and nothing ever arrives on the barrier -- the wait below must run out by itself and
  // report it (the bounded-wait path every kernel of this library relies on)
  if (tid == 0 && nk > 0) {
    const uint32_t a0 = smem_u32(a_s), b0 = smem_u32(b_s);
    for (int k = 0; k < nk; ++k) {
      const uint64_t da = a_desc | uint64_t(((a0 + uint32_t(a_off[k])) >> 4) & 0x3FFFu);
      const uint64_t db = b_desc | uint64_t(((b0 + uint32_t(b_off[k])) >> 4) & 0x3FFFu);
      if (tf32)
        umma_tf32(tmem + (uint32_t(d_lane) << 16), da, db, idesc, k > 0 ? 1u : 0u);
      else
        umma_f16(tmem + (uint32_t(d_lane) << 16), da, db, idesc, k > 0 ? 1u : 0u);
    }
    umma_commit(&bar);
  }
  const bool done = mbar_wait(&bar, 0);
  tc_fence_after();
  if (done) {
    for (int c0 = 0; c0 < ncols; c0 += 16) {
      float v[16];
      tmem_ld16(tmem_addr(tmem, warp, c0), v);
      tmem_ld_wait();
      for (int j = 0; j < 16; ++j) out[tid * ncols + c0 + j] = v[j];
    }
  } else if (tid == 0) {
    *status = kDevWaitTimeout;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

// One box of a tensor map -> shared memory -> `out`, byte for byte: what the copy engine wrote where.
__global__ void __launch_bounds__(128) selftest_tma_kernel(const __grid_constant__ CUtensorMap map, int x, int y,
                                                           int box_bytes, uint4* out, int32_t* status) {
  extern __shared__ uint8_t raw[];
  __shared__ uint64_t bar;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x;
  if (tid == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (tid == 0) {
    mbar_arrive_expect(&bar, uint32_t(box_bytes));
    tma_load_box(smem_u32(base), &map, x, y, &bar);
  }
  const bool done = mbar_wait(&bar, 0);
  if (done) {
    for (int i = tid; i < box_bytes / 16; i += 128) out[i] = reinterpret_cast<const uint4*>(base)[i];
  } else if (tid == 0) {
    *status = kDevWaitTimeout;
  }
}


// How long the tensor core takes for a run of instructions of one shape: `issuers` threads of different warps (1 or
// 2) each issue `count` products of contraction `kdim` into an accumulator of their own (or, with `interleave`, one
// thread issues twice as many, alternating between two accumulators), commit and wait; thread 0 reports the cycles
// from its first instruction to the last completion.  The operands are zeros (only addresses and
// shapes matter).
template <int M, int N>
__global__ void __launch_bounds__(128) umma_rate_kernel(int a_mn, int b_mn, int kdim, int count, int issuers,
                                                       int interleave, long long* cycles, int32_t* status) {
  extern __shared__ uint8_t raw[];
  __shared__ uint64_t bar[2];
  __shared__ uint32_t tmem_slot;
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x;
  for (int i = tid; i < 196608 / 16; i += 128) reinterpret_cast<uint4*>(sm)[i] = make_uint4(0u, 0u, 0u, 0u);
  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    fence_mbar_init();
  }
  if (tid < 32) tmem_alloc(&tmem_slot, 512);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot, sbase = smem_u32(sm);
  // K-major: [rows][128 columns] as two blocks of rows x 128 bytes; MN-major: [kdim rows][extent columns] as
  // blocks of 128 rows x 128 bytes
  const Operand a{sbase, a_mn ? 16384u : uint32_t(M) * 128u};
  const Operand b{sbase + 65536, b_mn ? 16384u : uint32_t(N) * 128u};
  bool ok = true;
  long long t0 = 0;
  const int who = tid >> 5;
  if (interleave) {  // one thread, the instructions alternating between two accumulators
    if (tid == 0) {
      t0 = clock64();
      for (int i = 0; i < count * int(kdim >> 4); ++i) {
        umma_gemm<M, N>(tmem, a, a_mn != 0, b, b_mn != 0, 16, true);
        umma_gemm<M, N>(tmem + 256, a, a_mn != 0, b, b_mn != 0, 16, true);
      }
      umma_commit(&bar[0]);
    }
    issuers = 1;
  } else if ((tid & 31) == 0 && who < issuers) {
    t0 = clock64();
    for (int i = 0; i < count; ++i) umma_gemm<M, N>(tmem + who * 256, a, a_mn != 0, b, b_mn != 0, kdim, true);
    umma_commit(&bar[who]);
  }
  for (int i = 0; i < issuers; ++i) ok = mbar_wait(&bar[i], 0) && ok;
  tc_fence_after();
  if (tid == 0) {
    cycles[0] = clock64() - t0;
    if (!ok) atomicExch(status, kDevWaitTimeout | (9 << 8));
  }
  tc_fence_before();
  __syncthreads();
  if (tid < 32) tmem_dealloc(tmem, 512);
}

}  // namespace mek

extern "C" {

int mek_build_cuda_version(void) { return CUDART_VERSION; }

const char* mek_last_error(void) { return mek::error_buffer(); }

int mek_check_device(int device) {
  int major = 0, minor = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device) != cudaSuccess) {
    cudaGetLastError();
    return mek::fail(MEK_ERR_CUDA, "cannot query the compute capability of device %d", device);
  }
  if (major != 10 || minor != 0)
    return mek::fail(MEK_ERR_UNSUPPORTED, "the kernels are built for sm_100a (B200), not compute capability %d.%d",
                     major, minor);
  return MEK_OK;
}

int mek_selftest_umma(const void* a_img, int a_bytes, const void* b_img, int b_bytes, uint64_t a_desc, uint64_t b_desc,
                      const int32_t* a_off, const int32_t* b_off, int nk, uint32_t idesc, int ncols, int d_lane,
                      int tf32, float* out, int32_t* status, void* stream) {
  using namespace mek;
  if (a_bytes <= 0 || b_bytes <= 0 || a_bytes > 65536 || b_bytes > 65536 || a_bytes % 16 || b_bytes % 16)
    return fail(MEK_ERR_INVALID, "selftest: operand images must be 16..65536 bytes, multiples of 16");
  if (ncols < 16 || ncols > 256 || ncols % 16 || nk < 0 || nk > 64)
    return fail(MEK_ERR_INVALID, "selftest: ncols in 16..256 (multiple of 16), nk in 0..64");
  if (d_lane != 0 && d_lane != 16) return fail(MEK_ERR_INVALID, "selftest: d_lane must be 0 or 16");
  const size_t smem = 2 * 65536 + 1024;
  if (int rc = want_smem(selftest_umma_kernel, smem, "selftest")) return rc;
  selftest_umma_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(a_img), a_bytes, static_cast<const uint4*>(b_img), b_bytes, a_desc, b_desc, a_off,
      b_off, nk, idesc, ncols, d_lane, tf32, out, status);
  return launched("selftest");
}

int mek_selftest_tma(const void* src, int64_t rows, int64_t cols, int box_rows, int x, int y, void* out,
                     int32_t* status, void* stream) {
  using namespace mek;
  if (rows <= 0 || cols <= 0 || box_rows < 8 || box_rows > 128 || box_rows % 8 || x % 8 || out == nullptr ||
      status == nullptr)
    return fail(MEK_ERR_INVALID, "selftest_tma: box_rows in 8..128 (multiple of 8), x a multiple of 8 elements");
  CUtensorMap map;
  if (int rc = make_tile_map(&map, src, uint64_t(rows), uint64_t(cols), uint32_t(box_rows), "selftest_tma")) return rc;
  const size_t smem = size_t(box_rows) * 128 + 1024;
  selftest_tma_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(map, x, y, box_rows * 128,
                                                                          static_cast<uint4*>(out), status);
  return launched("selftest_tma");
}

int mek_selftest_umma_rate(int m, int n, int a_mn, int b_mn, int kdim, int count, int issuers, int interleave,
                           long long* cycles, int32_t* status, void* stream) {
  using namespace mek;
  if (kdim < 16 || kdim > 128 || kdim % 16 || count < 1 || count > 4096 || issuers < 1 || issuers > 2)
    return fail(MEK_ERR_INVALID, "selftest rate: kdim in 16..128, count in 1..4096, 1 or 2 issuers");
  const size_t smem = 196608 + 1024;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define MEK_RATE(MM, NN)                                                                               \
  if (m == MM && n == NN) {                                                                            \
    if (int rc = want_smem(umma_rate_kernel<MM, NN>, smem, "selftest rate")) return rc;                \
    umma_rate_kernel<MM, NN><<<1, 128, smem, s>>>(a_mn, b_mn, kdim, count, issuers, interleave, cycles, \
                                                  status);                                             \
    return launched("selftest rate");                                                                  \
  }
  MEK_RATE(64, 64) MEK_RATE(64, 128) MEK_RATE(64, 256) MEK_RATE(128, 64) MEK_RATE(128, 128) MEK_RATE(128, 256)
#undef MEK_RATE
  return fail(MEK_ERR_UNSUPPORTED, "selftest rate: M in {64, 128}, N in {64, 128, 256}");
}

}  // extern "C"
