// An allocation-free forward of the gated delta rule for callers that must not allocate device memory.
//
// Who needs it: an inference server or a training runtime that reserves all of its device memory up front (a fixed
// memory plan, a real-time loop, a process without an allocator of its own such as a plain C host) cannot call
// cudaMalloc or a framework allocator between its setup and its hot loop.  The regular forward needs intermediate
// tensors (the cumulative gate, the WY tensors w and u, the corrected values v_new, the per-chunk state tape h and the
// per-chunk matrices A and Aqk) that its caller allocates.  Here they live in one file-scope device array of fixed
// size, so the call takes only its inputs and its outputs.
//
// Limits and rules of use:
//   * total_tokens * num_v_heads <= 8192 and num_chunks * num_v_heads <= 256 (about 18 MiB of scratch, held by every
//     GPU that loads the library until the process exits); larger calls are rejected with MEK_ERR_INVALID;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress); make that first call
//     before any stream capture;
//   * the array that is used is the CURRENT device's: the host thread's current device must be the one that owns the
//     operands and the stream (checked against q; a mismatch is MEK_ERR_INVALID);
//   * every call on a device uses the same array: two calls that overlap on the GPU (different streams) race, so
//     order them on one stream or with events; the array keeps the previous call's contents, and nothing in it has to
//     start at zero (every element a kernel reads was written earlier in the same call);
//   * no cudaMalloc, cudaFree or allocating library routine is called.
#include <mutex>

#include "common.cuh"

namespace {

constexpr int64_t kMaxTokenHeads = 8192;  // total_tokens * num_v_heads
constexpr int64_t kMaxChunkHeads = 256;   // num_chunks * num_v_heads
constexpr size_t kGcsBytes = kMaxTokenHeads * 4;
constexpr size_t kRowBytes = kMaxTokenHeads * 256;   // one [T, HV, 128] bf16 tensor
constexpr size_t kMatBytes = kMaxChunkHeads * 8192;  // one [NC, HV, 64, 64] bf16 tensor
constexpr size_t kTapeBytes = kMaxChunkHeads * 32768;  // [NC, HV, 128, 128] bf16
constexpr size_t kOffGcs = 0;
constexpr size_t kOffW = kOffGcs + kGcsBytes;
constexpr size_t kOffU = kOffW + kRowBytes;
constexpr size_t kOffVNew = kOffU + kRowBytes;
constexpr size_t kOffA = kOffVNew + kRowBytes;
constexpr size_t kOffAqk = kOffA + kMatBytes;
constexpr size_t kOffH = kOffAqk + kMatBytes;
constexpr size_t kScratchBytes = kOffH + kTapeBytes;

// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer to pass to a kernel.
static __device__ __align__(256) unsigned char g_forward_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_address[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

// The device address of the scratch array on the current device; looked up once per device.
int scratch_for_current_device(unsigned char** out) {
  using namespace mek;
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return fail(MEK_ERR_CUDA, "forward_static: cudaGetDevice: %s", cudaGetErrorString(err));
  if (device < 0 || device >= kMaxDevices)
    return fail(MEK_ERR_INVALID, "forward_static: device index %d is outside 0..%d", device, kMaxDevices - 1);
  std::lock_guard<std::mutex> guard(g_setup_mutex);
  if (g_scratch_address[device] == nullptr) {
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, g_forward_scratch);
    if (err != cudaSuccess || address == nullptr)
      return fail(MEK_ERR_CUDA, "forward_static: cudaGetSymbolAddress on device %d: %s", device,
                  cudaGetErrorString(err));
    g_scratch_address[device] = static_cast<unsigned char*>(address);
  }
  *out = g_scratch_address[device];
  return MEK_OK;
}

}  // namespace

extern "C" int mek_gdn_forward_static(const MekGdnDims* d, const void* q, const void* k, const void* v,
                                      const float* beta, const float* g, const float* h0, void* o, float* final_state,
                                      int32_t* status, void* stream) {
  using namespace mek;
  if (d == nullptr) return fail(MEK_ERR_INVALID, "forward_static: dims is null");
  if (!q || !k || !v || !beta || !g || !o || !status)
    return fail(MEK_ERR_INVALID, "forward_static: q, k, v, beta, g, o and status must not be null");
  if (d->total_tokens <= 0 || d->num_chunks <= 0 || d->num_v_heads <= 0)
    return fail(MEK_ERR_INVALID, "forward_static: no tokens");
  const int64_t token_heads = d->total_tokens * d->num_v_heads;
  const int64_t chunk_heads = int64_t(d->num_chunks) * d->num_v_heads;
  if (token_heads > kMaxTokenHeads || chunk_heads > kMaxChunkHeads)
    return fail(MEK_ERR_INVALID,
                "forward_static: total_tokens * num_v_heads = %lld (limit %lld) and num_chunks * num_v_heads = %lld "
                "(limit %lld): the call does not fit the fixed scratch; use the forward stages with caller-allocated "
                "tensors",
                (long long)token_heads, (long long)kMaxTokenHeads, (long long)chunk_heads, (long long)kMaxChunkHeads);
  {  // the scratch is the current device's: the operands must live there too
    int current = -1;
    cudaPointerAttributes where;
    if (cudaGetDevice(&current) != cudaSuccess || cudaPointerGetAttributes(&where, q) != cudaSuccess) {
      cudaGetLastError();
      return fail(MEK_ERR_CUDA, "forward_static: cannot tell which device holds q");
    }
    if (where.type != cudaMemoryTypeDevice || where.device != current)
      return fail(MEK_ERR_INVALID,
                  "forward_static: q is not in the memory of the current device (%d): set the device that owns the "
                  "operands and the stream before the call", current);
  }
  unsigned char* base = nullptr;
  if (int rc = scratch_for_current_device(&base)) return rc;
  float* g_cs = reinterpret_cast<float*>(base + kOffGcs);
  void *w = base + kOffW, *u = base + kOffU, *v_new = base + kOffVNew;
  void *a = base + kOffA, *aqk = base + kOffAqk, *h = base + kOffH;
  if (int rc = mek_gdn_gate_cumsum(d, g, g_cs, stream)) return rc;
  if (int rc = mek_gdn_wy_fwd(d, q, k, v, beta, g_cs, a, aqk, w, u, status, stream)) return rc;
  if (int rc = mek_gdn_fwd_h(d, k, w, u, g_cs, h0, h, v_new, final_state, status, stream)) return rc;
  return mek_gdn_fwd_o(d, q, aqk, v_new, h, g_cs, o, status, stream);
}
