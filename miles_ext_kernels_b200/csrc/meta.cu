// Chunk tables of a packed batch from its device `cu_seqlens`, without a host round trip: one launch, integer work
// only (reference: the `meta` kernel behind miles_ext_kernels/cake/_impl/gdn/ops.py:311-376, 1808-1858).
//
// The host cannot know the chunk count without reading cu_seqlens, so the tables have the padded extent
// bound = ceil(total_tokens / 64) + num_seqs (every sequence can add at most one ragged chunk); entries past the
// real chunk count are pad chunks: length 0, start 0, the last sequence's index.
#include "common.cuh"

namespace mek {

template <typename Offset>
__global__ void __launch_bounds__(1024) chunk_meta_kernel(const Offset* __restrict__ cu, int num_seqs, int bound,
                                                          int32_t* __restrict__ chunk_start,
                                                          int32_t* __restrict__ chunk_len,
                                                          int32_t* __restrict__ chunk_seq,
                                                          int32_t* __restrict__ seq_chunk_start) {
  __shared__ int s_part[1024];
  const int tid = threadIdx.x;
  // exclusive prefix sum of the sequences' chunk counts: a contiguous run of sequences per thread, then a scan of
  // the threads' partial sums
  const int per = (num_seqs + 1023) / 1024;
  const int begin = min(tid * per, num_seqs), end = min(begin + per, num_seqs);
  int mine = 0;
  for (int n = begin; n < end; ++n) {
    const long long len = (long long)cu[n + 1] - (long long)cu[n];
    mine += int((max(len, 0ll) + 63) / 64);
  }
  s_part[tid] = mine;
  __syncthreads();
  for (int offset = 1; offset < 1024; offset <<= 1) {
    const int add = tid >= offset ? s_part[tid - offset] : 0;
    __syncthreads();
    s_part[tid] += add;
    __syncthreads();
  }
  int first = s_part[tid] - mine;  // chunks before this thread's run
  const int total = s_part[1023];
  for (int n = begin; n < end; ++n) {
    const long long lo = cu[n], hi = cu[n + 1];
    const int chunks = int((max(hi - lo, 0ll) + 63) / 64);
    seq_chunk_start[n] = first;
    for (int c = 0; c < chunks; ++c) {
      if (first + c < bound) {
        chunk_start[first + c] = int32_t(lo + 64ll * c);
        chunk_len[first + c] = int32_t(min(64ll, hi - lo - 64ll * c));
        chunk_seq[first + c] = n;
      }
    }
    first += chunks;
  }
  if (tid == 0) seq_chunk_start[num_seqs] = total;
  for (int c = total + tid; c < bound; c += 1024) {  // pad chunks
    chunk_start[c] = 0;
    chunk_len[c] = 0;
    chunk_seq[c] = num_seqs - 1;
  }
}

}  // namespace mek

extern "C" int mek_gdn_chunk_meta(const void* cu_seqlens, int offsets_are_int64, int num_seqs, int bound,
                                  int32_t* chunk_start, int32_t* chunk_len, int32_t* chunk_seq,
                                  int32_t* seq_chunk_start, void* stream) {
  using namespace mek;
  if (!cu_seqlens || num_seqs <= 0 || bound <= 0 || !chunk_start || !chunk_len || !chunk_seq || !seq_chunk_start)
    return fail(MEK_ERR_INVALID, "chunk_meta: a null pointer, no sequences or no room for chunks");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (offsets_are_int64)
    chunk_meta_kernel<long long><<<1, 1024, 0, s>>>(static_cast<const long long*>(cu_seqlens), num_seqs, bound,
                                                    chunk_start, chunk_len, chunk_seq, seq_chunk_start);
  else
    chunk_meta_kernel<int><<<1, 1024, 0, s>>>(static_cast<const int*>(cu_seqlens), num_seqs, bound, chunk_start,
                                              chunk_len, chunk_seq, seq_chunk_start);
  return launched("chunk_meta");
}
