// Token / position embedding lookup and its gradient (dense nn.Embedding path).
//   forward : out[t, :] = wte[ids[t] - vocab_start, :] (+ wpe[t % seq, :]); rows whose id lies outside
//             this rank's vocabulary shard produce zeros (vocabulary-parallel: the shards are summed).
//   backward: dwte[id, :] += dout[t, :] (fp32 atomics), dwpe[pos, :] += dout[t, :].
// Reference counterparts: oneflow/user/kernels/embedding_kernel.cu, gather_kernel_util.cu,
// unsorted_segment_sum_kernel_util.cu.
#include "../common/host_utils.h"
#include "../common/ptx.cuh"
#include "ofb_kernels.h"

namespace ofb {

__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ wte,
                                     const __nv_bfloat16* __restrict__ wpe, __nv_bfloat16* __restrict__ out, long long tokens,
                                     int seq, int hidden, long long vocab_start, long long vocab_rows, int pos_offset) {
  const int vec = hidden >> 3;
  const long long total = tokens * vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec;
    const int c = static_cast<int>(i % vec) * 8;
    const long long id = ids[t] - vocab_start;
    float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const bool mine = id >= 0 && id < vocab_rows;
    if (mine) {
      uint4 q = *reinterpret_cast<const uint4*>(wte + id * hidden + c);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16x2(w[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
    }
    if (wpe) {
      const long long pos = (t % seq) + pos_offset;
      uint4 q = *reinterpret_cast<const uint4*>(wpe + pos * hidden + c);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16x2(w[j]); v[2 * j] += f.x; v[2 * j + 1] += f.y; }
    }
    *reinterpret_cast<uint4*>(out + t * hidden + c) =
        make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
  }
}

__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dwte, float* __restrict__ dwpe, long long tokens, int seq, int hidden,
                                     long long vocab_start, long long vocab_rows, int pos_offset) {
  const int vec = hidden >> 3;
  const long long total = tokens * vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vec;
    const int c = static_cast<int>(i % vec) * 8;
    uint4 q = *reinterpret_cast<const uint4*>(dout + t * hidden + c);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16x2(w[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
    const long long id = ids[t] - vocab_start;
    if (dwte && id >= 0 && id < vocab_rows) {
      float* dst = dwte + id * hidden + c;
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(dst + j, v[j]);
    }
    if (dwpe) {
      float* dst = dwpe + ((t % seq) + pos_offset) * hidden + c;
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(dst + j, v[j]);
    }
  }
}

}  // namespace ofb

using namespace ofb;

OFB_API int ofb_embedding_fwd(const long long* ids, const void* wte, const void* wpe, void* out, long long tokens, int seq,
                              int hidden, long long vocab_start, long long vocab_rows, int pos_offset, void* stream) {
  if (hidden % 8) return fail("embedding: hidden must be a multiple of 8");
  if (tokens == 0) return 0;
  long long blocks = (tokens * (hidden / 8) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  embedding_fwd_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      ids, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, (__nv_bfloat16*)out, tokens, seq, hidden, vocab_start,
      vocab_rows, pos_offset);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

OFB_API int ofb_embedding_bwd(const long long* ids, const void* dout, float* dwte, float* dwpe, long long tokens, int seq,
                              int hidden, long long vocab_start, long long vocab_rows, int pos_offset, void* stream) {
  if (hidden % 8) return fail("embedding: hidden must be a multiple of 8");
  if (tokens == 0) return 0;
  long long blocks = (tokens * (hidden / 8) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  embedding_bwd_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(ids, (const __nv_bfloat16*)dout, dwte, dwpe,
                                                                          tokens, seq, hidden, vocab_start, vocab_rows,
                                                                          pos_offset);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
