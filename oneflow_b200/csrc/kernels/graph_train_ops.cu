// Kernels that only the TRAINING form of the native graph runtime needs (csrc/api/graph_train_ops.cpp) beside the backward
// kernels the eager path already has (GEMM with transposed operands, attention / LayerNorm / softmax backward, embedding
// scatter-add, column sums, the multi-tensor optimizers): the derivative of the element-wise unary functions, a strided
// accumulate (the backward of every view copy: permute, slice, concatenation) that may widen bf16 to fp32 on the way, and
// deterministic reductions to one fp32 scalar for the loss value. All one-pass and HBM-bound.
//
// Reference counterparts: oneflow/core/ep/cuda/primitive/{elementwise_unary,broadcast_elementwise_binary}.cu (the *_grad
// functors in oneflow/core/ep/common/primitive/unary_functor.h), oneflow/user/kernels/slice_util.cu (slice_grad),
// oneflow/user/kernels/reduce_kernel.cpp.
#include <cuda_bf16.h>

#include "../common/dropout_hash.h"
#include "../common/host_utils.h"
#include "ofb_kernels.h"

namespace ofb {

using bf16 = __nv_bfloat16;

// y = x * keep / (1 - p); the call counter is read from device memory so that a recorded launch draws a new mask on every
// replay. 8 elements (two draws) per thread and iteration.
__global__ void gtr_dropout_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long n, unsigned long long seed,
                                   const unsigned long long* __restrict__ counter, unsigned int op_index, float p, bool vec) {
  const uint64_t base = dropout_base(seed, *counter, op_index);
  const uint32_t thr = dropout_threshold(p);
  const float scale = p < 1.f ? 1.f / (1.f - p) : 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long groups8 = (n + 7) / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < groups8; i += stride) {
    const uint64_t d0 = dropout_draw(base, 2 * i), d1 = dropout_draw(base, 2 * i + 1);
    if (vec && i * 8 + 8 <= n) {
      uint4 q = reinterpret_cast<const uint4*>(x)[i];
      bf16* e = reinterpret_cast<bf16*>(&q);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool keep = dropout_keep(j < 4 ? d0 : d1, j & 3, thr);
        e[j] = __float2bfloat16(keep ? __bfloat162float(e[j]) * scale : 0.f);
      }
      reinterpret_cast<uint4*>(y)[i] = q;
    } else {
      for (int j = 0; j < 8 && i * 8 + j < n; ++j) {
        const bool keep = dropout_keep(j < 4 ? d0 : d1, j & 3, thr);
        y[i * 8 + j] = __float2bfloat16(keep ? __bfloat162float(x[i * 8 + j]) * scale : 0.f);
      }
    }
  }
}

// d fn(x) / dx for the function codes of ofb_graph_unary
__device__ __forceinline__ float gtr_unary_grad(float x, int fn, float alpha) {
  switch (fn) {
    case 0: return alpha;
    case 1: return 0.5f * (1.f + erff(x * 0.7071067811865476f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
    case 2: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      const float t = tanhf(u);
      return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
    }
    case 3: return x > 0.f ? 1.f : 0.f;
    case 4: {
      const float t = tanhf(x);
      return 1.f - t * t;
    }
    case 5: {
      const float s = 1.f / (1.f + __expf(-x));
      return s * (1.f - s);
    }
    case 6: {
      const float s = 1.f / (1.f + __expf(-x));
      return s * (1.f + x * (1.f - s));
    }
    case 7: return 1.f;
    case 8: return __expf(x);
    case 9: return -0.5f * rsqrtf(x) / x;
    case 10: return 2.f * x;
    default: return 1.f;
  }
}

struct alignas(16) GtrBf16x8 {
  bf16 v[8];
};

__global__ void gtr_unary_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy, bf16* __restrict__ dx, long long n, int fn,
                                     float alpha, bool vec) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long nv = vec ? n / 8 : 0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += stride) {
    const GtrBf16x8 a = reinterpret_cast<const GtrBf16x8*>(x)[i], g = reinterpret_cast<const GtrBf16x8*>(dy)[i];
    GtrBf16x8 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = __float2bfloat16(__bfloat162float(g.v[j]) * gtr_unary_grad(__bfloat162float(a.v[j]), fn, alpha));
    reinterpret_cast<GtrBf16x8*>(dx)[i] = o;
  }
  for (long long i = nv * 8 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride)
    dx[i] = __float2bfloat16(__bfloat162float(dy[i]) * gtr_unary_grad(__bfloat162float(x[i]), fn, alpha));
}

struct AccView {
  long long shape[5], in_stride[5], out_stride[5], in_offset, out_offset;
};

__device__ __forceinline__ float gtr_load(const float* p, long long i) { return p[i]; }
__device__ __forceinline__ float gtr_load(const bf16* p, long long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void gtr_store(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void gtr_store(bf16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

// y[out view] += x[in view]; the out view must not visit an element twice (no zero strides over an extent > 1)
template <typename TI, typename TO>
__global__ void gtr_strided_acc_kernel(const TI* __restrict__ x, TO* __restrict__ y, AccView v, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
    long long r = i, in = v.in_offset, out = v.out_offset;
#pragma unroll
    for (int d = 4; d >= 0; --d) {
      const long long c = r % v.shape[d];
      r /= v.shape[d];
      in += c * v.in_stride[d];
      out += c * v.out_stride[d];
    }
    gtr_store(y, out, gtr_load(y, out) + gtr_load(x, in));
  }
}

// y[i] += x[i] on contiguous bf16 data, 8 elements (16 bytes) per access
__global__ void gtr_acc_bf16x8_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long nv) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += stride) {
    const GtrBf16x8 a = reinterpret_cast<const GtrBf16x8*>(x)[i];
    GtrBf16x8 b = reinterpret_cast<const GtrBf16x8*>(y)[i];
#pragma unroll
    for (int j = 0; j < 8; ++j) b.v[j] = __float2bfloat16(__bfloat162float(b.v[j]) + __bfloat162float(a.v[j]));
    reinterpret_cast<GtrBf16x8*>(y)[i] = b;
  }
}

__device__ __forceinline__ float gtr_block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    v = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  }
  __syncthreads();
  return v;   // valid in warp 0
}

// partial[b] = sum over this CTA's slice of (a - b)^2 (b given) or of x (fp32 input)
__global__ void gtr_sq_diff_partial_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, float* __restrict__ partial, long long n) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
    const float d = __bfloat162float(a[i]) - __bfloat162float(b[i]);
    acc += d * d;
  }
  acc = gtr_block_sum(acc, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}

// out[0] = scale * sum(x[0..n)), one CTA, fixed summation order (the same bits on every run)
__global__ void gtr_sum_f32_kernel(const float* __restrict__ x, float* __restrict__ out, long long n, float scale) {
  __shared__ float red[32];
  float acc = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) acc += x[i];
  acc = gtr_block_sum(acc, red);
  if (threadIdx.x == 0) out[0] = acc * scale;
}

static unsigned gtr_grid(long long work) {
  long long blocks = (work + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return blocks < 1 ? 1u : static_cast<unsigned>(blocks);
}

}  // namespace ofb

using namespace ofb;

// y = dropout(x) on n bf16 elements with the counter-based mask of common/dropout_hash.h; `counter` points to the call
// counter in device memory.
OFB_API int ofb_graph_dropout(const void* x, void* y, long long n, unsigned long long seed, const unsigned long long* counter,
                              unsigned int op_index, float p, void* stream) {
  if (n <= 0) return 0;
  if (!counter) return fail("graph_dropout: the call counter is required");
  if (!(p >= 0.f && p <= 1.f)) return fail("graph_dropout: p must be in [0, 1]");
  const bool vec = !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15);
  gtr_dropout_kernel<<<gtr_grid((n + 7) / 8), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, n, seed, counter, op_index, p, vec);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// dx = dy * fn'(x) on n bf16 elements; fn and alpha as in ofb_graph_unary.
OFB_API int ofb_graph_unary_bwd(const void* x, const void* dy, void* dx, long long n, int fn, float alpha, void* stream) {
  if (n <= 0) return 0;
  const bool vec = !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) & 15);
  gtr_unary_bwd_kernel<<<gtr_grid((n + 7) / 8), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (const bf16*)dy, (bf16*)dx, n, fn, alpha, vec);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// y[out view] += x[in view] over ndim <= 5 axes; dtype codes: 0 fp32, 1 bf16 (x and y may differ). The out view must be
// injective: an axis longer than 1 with out stride 0 is refused.
OFB_API int ofb_graph_strided_acc(const void* x, int x_dtype, void* y, int y_dtype, int ndim, const long long* shape,
                                  const long long* in_strides, long long in_offset, const long long* out_strides, long long out_offset,
                                  void* stream) {
  if (ndim < 1 || ndim > 5) return fail("graph_strided_acc: 1 to 5 axes");
  AccView v;
  long long n = 1;
  for (int d = 0; d < 5; ++d) {
    const int s = d - (5 - ndim);
    v.shape[d] = s >= 0 ? shape[s] : 1;
    v.in_stride[d] = s >= 0 ? in_strides[s] : 0;
    v.out_stride[d] = s >= 0 ? out_strides[s] : 0;
    if (v.shape[d] <= 0) return 0;
    if (v.shape[d] > 1 && v.out_stride[d] == 0) return fail("graph_strided_acc: the destination view repeats elements");
    n *= v.shape[d];
  }
  v.in_offset = in_offset;
  v.out_offset = out_offset;
  auto s = (cudaStream_t)stream;
  // both views contiguous (the usual case: a whole gradient added to a whole gradient): 16-byte accesses
  bool dense = x_dtype == 1 && y_dtype == 1 && n % 8 == 0;
  long long expect = 1;
  for (int d = 4; d >= 0 && dense; --d) {
    if (v.shape[d] > 1 && (v.in_stride[d] != expect || v.out_stride[d] != expect)) dense = false;
    expect *= v.shape[d];
  }
  if (dense) {
    const bf16* xs = (const bf16*)x + in_offset;
    bf16* ys = (bf16*)y + out_offset;
    if (((reinterpret_cast<uintptr_t>(xs) | reinterpret_cast<uintptr_t>(ys)) & 15) == 0) {
      gtr_acc_bf16x8_kernel<<<gtr_grid(n / 8), 256, 0, s>>>(xs, ys, n / 8);
      OFB_CUDA_OK(cudaGetLastError());
      return 0;
    }
  }
  const unsigned g = gtr_grid(n);
  if (x_dtype == 1 && y_dtype == 1) gtr_strided_acc_kernel<bf16, bf16><<<g, 256, 0, s>>>((const bf16*)x, (bf16*)y, v, n);
  else if (x_dtype == 1 && y_dtype == 0) gtr_strided_acc_kernel<bf16, float><<<g, 256, 0, s>>>((const bf16*)x, (float*)y, v, n);
  else if (x_dtype == 0 && y_dtype == 0) gtr_strided_acc_kernel<float, float><<<g, 256, 0, s>>>((const float*)x, (float*)y, v, n);
  else if (x_dtype == 0 && y_dtype == 1) gtr_strided_acc_kernel<float, bf16><<<g, 256, 0, s>>>((const float*)x, (bf16*)y, v, n);
  else return fail("graph_strided_acc: dtype codes are 0 (fp32) and 1 (bf16)");
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// Number of fp32 partial sums ofb_graph_mse needs as scratch.
OFB_API int ofb_graph_mse_parts(void) { return 148 * 4; }

// loss[0] = mean((a - b)^2) over n bf16 elements; scratch: ofb_graph_mse_parts() floats.
OFB_API int ofb_graph_mse(const void* a, const void* b, float* loss, float* scratch, long long n, void* stream) {
  if (n <= 0) return fail("graph_mse: empty input");
  long long blocks = (n + 1023) / 1024;
  if (blocks > 148 * 4) blocks = 148 * 4;
  gtr_sq_diff_partial_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const bf16*)a, (const bf16*)b, scratch, n);
  OFB_CUDA_OK(cudaGetLastError());
  gtr_sum_f32_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(scratch, loss, blocks, 1.f / static_cast<float>(n));
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// out[0] = scale * sum of n fp32 values (one CTA; meant for per-row losses and other short vectors).
OFB_API int ofb_graph_sum_f32(const float* x, float* out, long long n, float scale, void* stream) {
  if (n < 0) return fail("graph_sum_f32: negative length");
  gtr_sum_f32_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(x, out, n, scale);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
