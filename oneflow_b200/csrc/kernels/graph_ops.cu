// Small data-movement and element-wise kernels the native graph runtime (csrc/api/graph_runtime.cpp) needs beside the
// GEMM / attention / LayerNorm / softmax kernels: unary and binary element-wise ops on bf16 with row broadcasting, a
// strided copy (permute, slice, concatenation: any 5-D view -> contiguous), and a row gather for embeddings. All are
// HBM-bound one-pass kernels with 16-byte accesses where the layout allows.
//
// Reference counterparts: oneflow/core/ep/cuda/primitive/{elementwise_unary,broadcast_elementwise_binary,permute,copy_nd}.cu
// and oneflow/user/kernels/gather_kernel_util.cu.
#include <cuda_bf16.h>

#include "../common/host_utils.h"
#include "ofb_kernels.h"

namespace ofb {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float gop_unary(float x, int fn, float alpha) {
  switch (fn) {
    case 0: return x * alpha;                                             // scale
    case 1: return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));      // gelu (erf)
    case 2: {                                                             // gelu (tanh)
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanhf(u));
    }
    case 3: return fmaxf(x, 0.f);                                         // relu
    case 4: return tanhf(x);
    case 5: return 1.f / (1.f + __expf(-x));                              // sigmoid
    case 6: return x / (1.f + __expf(-x));                                // silu
    case 7: return x + alpha;                                             // add scalar
    case 8: return __expf(x);
    case 9: return rsqrtf(x);
    case 10: return x * x;
    default: return x;
  }
}
__device__ __forceinline__ float gop_binary(float a, float b, int op) {
  switch (op) {
    case 0: return a + b;
    case 1: return a - b;
    case 2: return a * b;
    case 3: return a / b;
    case 4: return fmaxf(a, b);
    default: return fminf(a, b);
  }
}

struct alignas(16) Bf16x8 {
  bf16 v[8];
};

__global__ void gop_unary_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long n, int fn, float alpha) {
  const long long nv = n / 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += stride) {
    Bf16x8 a = reinterpret_cast<const Bf16x8*>(x)[i], o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = __float2bfloat16(gop_unary(__bfloat162float(a.v[j]), fn, alpha));
    reinterpret_cast<Bf16x8*>(y)[i] = o;
  }
  for (long long i = nv * 8 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = __float2bfloat16(gop_unary(__bfloat162float(x[i]), fn, alpha));
}

// b_mode 0: b has n elements; 1: b has `cols` elements and repeats along the rows (y[r, c] = a[r, c] op b[c]);
// 2: b has n / cols elements, one per row (y[r, c] = a[r, c] op b[r]).
__global__ void gop_binary_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, bf16* __restrict__ y, long long n,
                                  long long cols, int b_mode, int op) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long bi = b_mode == 0 ? i : (b_mode == 1 ? i % cols : i / cols);
    y[i] = __float2bfloat16(gop_binary(__bfloat162float(a[i]), __bfloat162float(b[bi]), op));
  }
}
__global__ void gop_binary_vec_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, bf16* __restrict__ y, long long n,
                                      long long cols, int b_mode, int op) {
  // n, cols multiples of 8; b_mode 0 or 1
  const long long nv = n / 8, cv = cols / 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += stride) {
    const Bf16x8 av = reinterpret_cast<const Bf16x8*>(a)[i];
    const Bf16x8 bv = reinterpret_cast<const Bf16x8*>(b)[b_mode == 0 ? i : i % cv];
    Bf16x8 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = __float2bfloat16(gop_binary(__bfloat162float(av.v[j]), __bfloat162float(bv.v[j]), op));
    reinterpret_cast<Bf16x8*>(y)[i] = o;
  }
}

struct CopyView {
  long long shape[5];     // output shape (contiguous), padded with leading 1s
  long long stride[5];    // input strides in elements for the same axes
  long long in_offset;    // elements
  long long out_stride0[5];  // output strides (contiguous unless the copy writes into a slice of a larger tensor)
  long long out_offset;
};

template <typename T>
__global__ void gop_strided_copy_kernel(const T* __restrict__ x, T* __restrict__ y, CopyView v, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
    long long r = i, in = v.in_offset, out = v.out_offset;
#pragma unroll
    for (int d = 4; d >= 0; --d) {
      const long long c = r % v.shape[d];
      r /= v.shape[d];
      in += c * v.stride[d];
      out += c * v.out_stride0[d];
    }
    y[out] = x[in];
  }
}

__global__ void gop_gather_rows_kernel(const long long* __restrict__ ids, const bf16* __restrict__ table, bf16* __restrict__ out,
                                       long long n_ids, int cols, long long table_rows) {
  const int vec = cols / 8;
  const long long total = n_ids * vec;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / vec;
    const int c = static_cast<int>(i % vec);
    long long id = ids[r];
    Bf16x8 v;
    if (id >= 0 && id < table_rows) {
      v = reinterpret_cast<const Bf16x8*>(table + id * cols)[c];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v.v[j] = __float2bfloat16(0.f);
    }
    reinterpret_cast<Bf16x8*>(out + r * cols)[c] = v;
  }
}

static unsigned gop_grid(long long work) {
  long long blocks = (work + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return blocks < 1 ? 1u : static_cast<unsigned>(blocks);
}

}  // namespace ofb

using namespace ofb;

// y = fn(x) on n bf16 elements. fn: 0 scale by alpha, 1 gelu, 2 gelu(tanh), 3 relu, 4 tanh, 5 sigmoid, 6 silu, 7 add alpha,
// 8 exp, 9 rsqrt, 10 square.
OFB_API int ofb_graph_unary(const void* x, void* y, long long n, int fn, float alpha, void* stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) return fail("graph_unary: operands must be 16-byte aligned");
  gop_unary_kernel<<<gop_grid((n + 7) / 8), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, n, fn, alpha);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// y = a op b on n bf16 elements; op: 0 add, 1 sub, 2 mul, 3 div, 4 max, 5 min. b_mode: 0 same shape, 1 b is one row of
// `cols` elements repeated over the rows, 2 b is one value per row.
OFB_API int ofb_graph_binary(const void* a, const void* b, void* y, long long n, long long cols, int b_mode, int op, void* stream) {
  if (n <= 0) return 0;
  if (b_mode < 0 || b_mode > 2 || (b_mode != 0 && (cols <= 0 || n % cols))) return fail("graph_binary: bad broadcast description");
  const bool aligned = !((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(y)) & 15);
  if (aligned && b_mode != 2 && n % 8 == 0 && (b_mode == 0 || cols % 8 == 0))
    gop_binary_vec_kernel<<<gop_grid(n / 8), 256, 0, (cudaStream_t)stream>>>((const bf16*)a, (const bf16*)b, (bf16*)y, n, cols, b_mode, op);
  else
    gop_binary_kernel<<<gop_grid(n), 256, 0, (cudaStream_t)stream>>>((const bf16*)a, (const bf16*)b, (bf16*)y, n, cols, b_mode, op);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// Copies a strided view of x (ndim <= 5 axes: shape, element strides, element offset) into y, laid out with out_strides
// from out_offset (a contiguous tensor, or a slice of one: concatenation). elem_bytes: 2, 4 or 8.
OFB_API int ofb_graph_strided_copy(const void* x, void* y, int ndim, const long long* shape, const long long* in_strides,
                                   long long in_offset, const long long* out_strides, long long out_offset, int elem_bytes,
                                   void* stream) {
  if (ndim < 1 || ndim > 5) return fail("graph_strided_copy: 1 to 5 axes");
  CopyView v;
  long long n = 1;
  for (int d = 0; d < 5; ++d) {
    const int s = d - (5 - ndim);
    v.shape[d] = s >= 0 ? shape[s] : 1;
    v.stride[d] = s >= 0 ? in_strides[s] : 0;
    v.out_stride0[d] = s >= 0 ? out_strides[s] : 0;
    if (v.shape[d] <= 0) return 0;
    n *= v.shape[d];
  }
  v.in_offset = in_offset;
  v.out_offset = out_offset;
  auto s = (cudaStream_t)stream;
  if (elem_bytes == 2) gop_strided_copy_kernel<unsigned short><<<gop_grid(n), 256, 0, s>>>((const unsigned short*)x, (unsigned short*)y, v, n);
  else if (elem_bytes == 4) gop_strided_copy_kernel<unsigned int><<<gop_grid(n), 256, 0, s>>>((const unsigned int*)x, (unsigned int*)y, v, n);
  else if (elem_bytes == 8) gop_strided_copy_kernel<unsigned long long><<<gop_grid(n), 256, 0, s>>>((const unsigned long long*)x, (unsigned long long*)y, v, n);
  else return fail("graph_strided_copy: element size must be 2, 4 or 8 bytes");
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// out[i, :] = table[ids[i], :] (zeros for ids outside [0, table_rows)); cols a multiple of 8.
OFB_API int ofb_graph_gather_rows(const long long* ids, const void* table, void* out, long long n_ids, int cols, long long table_rows,
                                  void* stream) {
  if (cols % 8) return fail("graph_gather_rows: the row length must be a multiple of 8");
  if (n_ids <= 0) return 0;
  gop_gather_rows_kernel<<<gop_grid(n_ids * (cols / 8)), 256, 0, (cudaStream_t)stream>>>(ids, (const bf16*)table, (bf16*)out, n_ids, cols,
                                                                                       table_rows);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
