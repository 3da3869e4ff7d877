// Memory-bound fused elementwise kernels on bf16 activations: 16-byte vector accesses,
// grid sized to a multiple of the SM count, fp32 maths.
//
//   fused_bias_add_gelu(+grad)     oneflow/user/kernels/fused_bias_add_kernel.cu :381,:477
//   fused_bias_add_mask_scale      same file :431   (dropout: mask * (x+b) * scale (+addend))
//   fused_cast_scale               oneflow/user/kernels/fused_cast_scale_kernel.cu :144
//   column_sum (bias gradient)     the BGRADB epilogue of cublas_fused_mlp_grad_kernel.cu
//   dropout mask generation        oneflow/user/kernels/random_mask_generator.cu (philox)
#include <cuda_fp16.h>

#include "../common/host_utils.h"
#include "../common/ptx.cuh"
#include "ofb_kernels.h"

namespace ofb {

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 q = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16x2(w[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

__device__ __forceinline__ float act_fwd(float v, int act) {
  return act == 1 ? gelu_erf(v) : act == 2 ? gelu_tanh(v) : act == 3 ? fmaxf(v, 0.f) : v;
}
__device__ __forceinline__ float act_bwd(float h, int act) {
  return act == 1 ? gelu_erf_grad(h) : act == 2 ? gelu_tanh_grad(h) : act == 3 ? (h > 0.f ? 1.f : 0.f) : 1.f;
}

// y = act(x + bias[col])            (bias may be null)
__global__ void bias_act_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ bias,
                                    __nv_bfloat16* __restrict__ y, long long nvec, int cols, int act) {
  const int cvec = cols >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float v[8];
    load8(x + i * 8, v);
    if (bias) {
      float b[8];
      load8(bias + (i % cvec) * 8, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += b[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = act_fwd(v[j], act);
    store8(y + i * 8, v);
  }
}

// dx = dy * act'(x + bias[col])
__global__ void bias_act_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ bias,
                                    const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx,
                                    long long nvec, int cols, int act) {
  const int cvec = cols >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float v[8], g[8];
    load8(x + i * 8, v);
    load8(dy + i * 8, g);
    if (bias) {
      float b[8];
      load8(bias + (i % cvec) * 8, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += b[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= act_bwd(v[j], act);
    store8(dx + i * 8, g);
  }
}

// y = mask * (x + bias[col]) * scale (+ addend); mask is one byte per element.
__global__ void bias_mask_scale_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ bias,
                                       const uint8_t* __restrict__ mask, const __nv_bfloat16* __restrict__ addend,
                                       __nv_bfloat16* __restrict__ y, long long nvec, int cols, float scale) {
  const int cvec = cols >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float v[8];
    load8(x + i * 8, v);
    if (bias) {
      float b[8];
      load8(bias + (i % cvec) * 8, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += b[j];
    }
    if (mask) {
      uint2 m = *reinterpret_cast<const uint2*>(mask + i * 8);
      const uint32_t mw[2] = {m.x, m.y};
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = ((mw[j >> 2] >> ((j & 3) * 8)) & 0xff) ? v[j] * scale : 0.f;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] *= scale;
    }
    if (addend) {
      float a[8];
      load8(addend + i * 8, a);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += a[j];
    }
    store8(y + i * 8, v);
  }
}

// Philox-free counter hash (splitmix64) keep/drop mask: mask[i] = u(i) >= p. One byte per element.
__global__ void dropout_mask_kernel(uint8_t* __restrict__ mask, long long n, unsigned long long seed,
                                    unsigned long long offset, float p) {
  const uint32_t thr = static_cast<uint32_t>(fminf(fmaxf(p, 0.f), 1.f) * 4294967295.0f);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i * 8 < n; i += (long long)gridDim.x * blockDim.x) {
    unsigned long long z = seed + (offset + i) * 0x9E3779B97F4A7C15ull;
    uint8_t out[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      z += 0x9E3779B97F4A7C15ull;
      unsigned long long t = z;
      t = (t ^ (t >> 30)) * 0xBF58476D1CE4E5B9ull;
      t = (t ^ (t >> 27)) * 0x94D049BB133111EBull;
      t ^= t >> 31;
      // 4 x 16-bit lanes give four uniform draws each
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t u = static_cast<uint32_t>((t >> (16 * j)) & 0xffff) * 65537u;
        out[h * 4 + j] = u >= thr ? 1 : 0;
      }
    }
    if (i * 8 + 8 <= n) {
      *reinterpret_cast<uint2*>(mask + i * 8) = *reinterpret_cast<uint2*>(out);
    } else {
      for (int j = 0; i * 8 + j < n; ++j) mask[i * 8 + j] = out[j];
    }
  }
}

// y(out dtype) = cast(x) * scale * (scale_by_tensor ? *scale_by_tensor : 1)
template <typename TIn, typename TOut>
__global__ void cast_scale_kernel(const TIn* __restrict__ x, TOut* __restrict__ y, long long n, float scale,
                                  const float* __restrict__ scale_by_tensor) {
  const float s = scale * (scale_by_tensor ? *scale_by_tensor : 1.f);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] = static_cast<TOut>(static_cast<float>(x[i]) * s);
}

// out[c] (+)= sum_r x[r, c]; x bf16 [rows, cols]. Grid: (cols/256 column panels, row slabs); each
// CTA reduces its slab in registers/smem and adds the panel into out with one atomicAdd per column.
__global__ void column_sum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, int rows, int cols,
                                  int rows_per_cta) {
  // blockDim = (32 column-vectors, 8 row lanes); panel = 256 columns
  __shared__ float red[8][256 + 8];
  const int cv = blockIdx.x * 32 + threadIdx.x;  // vector index along columns
  const int r0 = blockIdx.y * rows_per_cta;
  const int r1 = min(rows, r0 + rows_per_cta);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (cv * 8 < cols) {
    for (int r = r0 + threadIdx.y; r < r1; r += 8) {
      float v[8];
      load8(x + static_cast<long long>(r) * cols + cv * 8, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[threadIdx.y][threadIdx.x * 8 + j] = acc[j];
  __syncthreads();
  const int t = threadIdx.y * 32 + threadIdx.x;  // 256 threads -> one column each
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) s += red[k][t];
  const int c = blockIdx.x * 256 + t;
  if (c < cols) atomicAdd(out + c, s);
}

static inline int ew_grid(long long work_items, int threads) {
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = 148ll * 8;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

// Binary cross entropy on logits, forward and backward in one pass (the loss head of click-through models;
// reference: binary_cross_entropy_with_logits(_reduce_mean) kernels). Row r reads logits[r * ld], adds its loss to
// *loss_sum (scaled) and writes grad_scale * (sigmoid(x) - y) to dlogits[r * ld], zeros to the ld - 1 columns beside it.
__global__ void __launch_bounds__(256)
bce_logits_kernel(const __nv_bfloat16* __restrict__ logits, int ld, const float* __restrict__ labels,
                  __nv_bfloat16* __restrict__ dlogits, float* loss_sum, long long rows, float loss_scale, float grad_scale) {
  float local = 0.f;
  for (long long r = blockIdx.x * (long long)blockDim.x + threadIdx.x; r < rows; r += (long long)gridDim.x * blockDim.x) {
    const float x = __bfloat162float(logits[r * ld]);
    const float y = labels[r];
    local += fmaxf(x, 0.f) - x * y + log1pf(__expf(-fabsf(x)));
    const float sig = 1.f / (1.f + __expf(-x));
    __nv_bfloat16* g = dlogits + r * ld;
    g[0] = __float2bfloat16(grad_scale * (sig - y));
    for (int c = 1; c < ld; ++c) g[c] = __float2bfloat16(0.f);
  }
  for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
  __shared__ float part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += part[w];
    atomicAdd(loss_sum, t * loss_scale);
  }
}

}  // namespace ofb

using namespace ofb;
typedef __nv_bfloat16 bf16;

OFB_API int ofb_bias_act_fwd(const void* x, const void* bias, void* y, long long n, int cols, int act, void* stream) {
  if (n % 8 || cols % 8) return fail("bias_act: sizes must be multiples of 8");
  if (n == 0) return 0;
  bias_act_fwd_kernel<<<ew_grid(n / 8, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (const bf16*)bias, (bf16*)y,
                                                                           n / 8, cols, act);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
OFB_API int ofb_bias_act_bwd(const void* x, const void* bias, const void* dy, void* dx, long long n, int cols, int act,
                             void* stream) {
  if (n % 8 || cols % 8) return fail("bias_act_bwd: sizes must be multiples of 8");
  if (n == 0) return 0;
  bias_act_bwd_kernel<<<ew_grid(n / 8, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (const bf16*)bias,
                                                                           (const bf16*)dy, (bf16*)dx, n / 8, cols, act);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
OFB_API int ofb_bias_mask_scale(const void* x, const void* bias, const void* mask, const void* addend, void* y,
                                long long n, int cols, float scale, void* stream) {
  if (n % 8 || cols % 8) return fail("bias_mask_scale: sizes must be multiples of 8");
  if (n == 0) return 0;
  bias_mask_scale_kernel<<<ew_grid(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)x, (const bf16*)bias, (const uint8_t*)mask, (const bf16*)addend, (bf16*)y, n / 8, cols, scale);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
OFB_API int ofb_dropout_mask(void* mask, long long n, unsigned long long seed, unsigned long long offset, float p,
                             void* stream) {
  if (n == 0) return 0;
  dropout_mask_kernel<<<ew_grid((n + 7) / 8, 256), 256, 0, (cudaStream_t)stream>>>((uint8_t*)mask, n, seed, offset, p);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
// dtype codes: 0 = fp32, 1 = bf16, 2 = fp16
OFB_API int ofb_cast_scale(const void* x, int in_dtype, void* y, int out_dtype, long long n, float scale,
                           const float* scale_by_tensor, void* stream) {
  if (n == 0) return 0;
  auto s = (cudaStream_t)stream;
  const int g = ew_grid(n, 256);
#define OFB_CS(TI, TO) cast_scale_kernel<TI, TO><<<g, 256, 0, s>>>((const TI*)x, (TO*)y, n, scale, scale_by_tensor)
  if (in_dtype == 0 && out_dtype == 0) OFB_CS(float, float);
  else if (in_dtype == 0 && out_dtype == 1) OFB_CS(float, bf16);
  else if (in_dtype == 1 && out_dtype == 0) OFB_CS(bf16, float);
  else if (in_dtype == 1 && out_dtype == 1) OFB_CS(bf16, bf16);
  else if (in_dtype == 2 && out_dtype == 0) OFB_CS(__half, float);
  else if (in_dtype == 0 && out_dtype == 2) OFB_CS(float, __half);
  else return fail("cast_scale: unsupported dtype pair");
#undef OFB_CS
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
// out must be zeroed by the caller unless accumulating into existing values is wanted.
OFB_API int ofb_column_sum(const void* x, float* out, int rows, int cols, void* stream) {
  if (cols % 8) return fail("column_sum: cols must be a multiple of 8");
  if (rows == 0) return 0;
  const int panels = (cols + 255) / 256;
  int slabs = (148 * 4 + panels - 1) / panels;
  if (slabs > (rows + 63) / 64) slabs = (rows + 63) / 64;
  if (slabs < 1) slabs = 1;
  const int rows_per_cta = (rows + slabs - 1) / slabs;
  column_sum_kernel<<<dim3(panels, slabs), dim3(32, 8), 0, (cudaStream_t)stream>>>((const bf16*)x, out, rows, cols,
                                                                                 rows_per_cta);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// loss_sum must be zeroed by the caller (it accumulates, so micro-batches can share it).
OFB_API int ofb_bce_logits(const void* logits, int ld, const float* labels, void* dlogits, float* loss_sum, long long rows,
                           float loss_scale, float grad_scale, void* stream) {
  if (rows == 0) return 0;
  if (ld < 1) return fail("bce_logits: bad leading dimension");
  bce_logits_kernel<<<ew_grid(rows, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)logits, ld, labels, (bf16*)dlogits, loss_sum,
                                                                          rows, loss_scale, grad_scale);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
