// Fused optimizer updates and gradient post-processing, multi-tensor: one launch walks a
// table of tensors (chunked so that every CTA gets the same amount of work), keeps fp32
// master weights / moments and writes the bf16 model copy in the same pass.
//
// Maths follow oneflow/user/kernels/model_update_kernel_util.h:25-140:
//   g = cast(grad) * scale + l1 * sign(w) + l2 * w
//   SGD      : w -= lr * (g + wd * w)
//   momentum : m = beta * m + (1 - dampening) * g ; g' = nesterov ? g + beta * m : m ;
//              w = w -/+ lr * g' - lr * wd * w
//   Adam(W)  : m, v EMAs ; denom = sqrt(v) / sqrt(bc2) + eps ; w -= (lr / bc1) * m / denom + lr * wd * w
// with `skip_if` (loss-scale overflow), lr / scale read from device memory when given.
// Reference kernels: model_update_kernel_util.cu (sgd :161, momentum :307, adam :487),
// multi_tensor_model_update_kernel_util.cu, multi_reduce_kernels.cu, count_not_finite_kernel.cu,
// fused_clip_grad.cu.
#include <cuda_fp16.h>

#include "../common/host_utils.h"
#include "../common/ptx.cuh"
#include "ofb_kernels.h"

namespace ofb {

constexpr int kMaxTensors = 48;
constexpr int kMaxChunk = 65536;  // largest chunk (elements): one CTA handles one chunk at a time
constexpr int kMinChunk = 4096;   // small problems get small chunks so that every SM has work

struct TensorTable {
  void* grad[kMaxTensors];
  float* master[kMaxTensors];
  void* model_copy[kMaxTensors];  // bf16 copy or null
  float* m[kMaxTensors];
  float* v[kMaxTensors];
  long long size[kMaxTensors];
  int first_chunk[kMaxTensors + 1];  // prefix sum of chunk counts
  int n;
  int chunk;                         // elements per chunk of this call
};

struct OptimHyper {
  float lr, beta1, beta2, eps, weight_decay, l1, l2, scale, bc1, bc2;
  float momentum, dampening;
  int nesterov, maximize, grad_is_bf16, amsgrad_unused;
  const float* lr_ptr;      // overrides lr when non-null
  const float* scale_ptr;   // multiplies scale when non-null (e.g. 1/loss_scale or clip factor)
  const long long* skip_if; // skip the whole update when *skip_if != 0
  const float* bc_ptr;      // {bc1, bc2} on the device: overrides the two values above when non-null, so that a step
                            // captured in a CUDA graph sees the bias corrections of the step it is replayed for
};

__device__ __forceinline__ int find_tensor(const TensorTable& t, int chunk) {
  int lo = 0, hi = t.n - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (t.first_chunk[mid] <= chunk) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ float load_grad(const void* g, long long i, int is_bf16) {
  return is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i]) : reinterpret_cast<const float*>(g)[i];
}

template <int MODE>  // 0 = adamw, 1 = sgd(momentum)
__global__ void __launch_bounds__(512) multi_tensor_update_kernel(const __grid_constant__ TensorTable tab, OptimHyper h) {
  if (h.skip_if && *h.skip_if != 0) return;
  const float lr = h.lr_ptr ? *h.lr_ptr : h.lr;
  const float scale = h.scale * (h.scale_ptr ? *h.scale_ptr : 1.f);
  const float bc1 = h.bc_ptr ? h.bc_ptr[0] : h.bc1, bc2 = h.bc_ptr ? h.bc_ptr[1] : h.bc2;
  for (int chunk = blockIdx.x; chunk < tab.first_chunk[tab.n]; chunk += gridDim.x) {
    const int ti = find_tensor(tab, chunk);
    const long long base = static_cast<long long>(chunk - tab.first_chunk[ti]) * tab.chunk;
    const long long end = min(tab.size[ti], base + tab.chunk);
    float* w = tab.master[ti];
    float* mm = tab.m[ti];
    float* vv = tab.v[ti];
    __nv_bfloat16* copy = reinterpret_cast<__nv_bfloat16*>(tab.model_copy[ti]);
    const void* gp = tab.grad[ti];
    // 4 elements per thread per iteration; tensors are at least 16-byte aligned by the allocator and
    // chunk bases are multiples of 4, so vector accesses stay aligned.
    for (long long i = base + threadIdx.x * 4; i < end; i += blockDim.x * 4) {
      float wv[4], gv[4], m4[4], v4[4];
      const int cnt = (end - i) >= 4 ? 4 : static_cast<int>(end - i);
      if (cnt == 4) {
        float4 t = *reinterpret_cast<const float4*>(w + i);
        wv[0] = t.x; wv[1] = t.y; wv[2] = t.z; wv[3] = t.w;
        if (h.grad_is_bf16) {
          uint2 q = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(gp) + i);
          float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y);
          gv[0] = a.x; gv[1] = a.y; gv[2] = b.x; gv[3] = b.y;
        } else {
          float4 q = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(gp) + i);
          gv[0] = q.x; gv[1] = q.y; gv[2] = q.z; gv[3] = q.w;
        }
        if (mm) { float4 q = *reinterpret_cast<const float4*>(mm + i); m4[0] = q.x; m4[1] = q.y; m4[2] = q.z; m4[3] = q.w; }
        if (MODE == 0) { float4 q = *reinterpret_cast<const float4*>(vv + i); v4[0] = q.x; v4[1] = q.y; v4[2] = q.z; v4[3] = q.w; }
      } else {
        for (int j = 0; j < cnt; ++j) {
          wv[j] = w[i + j];
          gv[j] = load_grad(gp, i + j, h.grad_is_bf16);
          if (mm) m4[j] = mm[i + j];
          if (MODE == 0) v4[j] = vv[i + j];
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j >= cnt) break;
        float g = gv[j] * scale;
        if (h.l1 != 0.f) g += h.l1 * (wv[j] > 0.f ? 1.f : (wv[j] < 0.f ? -1.f : 0.f));
        if (h.l2 != 0.f) g += h.l2 * wv[j];
        if (MODE == 0) {
          m4[j] = h.beta1 * m4[j] + (1.f - h.beta1) * g;
          v4[j] = h.beta2 * v4[j] + (1.f - h.beta2) * g * g;
          const float denom = sqrtf(v4[j]) / sqrtf(bc2) + h.eps;
          wv[j] = wv[j] - (lr / bc1) * (m4[j] / denom) - lr * h.weight_decay * wv[j];
        } else {
          if (mm) {
            m4[j] = h.momentum * m4[j] + (1.f - h.dampening) * g;
            g = h.nesterov ? g + h.momentum * m4[j] : m4[j];
          }
          const float step = lr * g;
          wv[j] = (h.maximize ? wv[j] + step : wv[j] - step) - lr * h.weight_decay * wv[j];
        }
      }
      if (cnt == 4) {
        *reinterpret_cast<float4*>(w + i) = make_float4(wv[0], wv[1], wv[2], wv[3]);
        if (mm) *reinterpret_cast<float4*>(mm + i) = make_float4(m4[0], m4[1], m4[2], m4[3]);
        if (MODE == 0) *reinterpret_cast<float4*>(vv + i) = make_float4(v4[0], v4[1], v4[2], v4[3]);
        if (copy) *reinterpret_cast<uint2*>(copy + i) = make_uint2(pack_bf16x2(wv[0], wv[1]), pack_bf16x2(wv[2], wv[3]));
      } else {
        for (int j = 0; j < cnt; ++j) {
          w[i + j] = wv[j];
          if (mm) mm[i + j] = m4[j];
          if (MODE == 0) vv[i + j] = v4[j];
          if (copy) copy[i + j] = __float2bfloat16(wv[j]);
        }
      }
    }
  }
}

// Per-CTA partial of sum |g|^2 (and a not-finite count) over a table of tensors; `partials`
// is scratch memory of gridDim.x * 2 floats that finish_norm_kernel folds.
__global__ void __launch_bounds__(512) multi_tensor_sqsum_kernel(const __grid_constant__ TensorTable tab, int grad_is_bf16,
                                                                 float* __restrict__ partials) {
  __shared__ float red[2][16];
  float s = 0.f, bad = 0.f;
  for (int chunk = blockIdx.x; chunk < tab.first_chunk[tab.n]; chunk += gridDim.x) {
    const int ti = find_tensor(tab, chunk);
    const long long base = static_cast<long long>(chunk - tab.first_chunk[ti]) * tab.chunk;
    const long long end = min(tab.size[ti], base + tab.chunk);
    const void* gp = tab.grad[ti];
    for (long long i = base + threadIdx.x; i < end; i += blockDim.x) {
      float g = load_grad(gp, i, grad_is_bf16);
      if (!isfinite(g)) bad += 1.f; else s += g * g;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { s += __shfl_xor_sync(0xffffffffu, s, o); bad += __shfl_xor_sync(0xffffffffu, bad, o); }
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = s; red[1][threadIdx.x >> 5] = bad; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    s = threadIdx.x < nw ? red[0][threadIdx.x] : 0.f;
    bad = threadIdx.x < nw ? red[1][threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { s += __shfl_xor_sync(0xffffffffu, s, o); bad += __shfl_xor_sync(0xffffffffu, bad, o); }
    if (threadIdx.x == 0) { partials[blockIdx.x * 2] = s; partials[blockIdx.x * 2 + 1] = bad; }
  }
}

// out[0] (+)= sum of squares, out[1] (+)= count of non-finite values. One CTA.
__global__ void finish_norm_kernel(const float* __restrict__ partials, int n, float* __restrict__ out, int accumulate) {
  __shared__ float red[2][32];
  float s = 0.f, bad = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) { s += partials[2 * i]; bad += partials[2 * i + 1]; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { s += __shfl_xor_sync(0xffffffffu, s, o); bad += __shfl_xor_sync(0xffffffffu, bad, o); }
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = s; red[1][threadIdx.x >> 5] = bad; }
  __syncthreads();
  if (threadIdx.x == 0) {
    s = 0.f; bad = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) { s += red[0][i]; bad += red[1][i]; }
    if (accumulate) { s += out[0]; bad += out[1]; }
    out[0] = s;
    out[1] = bad;
  }
}

// clip factor = min(1, max_norm / (sqrt(sqsum) + 1e-6)); also the "found inf" flag for skip_if.
__global__ void clip_factor_kernel(const float* __restrict__ sq_and_bad, float max_norm, float* __restrict__ factor,
                                   long long* __restrict__ found_inf, float* __restrict__ total_norm) {
  const float norm = sqrtf(sq_and_bad[0]);
  if (total_norm) *total_norm = norm;
  if (factor) *factor = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
  if (found_inf) *found_inf = sq_and_bad[1] > 0.f ? 1 : 0;
}

static int build_table(TensorTable& tab, int n, void* const* grads, float* const* masters, void* const* copies,
                       float* const* ms, float* const* vs, const long long* sizes) {
  if (n > kMaxTensors) return fail("multi-tensor table holds at most 48 tensors per launch");
  tab.n = n;
  long long total = 0;
  for (int i = 0; i < n; ++i) total += sizes[i];
  long long per = (total + 148 * 4 - 1) / (148 * 4);          // about four chunks per SM
  per = (per + kMinChunk - 1) / kMinChunk * kMinChunk;
  tab.chunk = static_cast<int>(per < kMinChunk ? kMinChunk : (per > kMaxChunk ? kMaxChunk : per));
  int chunks = 0;
  for (int i = 0; i < n; ++i) {
    tab.grad[i] = grads ? grads[i] : nullptr;
    tab.master[i] = masters ? masters[i] : nullptr;
    tab.model_copy[i] = copies ? copies[i] : nullptr;
    tab.m[i] = ms ? ms[i] : nullptr;
    tab.v[i] = vs ? vs[i] : nullptr;
    tab.size[i] = sizes[i];
    const uintptr_t all = reinterpret_cast<uintptr_t>(tab.grad[i]) | reinterpret_cast<uintptr_t>(tab.master[i]) |
                          reinterpret_cast<uintptr_t>(tab.model_copy[i]) | reinterpret_cast<uintptr_t>(tab.m[i]) |
                          reinterpret_cast<uintptr_t>(tab.v[i]);
    if (all & 15) return fail("multi-tensor kernels need 16-byte aligned tensors");
    tab.first_chunk[i] = chunks;
    chunks += static_cast<int>((sizes[i] + tab.chunk - 1) / tab.chunk);
  }
  tab.first_chunk[n] = chunks;
  return chunks;
}

}  // namespace ofb

using namespace ofb;

static int adamw_launch(int n, void* const* grads, float* const* masters, void* const* copies, float* const* ms,
                        float* const* vs, const long long* sizes, int grad_is_bf16, float lr, float beta1, float beta2, float eps,
                        float weight_decay, float l2, float scale, float bc1, float bc2, const float* lr_ptr, const float* scale_ptr,
                        const long long* skip_if, const float* bc_ptr, void* stream);

OFB_API int ofb_multi_tensor_adamw(int n, void* const* grads, float* const* masters, void* const* copies, float* const* ms,
                                   float* const* vs, const long long* sizes, int grad_is_bf16, float lr, float beta1,
                                   float beta2, float eps, float weight_decay, float l2, float scale, float bc1, float bc2,
                                   const float* lr_ptr, const float* scale_ptr, const long long* skip_if, void* stream) {
  return adamw_launch(n, grads, masters, copies, ms, vs, sizes, grad_is_bf16, lr, beta1, beta2, eps, weight_decay, l2, scale, bc1, bc2,
                      lr_ptr, scale_ptr, skip_if, nullptr, stream);
}

// The same update with the step-dependent scalars on the device: step[0] = learning rate, step[1] = 1 - beta1^t,
// step[2] = 1 - beta2^t; scale_ptr (optional) multiplies the gradients (a clip factor). Nothing in the launch depends on the
// step number, so it can be recorded in a CUDA graph.
OFB_API int ofb_multi_tensor_adamw_dev(int n, void* const* grads, float* const* masters, void* const* copies, float* const* ms,
                                       float* const* vs, const long long* sizes, int grad_is_bf16, float beta1, float beta2, float eps,
                                       float weight_decay, const float* step, const float* scale_ptr, void* stream) {
  if (!step) return fail("multi_tensor_adamw_dev: the step scalars are required");
  return adamw_launch(n, grads, masters, copies, ms, vs, sizes, grad_is_bf16, 0.f, beta1, beta2, eps, weight_decay, 0.f, 1.f, 1.f, 1.f, step,
                      scale_ptr, nullptr, step + 1, stream);
}

static int adamw_launch(int n, void* const* grads, float* const* masters, void* const* copies, float* const* ms,
                        float* const* vs, const long long* sizes, int grad_is_bf16, float lr, float beta1, float beta2, float eps,
                        float weight_decay, float l2, float scale, float bc1, float bc2, const float* lr_ptr, const float* scale_ptr,
                        const long long* skip_if, const float* bc_ptr, void* stream) {
  TensorTable tab;
  const int chunks = build_table(tab, n, grads, masters, copies, ms, vs, sizes);
  if (chunks < 0) return -1;
  if (chunks == 0) return 0;
  OptimHyper h;
  std::memset(&h, 0, sizeof(h));
  h.lr = lr; h.beta1 = beta1; h.beta2 = beta2; h.eps = eps; h.weight_decay = weight_decay; h.l2 = l2; h.scale = scale;
  h.bc1 = bc1; h.bc2 = bc2; h.grad_is_bf16 = grad_is_bf16; h.lr_ptr = lr_ptr; h.scale_ptr = scale_ptr; h.skip_if = skip_if;
  h.bc_ptr = bc_ptr;
  const int grid = chunks < 148 * 4 ? chunks : 148 * 4;
  multi_tensor_update_kernel<0><<<grid, 512, 0, (cudaStream_t)stream>>>(tab, h);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

OFB_API int ofb_multi_tensor_sgd(int n, void* const* grads, float* const* masters, void* const* copies, float* const* ms,
                                 const long long* sizes, int grad_is_bf16, float lr, float momentum, float dampening,
                                 int nesterov, int maximize, float weight_decay, float l1, float l2, float scale,
                                 const float* lr_ptr, const float* scale_ptr, const long long* skip_if, void* stream) {
  TensorTable tab;
  const int chunks = build_table(tab, n, grads, masters, copies, ms, nullptr, sizes);
  if (chunks < 0) return -1;
  if (chunks == 0) return 0;
  OptimHyper h;
  std::memset(&h, 0, sizeof(h));
  h.lr = lr; h.momentum = momentum; h.dampening = dampening; h.nesterov = nesterov; h.maximize = maximize;
  h.weight_decay = weight_decay; h.l1 = l1; h.l2 = l2; h.scale = scale; h.grad_is_bf16 = grad_is_bf16;
  h.lr_ptr = lr_ptr; h.scale_ptr = scale_ptr; h.skip_if = skip_if;
  const int grid = chunks < 148 * 4 ? chunks : 148 * 4;
  multi_tensor_update_kernel<1><<<grid, 512, 0, (cudaStream_t)stream>>>(tab, h);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// Number of floats of scratch ofb_multi_tensor_sqsum needs.
OFB_API int ofb_sqsum_scratch_floats(void) { return 2 * 148 * 4; }

// out[0] (+)= sum g^2 over finite entries, out[1] (+)= number of non-finite entries.
OFB_API int ofb_multi_tensor_sqsum(int n, void* const* grads, const long long* sizes, int grad_is_bf16, float* scratch,
                                   float* out, int accumulate, void* stream) {
  TensorTable tab;
  const int chunks = build_table(tab, n, grads, nullptr, nullptr, nullptr, nullptr, sizes);
  if (chunks < 0) return -1;
  auto s = (cudaStream_t)stream;
  if (chunks == 0) {
    if (!accumulate) OFB_CUDA_OK(cudaMemsetAsync(out, 0, 2 * sizeof(float), s));
    return 0;
  }
  const int grid = chunks < 148 * 4 ? chunks : 148 * 4;
  multi_tensor_sqsum_kernel<<<grid, 512, 0, s>>>(tab, grad_is_bf16, scratch);
  finish_norm_kernel<<<1, 256, 0, s>>>(scratch, grid, out, accumulate);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

OFB_API int ofb_clip_factor(const float* sq_and_bad, float max_norm, float* factor, long long* found_inf, float* total_norm,
                            void* stream) {
  clip_factor_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(sq_and_bad, max_norm, factor, found_inf, total_norm);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
