// Memory-bound companions of the convolution kernels for NHWC bf16 feature maps (C a multiple of 8, 16-byte
// accesses): batch normalisation (training) fused with the residual add and ReLU, 3x3/s2 max pooling, global
// average pooling, 2x spatial subsampling and its adjoint (stride-2 convolutions run as stride-1 + subsample or
// subsample + 1x1), and the im2col of the 7x7/s2 stem whose 3 input channels do not fill a TMA box.
//
// Reference: oneflow/user/kernels/normalization_kernel.cu (cuDNN BN + fused add/relu), pool_gpu_kernel / max_pool
// kernels, adaptive_avg_pool_gpu_kernel.cu.
#include "../common/host_utils.h"
#include "../common/ptx.cuh"
#include "ofb_kernels.h"

namespace ofb {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void ld8(const bf16* p, float (&v)[8]) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = unpack_bf16x2(w[j]);
    v[2 * j] = f.x;
    v[2 * j + 1] = f.y;
  }
}
__device__ __forceinline__ void st8(bf16* p, const float (&v)[8]) {
  uint4 o;
  o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
  o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

// ------------------------------------------------------------------------------------------------ batch norm
// Two per-channel sums over all rows in one pass. MODE 0: (x, x^2). MODE 1: (g, g * xhat) with
// g = dy (* [y > 0] when relu) and xhat = (x - mean) * rstd. Threads are laid out as [row lane][8-channel vector];
// a block reduces its row lanes in shared memory and adds the result to out[0..C) and out[C..2C).
template <int MODE>
__global__ void __launch_bounds__(256)
bn_reduce_kernel(const bf16* __restrict__ a, const bf16* __restrict__ x, const bf16* __restrict__ y, const float* __restrict__ mean,
                 const float* __restrict__ rstd, long long rows, int C, int relu, float* out) {
  const int vpr = C >> 3;                       // 8-channel vectors per row
  const int vec = threadIdx.x % vpr;
  const int rlane = threadIdx.x / vpr;
  const int rlanes = blockDim.x / vpr;
  float s1[8], s2[8], mu[8], rs[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s1[j] = s2[j] = 0.f;
  if (MODE == 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      mu[j] = mean[vec * 8 + j];
      rs[j] = rstd[vec * 8 + j];
    }
  }
  if (rlane < rlanes) {
    for (long long r = blockIdx.x * (long long)rlanes + rlane; r < rows; r += (long long)gridDim.x * rlanes) {
      float v[8];
      ld8(a + r * C + vec * 8, v);
      if (MODE == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s1[j] += v[j];
          s2[j] += v[j] * v[j];
        }
      } else {
        float xv[8];
        ld8(x + r * C + vec * 8, xv);
        if (relu) {
          float yv[8];
          ld8(y + r * C + vec * 8, yv);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = yv[j] > 0.f ? v[j] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s1[j] += v[j];
          s2[j] += v[j] * (xv[j] - mu[j]) * rs[j];
        }
      }
    }
  }
  __shared__ float red[256 * 16];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    red[threadIdx.x * 16 + j] = s1[j];
    red[threadIdx.x * 16 + 8 + j] = s2[j];
  }
  __syncthreads();
  // thread t < vpr * 16 sums one (vector, component) over the row lanes
  for (int i = threadIdx.x; i < vpr * 16; i += blockDim.x) {
    const int v = i / 16, comp = i % 16;
    float t = 0.f;
    for (int l = 0; l < rlanes; ++l) t += red[(l * vpr + v) * 16 + comp];
    atomicAdd(&out[(comp >> 3) * C + v * 8 + (comp & 7)], t);
  }
}

// sums[0..C) = sum x, sums[C..2C) = sum x^2  ->  mean, rstd, the folded affine map y = scale * x + shift
// (scale = gamma * rstd, shift = beta - mean * scale), and the running statistics when given.
__global__ void bn_finalize_kernel(const float* __restrict__ sums, float inv_rows, float eps, float momentum, float unbias, int C,
                                   const float* __restrict__ gamma, const float* __restrict__ beta, float* mean, float* rstd, float* scale,
                                   float* shift, float* running_mean, float* running_var) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float m = sums[c] * inv_rows;
  const float var = fmaxf(sums[C + c] * inv_rows - m * m, 0.f);
  const float rs = rsqrtf(var + eps);
  mean[c] = m;
  rstd[c] = rs;
  const float sc = gamma[c] * rs;
  scale[c] = sc;
  shift[c] = beta[c] - m * sc;
  if (running_mean) {
    running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * m;
    running_var[c] = (1.f - momentum) * running_var[c] + momentum * var * unbias;
  }
}

// Backward coefficients per channel: dx = a * g + b * x + c with
//   a = gamma rstd,  b = -a rstd s2 / rows,  c = -a s1 / rows - b mean      (s1 = sum g, s2 = sum g xhat)
__global__ void bn_bwd_coeffs_kernel(const float* __restrict__ sums, const float* __restrict__ mean, const float* __restrict__ rstd,
                                     const float* __restrict__ gamma, float inv_rows, int C, float* coef) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float a = gamma[c] * rstd[c];
  const float b = -a * rstd[c] * sums[C + c] * inv_rows;
  coef[c] = a;
  coef[C + c] = b;
  coef[2 * C + c] = -a * sums[c] * inv_rows - b * mean[c];
}

// Streaming kernels below: when the 8-channel vectors per row divide the block size, a thread keeps the same
// channels for every row it visits, so the per-channel coefficients are loaded into registers once.
__device__ __forceinline__ void load_coef8(const float* p, float (&v)[8]) {
  const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 4);
  v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
  v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
}

// y = [relu](scale * x + shift [+ residual])
__global__ void __launch_bounds__(256)
bn_apply_kernel(const bf16* __restrict__ x, const bf16* __restrict__ residual, const float* __restrict__ scale,
                const float* __restrict__ shift, long long vecs, int C, int relu, bf16* __restrict__ y) {
  const int vpr = C >> 3;
  const bool fixed = (blockDim.x % vpr) == 0;
  float sc[8], sh[8];
  if (fixed) {
    load_coef8(scale + (threadIdx.x % vpr) * 8, sc);
    load_coef8(shift + (threadIdx.x % vpr) * 8, sh);
  }
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < vecs; i += (long long)gridDim.x * blockDim.x) {
    if (!fixed) {
      const int c0 = static_cast<int>(i % vpr) * 8;
      load_coef8(scale + c0, sc);
      load_coef8(shift + c0, sh);
    }
    float v[8];
    ld8(x + i * 8, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = fmaf(v[j], sc[j], sh[j]);
    if (residual) {
      float r[8];
      ld8(residual + i * 8, r);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += r[j];
    }
    if (relu) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = fmaxf(v[j], 0.f);
    }
    st8(y + i * 8, v);
  }
}

// dx = a * g + b * x + c, g = dy (* [y > 0]); d_residual = g when wanted. coef = [a | b | c], each C long.
__global__ void __launch_bounds__(256)
bn_bwd_apply_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ y, const float* __restrict__ coef,
                    long long vecs, int C, int relu, bf16* __restrict__ dx, bf16* __restrict__ d_residual) {
  const int vpr = C >> 3;
  const bool fixed = (blockDim.x % vpr) == 0;
  float ca[8], cb[8], cc[8];
  if (fixed) {
    const int c0 = (threadIdx.x % vpr) * 8;
    load_coef8(coef + c0, ca);
    load_coef8(coef + C + c0, cb);
    load_coef8(coef + 2 * C + c0, cc);
  }
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < vecs; i += (long long)gridDim.x * blockDim.x) {
    if (!fixed) {
      const int c0 = static_cast<int>(i % vpr) * 8;
      load_coef8(coef + c0, ca);
      load_coef8(coef + C + c0, cb);
      load_coef8(coef + 2 * C + c0, cc);
    }
    float g[8], xv[8];
    ld8(dy + i * 8, g);
    ld8(x + i * 8, xv);
    if (relu) {
      float yv[8];
      ld8(y + i * 8, yv);
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = yv[j] > 0.f ? g[j] : 0.f;
    }
    if (d_residual) st8(d_residual + i * 8, g);
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = fmaf(ca[j], g[j], fmaf(cb[j], xv[j], cc[j]));
    st8(dx + i * 8, o);
  }
}

// ------------------------------------------------------------------------------------------------ pooling
// 3x3 window, stride 2, padding 1. idx keeps the winning tap (0..8) for the backward.
__global__ void __launch_bounds__(256)
maxpool_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, unsigned char* __restrict__ idx, int N, int H, int W, int C, int OH,
                   int OW) {
  const int vpr = C >> 3;
  const long long total = static_cast<long long>(N) * OH * OW * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = static_cast<int>(i % vpr);
    long long p = i / vpr;
    const int ow = static_cast<int>(p % OW);
    p /= OW;
    const int oh = static_cast<int>(p % OH);
    const int n = static_cast<int>(p / OH);
    float best[8];
    unsigned char bi[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      best[j] = -3.0e38f;
      bi[j] = 4;
    }
    for (int r = 0; r < 3; ++r) {
      const int h = 2 * oh + r - 1;
      if (h < 0 || h >= H) continue;
      for (int s = 0; s < 3; ++s) {
        const int w = 2 * ow + s - 1;
        if (w < 0 || w >= W) continue;
        float t[8];
        ld8(x + ((static_cast<long long>(n) * H + h) * W + w) * C + v * 8, t);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (t[j] > best[j]) {
            best[j] = t[j];
            bi[j] = static_cast<unsigned char>(r * 3 + s);
          }
      }
    }
    st8(y + i * 8, best);
    uint2 packed;
    packed.x = bi[0] | (bi[1] << 8) | (bi[2] << 16) | (bi[3] << 24);
    packed.y = bi[4] | (bi[5] << 8) | (bi[6] << 16) | (bi[7] << 24);
    *reinterpret_cast<uint2*>(idx + i * 8) = packed;
  }
}

// Gather form of the backward: every input pixel looks at the (up to four) windows that contain it.
__global__ void __launch_bounds__(256)
maxpool_bwd_kernel(const bf16* __restrict__ dy, const unsigned char* __restrict__ idx, bf16* __restrict__ dx, int N, int H, int W, int C,
                   int OH, int OW) {
  const int vpr = C >> 3;
  const long long total = static_cast<long long>(N) * H * W * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = static_cast<int>(i % vpr);
    long long p = i / vpr;
    const int w = static_cast<int>(p % W);
    p /= W;
    const int h = static_cast<int>(p % H);
    const int n = static_cast<int>(p / H);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int oh = h >> 1; oh <= (h + 1) >> 1; ++oh) {
      if (oh >= OH) continue;
      const int r = h - 2 * oh + 1;
      for (int ow = w >> 1; ow <= (w + 1) >> 1; ++ow) {
        if (ow >= OW) continue;
        const int s = w - 2 * ow + 1;
        const long long o = ((static_cast<long long>(n) * OH + oh) * OW + ow) * vpr + v;
        const uint2 packed = *reinterpret_cast<const uint2*>(idx + o * 8);
        float g[8];
        ld8(dy + o * 8, g);
        const unsigned int tap = r * 3 + s;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const unsigned int b = ((j < 4 ? packed.x : packed.y) >> (8 * (j & 3))) & 0xffu;
          if (b == tap) acc[j] += g[j];
        }
      }
    }
    st8(dx + i * 8, acc);
  }
}

// mean over the HW pixels of each image: x [N, HW, C] -> y [N, C]; backward broadcasts dy / HW.
__global__ void __launch_bounds__(256)
avgpool_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, int N, int HW, int C) {
  const int vpr = C >> 3;
  const long long total = static_cast<long long>(N) * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = static_cast<int>(i % vpr);
    const long long n = i / vpr;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int p = 0; p < HW; ++p) {
      float t[8];
      ld8(x + (n * HW + p) * C + v * 8, t);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += t[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= 1.f / HW;
    st8(y + i * 8, acc);
  }
}
__global__ void __launch_bounds__(256)
avgpool_bwd_kernel(const bf16* __restrict__ dy, bf16* __restrict__ dx, int N, int HW, int C) {
  const int vpr = C >> 3;
  const long long total = static_cast<long long>(N) * HW * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = static_cast<int>(i % vpr);
    const long long n = i / vpr / HW;
    float g[8];
    ld8(dy + (n * vpr + v) * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= 1.f / HW;
    st8(dx + i * 8, g);
  }
}

// ------------------------------------------------------------------------------------------------ stride 2 helpers
// y[n, oh, ow] = x[n, 2 oh, 2 ow]  (adjoint: dx = 0 except dx[n, 2 oh, 2 ow] = dy[n, oh, ow])
__global__ void __launch_bounds__(256)
subsample2_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, int N, int H, int W, int C, int OH, int OW) {
  const int vpr = C >> 3;
  const long long total = static_cast<long long>(N) * OH * OW * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = static_cast<int>(i % vpr);
    long long p = i / vpr;
    const int ow = static_cast<int>(p % OW);
    p /= OW;
    const int oh = static_cast<int>(p % OH);
    const long long n = p / OH;
    reinterpret_cast<uint4*>(y)[i] = *reinterpret_cast<const uint4*>(x + ((n * H + 2 * oh) * W + 2 * ow) * C + v * 8);
  }
}
__global__ void __launch_bounds__(256)
upsample2_zero_kernel(const bf16* __restrict__ dy, bf16* __restrict__ dx, int N, int H, int W, int C, int OH, int OW) {
  const int vpr = C >> 3;
  const long long total = static_cast<long long>(N) * H * W * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = static_cast<int>(i % vpr);
    long long p = i / vpr;
    const int w = static_cast<int>(p % W);
    p /= W;
    const int h = static_cast<int>(p % H);
    const long long n = p / H;
    uint4 q = make_uint4(0, 0, 0, 0);
    if (!(h & 1) && !(w & 1) && (h >> 1) < OH && (w >> 1) < OW)
      q = *reinterpret_cast<const uint4*>(dy + ((n * OH + (h >> 1)) * OW + (w >> 1)) * C + v * 8);
    reinterpret_cast<uint4*>(dx)[i] = q;
  }
}

// cols[(n, oh, ow)][(r * S + s) * Cin + c] = x[n, stride oh + r - pad, stride ow + s - pad, c] (zero outside and in
// the padding columns up to ldc). For small Cin (the RGB stem), one thread per 8 output columns.
// CIN_ / R_ / S_ > 0 fix the shape at compile time (constant divisors); 0 takes the runtime values.
template <int CIN_, int R_, int S_>
__global__ void __launch_bounds__(256)
im2col_small_kernel(const bf16* __restrict__ x, bf16* __restrict__ cols, int N, int H, int W, int Cin_rt, int R_rt, int S_rt, int stride,
                    int pad, int OH, int OW, int ldc) {
  const int Cin = CIN_ > 0 ? CIN_ : Cin_rt, R = R_ > 0 ? R_ : R_rt, S = S_ > 0 ? S_ : S_rt;
  const int vpr = ldc >> 3;
  const long long total = static_cast<long long>(N) * OH * OW * vpr;
  const int kcols = R * S * Cin;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = static_cast<int>(i % vpr);
    long long p = i / vpr;
    const int ow = static_cast<int>(p % OW);
    p /= OW;
    const int oh = static_cast<int>(p % OH);
    const long long n = p / OH;
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int col = v * 8 + j;
      float val = 0.f;
      if (col < kcols) {
        const int c = col % Cin, tap = col / Cin;
        const int h = stride * oh + tap / S - pad, w = stride * ow + tap % S - pad;
        if (h >= 0 && h < H && w >= 0 && w < W) val = __bfloat162float(x[((n * H + h) * W + w) * Cin + c]);
      }
      o[j] = val;
    }
    st8(cols + i * 8, o);
  }
}

}  // namespace ofb

using namespace ofb;

static inline int aux_grid(long long items) {
  long long b = (items + 255) / 256;
  if (b < 1) b = 1;
  if (b > 148 * 16) b = 148 * 16;
  return static_cast<int>(b);
}

// sums [2 C] fp32 must be zero on entry. mode 0: sums of x and x^2 (pass x as `a`). mode 1: sums of g and g * xhat.
OFB_API int ofb_bn_reduce(int mode, const void* a, const void* x, const void* y, const float* mean, const float* rstd, long long rows,
                          int C, int relu, float* sums, void* stream) {
  if (C % 8 || C > 2048) return fail("bn: channels must be a multiple of 8, at most 2048");
  if (rows == 0) return 0;
  const int vpr = C / 8;
  const int rlanes = 256 / vpr;
  long long blocks = (rows + rlanes * 16 - 1) / (rlanes * 16);
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  if (mode == 0)
    bn_reduce_kernel<0><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const bf16*)a, nullptr, nullptr, nullptr, nullptr, rows, C, 0, sums);
  else
    bn_reduce_kernel<1><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const bf16*)a, (const bf16*)x, (const bf16*)y, mean, rstd, rows, C,
                                                                         relu, sums);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

OFB_API int ofb_bn_finalize(const float* sums, long long rows, float eps, float momentum, int C, const float* gamma, const float* beta,
                            float* mean, float* rstd, float* scale, float* shift, float* running_mean, float* running_var, void* stream) {
  const float unbias = rows > 1 ? static_cast<float>(rows) / static_cast<float>(rows - 1) : 1.f;
  bn_finalize_kernel<<<(C + 127) / 128, 128, 0, (cudaStream_t)stream>>>(sums, 1.f / rows, eps, momentum, unbias, C, gamma, beta, mean, rstd,
                                                                       scale, shift, running_mean, running_var);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// y = [relu](scale * x + shift [+ residual]) with per-channel fp32 scale / shift.
OFB_API int ofb_bn_apply(const void* x, const void* residual, const float* scale, const float* shift, long long rows, int C, int relu,
                         void* y, void* stream) {
  if (C % 8) return fail("bn: channels must be a multiple of 8");
  const long long vecs = rows * (C / 8);
  if (vecs == 0) return 0;
  bn_apply_kernel<<<aux_grid(vecs), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (const bf16*)residual, scale, shift, vecs, C, relu,
                                                                  (bf16*)y);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// coef [3 C] is scratch written here. sums = [sum g | sum g xhat] from ofb_bn_reduce(mode 1).
OFB_API int ofb_bn_bwd_apply(const void* dy, const void* x, const void* y, const float* mean, const float* rstd, const float* gamma,
                             const float* sums, float* coef, long long rows, int C, int relu, void* dx, void* d_residual, void* stream) {
  if (C % 8) return fail("bn: channels must be a multiple of 8");
  const long long vecs = rows * (C / 8);
  if (vecs == 0) return 0;
  bn_bwd_coeffs_kernel<<<(C + 127) / 128, 128, 0, (cudaStream_t)stream>>>(sums, mean, rstd, gamma, 1.f / rows, C, coef);
  bn_bwd_apply_kernel<<<aux_grid(vecs), 256, 0, (cudaStream_t)stream>>>((const bf16*)dy, (const bf16*)x, (const bf16*)y, coef, vecs, C, relu,
                                                                      (bf16*)dx, (bf16*)d_residual);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

OFB_API int ofb_maxpool3x3s2_fwd(const void* x, void* y, void* idx, int N, int H, int W, int C, void* stream) {
  if (C % 8) return fail("maxpool: channels must be a multiple of 8");
  const int OH = (H + 1) / 2, OW = (W + 1) / 2;
  maxpool_fwd_kernel<<<aux_grid((long long)N * OH * OW * (C / 8)), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y,
                                                                                                 (unsigned char*)idx, N, H, W, C, OH, OW);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
OFB_API int ofb_maxpool3x3s2_bwd(const void* dy, const void* idx, void* dx, int N, int H, int W, int C, void* stream) {
  if (C % 8) return fail("maxpool: channels must be a multiple of 8");
  const int OH = (H + 1) / 2, OW = (W + 1) / 2;
  maxpool_bwd_kernel<<<aux_grid((long long)N * H * W * (C / 8)), 256, 0, (cudaStream_t)stream>>>((const bf16*)dy, (const unsigned char*)idx,
                                                                                               (bf16*)dx, N, H, W, C, OH, OW);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
OFB_API int ofb_avgpool_fwd(const void* x, void* y, int N, int HW, int C, void* stream) {
  if (C % 8) return fail("avgpool: channels must be a multiple of 8");
  avgpool_fwd_kernel<<<aux_grid((long long)N * (C / 8)), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, N, HW, C);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
OFB_API int ofb_avgpool_bwd(const void* dy, void* dx, int N, int HW, int C, void* stream) {
  if (C % 8) return fail("avgpool: channels must be a multiple of 8");
  avgpool_bwd_kernel<<<aux_grid((long long)N * HW * (C / 8)), 256, 0, (cudaStream_t)stream>>>((const bf16*)dy, (bf16*)dx, N, HW, C);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
OFB_API int ofb_subsample2(const void* x, void* y, int N, int H, int W, int C, void* stream) {
  if (C % 8) return fail("subsample: channels must be a multiple of 8");
  const int OH = (H + 1) / 2, OW = (W + 1) / 2;
  subsample2_kernel<<<aux_grid((long long)N * OH * OW * (C / 8)), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, N, H, W, C, OH, OW);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
OFB_API int ofb_upsample2_zero(const void* dy, void* dx, int N, int H, int W, int C, void* stream) {
  if (C % 8) return fail("upsample: channels must be a multiple of 8");
  const int OH = (H + 1) / 2, OW = (W + 1) / 2;
  upsample2_zero_kernel<<<aux_grid((long long)N * H * W * (C / 8)), 256, 0, (cudaStream_t)stream>>>((const bf16*)dy, (bf16*)dx, N, H, W, C, OH,
                                                                                                  OW);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
OFB_API int ofb_im2col_small(const void* x, void* cols, int N, int H, int W, int Cin, int R, int S, int stride, int pad, int ldc,
                             void* stream) {
  if (ldc % 8 || ldc < R * S * Cin) return fail("im2col: leading dimension must be a multiple of 8 covering R S Cin");
  const int OH = (H + 2 * pad - R) / stride + 1, OW = (W + 2 * pad - S) / stride + 1;
  const int grid = aux_grid((long long)N * OH * OW * (ldc / 8));
  if (Cin == 3 && R == 7 && S == 7)
    im2col_small_kernel<3, 7, 7><<<grid, 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)cols, N, H, W, Cin, R, S, stride, pad, OH, OW, ldc);
  else
    im2col_small_kernel<0, 0, 0><<<grid, 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)cols, N, H, W, Cin, R, S, stride, pad, OH, OW, ldc);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
