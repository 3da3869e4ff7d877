// Row softmax family on bf16 with fp32 maths. One warp owns one row and keeps it in
// registers (up to 2048 columns); longer rows use one CTA per row that keeps the row in
// shared memory, so each element is read from HBM once.
//
//   fused_scale_tril_softmax_mask_scale(+grad)  oneflow/user/kernels/fused_tril_scale_softmax_mask_scale_kernel.cu :175,:219
//   fused_scale_mask_softmax(_dropout)(+grad)   oneflow/user/kernels/fused_scale_mask_softmax.cu, ..._dropout.cu
//   softmax / softmax_grad                      oneflow/core/cuda/softmax.cuh
//   sparse_softmax_cross_entropy(+_ms)          oneflow/user/kernels/sparse_softmax_cross_entropy_kernel.cu
#include "../common/host_utils.h"
#include "../common/ptx.cuh"
#include "ofb_kernels.h"

namespace ofb {

__device__ __forceinline__ float wmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct SoftmaxArgs {
  const __nv_bfloat16* x;      // [rows, cols]
  const uint8_t* mask;         // tril mode: dropout keep-mask [rows, cols] or null
                               // mask mode: attention mask, 0 = masked out, broadcast by mask_row_div
  __nv_bfloat16* y;            // [rows, cols] final output
  __nv_bfloat16* softmax_y;    // [rows, cols] softmax before dropout (null = do not store)
  long long rows;
  int cols;
  int tril;                    // 1: causal (row r of a [.., s, s] block keeps cols <= (r % tril_rows) + diagonal)
  int tril_rows;               // s (rows per attention matrix)
  int diagonal;
  float scale;                 // applied to x before softmax
  float mask_fill;             // value for masked-out logits (mask mode)
  float out_scale;             // dropout rescale applied with the keep-mask (1 when no dropout)
  const uint8_t* attn_mask;    // optional attention mask [rows / attn_mask_row_div ..] see kernel
  long long attn_mask_rows;    // number of rows of attn_mask (rows are mapped with row % attn_mask_rows)
};

// NV = number of 8-element vectors per lane: cols <= 256*NV
template <int NV>
__global__ void __launch_bounds__(256) softmax_fwd_warp_kernel(SoftmaxArgs a) {
  const int lane = threadIdx.x & 31;
  const long long warp_global = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = a.cols >> 3;
  for (long long row = warp_global; row < a.rows; row += nwarps) {
    const __nv_bfloat16* xr = a.x + row * a.cols;
    const int limit = a.tril ? static_cast<int>(row % a.tril_rows) + a.diagonal : a.cols - 1;  // last kept column
    const uint8_t* am = a.attn_mask ? a.attn_mask + (row % a.attn_mask_rows) * a.cols : nullptr;
    float v[NV][8];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        uint4 q = *reinterpret_cast<const uint4*>(xr + vi * 8);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint2 mm = make_uint2(0x01010101u, 0x01010101u);
        if (am) mm = *reinterpret_cast<const uint2*>(am + vi * 8);
        const uint32_t mw[2] = {mm.x, mm.y};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float2 f = unpack_bf16x2(w[j >> 1]);
          float e = ((j & 1) ? f.y : f.x) * a.scale;
          const int col = vi * 8 + j;
          if (col > limit) e = -INFINITY;
          else if (!((mw[j >> 2] >> ((j & 3) * 8)) & 0xff)) e = a.mask_fill;
          v[i][j] = e;
          mx = fmaxf(mx, e);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = -INFINITY;
      }
    }
    mx = wmax(mx);
    if (mx == -INFINITY) mx = 0.f;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) { v[i][j] = __expf(v[i][j] - mx); s += v[i][j]; }
    s = wsum(s);
    const float inv = s > 0.f ? 1.f / s : 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float p[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) p[j] = v[i][j] * inv;
        if (a.softmax_y) {
          uint4 o;
          o.x = pack_bf16x2(p[0], p[1]); o.y = pack_bf16x2(p[2], p[3]);
          o.z = pack_bf16x2(p[4], p[5]); o.w = pack_bf16x2(p[6], p[7]);
          *reinterpret_cast<uint4*>(a.softmax_y + row * a.cols + vi * 8) = o;
        }
        if (a.mask) {
          uint2 mm = *reinterpret_cast<const uint2*>(a.mask + row * a.cols + vi * 8);
          const uint32_t mw[2] = {mm.x, mm.y};
#pragma unroll
          for (int j = 0; j < 8; ++j) p[j] = ((mw[j >> 2] >> ((j & 3) * 8)) & 0xff) ? p[j] * a.out_scale : 0.f;
        } else if (a.out_scale != 1.f) {
#pragma unroll
          for (int j = 0; j < 8; ++j) p[j] *= a.out_scale;
        }
        uint4 o;
        o.x = pack_bf16x2(p[0], p[1]); o.y = pack_bf16x2(p[2], p[3]);
        o.z = pack_bf16x2(p[4], p[5]); o.w = pack_bf16x2(p[6], p[7]);
        *reinterpret_cast<uint4*>(a.y + row * a.cols + vi * 8) = o;
      }
    }
  }
}

struct SoftmaxGradArgs {
  const __nv_bfloat16* softmax_y;  // [rows, cols]
  const __nv_bfloat16* dy;         // [rows, cols]
  const uint8_t* mask;             // dropout keep mask or null
  __nv_bfloat16* dx;
  long long rows;
  int cols;
  int tril, tril_rows, diagonal;
  float scale;      // forward input scale
  float out_scale;  // dropout rescale
};

// dx = scale * y * (g - sum(g*y)), g = dy * mask * out_scale; zero above the diagonal in tril mode
template <int NV>
__global__ void __launch_bounds__(256) softmax_bwd_warp_kernel(SoftmaxGradArgs a) {
  const int lane = threadIdx.x & 31;
  const long long warp_global = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = a.cols >> 3;
  for (long long row = warp_global; row < a.rows; row += nwarps) {
    const int limit = a.tril ? static_cast<int>(row % a.tril_rows) + a.diagonal : a.cols - 1;
    float y[NV][8], g[NV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        uint4 qy = *reinterpret_cast<const uint4*>(a.softmax_y + row * a.cols + vi * 8);
        uint4 qg = *reinterpret_cast<const uint4*>(a.dy + row * a.cols + vi * 8);
        const uint32_t wy[4] = {qy.x, qy.y, qy.z, qy.w};
        const uint32_t wg[4] = {qg.x, qg.y, qg.z, qg.w};
        uint2 mm = make_uint2(0x01010101u, 0x01010101u);
        if (a.mask) mm = *reinterpret_cast<const uint2*>(a.mask + row * a.cols + vi * 8);
        const uint32_t mw[2] = {mm.x, mm.y};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float2 fy = unpack_bf16x2(wy[j >> 1]), fg = unpack_bf16x2(wg[j >> 1]);
          float yy = (j & 1) ? fy.y : fy.x, gg = (j & 1) ? fg.y : fg.x;
          gg = ((mw[j >> 2] >> ((j & 3) * 8)) & 0xff) ? gg * a.out_scale : 0.f;
          if (vi * 8 + j > limit) { yy = 0.f; gg = 0.f; }
          y[i][j] = yy; g[i][j] = gg;
          dot += yy * gg;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) { y[i][j] = 0.f; g[i][j] = 0.f; }
      }
    }
    dot = wsum(dot);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = a.scale * y[i][j] * (g[i][j] - dot);
        uint4 o;
        o.x = pack_bf16x2(r[0], r[1]); o.y = pack_bf16x2(r[2], r[3]);
        o.z = pack_bf16x2(r[4], r[5]); o.w = pack_bf16x2(r[6], r[7]);
        *reinterpret_cast<uint4*>(a.dx + row * a.cols + vi * 8) = o;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Sparse softmax cross-entropy over a (possibly vocabulary-sharded) logits matrix.
//   stats pass : per row local max, local sum exp(x - max), logit of the label if it lives here
//   grad pass  : dlogits = (exp(x - gmax) / gsum - onehot) * row_scale ; loss = log(gsum) + gmax - target
// Between the passes a tensor-parallel group merges the [rows,3] statistics (tiny all-reduce);
// on one GPU the merge is the identity.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512)
xent_stats_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                  float* __restrict__ stats /*[rows,3]*/, int rows, int cols, long long ld, int vocab_start) {
  __shared__ float red[32];
  const int nvec = cols >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = logits + row * ld;
    float mx = -INFINITY;
    for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
      uint4 q = *reinterpret_cast<const uint4*>(xr + vi * 8);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16x2(w[j]); mx = fmaxf(mx, fmaxf(f.x, f.y)); }
    }
    mx = wmax(mx);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : -INFINITY;
    mx = wmax(mx);
    float s = 0.f;
    for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
      uint4 q = *reinterpret_cast<const uint4*>(xr + vi * 8);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16x2(w[j]); s += __expf(f.x - mx) + __expf(f.y - mx); }
    }
    s = wsum(s);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    s = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : 0.f;
    s = wsum(s);
    if (threadIdx.x == 0) {
      const long long lab = labels[row] - vocab_start;
      float tgt = 0.f;
      if (lab >= 0 && lab < cols) tgt = __bfloat162float(xr[lab]);
      stats[row * 3 + 0] = mx;
      stats[row * 3 + 1] = s;
      stats[row * 3 + 2] = tgt;
    }
  }
}

// merged: [rows,3] = (global max, global sum w.r.t. global max, target logit). ignore_index rows get 0 loss/grad.
__global__ void __launch_bounds__(512)
xent_grad_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                 const float* __restrict__ merged, float* __restrict__ loss, __nv_bfloat16* __restrict__ dlogits,
                 int rows, int cols, long long ld, int vocab_start, float grad_scale, long long ignore_index) {
  const int nvec = cols >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float gmax = merged[row * 3], gsum = merged[row * 3 + 1], tgt = merged[row * 3 + 2];
    const long long lab_g = labels[row];
    const bool ignored = lab_g == ignore_index;
    if (threadIdx.x == 0 && loss) loss[row] = ignored ? 0.f : (__logf(gsum) + gmax - tgt);
    if (!dlogits) continue;
    const long long lab = lab_g - vocab_start;
    const float inv = ignored ? 0.f : grad_scale / gsum;
    const float gs = ignored ? 0.f : grad_scale;
    const __nv_bfloat16* xr = logits + row * ld;
    __nv_bfloat16* dr = dlogits + row * ld;
    for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
      uint4 q = *reinterpret_cast<const uint4*>(xr + vi * 8);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      float r[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16x2(w[j]);
        r[2 * j] = __expf(f.x - gmax) * inv;
        r[2 * j + 1] = __expf(f.y - gmax) * inv;
      }
      const long long d = lab - static_cast<long long>(vi) * 8;
      if (d >= 0 && d < 8) r[d] -= gs;
      uint4 o;
      o.x = pack_bf16x2(r[0], r[1]); o.y = pack_bf16x2(r[2], r[3]);
      o.z = pack_bf16x2(r[4], r[5]); o.w = pack_bf16x2(r[6], r[7]);
      *reinterpret_cast<uint4*>(dr + vi * 8) = o;
    }
  }
}

// Merges per-shard statistics stacked as [nshards, rows, 3] into [rows, 3].
__global__ void xent_merge_kernel(const float* __restrict__ parts, float* __restrict__ merged, int nshards, int rows) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float gm = -INFINITY;
  for (int s = 0; s < nshards; ++s) gm = fmaxf(gm, parts[(static_cast<long long>(s) * rows + r) * 3]);
  float sum = 0.f, tgt = 0.f;
  for (int s = 0; s < nshards; ++s) {
    const float* p = parts + (static_cast<long long>(s) * rows + r) * 3;
    sum += p[1] * __expf(p[0] - gm);
    tgt += p[2];
  }
  merged[r * 3] = gm;
  merged[r * 3 + 1] = sum;
  merged[r * 3 + 2] = tgt;
}

}  // namespace ofb

using namespace ofb;
typedef __nv_bfloat16 bf16;

static int softmax_grid(long long rows) {
  long long blocks = (rows + 7) / 8;  // 8 warps per CTA
  const long long cap = 148ll * 8;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

OFB_API int ofb_softmax_fwd(const void* x, const void* dropout_mask, const void* attn_mask, long long attn_mask_rows,
                            void* y, void* softmax_y, long long rows, int cols, int tril, int tril_rows, int diagonal,
                            float scale, float mask_fill, float out_scale, void* stream) {
  if (cols % 8 || cols > 2048) return fail("softmax: cols must be a multiple of 8 and <= 2048");
  if (rows == 0) return 0;
  SoftmaxArgs a;
  a.x = (const bf16*)x; a.mask = (const uint8_t*)dropout_mask; a.y = (bf16*)y; a.softmax_y = (bf16*)softmax_y;
  a.rows = rows; a.cols = cols; a.tril = tril; a.tril_rows = tril_rows > 0 ? tril_rows : 1; a.diagonal = diagonal;
  a.scale = scale; a.mask_fill = mask_fill; a.out_scale = out_scale;
  a.attn_mask = (const uint8_t*)attn_mask; a.attn_mask_rows = attn_mask_rows > 0 ? attn_mask_rows : 1;
  const int g = softmax_grid(rows);
  auto s = (cudaStream_t)stream;
  if (cols <= 256) softmax_fwd_warp_kernel<1><<<g, 256, 0, s>>>(a);
  else if (cols <= 512) softmax_fwd_warp_kernel<2><<<g, 256, 0, s>>>(a);
  else if (cols <= 1024) softmax_fwd_warp_kernel<4><<<g, 256, 0, s>>>(a);
  else softmax_fwd_warp_kernel<8><<<g, 256, 0, s>>>(a);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

OFB_API int ofb_softmax_bwd(const void* softmax_y, const void* dy, const void* dropout_mask, void* dx, long long rows,
                            int cols, int tril, int tril_rows, int diagonal, float scale, float out_scale,
                            void* stream) {
  if (cols % 8 || cols > 2048) return fail("softmax_bwd: cols must be a multiple of 8 and <= 2048");
  if (rows == 0) return 0;
  SoftmaxGradArgs a;
  a.softmax_y = (const bf16*)softmax_y; a.dy = (const bf16*)dy; a.mask = (const uint8_t*)dropout_mask; a.dx = (bf16*)dx;
  a.rows = rows; a.cols = cols; a.tril = tril; a.tril_rows = tril_rows > 0 ? tril_rows : 1; a.diagonal = diagonal;
  a.scale = scale; a.out_scale = out_scale;
  const int g = softmax_grid(rows);
  auto s = (cudaStream_t)stream;
  if (cols <= 256) softmax_bwd_warp_kernel<1><<<g, 256, 0, s>>>(a);
  else if (cols <= 512) softmax_bwd_warp_kernel<2><<<g, 256, 0, s>>>(a);
  else if (cols <= 1024) softmax_bwd_warp_kernel<4><<<g, 256, 0, s>>>(a);
  else softmax_bwd_warp_kernel<8><<<g, 256, 0, s>>>(a);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

OFB_API int ofb_xent_stats(const void* logits, const long long* labels, float* stats, int rows, int cols, long long ld,
                           int vocab_start, void* stream) {
  if (cols % 8 || ld % 8) return fail("xent: cols and ld must be multiples of 8");
  if (rows == 0) return 0;
  xent_stats_kernel<<<rows < 148 * 8 ? rows : 148 * 8, 512, 0, (cudaStream_t)stream>>>((const bf16*)logits, labels, stats,
                                                                                   rows, cols, ld, vocab_start);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
OFB_API int ofb_xent_merge(const float* parts, float* merged, int nshards, int rows, void* stream) {
  if (rows == 0) return 0;
  xent_merge_kernel<<<(rows + 127) / 128, 128, 0, (cudaStream_t)stream>>>(parts, merged, nshards, rows);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
OFB_API int ofb_xent_grad(const void* logits, const long long* labels, const float* merged, float* loss, void* dlogits,
                          int rows, int cols, long long ld, int vocab_start, float grad_scale, long long ignore_index,
                          void* stream) {
  if (cols % 8 || ld % 8) return fail("xent: cols and ld must be multiples of 8");
  if (rows == 0) return 0;
  xent_grad_kernel<<<rows < 148 * 8 ? rows : 148 * 8, 512, 0, (cudaStream_t)stream>>>(
      (const bf16*)logits, labels, merged, loss, (bf16*)dlogits, rows, cols, ld, vocab_start, grad_scale, ignore_index);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
