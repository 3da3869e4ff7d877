// DLRM dot feature interaction, forward and backward, one warp per sample.
//   X = [dense ; sparse_0 .. sparse_{T-1}]  (F = T + 1 rows of D bf16 values)
//   out = [ dense (D values) | Z[i][j] for i > j (or i >= j with self-interaction), row by row | zero padding ]
//   with Z = X X^T.
// The sample's feature matrix is staged once in shared memory (fp32, padded rows), every lane owns pairs
// (forward) or columns (backward), so each input byte is read from HBM exactly once; at F = 27, D = 128 the
// kernel moves 7 KB per sample for 45 k FMAs and is bound by HBM, not by arithmetic, which is why it runs
// on the CUDA cores instead of padding 27 x 27 products up to a 128-row tensor-core tile.
//
// Reference: oneflow/user/kernels/fused_dot_feature_interaction_kernel.cu (wmma, one CTA per sample,
// fwd :1141,1277, grad :1377,1413).
#include "../common/host_utils.h"
#include "../common/ptx.cuh"
#include "ofb_kernels.h"

namespace ofb {

constexpr int kIntMaxF = 32;
constexpr int kIntMaxD = 128;
constexpr int kIntWarps = 2;   // 2 x (32 x 129 + 32 x 32) floats = 41 KB of static shared memory

__device__ __forceinline__ void stage_features(float* sx, const __nv_bfloat16* dense, const __nv_bfloat16* sparse, int T, int D,
                                               int lane) {
  const int F = T + 1;
  const int vec = D >> 3;
  for (int e = lane; e < F * vec; e += 32) {
    const int row = e / vec, c = (e % vec) * 8;
    const __nv_bfloat16* src = row == 0 ? dense + c : sparse + static_cast<long long>(row - 1) * D + c;
    const uint4 q = *reinterpret_cast<const uint4*>(src);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    float* dst = sx + row * (kIntMaxD + 1) + c;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(w[j]);
      dst[2 * j] = f.x;
      dst[2 * j + 1] = f.y;
    }
  }
}

__global__ void __launch_bounds__(32 * kIntWarps)
interaction_fwd_kernel(const __nv_bfloat16* __restrict__ dense, const __nv_bfloat16* __restrict__ sparse,
                       __nv_bfloat16* __restrict__ out, long long batch, int T, int D, int self_inter, int out_dim) {
  __shared__ float sx_all[kIntWarps][kIntMaxF * (kIntMaxD + 1)];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* sx = sx_all[warp];
  const int F = T + 1;
  const int npairs = self_inter ? F * (F + 1) / 2 : F * (F - 1) / 2;
  for (long long s = blockIdx.x * (long long)kIntWarps + warp; s < batch; s += (long long)gridDim.x * kIntWarps) {
    __syncwarp();
    stage_features(sx, dense + s * D, sparse + s * T * D, T, D, lane);
    __syncwarp();
    __nv_bfloat16* o = out + s * out_dim;
    for (int c = lane; c < D; c += 32) o[c] = __float2bfloat16(sx[c]);  // concatenated dense vector
    for (int pidx = lane; pidx < npairs; pidx += 32) {
      // invert pidx -> (i, j) of the row-major lower triangle
      int i, j;
      if (self_inter) {
        i = static_cast<int>((sqrtf(8.f * pidx + 1.f) - 1.f) * 0.5f);
        while ((i + 1) * (i + 2) / 2 <= pidx) ++i;
        while (i * (i + 1) / 2 > pidx) --i;
        j = pidx - i * (i + 1) / 2;
      } else {
        i = static_cast<int>((sqrtf(8.f * pidx + 1.f) + 1.f) * 0.5f);
        while (i * (i + 1) / 2 <= pidx) ++i;
        while (i * (i - 1) / 2 > pidx) --i;
        j = pidx - i * (i - 1) / 2;
      }
      const float* a = sx + i * (kIntMaxD + 1);
      const float* b = sx + j * (kIntMaxD + 1);
      float acc0 = 0.f, acc1 = 0.f;
      for (int d = 0; d < D; d += 2) {
        acc0 += a[d] * b[d];
        acc1 += a[d + 1] * b[d + 1];
      }
      o[D + pidx] = __float2bfloat16(acc0 + acc1);
    }
    for (int c = D + npairs + lane; c < out_dim; c += 32) o[c] = __float2bfloat16(0.f);
  }
}

__global__ void __launch_bounds__(32 * kIntWarps)
interaction_bwd_kernel(const __nv_bfloat16* __restrict__ dense, const __nv_bfloat16* __restrict__ sparse,
                       const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ d_dense,
                       __nv_bfloat16* __restrict__ d_sparse, long long batch, int T, int D, int self_inter, int out_dim) {
  __shared__ float sx_all[kIntWarps][kIntMaxF * (kIntMaxD + 1)];
  __shared__ float sg_all[kIntWarps][kIntMaxF * kIntMaxF];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* sx = sx_all[warp];
  float* sg = sg_all[warp];
  const int F = T + 1;
  for (long long s = blockIdx.x * (long long)kIntWarps + warp; s < batch; s += (long long)gridDim.x * kIntWarps) {
    __syncwarp();
    stage_features(sx, dense + s * D, sparse + s * T * D, T, D, lane);
    const __nv_bfloat16* g = dout + s * out_dim;
    // symmetric gradient matrix: dZ[i][j] = dZ[j][i] = grad of the pair (diagonal counts twice: d(x.x) = 2x)
    for (int e = lane; e < F * F; e += 32) {
      const int i = e / F, j = e % F;
      const int hi = max(i, j), lo = min(i, j);
      float v = 0.f;
      if (self_inter) {
        v = __bfloat162float(g[D + hi * (hi + 1) / 2 + lo]);
        if (i == j) v *= 2.f;
      } else if (i != j) {
        v = __bfloat162float(g[D + hi * (hi - 1) / 2 + lo]);
      }
      sg[i * kIntMaxF + j] = v;
    }
    __syncwarp();
    for (int row = 0; row < F; ++row) {
      const float* gr = sg + row * kIntMaxF;
      for (int c = lane; c < D; c += 32) {
        float acc = 0.f;
        for (int j = 0; j < F; ++j) acc += gr[j] * sx[j * (kIntMaxD + 1) + c];
        if (row == 0) {
          acc += __bfloat162float(g[c]);  // gradient of the concatenated dense vector
          d_dense[s * D + c] = __float2bfloat16(acc);
        } else {
          d_sparse[(s * T + (row - 1)) * D + c] = __float2bfloat16(acc);
        }
      }
    }
  }
}

}  // namespace ofb

using namespace ofb;

static int interaction_check(int T, int D, int out_dim, int self_inter) {
  const int F = T + 1;
  if (F > kIntMaxF || D > kIntMaxD || D % 8) return fail("interaction: supports up to 32 features of dim <= 128 (multiple of 8)");
  const int npairs = self_inter ? F * (F + 1) / 2 : F * (F - 1) / 2;
  if (out_dim < D + npairs) return fail("interaction: output row too short");
  return 0;
}

OFB_API int ofb_interaction_fwd(const void* dense, const void* sparse, void* out, long long batch, int T, int D, int self_inter,
                                int out_dim, void* stream) {
  if (interaction_check(T, D, out_dim, self_inter)) return -1;
  if (batch == 0) return 0;
  long long blocks = (batch + kIntWarps - 1) / kIntWarps;
  if (blocks > 148 * 8) blocks = 148 * 8;
  interaction_fwd_kernel<<<(unsigned)blocks, 32 * kIntWarps, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dense, (const __nv_bfloat16*)sparse, (__nv_bfloat16*)out, batch, T, D, self_inter, out_dim);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

OFB_API int ofb_interaction_bwd(const void* dense, const void* sparse, const void* dout, void* d_dense, void* d_sparse,
                                long long batch, int T, int D, int self_inter, int out_dim, void* stream) {
  if (interaction_check(T, D, out_dim, self_inter)) return -1;
  if (batch == 0) return 0;
  long long blocks = (batch + kIntWarps - 1) / kIntWarps;
  if (blocks > 148 * 4) blocks = 148 * 4;
  interaction_bwd_kernel<<<(unsigned)blocks, 32 * kIntWarps, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dense, (const __nv_bfloat16*)sparse, (const __nv_bfloat16*)dout, (__nv_bfloat16*)d_dense,
      (__nv_bfloat16*)d_sparse, batch, T, D, self_inter, out_dim);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
