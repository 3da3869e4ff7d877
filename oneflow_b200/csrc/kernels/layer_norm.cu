// LayerNorm forward / backward for bf16 activations (fp32 statistics), written for B200:
// one CTA per row with the row held in registers as 16-byte vectors, so every element
// is read from HBM exactly once per pass; the backward accumulates the gamma/beta
// gradients of many rows in registers and leaves one partial row per CTA in a scratch
// buffer that a second tiny kernel folds.
//
// Reference counterparts: oneflow/core/cuda/layer_norm.cuh (three-tier dispatch) and
// oneflow/user/kernels/layer_norm_gpu_kernel.cu (layer_norm :330, layer_norm_grad :376,
// layer_norm_param_grad :454).
#include <cstdlib>

#include "../common/host_utils.h"
#include "../common/ptx.cuh"
#include "ofb_kernels.h"

namespace ofb {

constexpr int kLnMaxVecPerThread = 4;  // 4 x 8 elements x up to 1024 threads = 32768 columns

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide sum of two values at once; `red` holds 2*32 floats.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* red) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) { red[warp] = a; red[32 + warp] = b; }
  __syncthreads();
  float x = lane < nw ? red[lane] : 0.f, y = lane < nw ? red[32 + lane] : 0.f;
  a = warp_sum(x);
  b = warp_sum(y);
}

// 1-D bulk asynchronous copy global -> shared, completion counted in bytes on an mbarrier (addresses and size are
// multiples of 16 bytes).
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// (count, mean, M2) of two disjoint sets of values merged into one (Chan et al.): the variance comes out of ONE reduction
// without the cancellation of E[x^2] - mean^2.
__device__ __forceinline__ void welford_merge(float& n, float& mean, float& m2, float nb, float meanb, float m2b) {
  const float nt = n + nb;
  if (nt > 0.f) {
    const float delta = meanb - mean;
    const float fb = nb / nt;
    mean += delta * fb;
    m2 += m2b + delta * delta * n * fb;
  }
  n = nt;
}

// Block-wide merge of per-thread (count, mean, M2); `red` holds 3*32 floats. Every thread gets the total.
__device__ __forceinline__ void block_welford(float& n, float& mean, float& m2, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float nb = __shfl_xor_sync(0xffffffffu, n, o), mb = __shfl_xor_sync(0xffffffffu, mean, o), qb = __shfl_xor_sync(0xffffffffu, m2, o);
    welford_merge(n, mean, m2, nb, mb, qb);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();   // the previous row's readers of `red` are done
  if (lane == 0) { red[warp] = n; red[32 + warp] = mean; red[64 + warp] = m2; }
  __syncthreads();
  n = lane < nw ? red[lane] : 0.f;
  mean = lane < nw ? red[32 + lane] : 0.f;
  m2 = lane < nw ? red[64 + lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float nb = __shfl_xor_sync(0xffffffffu, n, o), mb = __shfl_xor_sync(0xffffffffu, mean, o), qb = __shfl_xor_sync(0xffffffffu, m2, o);
    welford_merge(n, mean, m2, nb, mb, qb);
  }
}

// The same merge when every thread of the CTA holds the same number of values and the CTA has a power-of-two number of
// warps (the usual case: cols = 8 * NV * threads): two sets of equal size n merge without a division,
// mean = (ma + mb) / 2, M2 = M2a + M2b + (mb - ma)^2 * n / 2. The general form above costs a division per round and
// thread, which made the forward kernel bound by instruction issue (72 % issue slots busy at 2.8 TB/s).
__device__ __forceinline__ void block_welford_equal(float n, float& mean, float& m2, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float mb = __shfl_xor_sync(0xffffffffu, mean, o), qb = __shfl_xor_sync(0xffffffffu, m2, o);
    const float delta = mb - mean;
    mean = 0.5f * (mean + mb);
    m2 += qb + delta * delta * (0.5f * n);
    n *= 2.f;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) { red[32 + warp] = mean; red[64 + warp] = m2; }
  __syncthreads();
  mean = red[32 + (lane & (nw - 1))];      // every lane group of nw lanes holds the nw warp results
  m2 = red[64 + (lane & (nw - 1))];
  for (int o = nw >> 1; o > 0; o >>= 1) {
    const float mb = __shfl_xor_sync(0xffffffffu, mean, o), qb = __shfl_xor_sync(0xffffffffu, m2, o);
    const float delta = mb - mean;
    mean = 0.5f * (mean + mb);
    m2 += qb + delta * delta * (0.5f * n);
    n *= 2.f;
  }
}

// One CTA per row at a time; the row lives in registers as packed 16-byte vectors. The loads of the CTA's NEXT row are
// issued before the current row's reduction, so a CTA always has a row in flight while it computes (the reduction and
// its barriers no longer sit between two dependent HBM round trips); mean and variance come from one merged reduction.
// Measured on 32768 x 4096 (CUDA events): 185 us with two block reductions and no prefetch, 190 us with the prefetch
// and the general merge (72 % of the issue slots busy: a division per merge round and thread), 117 us = 4.6 TB/s with
// the division-free merge. A variant fed through a shared-memory ring of bulk copies measured 122 us: no gain, left out.
template <int NV>
__global__ void __launch_bounds__(NV == 4 ? 1024 : 256)
layer_norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                      const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                      float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int cols, float eps) {
  __shared__ float red[96];
  const int nvec = cols >> 3;
  const bool equal_counts = nvec == NV * static_cast<int>(blockDim.x) && ((blockDim.x >> 5) & ((blockDim.x >> 5) - 1)) == 0;
  uint4 nxt[NV];
  auto load_row = [&](int row) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * cols);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      nxt[i] = vi < nvec ? __ldcs(xr + vi) : make_uint4(0, 0, 0, 0);
    }
  };
  if (static_cast<int>(blockIdx.x) < rows) load_row(blockIdx.x);
  // gamma and beta stay in registers (packed) for all of the CTA's rows: fetched per row they cost twice the row's own
  // bytes in L2 traffic. The 1024-thread form has no registers to spare and reads them per row.
  constexpr bool kKeepParams = NV < 4;
  uint4 gq[kKeepParams ? NV : 1], bq[kKeepParams ? NV : 1];
  if constexpr (kKeepParams) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      const bool in = vi < nvec;
      gq[i] = (gamma && in) ? __ldg(reinterpret_cast<const uint4*>(gamma) + vi) : make_uint4(0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u);
      bq[i] = (beta && in) ? __ldg(reinterpret_cast<const uint4*>(beta) + vi) : make_uint4(0, 0, 0, 0);
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float v[NV][8];
    float s = 0.f, cnt = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      const uint32_t w[4] = {nxt[i].x, nxt[i].y, nxt[i].z, nxt[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16x2(w[j]);
        v[i][2 * j] = f.x; v[i][2 * j + 1] = f.y;
        s += f.x + f.y;
      }
      if (vi < nvec) cnt += 8.f;
    }
    if (row + static_cast<int>(gridDim.x) < rows) load_row(row + gridDim.x);   // next row in flight under this row's math
    float mean = cnt > 0.f ? s / cnt : 0.f;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { float d = v[i][j] - mean; q += d * d; }
      }
    }
    if (equal_counts) block_welford_equal(cnt, mean, q, red);
    else block_welford(cnt, mean, q, red);
    const float rstd = rsqrtf(q / cols + eps);
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    uint4* yr = reinterpret_cast<uint4*>(y + static_cast<long long>(row) * cols);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
        float g[8], b[8];
        if constexpr (kKeepParams) {
          const uint32_t wg[4] = {gq[i].x, gq[i].y, gq[i].z, gq[i].w};
          const uint32_t wb[4] = {bq[i].x, bq[i].y, bq[i].z, bq[i].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 fg = unpack_bf16x2(wg[j]), fb = unpack_bf16x2(wb[j]);
            g[2 * j] = fg.x; g[2 * j + 1] = fg.y;
            b[2 * j] = fb.x; b[2 * j + 1] = fb.y;
          }
        } else {
          if (gamma) {
            uint4 p = __ldg(reinterpret_cast<const uint4*>(gamma) + vi);
            const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16x2(w[j]); g[2 * j] = f.x; g[2 * j + 1] = f.y; }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) g[j] = 1.f;
          }
          if (beta) {
            uint4 p = __ldg(reinterpret_cast<const uint4*>(beta) + vi);
            const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16x2(w[j]); b[2 * j] = f.x; b[2 * j + 1] = f.y; }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) b[j] = 0.f;
          }
        }
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          ow[j] = pack_bf16x2((v[i][2 * j] - mean) * rstd * g[2 * j] + b[2 * j],
                              (v[i][2 * j + 1] - mean) * rstd * g[2 * j + 1] + b[2 * j + 1]);
        __stcs(yr + vi, o);
      }
    }
  }
}

// dx = rstd * (g*dy - mean_c(g*dy) - xhat * mean_c(g*dy*xhat)); each CTA also accumulates
// sum_rows(dy*xhat) and sum_rows(dy) for its rows and writes them to partial[blockIdx.x].
template <int NV>
__global__ void __launch_bounds__(NV == 4 ? 1024 : 256, NV == 4 ? 1 : 2)
layer_norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                      const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean,
                      const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ add_to_dx,
                      __nv_bfloat16* __restrict__ dx, float* __restrict__ partial_dgamma,
                      float* __restrict__ partial_dbeta, int rows, int cols) {
  __shared__ float red[64];
  const int nvec = cols >> 3;
  float acc_g[NV][8], acc_b[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc_g[i][j] = 0.f; acc_b[i][j] = 0.f; }
  float g[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * blockDim.x;
    if (gamma && vi < nvec) {
      uint4 p = __ldg(reinterpret_cast<const uint4*>(gamma) + vi);
      const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16x2(w[j]); g[i][2 * j] = f.x; g[i][2 * j + 1] = f.y; }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[i][j] = 1.f;
    }
  }
  // The loads of the NEXT row (x, dy, the addend, its statistics) are issued before this row's block-wide reduction:
  // one row per CTA in flight leaves the memory system idle during the reduction (measured 0.27-0.38 of the HBM rate),
  // two keep it busy.
  uint4 nx[NV], nd[NV], na[NV];
  float nmu = 0.f, nrs = 0.f;
  auto prefetch = [&](int r) {
    const long long o = static_cast<long long>(r) * cols;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
        nx[i] = reinterpret_cast<const uint4*>(x + o)[vi];
        nd[i] = reinterpret_cast<const uint4*>(dy + o)[vi];
        if (add_to_dx) na[i] = reinterpret_cast<const uint4*>(add_to_dx + o)[vi];
      }
    }
    nmu = mean[r];
    nrs = rstd[r];
  };
  constexpr bool kPrefetch = NV < 4;   // the 1024-thread form has 64 registers per thread: no room for a second row
  if (blockIdx.x < rows) prefetch(blockIdx.x);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long off = static_cast<long long>(row) * cols;
    const float mu = nmu, rs = nrs;
    uint4 cx[NV], cd[NV], ca[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) { cx[i] = nx[i]; cd[i] = nd[i]; ca[i] = na[i]; }
    if (kPrefetch) {
      if (row + static_cast<int>(gridDim.x) < rows) prefetch(row + gridDim.x);
    }
    float xh[NV][8], gd[NV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
        const uint4 px = cx[i], pd = cd[i];
        const uint32_t wx[4] = {px.x, px.y, px.z, px.w};
        const uint32_t wd[4] = {pd.x, pd.y, pd.z, pd.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 fx = unpack_bf16x2(wx[j]), fd = unpack_bf16x2(wd[j]);
          float h0 = (fx.x - mu) * rs, h1 = (fx.y - mu) * rs;
          xh[i][2 * j] = h0; xh[i][2 * j + 1] = h1;
          acc_g[i][2 * j] += fd.x * h0; acc_g[i][2 * j + 1] += fd.y * h1;
          acc_b[i][2 * j] += fd.x; acc_b[i][2 * j + 1] += fd.y;
          float a0 = fd.x * g[i][2 * j], a1 = fd.y * g[i][2 * j + 1];
          gd[i][2 * j] = a0; gd[i][2 * j + 1] = a1;
          s1 += a0 + a1;
          s2 += a0 * h0 + a1 * h1;
        }
      }
    }
    block_sum2(s1, s2, red);
    const float m1 = s1 / cols, m2 = s2 / cols;
    uint4* dxr = reinterpret_cast<uint4*>(dx + off);
    if (!kPrefetch) {
      if (row + static_cast<int>(gridDim.x) < rows) prefetch(row + gridDim.x);   // after the reduction: registers are free again
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
        float r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = rs * (gd[i][j] - m1 - xh[i][j] * m2);
        if (add_to_dx) {
          const uint4 pa = ca[i];
          const uint32_t wa[4] = {pa.x, pa.y, pa.z, pa.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16x2(wa[j]); r[2 * j] += f.x; r[2 * j + 1] += f.y; }
        }
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) ow[j] = pack_bf16x2(r[2 * j], r[2 * j + 1]);
        dxr[vi] = o;
      }
    }
  }
  if (partial_dgamma) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
        float* pg = partial_dgamma + static_cast<long long>(blockIdx.x) * cols + vi * 8;
        float* pb = partial_dbeta + static_cast<long long>(blockIdx.x) * cols + vi * 8;
        *reinterpret_cast<float4*>(pg) = make_float4(acc_g[i][0], acc_g[i][1], acc_g[i][2], acc_g[i][3]);
        *reinterpret_cast<float4*>(pg + 4) = make_float4(acc_g[i][4], acc_g[i][5], acc_g[i][6], acc_g[i][7]);
        *reinterpret_cast<float4*>(pb) = make_float4(acc_b[i][0], acc_b[i][1], acc_b[i][2], acc_b[i][3]);
        *reinterpret_cast<float4*>(pb + 4) = make_float4(acc_b[i][4], acc_b[i][5], acc_b[i][6], acc_b[i][7]);
      }
    }
  }
}

// The same backward for rows of up to 8192 columns, fed through shared memory: one elected thread streams the CTA's rows
// (x, dy and the optional addend) into a ring of stages with 1-D bulk asynchronous copies (cp.async.bulk, completion on
// an mbarrier), kStages rows ahead of the row being computed. The register-prefetch form above can keep only one row
// per CTA in flight (its registers are full: two CTAs x 16 KB per SM = 4.7 MB on the chip, which at the HBM latency gives
// the ~3 TB/s it measures); the ring keeps kStages of them in flight without holding them in registers.
constexpr int kLnRingStages = 4;


template <int NV>
__global__ void __launch_bounds__(256, 2)
layer_norm_bwd_ring_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                           const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean,
                           const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ add_to_dx,
                           __nv_bfloat16* __restrict__ dx, float* __restrict__ partial_dgamma,
                           float* __restrict__ partial_dbeta, int rows, int cols, int* status) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ float red[64];
  __shared__ uint64_t full[kLnRingStages];
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;
  const int nvec = cols >> 3;
  const uint32_t row_bytes = static_cast<uint32_t>(cols) * 2u;
  const int ntens = add_to_dx ? 3 : 2;
  const uint32_t stage_bytes = row_bytes * 3u;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kLnRingStages; ++s) mbar_init(&full[s], 1);
    abort_flag_s = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const int my_rows = static_cast<int>(blockIdx.x) < rows ? (rows - 1 - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x) + 1 : 0;
  auto issue = [&](int k) {   // thread 0 only: row number k of this CTA into stage k % kStages
    const int s = k % kLnRingStages;
    const long long o = (static_cast<long long>(blockIdx.x) + static_cast<long long>(k) * gridDim.x) * cols;
    uint8_t* st = ring + static_cast<size_t>(s) * stage_bytes;
    mbar_arrive_expect_tx(&full[s], row_bytes * static_cast<uint32_t>(ntens));
    bulk_load_1d(st, x + o, row_bytes, &full[s]);
    bulk_load_1d(st + row_bytes, dy + o, row_bytes, &full[s]);
    if (add_to_dx) bulk_load_1d(st + 2 * row_bytes, add_to_dx + o, row_bytes, &full[s]);
  };
  if (threadIdx.x == 0)
    for (int k = 0; k < kLnRingStages && k < my_rows; ++k) issue(k);

  float acc_g[NV][8], acc_b[NV][8], g[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = threadIdx.x + i * blockDim.x;
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc_g[i][j] = 0.f; acc_b[i][j] = 0.f; g[i][j] = 1.f; }
    if (gamma && vi < nvec) {
      uint4 p = __ldg(reinterpret_cast<const uint4*>(gamma) + vi);
      const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16x2(w[j]); g[i][2 * j] = f.x; g[i][2 * j + 1] = f.y; }
    }
  }
  bool ok = true;
  for (int k = 0; k < my_rows; ++k) {
    const int row = static_cast<int>(blockIdx.x) + k * static_cast<int>(gridDim.x);
    const int s = k % kLnRingStages;
    const float mu = mean[row], rs = rstd[row];
    if (!mbar_wait(&full[s], static_cast<uint32_t>(k / kLnRingStages) & 1u, abort_flag)) { ok = false; break; }
    const uint8_t* st = ring + static_cast<size_t>(s) * stage_bytes;
    float xh[NV][8], gd[NV][8];
    uint4 ca[NV];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
        const uint4 px = reinterpret_cast<const uint4*>(st)[vi];
        const uint4 pd = reinterpret_cast<const uint4*>(st + row_bytes)[vi];
        if (add_to_dx) ca[i] = reinterpret_cast<const uint4*>(st + 2 * row_bytes)[vi];
        const uint32_t wx[4] = {px.x, px.y, px.z, px.w};
        const uint32_t wd[4] = {pd.x, pd.y, pd.z, pd.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 fx = unpack_bf16x2(wx[j]), fd = unpack_bf16x2(wd[j]);
          float h0 = (fx.x - mu) * rs, h1 = (fx.y - mu) * rs;
          xh[i][2 * j] = h0; xh[i][2 * j + 1] = h1;
          acc_g[i][2 * j] += fd.x * h0; acc_g[i][2 * j + 1] += fd.y * h1;
          acc_b[i][2 * j] += fd.x; acc_b[i][2 * j + 1] += fd.y;
          float a0 = fd.x * g[i][2 * j], a1 = fd.y * g[i][2 * j + 1];
          gd[i][2 * j] = a0; gd[i][2 * j + 1] = a1;
          s1 += a0 + a1;
          s2 += a0 * h0 + a1 * h1;
        }
      }
    }
    block_sum2(s1, s2, red);   // its barriers also order every thread's reads of this stage before the refill below
    if (threadIdx.x == 0 && k + kLnRingStages < my_rows) issue(k + kLnRingStages);
    const float m1 = s1 / cols, m2 = s2 / cols;
    uint4* dxr = reinterpret_cast<uint4*>(dx + static_cast<long long>(row) * cols);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
        float r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = rs * (gd[i][j] - m1 - xh[i][j] * m2);
        if (add_to_dx) {
          const uint32_t wa[4] = {ca[i].x, ca[i].y, ca[i].z, ca[i].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16x2(wa[j]); r[2 * j] += f.x; r[2 * j + 1] += f.y; }
        }
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) ow[j] = pack_bf16x2(r[2 * j], r[2 * j + 1]);
        __stcs(dxr + vi, o);
      }
    }
  }
  if (!ok) {
    // a copy never completed: report it; the copies still in flight land in this CTA's own shared memory, so give them a
    // bounded moment before the CTA ends
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, (int)kStatusMbarTimeout);
  }
  if (partial_dgamma) {
    float* pg = partial_dgamma + static_cast<long long>(blockIdx.x) * cols;
    float* pb = partial_dbeta + static_cast<long long>(blockIdx.x) * cols;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
        float4* a = reinterpret_cast<float4*>(pg + vi * 8);
        float4* b = reinterpret_cast<float4*>(pb + vi * 8);
        a[0] = make_float4(acc_g[i][0], acc_g[i][1], acc_g[i][2], acc_g[i][3]);
        a[1] = make_float4(acc_g[i][4], acc_g[i][5], acc_g[i][6], acc_g[i][7]);
        b[0] = make_float4(acc_b[i][0], acc_b[i][1], acc_b[i][2], acc_b[i][3]);
        b[1] = make_float4(acc_b[i][4], acc_b[i][5], acc_b[i][6], acc_b[i][7]);
      }
    }
  }
}

// Folds partial[nparts, cols] into out[cols] (fp32, optionally accumulating). Block = 32 columns x 8 part
// lanes: the 8 lanes of a column stride over the parts, then a shared-memory step adds them.
__global__ void __launch_bounds__(256)
fold_partials_kernel(const float* __restrict__ pa, const float* __restrict__ pb, float* __restrict__ outa,
                     float* __restrict__ outb, int nparts, int cols, int accumulate) {
  __shared__ float sa[8][33], sb[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float a = 0.f, b = 0.f;
  if (c < cols) {
    for (int p = ty; p < nparts; p += 8) {
      a += pa[static_cast<long long>(p) * cols + c];
      b += pb[static_cast<long long>(p) * cols + c];
    }
  }
  sa[ty][tx] = a;
  sb[ty][tx] = b;
  __syncthreads();
  if (ty == 0 && c < cols) {
#pragma unroll
    for (int k = 1; k < 8; ++k) { a += sa[k][tx]; b += sb[k][tx]; }
    if (accumulate) { a += outa[c]; b += outb[c]; }
    outa[c] = a;
    outb[c] = b;
  }
}

static int ln_block_threads(int cols, int& nv) {
  const int nvec = cols / 8;
  nv = 1;
  while (nv < kLnMaxVecPerThread && (nvec + nv - 1) / nv > 256) nv *= 2;  // aim for <=256 threads
  int threads = (nvec + nv - 1) / nv;
  if (threads > 1024) { nv = kLnMaxVecPerThread; threads = (nvec + nv - 1) / nv; }
  threads = ((threads + 31) / 32) * 32;
  return threads;
}

}  // namespace ofb

using namespace ofb;

OFB_API int ofb_layer_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                               int rows, int cols, float eps, void* stream) {
  if (cols % 8 != 0 || cols > 8 * kLnMaxVecPerThread * 1024) return fail("layer_norm: cols must be a multiple of 8 and <= 32768");
  if (rows <= 0) return 0;
  int nv;
  const int threads = ln_block_threads(cols, nv);
  const int grid = rows < 148 * 16 ? rows : 148 * 16;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto G = reinterpret_cast<const __nv_bfloat16*>(gamma);
  auto B = reinterpret_cast<const __nv_bfloat16*>(beta);
  auto Y = reinterpret_cast<__nv_bfloat16*>(y);
  switch (nv) {
    case 1: layer_norm_fwd_kernel<1><<<grid, threads, 0, s>>>(X, G, B, Y, mean, rstd, rows, cols, eps); break;
    case 2: layer_norm_fwd_kernel<2><<<grid, threads, 0, s>>>(X, G, B, Y, mean, rstd, rows, cols, eps); break;
    default: layer_norm_fwd_kernel<4><<<grid, threads, 0, s>>>(X, G, B, Y, mean, rstd, rows, cols, eps); break;
  }
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// Number of partial rows ofb_layer_norm_bwd writes: scratch must hold 2 * this * cols floats.
OFB_API int ofb_layer_norm_bwd_parts(int rows) { return rows < 296 ? rows : 296; }

OFB_API int ofb_layer_norm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                               const void* add_to_dx, void* dx, float* dgamma, float* dbeta, float* scratch,
                               int accumulate_param_grads, int rows, int cols, void* stream) {
  if (cols <= 0 || cols % 8 != 0 || cols > 8 * kLnMaxVecPerThread * 1024)
    return fail("layer_norm_bwd: cols must be a positive multiple of 8 and <= 32768");
  if ((dgamma == nullptr) != (dbeta == nullptr)) return fail("layer_norm_bwd: dgamma and dbeta must be given together or not at all");
  if (rows <= 0) return 0;
  if (dgamma && !scratch) return fail("layer_norm_bwd: scratch required for parameter gradients");
  int nv;
  const int threads = ln_block_threads(cols, nv);
  const int grid = ofb_layer_norm_bwd_parts(rows);
  auto s = reinterpret_cast<cudaStream_t>(stream);
  float* pg = dgamma ? scratch : nullptr;
  float* pb = dgamma ? scratch + static_cast<long long>(grid) * cols : nullptr;
  auto DY = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto G = reinterpret_cast<const __nv_bfloat16*>(gamma);
  auto AD = reinterpret_cast<const __nv_bfloat16*>(add_to_dx);
  auto DX = reinterpret_cast<__nv_bfloat16*>(dx);
  // rows of up to 4096 columns stream through the shared-memory ring (bulk copies need 16-byte aligned rows)
  const bool aligned16 = !((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(add_to_dx)) & 15);
  static const bool ring_off = std::getenv("OFB_LN_BWD_RING") && std::getenv("OFB_LN_BWD_RING")[0] == '0';
  if (nv <= 2 && aligned16 && !ring_off) {
    const int smem = kLnRingStages * 3 * cols * 2;
    static bool configured = false;
    if (!configured) {
      OFB_CUDA_OK(cudaFuncSetAttribute(layer_norm_bwd_ring_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kLnRingStages * 3 * 4096 * 2));
      OFB_CUDA_OK(cudaFuncSetAttribute(layer_norm_bwd_ring_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kLnRingStages * 3 * 4096 * 2));
      configured = true;
    }
    int* status = device_status_ptr();
    if (nv == 1) layer_norm_bwd_ring_kernel<1><<<grid, threads, smem, s>>>(DY, X, G, mean, rstd, AD, DX, pg, pb, rows, cols, status);
    else layer_norm_bwd_ring_kernel<2><<<grid, threads, smem, s>>>(DY, X, G, mean, rstd, AD, DX, pg, pb, rows, cols, status);
  } else {
    switch (nv) {
      case 1: layer_norm_bwd_kernel<1><<<grid, threads, 0, s>>>(DY, X, G, mean, rstd, AD, DX, pg, pb, rows, cols); break;
      case 2: layer_norm_bwd_kernel<2><<<grid, threads, 0, s>>>(DY, X, G, mean, rstd, AD, DX, pg, pb, rows, cols); break;
      default: layer_norm_bwd_kernel<4><<<grid, threads, 0, s>>>(DY, X, G, mean, rstd, AD, DX, pg, pb, rows, cols); break;
    }
  }
  OFB_CUDA_OK(cudaGetLastError());
  if (dgamma) {
    fold_partials_kernel<<<(cols + 31) / 32, 256, 0, s>>>(pg, pb, dgamma, dbeta, grid, cols, accumulate_param_grads);
    OFB_CUDA_OK(cudaGetLastError());
  }
  return 0;
}

// ------------------------------------------------------------------------------------------------
// LayerNorm backward for callers that must not allocate (declared in ofb_noalloc.h).
//
// The regular entry point above takes its partial-sum scratch from the caller, who normally gets it
// from an allocator. Some callers have none they may touch at that moment: code running inside a
// latency-critical serving loop that has frozen its memory pool, a plug-in that is handed raw device
// pointers by a host application and is forbidden to call cudaMalloc, or a step replayed under a
// memory budget that is already spoken for. For them the scratch lives in the library image itself.
//
// The array below is ordinary device memory reserved when the library is loaded: every GPU that loads
// libofb_kernels.so keeps kNoAllocScratchFloats * 4 bytes (9.25 MiB) until the process exits.
// Its size bounds the problem: cols <= kNoAllocMaxCols (rows are unlimited - the number of partial rows
// is capped at 296 whatever the row count).
//
// All calls share the one array and it keeps whatever the last call left in it. Nothing in it has to
// start at zero (each CTA overwrites its whole partial row before the fold reads it), so no clearing
// pass runs; but two calls that overlap on the GPU (different streams, or different threads launching
// at once) would write the same partial rows and race. Issue the calls on one stream, or order them
// with events.
//
// The first call on a device resolves the array's device address (cudaGetSymbolAddress, with that
// device current) and remembers it; that first call should therefore happen before any stream capture
// begins. No call here allocates or frees memory itself. One caveat comes from the CUDA runtime, not from
// this code: with lazy module loading (the default) the driver may load this library's module image,
// the 9.25 MiB array included, at the first call that touches it on a device, and that load can fail
// when the device has no memory left. A caller that freezes its memory should make one call (or load
// the module eagerly, CUDA_MODULE_LOADING=EAGER) before it does so.
// ------------------------------------------------------------------------------------------------
namespace {
constexpr int kNoAllocMaxCols = 4096;
constexpr int kNoAllocMaxParts = 296;
constexpr long long kNoAllocScratchFloats = 2ll * kNoAllocMaxParts * kNoAllocMaxCols;
static __device__ __align__(256) float g_ln_bwd_scratch[kNoAllocScratchFloats];

// In host code `g_ln_bwd_scratch` only names the symbol; the device address has to be asked for,
// once per device, while that device is current.
int noalloc_scratch_ptr(float** out) {
  static float* ptrs[64] = {nullptr};
  static std::mutex mu;
  int dev = -1;
  OFB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return ::ofb::fail("layer_norm_bwd_noalloc: unsupported device ordinal");
  std::lock_guard<std::mutex> g(mu);
  if (!ptrs[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_ln_bwd_scratch);
    if (e != cudaSuccess) return ::ofb::fail(std::string("cudaGetSymbolAddress(g_ln_bwd_scratch): ") + cudaGetErrorString(e));
    ptrs[dev] = static_cast<float*>(p);
  }
  *out = ptrs[dev];
  return 0;
}
}  // namespace

OFB_API int ofb_layer_norm_bwd_noalloc_max_cols(void) { return kNoAllocMaxCols; }

OFB_API int ofb_layer_norm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* mean,
                                       const float* rstd, const void* add_to_dx, void* dx, float* dgamma, float* dbeta,
                                       int accumulate_param_grads, int rows, int cols, void* stream) {
  if (cols > kNoAllocMaxCols)
    return fail("layer_norm_bwd_noalloc: cols = " + std::to_string(cols) + " exceeds the built-in scratch (max " +
                std::to_string(kNoAllocMaxCols) + " columns); use ofb_layer_norm_bwd with caller-provided scratch");
  if (cols <= 0 || cols % 8 != 0) return fail("layer_norm_bwd_noalloc: cols must be a positive multiple of 8");
  if ((dgamma == nullptr) != (dbeta == nullptr))
    return fail("layer_norm_bwd_noalloc: dgamma and dbeta must be given together or not at all");
  if (rows <= 0) return 0;
  float* scratch = nullptr;
  if (noalloc_scratch_ptr(&scratch)) return -1;
  int nv;
  const int threads = ln_block_threads(cols, nv);
  const int grid = rows < kNoAllocMaxParts ? rows : kNoAllocMaxParts;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  float* pg = dgamma ? scratch : nullptr;
  float* pb = dgamma ? scratch + static_cast<long long>(grid) * cols : nullptr;
  auto DY = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto G = reinterpret_cast<const __nv_bfloat16*>(gamma);
  auto AD = reinterpret_cast<const __nv_bfloat16*>(add_to_dx);
  auto DX = reinterpret_cast<__nv_bfloat16*>(dx);
  switch (nv) {
    case 1: layer_norm_bwd_kernel<1><<<grid, threads, 0, s>>>(DY, X, G, mean, rstd, AD, DX, pg, pb, rows, cols); break;
    case 2: layer_norm_bwd_kernel<2><<<grid, threads, 0, s>>>(DY, X, G, mean, rstd, AD, DX, pg, pb, rows, cols); break;
    default: layer_norm_bwd_kernel<4><<<grid, threads, 0, s>>>(DY, X, G, mean, rstd, AD, DX, pg, pb, rows, cols); break;
  }
  OFB_CUDA_OK(cudaGetLastError());
  if (dgamma) {
    fold_partials_kernel<<<(cols + 31) / 32, 256, 0, s>>>(pg, pb, dgamma, dbeta, grid, cols, accumulate_param_grads);
    OFB_CUDA_OK(cudaGetLastError());
  }
  return 0;
}
