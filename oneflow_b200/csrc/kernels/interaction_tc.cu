// DLRM dot feature interaction on the tensor cores (tcgen05 + TMEM + TMA), embedding dim 128.
//
// Three samples share one 128-row operand tile X (bf16, K-major, 128-byte swizzle, two 64-column halves):
//     rows 32 s + t   (s = 0..2, t < T)  sparse feature t of sample s      (TMA box of T rows per sample and half)
//     rows 96 + s                         dense vector of sample s          (one TMA box of 3 rows per half)
//     all other rows                      zero (cleared once; no copy ever writes them)
// Forward:  G = X X^T is one 128 x 128 x 128 MMA chain with X as both operands; the pair products of sample s sit
//           in the diagonal block (rows/cols 32 s ..) and in column 96 + s, so the epilogue warp that owns TMEM
//           lanes 32 s .. 32 s + 31 reads its block with two tcgen05.ld, scatters the lower triangle into a
//           staging row in shared memory and writes the output row with full 16-byte pieces.
// Backward: dX = A X with the same X tile as the (MN-major) B operand and A = the symmetric gradient matrix of the
//           three samples laid out block-diagonally (plus row/column 96 + s for the dense vector), which three
//           builder warps assemble in shared memory from dout while the previous tile runs.
// Roles per CTA: warp 0 TMA producer, warp 1 MMA issuer, then builder (backward only: 4) and epilogue warps (backward: 8); the
// tiles flow through a multi-stage shared-memory ring and two TMEM accumulators, every wait is bounded.
//
// Reference: oneflow/user/kernels/fused_dot_feature_interaction_kernel.cu (wmma, one CTA per sample).
#include "../common/host_utils.h"
#include "../common/ptx.cuh"
#include "gemm_tcgen05.cuh"
#include "ofb_kernels.h"

namespace ofb {

constexpr int kItD = 128;
constexpr int kItHalfBytes = 128 * 128;          // [128 rows][64 columns] bf16
constexpr int kItTileBytes = 2 * kItHalfBytes;   // 32 KB
constexpr int kItSamples = 3;

struct ItParams {
  long long batch;
  int T;         // sparse features per sample (<= 31)
  int out_dim;   // elements per output row: 128 + T (T + 1) / 2 + padding, multiple of 8
  int groups;    // ceil(batch / 3)
};

__device__ __forceinline__ uint32_t it_swz(uint32_t tile, int row, int chunk) {
  return tile + row * 128 + ((chunk ^ (row & 7)) << 4);
}

// ------------------------------------------------------------------------------------------------ forward
template <int STAGES>
__global__ void __launch_bounds__(192, 2)
interaction_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmD,
                          const __nv_bfloat16* __restrict__ dense, __nv_bfloat16* __restrict__ out, ItParams p, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  __nv_bfloat16* ostage = reinterpret_cast<__nv_bfloat16*>(smem + STAGES * kItTileBytes);  // [3][512]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * kItTileBytes + 3 * 1024);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int i = threadIdx.x; i < STAGES * kItTileBytes / 16; i += blockDim.x) reinterpret_cast<uint4*>(tiles)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], kItSamples);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmS);
    tma_prefetch_desc(&tmD);
  }
  fence_proxy_async_smem();  // the zero fill above must be ordered before the first TMA write into the tiles
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tx_bytes = 2u * (kItSamples * p.T * 128u + kItSamples * 128u);
  constexpr uint32_t IDESC = make_idesc_bf16(128, 128, 0, 0);

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (int g = blockIdx.x; g < p.groups; g += gridDim.x) {
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) break;
        mbar_arrive_expect_tx(&full[stage], tx_bytes);
        uint8_t* tile = tiles + stage * kItTileBytes;
        for (int h = 0; h < 2; ++h) {
          for (int s = 0; s < kItSamples; ++s)
            tma_load_2d(tile + h * kItHalfBytes + s * 32 * 128, &tmS, &full[stage], h * 64, (g * kItSamples + s) * p.T);
          tma_load_2d(tile + h * kItHalfBytes + 96 * 128, &tmD, &full[stage], h * 64, g * kItSamples);
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int g = blockIdx.x; g < p.groups; g += gridDim.x) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) break;
        if (!mbar_wait(&full[stage], phase, abort_flag)) break;
        tc_fence_after();
        const uint32_t base = smem_u32(tiles + stage * kItTileBytes);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t d = make_smem_desc_sw128(base + (k >> 2) * kItHalfBytes + (k & 3) * 32, 16, 1024);
          umma_bf16_ss(tmem_base + acc * 128, d, d, IDESC, k != 0 ? 1u : 0u);
        }
        umma_commit(&empty[stage]);
        umma_commit(&tfull[acc]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    __syncwarp();
  } else if ((warp & 3) < kItSamples) {
    const int q = warp & 3;  // TMEM lane quadrant = sample of the group
    __nv_bfloat16* sp = ostage + q * 512;
    const int npairs = p.T * (p.T + 1) / 2;
    const int tail = p.out_dim - kItD;  // elements after the dense part
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int g = blockIdx.x; g < p.groups; g += gridDim.x) {
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) break;
      tc_fence_after();
      uint32_t r[32], r2[16];
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * 128;
      tmem_ld_32x32(taddr + q * 32, r);
      tmem_ld_32x16(taddr + 96, r2);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
      const long long b = static_cast<long long>(g) * kItSamples + q;
      if (b < p.batch) {
        // feature order of the output: dense = 0, sparse t = t + 1; pair (i > j) sits at i (i - 1) / 2 + j
        if (lane < p.T) {
          const int base = lane * (lane + 1) / 2;
          const uint32_t gd = q == 0 ? r2[0] : (q == 1 ? r2[1] : r2[2]);
          sp[base] = __float2bfloat16(__uint_as_float(gd));
#pragma unroll
          for (int u = 0; u < 31; ++u)
            if (u < lane) sp[base + 1 + u] = __float2bfloat16(__uint_as_float(r[u]));
        }
        for (int i = npairs + lane; i < tail; i += 32) sp[i] = __float2bfloat16(0.f);
        __syncwarp();
        __nv_bfloat16* o = out + b * p.out_dim;
        if (lane < 16) reinterpret_cast<uint4*>(o)[lane] = __ldg(reinterpret_cast<const uint4*>(dense + b * kItD) + lane);
        for (int i = lane; i < tail / 8; i += 32) reinterpret_cast<uint4*>(o + kItD)[i] = reinterpret_cast<const uint4*>(sp)[i];
        __syncwarp();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);  // let copies in flight land before the shared memory goes away
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, (int)kStatusMbarTimeout);
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem_base, 256);
}

// ------------------------------------------------------------------------------------------------ backward
template <int STAGES>
__global__ void __launch_bounds__(448, 1)
interaction_bwd_tc_kernel(const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmD,
                          const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ d_dense,
                          __nv_bfloat16* __restrict__ d_sparse, ItParams p, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* xt = smem;                              // [STAGES] X tiles
  uint8_t* at = smem + STAGES * kItTileBytes;      // [STAGES] A tiles
  uint8_t* epi = at + STAGES * kItTileBytes;       // [8] epilogue staging, 4 KB each
  __nv_bfloat16* gbuf = reinterpret_cast<__nv_bfloat16*>(epi + 8 * kEpiStageBytesPerWarp);  // [3][512]
  uint64_t* x_full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(gbuf) + 3 * 1024);
  uint64_t* a_full = x_full + STAGES;
  uint64_t* empty = a_full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int i = threadIdx.x; i < 2 * STAGES * kItTileBytes / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&x_full[s], 1);
      mbar_init(&a_full[s], kItSamples);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmS);
    tma_prefetch_desc(&tmD);
  }
  fence_proxy_async_smem();
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tx_bytes = 2u * (kItSamples * p.T * 128u + kItSamples * 128u);
  constexpr uint32_t IDESC = make_idesc_bf16(128, 128, 0, 1);
  const int T = p.T;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (int g = blockIdx.x; g < p.groups; g += gridDim.x) {
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) break;
        mbar_arrive_expect_tx(&x_full[stage], tx_bytes);
        uint8_t* tile = xt + stage * kItTileBytes;
        for (int h = 0; h < 2; ++h) {
          for (int s = 0; s < kItSamples; ++s)
            tma_load_2d(tile + h * kItHalfBytes + s * 32 * 128, &tmS, &x_full[stage], h * 64, (g * kItSamples + s) * T);
          tma_load_2d(tile + h * kItHalfBytes + 96 * 128, &tmD, &x_full[stage], h * 64, g * kItSamples);
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int g = blockIdx.x; g < p.groups; g += gridDim.x) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) break;
        if (!mbar_wait(&x_full[stage], phase, abort_flag)) break;
        if (!mbar_wait(&a_full[stage], phase, abort_flag)) break;
        tc_fence_after();
        const uint32_t a_base = smem_u32(at + stage * kItTileBytes);
        const uint32_t b_base = smem_u32(xt + stage * kItTileBytes);
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // K = the 128 tile rows, 16 per instruction
          const uint64_t da = make_smem_desc_sw128(a_base + (k >> 2) * kItHalfBytes + (k & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(b_base + k * 2048, kItHalfBytes, 1024);
          umma_bf16_ss(tmem_base + acc * 128, da, db, IDESC, k != 0 ? 1u : 0u);
        }
        umma_commit(&empty[stage]);
        umma_commit(&tfull[acc]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ---------------------------------------------------------------- builders of the gradient operand
    const int q = warp & 3;
    if (q < kItSamples) {
      __nv_bfloat16* gb = gbuf + q * 512;
      const int npairs = T * (T + 1) / 2;
      int stage = 0;
      uint32_t phase = 0;
      for (int g = blockIdx.x; g < p.groups; g += gridDim.x) {
        const long long b = static_cast<long long>(g) * kItSamples + q;
        // pair gradients of this sample, fetched before the wait so that the load latency overlaps it
        uint4 v0 = make_uint4(0, 0, 0, 0), v1 = v0;
        if (b < p.batch) {
          const uint4* src = reinterpret_cast<const uint4*>(dout + b * p.out_dim + kItD);
          if (lane * 8 < npairs) v0 = __ldg(src + lane);
          if ((lane + 32) * 8 < npairs) v1 = __ldg(src + lane + 32);
        }
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) break;
        reinterpret_cast<uint4*>(gb)[lane] = v0;
        reinterpret_cast<uint4*>(gb)[lane + 32] = v1;
        __syncwarp();
        const uint32_t a_tile = smem_u32(at + stage * kItTileBytes);
        const int t = lane;
        const int row = 32 * q + t;
        const __nv_bfloat16 zero = __float2bfloat16(0.f);
        // row (q, t): columns (q, u) of the diagonal block, feature order dense = 0, sparse u = u + 1
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __nv_bfloat16 e[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int u = 8 * j + i;
            const int hi = (t > u ? t : u) + 1, lo = (t > u ? u : t) + 1;
            const int idx = hi * (hi - 1) / 2 + lo;
            e[i] = (t < T && u < T && u != t && idx < npairs) ? gb[idx] : zero;
          }
          uint4 qv;
          qv.x = (uint32_t)__bfloat16_as_ushort(e[0]) | ((uint32_t)__bfloat16_as_ushort(e[1]) << 16);
          qv.y = (uint32_t)__bfloat16_as_ushort(e[2]) | ((uint32_t)__bfloat16_as_ushort(e[3]) << 16);
          qv.z = (uint32_t)__bfloat16_as_ushort(e[4]) | ((uint32_t)__bfloat16_as_ushort(e[5]) << 16);
          qv.w = (uint32_t)__bfloat16_as_ushort(e[6]) | ((uint32_t)__bfloat16_as_ushort(e[7]) << 16);
          epi_sts(it_swz(a_tile + (q >> 1) * kItHalfBytes, row, (q & 1) * 4 + j), qv);
        }
        // row (q, t), column 96 + q: the pair with the dense vector
        {
          const __nv_bfloat16 gd = t < T ? gb[t * (t + 1) / 2] : zero;
          const uint32_t hv = __bfloat16_as_ushort(gd);
          uint4 qv = make_uint4(0, 0, 0, 0);
          if (q == 0) qv.x = hv;
          if (q == 1) qv.x = hv << 16;
          if (q == 2) qv.y = hv;
          epi_sts(it_swz(a_tile + kItHalfBytes, row, 4), qv);
        }
        // row 96 + q: the same pair gradients along the columns (q, u)
        if (lane < 4) {
          __nv_bfloat16 e[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int u = 8 * lane + i;
            e[i] = u < T ? gb[u * (u + 1) / 2] : zero;
          }
          uint4 qv;
          qv.x = (uint32_t)__bfloat16_as_ushort(e[0]) | ((uint32_t)__bfloat16_as_ushort(e[1]) << 16);
          qv.y = (uint32_t)__bfloat16_as_ushort(e[2]) | ((uint32_t)__bfloat16_as_ushort(e[3]) << 16);
          qv.z = (uint32_t)__bfloat16_as_ushort(e[4]) | ((uint32_t)__bfloat16_as_ushort(e[5]) << 16);
          qv.w = (uint32_t)__bfloat16_as_ushort(e[6]) | ((uint32_t)__bfloat16_as_ushort(e[7]) << 16);
          epi_sts(it_swz(a_tile + (q >> 1) * kItHalfBytes, 96 + q, (q & 1) * 4 + lane), qv);
        }
        fence_proxy_async_smem();  // generic-proxy stores above -> tensor-core (async proxy) reads
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_full[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 6..13): two warps per TMEM lane
    // quadrant, each draining two of the four 32-column chunks (one warp per scheduler alone cannot keep up)
    const int q = warp & 3;
    const int half = (warp - 6) >> 2;
    const uint32_t stage_sm = smem_u32(epi + (warp - 6) * kEpiStageBytesPerWarp);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int g = blockIdx.x; g < p.groups; g += gridDim.x) {
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) break;
      tc_fence_after();
      const long long b0 = static_cast<long long>(g) * kItSamples;
#pragma unroll 1
      for (int c = half * 2; c < half * 2 + 2; ++c) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * 128 + c * 32, r);
        tmem_wait_ld();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (q < kItSamples) {
          const long long b = b0 + q;
          epi_store_bf16(stage_sm, lane, v, d_sparse + b * T * kItD + c * 32, kItD, b < p.batch ? T : 0, 32, false);
        } else {
          long long left = p.batch - b0;
          const int rv = left >= kItSamples ? kItSamples : (left > 0 ? static_cast<int>(left) : 0);
          float h[32];
          epi_load_bf16(stage_sm, lane, dout + b0 * p.out_dim + c * 32, p.out_dim, rv, 32, h);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += h[j];
          epi_store_bf16(stage_sm, lane, v, d_dense + b0 * kItD + c * 32, kItD, rv, 32, false);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, (int)kStatusMbarTimeout);
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem_base, 256);
}

}  // namespace ofb

using namespace ofb;

static int it_sm_count() {
  static int sm = 0;
  if (sm == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sm = 148;
  }
  return sm;
}

static int it_check(long long batch, int T, int D, int out_dim) {
  if (D != kItD) return fail("interaction_tc: embedding dim must be 128");
  if (T < 1 || T > 31) return fail("interaction_tc: 1..31 sparse features");
  if (out_dim % 8 || out_dim < D + T * (T + 1) / 2 || out_dim - D > 512) return fail("interaction_tc: bad output row length");
  if (batch * T >= (1ll << 31) - 64) return fail("interaction_tc: batch too large for the tensor map coordinates");
  return 0;
}

static int it_maps(CUtensorMap* tmS, CUtensorMap* tmD, const void* dense, const void* sparse, long long batch, int T) {
  if (get_tensor_map(tmS, sparse, 2, 2, kItD, static_cast<uint64_t>(batch) * T, 0, kItD * 2, 0, 64, T, 0, 3)) return -1;
  if (get_tensor_map(tmD, dense, 2, 2, kItD, static_cast<uint64_t>(batch), 0, kItD * 2, 0, 64, kItSamples, 0, 3)) return -1;
  return 0;
}

// out[b] = [dense[b] | sparse/dense pair products, lower triangle row by row | zero padding], no self-interaction.
OFB_API int ofb_interaction_tc_fwd(const void* dense, const void* sparse, void* out, long long batch, int T, int D, int out_dim,
                                   void* stream) {
  if (it_check(batch, T, D, out_dim)) return -1;
  if (batch == 0) return 0;
  CUtensorMap tmS, tmD;
  if (it_maps(&tmS, &tmD, dense, sparse, batch, T)) return -1;
  constexpr int STAGES = 3;
  constexpr int SMEM = STAGES * kItTileBytes + 3 * 1024 + 256 + 1024;
  auto kern = interaction_fwd_tc_kernel<STAGES>;
  static bool configured = false;
  if (!configured) {
    OFB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured = true;
  }
  ItParams p{batch, T, out_dim, static_cast<int>((batch + kItSamples - 1) / kItSamples)};
  int grid = 2 * it_sm_count();
  if (grid > p.groups) grid = p.groups;
  kern<<<grid, 192, SMEM, reinterpret_cast<cudaStream_t>(stream)>>>(tmS, tmD, reinterpret_cast<const __nv_bfloat16*>(dense),
                                                                    reinterpret_cast<__nv_bfloat16*>(out), p, device_status_ptr());
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

OFB_API int ofb_interaction_tc_bwd(const void* dense, const void* sparse, const void* dout, void* d_dense, void* d_sparse,
                                   long long batch, int T, int D, int out_dim, void* stream) {
  if (it_check(batch, T, D, out_dim)) return -1;
  if (batch == 0) return 0;
  CUtensorMap tmS, tmD;
  if (it_maps(&tmS, &tmD, dense, sparse, batch, T)) return -1;
  constexpr int STAGES = 2;
  constexpr int SMEM = 2 * STAGES * kItTileBytes + 8 * kEpiStageBytesPerWarp + 3 * 1024 + 256 + 1024;
  auto kern = interaction_bwd_tc_kernel<STAGES>;
  static bool configured = false;
  if (!configured) {
    OFB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured = true;
  }
  ItParams p{batch, T, out_dim, static_cast<int>((batch + kItSamples - 1) / kItSamples)};
  int grid = it_sm_count();
  if (grid > p.groups) grid = p.groups;
  kern<<<grid, 448, SMEM, reinterpret_cast<cudaStream_t>(stream)>>>(
      tmS, tmD, reinterpret_cast<const __nv_bfloat16*>(dout), reinterpret_cast<__nv_bfloat16*>(d_dense),
      reinterpret_cast<__nv_bfloat16*>(d_sparse), p, device_status_ptr());
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
