// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   D[M,N] = epilogue( alpha * sum_k A[m,k] * B[n,k] )
//
// * operands are fetched by TMA (128-byte swizzle, tiled mode, never multicast) into a
//   multi-stage shared-memory ring,
// * one elected thread issues tcgen05.mma (cta_group::1, 128 x BN x 16 per instruction),
//   accumulating in TMEM; two TMEM accumulators are ping-ponged so that the epilogue of
//   tile i overlaps the main loop of tile i+1,
// * four epilogue warps read TMEM with tcgen05.ld (one accumulator row per thread) and
//   apply the fused epilogue (bias, GELU/ReLU, activation-gradient multiply, residual
//   add, accumulate, optional second output with the pre-activation, optional stores to
//   peer GPUs for the fused collectives).
//
// Either operand may be "K-major" (the reduction index is the contiguous one: A stored
// [M,K], B stored [N,K] like a torch Linear weight) or "MN-major" (A stored [K,M], B
// stored [K,N]); this covers forward, data-gradient and weight-gradient products
// without any transposition pass.
//
// Plays the role of the reference's cuBLAS/cuBLASLt matmul family
// (oneflow/user/kernels/matmul_kernels.cpp, cublas_fused_mlp_kernel.cu,
// fused_matmul_bias_kernel.cu), written for tcgen05 instead of calling a library.
#pragma once
#include "../common/ptx.cuh"

namespace ofb {

enum GemmAct : int { kActNone = 0, kActGeluErf = 1, kActGeluTanh = 2, kActRelu = 3 };

struct GemmEpilogue {
  void* C;                        // [M, ldc] bf16 (or fp32 when out_fp32)
  long long ldc;
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldr] or null: added after the activation
  long long ldr;
  const __nv_bfloat16* aux_in;    // [M, ld_aux] pre-activation; result *= act'(aux_in)
  __nv_bfloat16* aux_out;         // [M, ld_aux] receives the pre-activation (bias included)
  long long ld_aux;
  float alpha;
  int act;                        // GemmAct applied to (alpha*acc + bias)
  int out_fp32;                   // C is fp32
  int accumulate;                 // C += result
};

struct GemmShape {
  int M, N, K;
  int splits;  // > 1: the K range is cut into this many pieces whose partial sums are added atomically into an fp32 C
};

}  // namespace ofb
#include "gemm_epilogue.cuh"
namespace ofb {

// ST = 0 picks the deep ring for compute-bound problems (one CTA per SM); a short ring (2) leaves room for two CTAs
// per SM, which doubles the epilogue throughput of problems with few K blocks.
template <int BN, int ST = 0>
struct GemmCfg {
  static constexpr int BM = 128;
  static constexpr int BK = 64;
  static constexpr int STAGES = ST > 0 ? ST : ((BN == 256) ? 4 : 6);
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int TMEM_COLS = (2 * BN <= 256) ? 256 : 512;
  static constexpr int EPI_BYTES = 4 * 32 * 128;  // staging tile of each epilogue warp (gemm_epilogue.cuh)
  static constexpr int SMEM_BYTES = STAGES * (A_BYTES + B_BYTES) + EPI_BYTES + 256 /*barriers*/ + 1024 /*alignment*/;
  static constexpr int THREADS = 192;
};

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case kActGeluErf: return gelu_erf(v);
    case kActGeluTanh: return gelu_tanh(v);
    case kActRelu: return v > 0.f ? v : 0.f;
    default: return v;
  }
}
__device__ __forceinline__ float apply_act_grad(float h, int act) {
  switch (act) {
    case kActGeluErf: return gelu_erf_grad(h);
    case kActGeluTanh: return gelu_tanh_grad(h);
    case kActRelu: return h > 0.f ? 1.f : 0.f;
    default: return 1.f;
  }
}

// Grouped rasterisation: consecutive tile ids walk down a band of GROUP_M row-tiles so
// that the CTAs running at the same time share A and B tiles in L2.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int GROUP_M = 16;
  int per_group = GROUP_M * tiles_n;
  int g = t / per_group;
  int first_m = g * GROUP_M;
  int gsz = min(tiles_m - first_m, GROUP_M);
  int r = t - g * per_group;
  tm = first_m + (r % gsz);
  tn = r / gsz;
}

template <int BN, int A_MN, int B_MN, int ST = 0, int MINB = 1>
__global__ void __launch_bounds__(192, MINB)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         GemmShape shp, GemmEpilogue ep, int* status) {
  using Cfg = GemmCfg<BN, ST>;
  constexpr int BM = Cfg::BM, BK = Cfg::BK, STAGES = Cfg::STAGES;
  constexpr int A_BYTES = Cfg::A_BYTES, B_BYTES = Cfg::B_BYTES;
  constexpr uint32_t IDESC = make_idesc_bf16(BM, BN, A_MN, B_MN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint8_t* epi_stage = smem + STAGES * (A_BYTES + B_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(epi_stage + Cfg::EPI_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (shp.M + BM - 1) / BM;
  const int tiles_n = (shp.N + BN - 1) / BN;
  const int total_tiles = tiles_m * tiles_n;
  const int kblocks = (shp.K + BK - 1) / BK;
  // split-K: unit u = (tile u % total_tiles, K piece u / total_tiles); no piece is empty
  const int kb_per = (kblocks + max(shp.splits, 1) - 1) / max(shp.splits, 1);
  const int splits = (kblocks + kb_per - 1) / kb_per;
  const int total_units = total_tiles * splits;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        int tm, tn;
        tile_coords(u % total_tiles, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        const int kb0 = (u / total_tiles) * kb_per, kb1 = min(kblocks, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&full[stage], A_BYTES + B_BYTES);
          uint8_t* a_dst = sA + stage * A_BYTES;
          uint8_t* b_dst = sB + stage * B_BYTES;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(a_dst + c * (BK * 128), &tmA, &full[stage], m0 + c * 64, kb * BK);
          } else {
            tma_load_2d(a_dst, &tmA, &full[stage], kb * BK, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(b_dst + c * (BK * 128), &tmB, &full[stage], n0 + c * 64, kb * BK);
          } else {
            tma_load_2d(b_dst, &tmB, &full[stage], kb * BK, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int kb0 = (u / total_tiles) * kb_per, kb1 = min(kblocks, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + stage * A_BYTES);
          const uint32_t b_base = smem_u32(sB + stage * B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(a_base + k * 2048, BK * 128, 1024)
                                     : make_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_base + k * 2048, BK * 128, 1024)
                                     : make_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_bf16_ss(d_tmem, da, db, IDESC, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);  // frees the smem stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    const uint32_t stage = smem_u32(epi_stage + quad * kEpiStageBytesPerWarp);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int u = blockIdx.x; u < total_units; u += gridDim.x) {
      int tm, tn;
      tile_coords(u % total_tiles, tiles_m, tiles_n, tm, tn);
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) break;
      tc_fence_after();
      gemm_epilogue_warp<BN>(ep, shp, tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN, tm * BM + quad * 32, tn * BN,
                             lane, stage, splits > 1);
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
    // Something upstream never arrived: let copies that may still be in flight land before the
    // shared memory is released, then report.
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, (int)kStatusMbarTimeout);
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace ofb
