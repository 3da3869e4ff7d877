// Two-SM variant of the bf16 GEMM: a cluster of two CTAs (a "CTA pair") computes one 256 x 256 tile with
// `tcgen05.mma.cta_group::2`. Each CTA stages its own 128 rows of A and HALF of the B tile (128 of the 256
// columns); the pair's tensor cores read both halves, so the L2 -> shared-memory traffic per flop drops by a
// third compared with the one-SM 128 x 256 tile (64 instead of 96 bytes per tensor-core cycle per SM) and the
// ring holds 6 stages instead of 4. Only the leader CTA (cluster rank 0) issues MMAs; completion is signalled
// to both CTAs with `tcgen05.commit ... multicast::cluster`. TMA loads are plain (non-multicast) tile loads
// issued by each CTA for its own shared memory, with their byte counts landing on the leader's mbarrier.
//
// Roles per CTA (192 threads): warp 0 TMA producer, warp 1 MMA issuer (leader only; both allocate TMEM),
// warps 2..5 epilogue for the CTA's own 128 accumulator rows (same fused epilogue as the one-SM kernel).
#pragma once
#include "gemm_tcgen05.cuh"

namespace ofb {

struct Gemm2Cfg {
  static constexpr int BM = 128;       // rows per CTA (256 per pair)
  static constexpr int BN = 256;       // columns per pair
  static constexpr int BNH = 128;      // columns of B staged by each CTA
  static constexpr int BK = 64;
  static constexpr int STAGES = 6;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BNH * BK * 2;
  static constexpr int EPI_BYTES = 4 * 32 * 128;  // staging tile of each epilogue warp (gemm_epilogue.cuh)
  static constexpr int SMEM_BYTES = STAGES * (A_BYTES + B_BYTES) + EPI_BYTES + 256 + 1024;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load whose completion bytes are credited to an mbarrier given by its shared::cluster address
// (it may live in the peer CTA of the pair). No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive (once all MMAs issued so far have completed) on the mbarrier at this shared-memory offset in BOTH CTAs.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 0x3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}

template <int A_MN, int B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmShape shp,
                      GemmEpilogue ep, int* status) {
  using Cfg = Gemm2Cfg;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BNH = Cfg::BNH, BK = Cfg::BK, STAGES = Cfg::STAGES;
  constexpr int A_BYTES = Cfg::A_BYTES, B_BYTES = Cfg::B_BYTES;
  constexpr uint32_t IDESC = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint8_t* epi_stage = smem + STAGES * (A_BYTES + B_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(epi_stage + Gemm2Cfg::EPI_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();   // 0 = leader
  const bool leader = cta == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);     // leader's producer arrives once (expect_tx for the bytes of both CTAs)
      mbar_init(&empty[s], 1);    // one multicast commit per phase
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);   // 4 epilogue warps of each CTA of the pair (only the leader's copy is waited on)
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers are initialised before anybody signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (shp.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (shp.N + BN - 1) / BN;
  const int total_tiles = tiles_m * tiles_n;
  const int kblocks = (shp.K + BK - 1) / BK;
  const int pair = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += n_pairs) {
        int tm, tn;
        tile_coords(t, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * 2 * BM + static_cast<int>(cta) * BM;   // this CTA's rows
        const int n0 = tn * BN + static_cast<int>(cta) * BNH;      // this CTA's half of the B tile
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          if (leader) mbar_arrive_expect_tx(&full[stage], 2 * (A_BYTES + B_BYTES));
          const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0);
          uint8_t* a_dst = sA + stage * A_BYTES;
          uint8_t* b_dst = sB + stage * B_BYTES;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d_pair(a_dst + c * (BK * 128), &tmA, bar, m0 + c * 64, kb * BK);
          } else {
            tma_load_2d_pair(a_dst, &tmA, bar, kb * BK, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BNH / 64; ++c) tma_load_2d_pair(b_dst + c * (BK * 128), &tmB, bar, n0 + c * 64, kb * BK);
          } else {
            tma_load_2d_pair(b_dst, &tmB, bar, kb * BK, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader CTA only)
    if (leader && elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += n_pairs) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
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
            umma_bf16_ss_pair(d_tmem, da, db, IDESC, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5, both CTAs)
    const int quad = warp & 3;
    const uint32_t stage = smem_u32(epi_stage + quad * kEpiStageBytesPerWarp);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = pair; t < total_tiles; t += n_pairs) {
      int tm, tn;
      tile_coords(t, tiles_m, tiles_n, tm, tn);
      const int m0 = tm * 2 * BM + static_cast<int>(cta) * BM, n0 = tn * BN;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) break;
      tc_fence_after();
      gemm_epilogue_warp<BN>(ep, shp, tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN, m0 + quad * 32, n0, lane, stage,
                             false);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&tempty[acc]), 0));   // the leader owns the accumulator hand-off
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  // Neither CTA may leave (and release its shared memory / barriers) while the other can still signal it.
  cluster_sync_all();
  tc_fence_after();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    if (threadIdx.x == 0 && status) {
      if (atomicCAS(status, 0, (int)kStatusMbarTimeout) == 0) status[1] = 2000 + static_cast<int>(cta);
    }
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

}  // namespace ofb
