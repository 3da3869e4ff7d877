// GEMM fused with its collective over NVSwitch peer memory (tensor parallel with sequence-parallel
// activations). One persistent tcgen05 kernel per call does the tensor-core tiles AND the transfer:
//
//   MODE_RS  "GEMM -> reduce-scatter" (row-parallel Linear forward, column-parallel dX):
//       every rank computes its partial C[T, N] tile by tile, owners interleaved (peer, ..., peer, self, ...). The
//       epilogue of a peer's tile stores it (bf16) straight into the staging buffer of the rank that owns those
//       rows (plain P2P stores over NVLink) and publishes a per-(tile, quadrant) flag there. The epilogue of an own
//       tile waits (bounded) for the peers' flags of that tile and finishes the reduction in registers:
//       out = alpha * acc + the peers' partials + bias + residual shard. No separate reduction pass exists and the
//       transfers are spread over the whole kernel.
//   MODE_AG  "all-gather -> GEMM" (column-parallel Linear forward, row-parallel dX, ZeRO parameter gather
//       in front of the first consuming GEMM):
//       two extra copier warps per CTA pull the peers' row shards into this GPU's gathered buffer (each
//       remote tile crosses NVLink once); the TMA producer starts with the local rows and waits (bounded)
//       on a per-peer arrival counter before it loads rows that came from that peer. TMA only ever reads
//       local memory.
//
// Synchronisation uses monotonic epochs in the SignalBlock (comm_common.cuh); staging and gathered
// buffers are double-buffered by epoch parity and guarded by "consumed"/"pulled" acknowledgements, so a
// fast rank can run at most two calls ahead of a slow one. No NCCL, no TMA multicast.
//
// Reference counterparts: matmul + `_nccl_logical_reduce_scatter` / `_nccl_logical_all_gather` ops
// (oneflow/user/kernels/nccl_logical_kernels.cpp:199-352) inserted by insert_nccl_logical_op_pass.cpp.
#include <cstdlib>

#include "../common/host_utils.h"
#include "../kernels/gemm_2cta.cuh"
#include "comm_common.cuh"
#include "ofb_comm.h"

namespace ofb {

enum { MODE_RS = 1, MODE_AG = 2 };

struct GemmCommParams {
  int n, rank;
  int rows_per_rank;           // T / n, multiple of 128
  unsigned int epoch;          // per-mode call counter (1, 2, ...), identical on all ranks
  SignalBlock* sig[kMaxPeers];
  int* status;
  // ---- MODE_RS
  __nv_bfloat16* stage[kMaxPeers];    // staging of every rank: [2 parity][n src][rows_per_rank][N]
  unsigned int* flags[kMaxPeers];     // flags of every rank:   [2 parity][n src][flag_stride]
  int flag_stride;
  __nv_bfloat16* out;                 // [rows_per_rank, ldc] local result
  long long ldc;
  const __nv_bfloat16* bias;          // [N] or null (added once, after the reduction)
  const __nv_bfloat16* residual;      // [rows_per_rank, ldr] or null
  long long ldr;
  int done_slot;                      // local counter slot used to detect the last reducing CTA
  unsigned int done_target;
  // ---- MODE_AG
  const __nv_bfloat16* x_local;       // [rows_per_rank, K] this rank's shard (private memory)
  __nv_bfloat16* gathered[kMaxPeers]; // gathered buffers of every rank: [2 parity][T][K] (only peers' own rows are read)
  long long k_cols;                   // K (row length of the gathered matrix)
  unsigned int pull_target;           // cumulative arrival count expected on the per-peer pull counters
  int pull_slot;                      // first local counter slot of the per-peer pull counters
  // Element offset of the parity-1 half of the staging / gathered buffers. It is a property of the buffer (half of
  // its capacity), not of the current problem: consecutive calls with different shapes then never place one call's
  // parity-1 data over the parity-0 data of the previous call that a slow peer may still be reading.
  long long parity_stride;
  int tune;                           // OFB_GEMM_COMM_TUNE bit mask, experiments only (0 in normal use)
  unsigned int* ag_flags[kMaxPeers];  // pair kernel, MODE_AG: per rank [n owners][256] "CTA b of owner o has pushed its slice" epochs
  int ag_done_slot;                   // local counter slot that detects the last CTA of an all-gather call
};

template <int BN>
struct GemmCommCfg {
  static constexpr int THREADS_RS = 192;
  static constexpr int THREADS_AG = 256;
};

__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

template <int BN, int B_MN, int MODE>
__global__ void __launch_bounds__(MODE == MODE_AG ? 256 : 320, 1)
gemm_comm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmAlocal,
                 const __grid_constant__ CUtensorMap tmB, GemmShape shp, GemmEpilogue ep, GemmCommParams cp) {
  using Cfg = GemmCfg<BN>;
  constexpr int BM = Cfg::BM, BK = Cfg::BK, STAGES = Cfg::STAGES;
  constexpr int A_BYTES = Cfg::A_BYTES, B_BYTES = Cfg::B_BYTES;
  constexpr uint32_t IDESC = make_idesc_bf16(BM, BN, 0, B_MN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  // MODE_RS drains every accumulator with eight warps (two per TMEM lane quadrant, half of the columns each): its
  // epilogue carries the P2P stores and the reduction of the own rows and would otherwise bound short-K problems.
  constexpr int EPI_WARPS = MODE == MODE_RS ? 8 : 4;
  uint8_t* epi_stage = smem + STAGES * (A_BYTES + B_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(epi_stage + EPI_WARPS * kEpiStageBytesPerWarp);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  SignalBlock* my_sig = cp.sig[cp.rank];
  const int parity = cp.epoch & 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], EPI_WARPS);
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
  const int tiles_m_per_rank = cp.rows_per_rank / BM;
  // Row-tile order. MODE_AG starts with the local rows (the peers' shards arrive meanwhile). MODE_RS interleaves the
  // owners tile by tile (peer, ..., peer, self, peer, ...), so that the P2P stores are spread evenly over the whole
  // kernel instead of saturating NVLink during its first part; every round ends with this rank's own rows.
  auto map_tm = [&](int tm) {
    if (MODE == MODE_AG) return (tm + cp.rank * tiles_m_per_rank) % tiles_m;
    const int o = (cp.rank + 1 + tm % cp.n) % cp.n;
    return o * tiles_m_per_rank + tm / cp.n;
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int ready_owner = cp.rank;  // rows of this owner are known to be present
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(t, tiles_m, tiles_n, tm, tn);
        tm = map_tm(tm);
        const int m0 = tm * BM, n0 = tn * BN;
        const int owner = tm / tiles_m_per_rank;
        if (MODE == MODE_AG && owner != cp.rank && owner != ready_owner) {
          if (!wait_local_ge(&my_sig->local_cnt[cp.pull_slot + owner], cp.pull_target, cp.status, 200 + owner)) {
            *abort_flag = 1;
            ok = false;
            break;
          }
          fence_proxy_async_global();
          ready_owner = owner;
        }
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&full[stage], A_BYTES + B_BYTES);
          uint8_t* a_dst = sA + stage * A_BYTES;
          uint8_t* b_dst = sB + stage * B_BYTES;
          if (MODE == MODE_AG && owner == cp.rank) {
            tma_load_2d(a_dst, &tmAlocal, &full[stage], kb * BK, m0 - cp.rank * cp.rows_per_rank);
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
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
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
            const uint64_t da = make_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_base + k * 2048, BK * 128, 1024)
                                     : make_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_bf16_ss(d_tmem, da, db, IDESC, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    __syncwarp();
  } else if (warp < 2 + EPI_WARPS) {
    // ---------------------------------------------------------------- epilogue (warps 2..5, MODE_RS: 2..9)
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;                       // which half of the tile's columns (MODE_RS)
    constexpr int CPW = (BN / 32) / (EPI_WARPS / 4);         // 32-column chunks per warp
    const int c_begin = half * CPW, c_end = c_begin + CPW;
    int acc = 0;
    uint32_t acc_phase = 0;
    unsigned int cleared_owners = 0;  // owners whose staging slab of this parity is known to be free
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      int tm, tn;
      tile_coords(t, tiles_m, tiles_n, tm, tn);
      tm = map_tm(tm);
      const int m0 = tm * BM, n0 = tn * BN;
      const int owner = tm / tiles_m_per_rank;
      if (MODE == MODE_RS && !((cleared_owners >> owner) & 1u)) {
        // The owner must have finished reducing what we stored into this parity two calls ago.
        int ok_w = 1;
        if (lane == 0 && cp.epoch > 2)
          ok_w = wait_flag_ge(&my_sig->rs_consumed[owner], cp.epoch - 2, cp.status, 300 + owner) ? 1 : 0;
        ok_w = __shfl_sync(0xffffffffu, ok_w, 0);
        if (!ok_w) { *abort_flag = 1; break; }
        cleared_owners |= 1u << owner;
      }
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      const uint32_t stage_sm = smem_u32(epi_stage + (warp - 2) * kEpiStageBytesPerWarp);
      const int tile_local = (tm - owner * tiles_m_per_rank) * tiles_n + tn;
      const bool remote_path = owner != cp.rank;
      if (MODE == MODE_RS && remote_path) {
        // The raw partial tile goes to the slab this rank owns in the staging buffer of the rows' owner (plain P2P
        // stores over NVLink, full 64-byte row segments); the owner adds it in the epilogue of its own tile.
        GemmEpilogue pe;
        pe.C = cp.stage[owner] + parity * cp.parity_stride + static_cast<long long>(cp.rank) * cp.rows_per_rank * shp.N;
        pe.ldc = shp.N;
        pe.bias = nullptr; pe.residual = nullptr; pe.aux_in = nullptr; pe.aux_out = nullptr;
        pe.ldr = 0; pe.ld_aux = 0;
        pe.alpha = ep.alpha; pe.act = kActNone; pe.out_fp32 = 0; pe.accumulate = 0;
        GemmShape slab{cp.rows_per_rank, shp.N, shp.K, 1};
        if (!(cp.tune & 1))
          gemm_epilogue_warp<BN>(pe, slab, taddr, m0 - owner * cp.rows_per_rank + quad * 32, n0, lane, stage_sm, false, c_begin, c_end);
      } else if (MODE == MODE_RS) {
        // Own rows: wait (bounded) until every peer's partial of this tile quadrant has landed in the local staging
        // buffer, then finish the reduction here: out = alpha * acc + sum of the peers' partials + bias + residual.
        int ok_w = 1;
        if (lane == 0 && !(cp.tune & 4)) {
          for (int s = 0; s < cp.n && ok_w; ++s) {
            if (s == cp.rank) continue;
            const unsigned int* f =
                cp.flags[cp.rank] + (static_cast<long long>(parity) * cp.n + s) * cp.flag_stride + tile_local * 8 + half * 4 + quad;
            ok_w = wait_flag_ge(f, cp.epoch, cp.status, 600 + s) ? 1 : 0;
          }
        }
        ok_w = __shfl_sync(0xffffffffu, ok_w, 0);
        if (!ok_w) { *abort_flag = 1; break; }
        const int lrow0 = m0 - owner * cp.rows_per_rank + quad * 32;
        const __nv_bfloat16* my_stage = cp.stage[cp.rank] + parity * cp.parity_stride;
        const int rows_valid = cp.rows_per_rank - lrow0;
        GemmEpilogue pe;
        pe.C = cp.out; pe.ldc = cp.ldc;
        pe.bias = cp.bias; pe.residual = nullptr; pe.ldr = 0;
        pe.aux_in = nullptr; pe.aux_out = nullptr; pe.ld_aux = 0;
        pe.alpha = 1.f; pe.act = kActNone; pe.out_fp32 = 0; pe.accumulate = 0;
#pragma unroll 1
        for (int c = c_begin; c < c_end; ++c) {
          const int col0 = n0 + c * 32;
          const int cols_valid = shp.N - col0;
          if (cols_valid <= 0) break;
          // the peers' partials and the residual shard, summed in fp32 with all their loads in flight together
          float h[32];
          epi_load_sum_bf16(stage_sm, lane, my_stage + static_cast<long long>(lrow0) * shp.N + col0,
                            static_cast<long long>(cp.rows_per_rank) * shp.N, (cp.tune & 8) ? 0 : cp.n, cp.rank, shp.N,
                            cp.residual ? cp.residual + static_cast<long long>(lrow0) * cp.ldr + col0 : nullptr, cp.ldr, rows_valid, cols_valid, h);
          uint32_t r[32];
          __syncwarp();
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(fmaf(__uint_as_float(r[j]), ep.alpha, h[j]));
          gemm_epilogue_chunk(pe, r, lrow0, col0, rows_valid, cols_valid, lane, stage_sm, false);
        }
      } else {
        gemm_epilogue_warp<BN>(ep, shp, taddr, m0 + quad * 32, n0, lane, stage_sm, false);
      }
      tc_fence_before();
      if (MODE == MODE_RS && remote_path && !(cp.tune & 2)) __threadfence_system();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&tempty[acc]);
        if (MODE == MODE_RS && remote_path) {
          // per (tile, quadrant) flag holding the call number: never reset, older calls left smaller values
          st_release_sys(cp.flags[owner] + (static_cast<long long>(parity) * cp.n + cp.rank) * cp.flag_stride + tile_local * 8 + half * 4 + quad,
                         cp.epoch);
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  } else if (MODE == MODE_AG) {
    // ---------------------------------------------------------------- copiers (warps 6, 7)
    const int ct = threadIdx.x - 192;  // 0..63
    const long long shard_vecs = static_cast<long long>(cp.rows_per_rank) * cp.k_cols / 8;
    const long long per_cta = (shard_vecs + gridDim.x - 1) / gridDim.x;
    const long long v0 = per_cta * blockIdx.x;
    const long long v1 = min(shard_vecs, v0 + per_cta);
    __nv_bfloat16* my_gathered = cp.gathered[cp.rank] + parity * cp.parity_stride;
    bool ok = true;
    // 1. publish the local shard: peers must have finished pulling what this parity held two calls ago
    if (ct == 0 && cp.epoch > 2) {
      for (int p = 0; p < cp.n && ok; ++p)
        if (p != cp.rank) ok = wait_flag_ge(&my_sig->ag_pulled[p], cp.epoch - 2, cp.status, 400 + p);
    }
    asm volatile("bar.sync 1, 64;" ::: "memory");
    {
      const uint4* src = reinterpret_cast<const uint4*>(cp.x_local);
      uint4* dst = reinterpret_cast<uint4*>(my_gathered + static_cast<long long>(cp.rank) * cp.rows_per_rank * cp.k_cols);
      for (long long i = v0 + ct; i < v1; i += 64) dst[i] = src[i];
    }
    __threadfence_system();
    asm volatile("bar.sync 1, 64;" ::: "memory");
    if (ct == 0) {
      const unsigned int arrived = atomicAdd(&my_sig->local_cnt[cp.pull_slot + cp.rank], 1u) + 1u;
      if (arrived == cp.pull_target) {  // last CTA: the whole local shard is readable by the peers
        for (int p = 0; p < cp.n; ++p)
          if (p != cp.rank) st_release_sys(&cp.sig[p]->ag_ready[cp.rank], cp.epoch);
      }
    }
    // 2. pull the peers' shards, nearest successor first (the order the GEMM consumes them in)
    for (int k = 1; k < cp.n; ++k) {
      const int o = (cp.rank + k) % cp.n;
      int okw = 1;
      if (ct == 0) okw = (ok && wait_flag_ge(&my_sig->ag_ready[o], cp.epoch, cp.status, 500 + o)) ? 1 : 0;
      __shared__ int ok_shared;
      if (ct == 0) ok_shared = okw;
      asm volatile("bar.sync 1, 64;" ::: "memory");
      if (!ok_shared) { *abort_flag = 1; break; }
      const uint4* src = reinterpret_cast<const uint4*>(cp.gathered[o] + parity * cp.parity_stride +
                                                        static_cast<long long>(o) * cp.rows_per_rank * cp.k_cols);
      uint4* dst = reinterpret_cast<uint4*>(my_gathered + static_cast<long long>(o) * cp.rows_per_rank * cp.k_cols);
      long long i = v0 + ct;
      // 8 independent 16-byte loads in flight per thread before the first store (16 measured slower at TP4: the
      // deeper read queue competes with the TMA loads of the MMA loop)
      for (; i + 7 * 64 < v1; i += 8 * 64) {
        uint4 t[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) t[u] = src[i + u * 64];
#pragma unroll
        for (int u = 0; u < 8; ++u) dst[i + u * 64] = t[u];
      }
      for (; i < v1; i += 64) dst[i] = src[i];
      __threadfence();
      asm volatile("bar.sync 1, 64;" ::: "memory");
      if (ct == 0) {
        const unsigned int arrived = atomicAdd(&my_sig->local_cnt[cp.pull_slot + o], 1u) + 1u;
        if (arrived == cp.pull_target) st_release_sys(&cp.sig[o]->ag_pulled[cp.rank], cp.epoch);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (MODE == MODE_RS && !*abort_flag) {
    // Tell the senders that this parity of the staging buffer may be reused.
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int arrived = atomicAdd(&my_sig->local_cnt[cp.done_slot], 1u) + 1u;
      if (arrived == cp.done_target)
        for (int p = 0; p < cp.n; ++p) st_release_sys(&cp.sig[p]->rs_consumed[cp.rank], cp.epoch);
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    if (threadIdx.x == 0 && cp.status) atomicCAS(cp.status, 0, (int)kStatusMbarTimeout);
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// ------------------------------------------------------------------------------------------------
// Drains a 32-row x 256-column strip of an accumulator (this warp's TMEM lane quadrant) as bf16 to `dst` with full-row
// stores: the strip is staged in shared memory (512 bytes per row, 16-byte pieces XOR-swizzled by the row so that both the
// row-per-thread writes and the row-per-instruction reads are conflict free), then every store instruction of the warp
// writes ONE whole row of 512 contiguous bytes and the 32 rows go out back to back. Over NVLink this is what reaches the
// link rate from few warps: stores of 64-byte row segments with a TMEM read between them measured about half of it.
__device__ __forceinline__ void rs_store_strip_wide(uint32_t smem_strip, uint32_t taddr, float alpha, __nv_bfloat16* dst, long long ld,
                                                    int rows_valid, int cols_valid, int lane) {
#pragma unroll 1
  for (int c = 0; c < 8; ++c) {
    uint32_t r[32];
    __syncwarp();
    tmem_ld_32x32(taddr + c * 32, r);
    tmem_wait_ld();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 q;
      q.x = pack_bf16x2(__uint_as_float(r[j * 8 + 0]) * alpha, __uint_as_float(r[j * 8 + 1]) * alpha);
      q.y = pack_bf16x2(__uint_as_float(r[j * 8 + 2]) * alpha, __uint_as_float(r[j * 8 + 3]) * alpha);
      q.z = pack_bf16x2(__uint_as_float(r[j * 8 + 4]) * alpha, __uint_as_float(r[j * 8 + 5]) * alpha);
      q.w = pack_bf16x2(__uint_as_float(r[j * 8 + 6]) * alpha, __uint_as_float(r[j * 8 + 7]) * alpha);
      epi_sts(smem_strip + lane * 512 + ((((c * 4 + j) ^ lane) & 31) << 4), q);
    }
  }
  __syncwarp();
  const bool col_ok = lane * 8 < cols_valid;
#pragma unroll 8
  for (int rr = 0; rr < 32; ++rr) {
    const uint4 q = epi_lds(smem_strip + rr * 512 + (((lane ^ rr) & 31) << 4));
    if (col_ok && rr < rows_valid) *reinterpret_cast<uint4*>(dst + rr * ld + lane * 8) = q;
  }
  __syncwarp();
}

// Two-SM versions (cta_group::2, 256 x 256 tiles over a CTA pair, 6-stage ring: the main loop of gemm_2cta.cuh).
// The one-SM kernels above spend most of their time in their own main loop (about 1.1 PFLOP/s against 1.5 for the
// pair kernel), so the exchange is moved onto the faster loop:
//
//   MODE_RS  Tiles are walked owner by owner, (rank+1), (rank+2), ..., this rank's own rows LAST. Partial tiles of the
//            other owners go straight to their staging slabs with plain P2P stores of whole 512-byte rows (from a 16 KB
//            shared-memory strip per epilogue warp) and NO fence per tile (a system
//            fence after every tile stalls the epilogue for a NVLink round trip each time; measured: 46 us of a
//            182 us call at two ranks). Each epilogue warp fences ONCE, after its last remote tile, and then
//            publishes the flags of all the tiles it sent. The own tiles come last, when the peers' partials are
//            already there or about to be, and are reduced in the epilogue as before.
//   MODE_AG  Copier warps PUSH this rank's shard into the peers' gathered buffers while the pair starts on the local
//            rows; per-CTA arrival flags let the TMA producer start on an owner's rows as soon as they are complete.
// rows_per_rank must be a multiple of 256 (a pair's tile never straddles two owners).
template <int B_MN, int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MODE == MODE_AG ? 256 : 192, 1)
gemm_comm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmAlocal,
                  const __grid_constant__ CUtensorMap tmB, GemmShape shp, GemmEpilogue ep, GemmCommParams cp) {
  using Cfg = Gemm2Cfg;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BNH = Cfg::BNH, BK = Cfg::BK;
  // MODE_RS gives one ring stage up for a 16 KB staging strip per epilogue warp (full-row stores to the peers)
  constexpr int STAGES = MODE == MODE_RS ? 5 : Cfg::STAGES;
  constexpr int EPI_PER_WARP = MODE == MODE_RS ? 32 * 512 : kEpiStageBytesPerWarp;
  constexpr int A_BYTES = Cfg::A_BYTES, B_BYTES = Cfg::B_BYTES;
  constexpr uint32_t IDESC = make_idesc_bf16(2 * BM, BN, 0, B_MN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint8_t* epi_stage = smem + STAGES * (A_BYTES + B_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(epi_stage + 4 * EPI_PER_WARP);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* ok_shared = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 2));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();
  const bool leader = cta == 0;
  SignalBlock* my_sig = cp.sig[cp.rank];
  const int parity = cp.epoch & 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);
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
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = shp.M / (2 * BM);
  const int tiles_n = (shp.N + BN - 1) / BN;
  const int total_tiles = tiles_m * tiles_n;
  const int kblocks = (shp.K + BK - 1) / BK;
  const int tmpr = cp.rows_per_rank / (2 * BM);   // row tiles per owner
  const int pair = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  // Raster: bands of `band` row tiles that never straddle two owners, walked down the band first (the CTAs running at
  // the same time share A and B tiles in L2); the owners are taken in the order given above.
  int band = tmpr;
  while (band > 16) band = (band % 2 == 0) ? band / 2 : 1;
  if (band < 1) band = 1;
  const int first_owner = MODE == MODE_AG ? cp.rank : (cp.rank + 1) % cp.n;
  auto coords = [&](int t, int& tm, int& tn) {
    const int per_band = band * tiles_n;
    const int g = t / per_band, r = t - g * per_band;
    const int seq_tm = g * band + r % band;                       // position in the owner-ordered sequence
    tn = r / band;
    tm = (seq_tm + first_owner * tmpr) % tiles_m;                 // physical row tile
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int ready_owner = cp.rank;
      for (int t = pair; t < total_tiles && ok; t += n_pairs) {
        int tm, tn;
        coords(t, tm, tn);
        const int m0 = tm * 2 * BM + static_cast<int>(cta) * BM;
        const int n0 = tn * BN + static_cast<int>(cta) * BNH;
        const int owner = tm / tmpr;
        if (MODE == MODE_AG && owner != cp.rank && owner != ready_owner) {
          if (!wait_local_ge(&my_sig->local_cnt[cp.pull_slot + owner], cp.pull_target, cp.status, 200 + owner)) {
            *abort_flag = 1;
            ok = false;
            break;
          }
          fence_proxy_async_global();
          ready_owner = owner;
        }
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          if (leader) mbar_arrive_expect_tx(&full[stage], 2 * (A_BYTES + B_BYTES));
          const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0);
          uint8_t* a_dst = sA + stage * A_BYTES;
          uint8_t* b_dst = sB + stage * B_BYTES;
          if (MODE == MODE_AG && owner == cp.rank) {
            tma_load_2d_pair(a_dst, &tmAlocal, bar, kb * BK, m0 - cp.rank * cp.rows_per_rank);
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
            const uint64_t da = make_smem_desc_sw128(a_base + k * 32, 16, 1024);
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
  } else if (warp < 6) {
    // ---------------------------------------------------------------- epilogue (warps 2..5 of both CTAs)
    const int quad = warp & 3;
    const uint32_t stage_sm = smem_u32(epi_stage + quad * EPI_PER_WARP);
    int acc = 0;
    uint32_t acc_phase = 0;
    unsigned int cleared_owners = 0;
    bool published = MODE != MODE_RS;   // the flags of this warp's remote tiles are out
    bool bail = false;
    auto flag_of = [&](int dst_rank, int src_rank, int tile_local) {
      return cp.flags[dst_rank] + (static_cast<long long>(parity) * cp.n + src_rank) * cp.flag_stride + tile_local * 8 +
             static_cast<int>(cta) * 4 + quad;
    };
    auto publish = [&]() {
      // one fence for everything this warp stored to peers, then the flag of every tile it sent
      __threadfence_system();
      __syncwarp();
      if (lane == 0) {
        for (int t = pair; t < total_tiles; t += n_pairs) {
          int tm, tn;
          coords(t, tm, tn);
          const int owner = tm / tmpr;
          if (owner == cp.rank) break;
          st_release_sys(flag_of(owner, cp.rank, (tm - owner * tmpr) * tiles_n + tn), cp.epoch);
        }
      }
      __syncwarp();
      published = true;
    };
    for (int t = pair; t < total_tiles; t += n_pairs) {
      int tm, tn;
      coords(t, tm, tn);
      const int m0 = tm * 2 * BM + static_cast<int>(cta) * BM, n0 = tn * BN;
      const int owner = tm / tmpr;
      const bool remote_path = MODE == MODE_RS && owner != cp.rank;
      if (MODE == MODE_RS && !remote_path && !published) publish();
      if (remote_path && !((cleared_owners >> owner) & 1u)) {
        int ok_w = 1;
        if (lane == 0 && cp.epoch > 2)
          ok_w = wait_flag_ge(&my_sig->rs_consumed[owner], cp.epoch - 2, cp.status, 300 + owner) ? 1 : 0;
        ok_w = __shfl_sync(0xffffffffu, ok_w, 0);
        if (!ok_w) { *abort_flag = 1; bail = true; break; }
        cleared_owners |= 1u << owner;
      }
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) { bail = true; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      const int tile_local = (tm - owner * tmpr) * tiles_n + tn;
      if (remote_path) {
        GemmEpilogue pe;
        pe.C = cp.stage[owner] + parity * cp.parity_stride + static_cast<long long>(cp.rank) * cp.rows_per_rank * shp.N;
        pe.ldc = shp.N;
        pe.bias = nullptr; pe.residual = nullptr; pe.aux_in = nullptr; pe.aux_out = nullptr;
        pe.ldr = 0; pe.ld_aux = 0;
        pe.alpha = ep.alpha; pe.act = kActNone; pe.out_fp32 = 0; pe.accumulate = 0;
        GemmShape slab{cp.rows_per_rank, shp.N, shp.K, 1};
        const int lrow = m0 - owner * cp.rows_per_rank + quad * 32;
        if (cp.tune & 16) {
          gemm_epilogue_warp<BN>(pe, slab, taddr, lrow, n0, lane, stage_sm, false);      // 64-byte segments (comparison)
        } else if (!(cp.tune & 1)) {
          rs_store_strip_wide(stage_sm, taddr, ep.alpha, reinterpret_cast<__nv_bfloat16*>(pe.C) + static_cast<long long>(lrow) * shp.N + n0,
                              shp.N, cp.rows_per_rank - lrow, shp.N - n0, lane);
        }
      } else if (MODE == MODE_RS) {
        int ok_w = 1;
        if (lane == 0 && !(cp.tune & 4)) {
          for (int s = 0; s < cp.n && ok_w; ++s) {
            if (s == cp.rank) continue;
            ok_w = wait_flag_ge(flag_of(cp.rank, s, tile_local), cp.epoch, cp.status, 600 + s) ? 1 : 0;
          }
        }
        ok_w = __shfl_sync(0xffffffffu, ok_w, 0);
        if (!ok_w) { *abort_flag = 1; bail = true; break; }
        const int lrow0 = m0 - owner * cp.rows_per_rank + quad * 32;
        const __nv_bfloat16* my_stage = cp.stage[cp.rank] + parity * cp.parity_stride;
        const int rows_valid = cp.rows_per_rank - lrow0;
        GemmEpilogue pe;
        pe.C = cp.out; pe.ldc = cp.ldc;
        pe.bias = cp.bias; pe.residual = nullptr; pe.ldr = 0;
        pe.aux_in = nullptr; pe.aux_out = nullptr; pe.ld_aux = 0;
        pe.alpha = 1.f; pe.act = kActNone; pe.out_fp32 = 0; pe.accumulate = 0;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = n0 + c * 32;
          const int cols_valid = shp.N - col0;
          if (cols_valid <= 0) break;
          float h[32];
          epi_load_sum_bf16(stage_sm, lane, my_stage + static_cast<long long>(lrow0) * shp.N + col0,
                            static_cast<long long>(cp.rows_per_rank) * shp.N, (cp.tune & 8) ? 0 : cp.n, cp.rank, shp.N,
                            cp.residual ? cp.residual + static_cast<long long>(lrow0) * cp.ldr + col0 : nullptr, cp.ldr, rows_valid, cols_valid, h);
          uint32_t r[32];
          __syncwarp();
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(fmaf(__uint_as_float(r[j]), ep.alpha, h[j]));
          gemm_epilogue_chunk(pe, r, lrow0, col0, rows_valid, cols_valid, lane, stage_sm, false);
        }
      } else {
        gemm_epilogue_warp<BN>(ep, shp, taddr, m0 + quad * 32, n0, lane, stage_sm, false);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&tempty[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (MODE == MODE_RS && !published && !bail) publish();   // a pair that had no own tile at the end of its sequence
  } else if (MODE == MODE_AG) {
    // ---------------------------------------------------------------- copiers (warps 6, 7 of both CTAs): PUSH
    // Every CTA owns one slice of this rank's shard and stores it into the gathered buffer of every peer (plain P2P
    // stores, 512 contiguous bytes per warp instruction, several in flight: stores reach the link rate from these few
    // threads, loads of the same width measured about half of it), nearest consumer first. After a system fence it
    // raises its flag on that peer; the peer's CTA with the same index sees it and counts the slice as arrived.
    const int ct = threadIdx.x - 192;  // 0..63
    const long long shard_vecs = static_cast<long long>(cp.rows_per_rank) * cp.k_cols / 8;
    const long long per_cta = (shard_vecs + gridDim.x - 1) / gridDim.x;
    const long long v0 = per_cta * blockIdx.x;
    const long long v1 = min(shard_vecs, v0 + per_cta);
    const long long my_rows_off = static_cast<long long>(cp.rank) * cp.rows_per_rank * cp.k_cols;
    const uint4* src = reinterpret_cast<const uint4*>(cp.x_local);
    // the peers must be done with what this parity of their buffers held two calls ago
    if (ct == 0) {
      int okc = 1;
      if (cp.epoch > 2)
        for (int p = 0; p < cp.n && okc; ++p)
          if (p != cp.rank) okc = wait_flag_ge(&my_sig->ag_pulled[p], cp.epoch - 2, cp.status, 400 + p) ? 1 : 0;
      *ok_shared = okc;
    }
    asm volatile("bar.sync 1, 64;" ::: "memory");
    bool okc = *ok_shared != 0;
    if (!okc) *abort_flag = 1;
    if (ct == 0 && okc) atomicAdd(&my_sig->local_cnt[cp.pull_slot + cp.rank], 1u);   // keeps this counter in step with the one-SM kernel
    for (int k = 0; k < cp.n && okc; ++k) {
      const int p = (cp.rank - k + cp.n) % cp.n;   // k = 0: the local copy (kept for the weight gradient)
      uint4* dst = reinterpret_cast<uint4*>(cp.gathered[p] + parity * cp.parity_stride + my_rows_off);
      long long i = (cp.tune & 32) && k ? v1 : v0 + ct;
      for (; i + 3 * 64 < v1; i += 4 * 64) {
        const uint4 t0 = src[i], t1 = src[i + 64], t2 = src[i + 128], t3 = src[i + 192];
        dst[i] = t0; dst[i + 64] = t1; dst[i + 128] = t2; dst[i + 192] = t3;
      }
      for (; i < v1; i += 64) dst[i] = src[i];
      if (k) {
        __threadfence_system();
        asm volatile("bar.sync 1, 64;" ::: "memory");
        if (ct == 0) {
          st_release_sys(cp.ag_flags[p] + cp.rank * 256 + blockIdx.x, cp.epoch);
          // Arrivals are counted between the pushes, in the order the GEMM needs the owners: by now the k-th owner
          // after this rank has had the time of k pushes to deliver its slice, and the TMA producer must not wait for
          // this thread to finish all of its own pushes first. This CTA vouches for the slice of the CTA with its
          // index on that owner.
          const int o = (cp.rank + k) % cp.n;
          if (!wait_flag_ge(cp.ag_flags[cp.rank] + o * 256 + blockIdx.x, cp.epoch, cp.status, 500 + o)) {
            *abort_flag = 1;
            okc = false;
          } else {
            __threadfence();
            atomicAdd(&my_sig->local_cnt[cp.pull_slot + o], 1u);
          }
          *ok_shared = okc ? 1 : 0;
        }
        // all 64 copier threads leave together when the wait gave up (nobody may be left alone at the named barrier)
        asm volatile("bar.sync 1, 64;" ::: "memory");
        okc = *ok_shared != 0;
      }
    }
  }

  tc_fence_before();
  __syncthreads();

  if (MODE == MODE_RS && !*abort_flag) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int arrived = atomicAdd(&my_sig->local_cnt[cp.done_slot], 1u) + 1u;
      if (arrived == cp.done_target)
        for (int p = 0; p < cp.n; ++p) st_release_sys(&cp.sig[p]->rs_consumed[cp.rank], cp.epoch);
    }
  }
  if (MODE == MODE_AG && !*abort_flag) {
    // every tile of this rank has been computed from its gathered buffer: the peers may write this parity again
    if (threadIdx.x == 0) {
      const unsigned int arrived = atomicAdd(&my_sig->local_cnt[cp.ag_done_slot], 1u) + 1u;
      if (arrived % gridDim.x == 0)     // the last CTA of this call (only this kernel counts on this slot)
        for (int p = 0; p < cp.n; ++p)
          if (p != cp.rank) st_release_sys(&cp.sig[p]->ag_pulled[cp.rank], cp.epoch);
    }
  }
  cluster_sync_all();
  tc_fence_after();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    if (threadIdx.x == 0 && cp.status) {
      if (atomicCAS(cp.status, 0, (int)kStatusMbarTimeout) == 0) cp.status[1] = 2100 + static_cast<int>(cta);
    }
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

template <int B_MN, int MODE>
static int launch_gemm_comm2(const CUtensorMap& tmA, const CUtensorMap& tmAl, const CUtensorMap& tmB, const GemmShape& shp,
                             const GemmEpilogue& ep, const GemmCommParams& cp, int grid, cudaStream_t stream) {
  auto kern = gemm_comm2_kernel<B_MN, MODE>;
  constexpr int smem_bytes = MODE == MODE_RS ? 5 * (Gemm2Cfg::A_BYTES + Gemm2Cfg::B_BYTES) + 4 * 32 * 512 + 256 + 1024 : Gemm2Cfg::SMEM_BYTES;
  static bool configured = false;
  if (!configured) {
    OFB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    configured = true;
  }
  kern<<<grid & ~1, MODE == MODE_AG ? 256 : 192, smem_bytes, stream>>>(tmA, tmAl, tmB, shp, ep, cp);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// The pair kernels are used when a pair's 256-row tile cannot straddle two owners (OFB_GEMM_COMM_2CTA=0 turns them off).
static bool use_pair_kernel(int T, int n) {
  static int mode = -1;
  if (mode < 0) {
    const char* e = std::getenv("OFB_GEMM_COMM_2CTA");
    mode = e ? std::atoi(e) : 1;
  }
  return mode != 0 && T % (n * 256) == 0;
}

template <int BN, int B_MN, int MODE>
static int launch_gemm_comm(const CUtensorMap& tmA, const CUtensorMap& tmAl, const CUtensorMap& tmB, const GemmShape& shp,
                            const GemmEpilogue& ep, const GemmCommParams& cp, int grid, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_comm_kernel<BN, B_MN, MODE>;
  static bool configured = false;
  if (!configured) {
    OFB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg::SMEM_BYTES + (MODE == MODE_RS ? 4 * kEpiStageBytesPerWarp : 0)));
    configured = true;
  }
  kern<<<grid, MODE == MODE_AG ? 256 : 320, Cfg::SMEM_BYTES + (MODE == MODE_RS ? 4 * kEpiStageBytesPerWarp : 0), stream>>>(tmA, tmAl, tmB, shp, ep, cp);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace ofb

using namespace ofb;

// The grid of the fused kernels is fixed per device (one CTA per SM, capped by the tile count is NOT
// applied) so that the per-call arrival targets are simple multiples of it.
OFB_API int ofb_gemm_comm_grid(int* out) {
  int dev = 0, sms = 0;
  OFB_CUDA_OK(cudaGetDevice(&dev));
  OFB_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  *out = sms;
  return 0;
}

// C[T/n, N] = reduce_scatter_rows( A[T, K] @ B^T ) + bias + residual.
//   a: bf16 [T, lda] local; b: bf16 [N, ldb] ("nk") or [K, ldb] ("kn"); out: bf16 [T/n, ldc] local.
//   stage_off / flag_off: byte offsets of the staging and flag regions inside every rank's arena.
OFB_API int ofb_gemm_rs(const OfbCommCtx* ctx, const void* a, long long lda, const void* b, long long ldb, int b_mn_major,
                        void* out, long long ldc, const void* bias, const void* residual, long long ldr, int T, int N, int K,
                        float alpha, long long stage_off, long long stage_bytes, long long flag_off, int flag_stride,
                        unsigned int epoch, int done_slot, void* stream) {
  const int n = ctx->n;
  if (n < 1 || n > kMaxPeers) return fail("gemm_rs: group size must be 1..8");
  if (T % (n * 128)) return fail("gemm_rs: rows must be a multiple of 128 * group size");
  if (N % 8 || K % 8) return fail("gemm_rs: N and K must be multiples of 8");
  const int bn = 256;
  const int tiles_local = (T / n / 128) * ((N + bn - 1) / bn);
  if (8 * tiles_local > flag_stride) return fail("gemm_rs: flag region too small for this problem");
  if (2ll * T * N * 2 > stage_bytes) return fail("gemm_rs: staging region too small for this problem");
  CUtensorMap tmA, tmB;
  if (get_tensor_map(&tmA, a, 2, 2, K, T, 0, (uint64_t)lda * 2, 0, 64, 128, 0, 3)) return -1;
  if (!b_mn_major) {
    if (get_tensor_map(&tmB, b, 2, 2, K, N, 0, (uint64_t)ldb * 2, 0, 64, bn, 0, 3)) return -1;
  } else {
    if (get_tensor_map(&tmB, b, 2, 2, N, K, 0, (uint64_t)ldb * 2, 0, 64, 64, 0, 3)) return -1;
  }
  int grid = 0;
  if (ofb_gemm_comm_grid(&grid)) return -1;
  GemmShape shp{T, N, K};
  GemmEpilogue ep;
  std::memset(&ep, 0, sizeof(ep));
  ep.alpha = alpha;
  GemmCommParams cp;
  std::memset(&cp, 0, sizeof(cp));
  cp.n = n; cp.rank = ctx->rank; cp.rows_per_rank = T / n; cp.epoch = epoch; cp.status = device_status_ptr();
  for (int i = 0; i < n; ++i) {
    cp.sig[i] = reinterpret_cast<SignalBlock*>(ctx->signals[i]);
    cp.stage[i] = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<unsigned char*>(ctx->arena[i]) + stage_off);
    cp.flags[i] = reinterpret_cast<unsigned int*>(reinterpret_cast<unsigned char*>(ctx->arena[i]) + flag_off);
  }
  cp.flag_stride = flag_stride;
  cp.out = reinterpret_cast<__nv_bfloat16*>(out); cp.ldc = ldc;
  cp.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  cp.residual = reinterpret_cast<const __nv_bfloat16*>(residual); cp.ldr = ldr;
  cp.done_slot = done_slot; cp.done_target = epoch * static_cast<unsigned int>(grid);
  cp.parity_stride = stage_bytes / 4;  // half of the region, in bf16 elements
  if (const char* e = std::getenv("OFB_GEMM_COMM_TUNE")) cp.tune = std::atoi(e);
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (use_pair_kernel(T, n)) {
    // each CTA of a pair stages 128 of the tile's 256 B columns
    if (!b_mn_major && get_tensor_map(&tmB, b, 2, 2, K, N, 0, (uint64_t)ldb * 2, 0, 64, 128, 0, 3)) return -1;
    cp.done_target = epoch * static_cast<unsigned int>(grid & ~1);
    return b_mn_major ? launch_gemm_comm2<1, MODE_RS>(tmA, tmA, tmB, shp, ep, cp, grid, s)
                      : launch_gemm_comm2<0, MODE_RS>(tmA, tmA, tmB, shp, ep, cp, grid, s);
  }
  return b_mn_major ? launch_gemm_comm<256, 1, MODE_RS>(tmA, tmA, tmB, shp, ep, cp, grid, s)
                    : launch_gemm_comm<256, 0, MODE_RS>(tmA, tmA, tmB, shp, ep, cp, grid, s);
}

// C[T, N] = epilogue( all_gather_rows(x_local[T/n, K]) @ B^T ); the gathered matrix of this call stays in
// this rank's gathered buffer (parity = epoch & 1) for later kernels (weight gradients).
OFB_API int ofb_ag_gemm(const OfbCommCtx* ctx, const void* x_local, const void* b, long long ldb, int b_mn_major, void* out,
                        long long ldc, const void* bias, const void* aux_in, void* aux_out, long long ld_aux, int act, int T,
                        int N, int K, float alpha, long long gathered_off, long long gathered_bytes, long long ag_flag_off,
                        unsigned int epoch, int pull_slot, void* stream) {
  const int n = ctx->n;
  if (n < 1 || n > kMaxPeers) return fail("ag_gemm: group size must be 1..8");
  if (T % (n * 128)) return fail("ag_gemm: rows must be a multiple of 128 * group size");
  if (N % 8 || K % 8) return fail("ag_gemm: N and K must be multiples of 8");
  const int bn = 256;
  int grid = 0;
  if (ofb_gemm_comm_grid(&grid)) return -1;
  if (2ll * T * K * 2 > gathered_bytes) return fail("ag_gemm: gathered region too small for this problem");
  const long long parity_stride = gathered_bytes / 4;  // half of the region, in bf16 elements
  auto* my_g = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<unsigned char*>(ctx->arena[ctx->rank]) + gathered_off) +
               (epoch & 1) * parity_stride;
  CUtensorMap tmA, tmAl, tmB;
  if (get_tensor_map(&tmA, my_g, 2, 2, K, T, 0, (uint64_t)K * 2, 0, 64, 128, 0, 3)) return -1;
  if (get_tensor_map(&tmAl, x_local, 2, 2, K, T / n, 0, (uint64_t)K * 2, 0, 64, 128, 0, 3)) return -1;
  if (!b_mn_major) {
    if (get_tensor_map(&tmB, b, 2, 2, K, N, 0, (uint64_t)ldb * 2, 0, 64, bn, 0, 3)) return -1;
  } else {
    if (get_tensor_map(&tmB, b, 2, 2, N, K, 0, (uint64_t)ldb * 2, 0, 64, 64, 0, 3)) return -1;
  }
  GemmShape shp{T, N, K};
  GemmEpilogue ep;
  std::memset(&ep, 0, sizeof(ep));
  ep.C = out; ep.ldc = ldc; ep.alpha = alpha; ep.act = act;
  ep.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  ep.aux_in = reinterpret_cast<const __nv_bfloat16*>(aux_in);
  ep.aux_out = reinterpret_cast<__nv_bfloat16*>(aux_out);
  ep.ld_aux = ld_aux;
  GemmCommParams cp;
  std::memset(&cp, 0, sizeof(cp));
  cp.n = n; cp.rank = ctx->rank; cp.rows_per_rank = T / n; cp.epoch = epoch; cp.status = device_status_ptr();
  for (int i = 0; i < n; ++i) {
    cp.sig[i] = reinterpret_cast<SignalBlock*>(ctx->signals[i]);
    cp.gathered[i] = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<unsigned char*>(ctx->arena[i]) + gathered_off);
    cp.ag_flags[i] = reinterpret_cast<unsigned int*>(reinterpret_cast<unsigned char*>(ctx->arena[i]) + ag_flag_off);
  }
  cp.ag_done_slot = 3;
  cp.x_local = reinterpret_cast<const __nv_bfloat16*>(x_local);
  cp.k_cols = K;
  cp.pull_slot = pull_slot;
  cp.pull_target = epoch * static_cast<unsigned int>(grid);
  cp.parity_stride = parity_stride;
  if (const char* e = std::getenv("OFB_GEMM_COMM_TUNE")) cp.tune = std::atoi(e);
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (use_pair_kernel(T, n) && ag_flag_off > 0 && grid <= 256) {
    if (!b_mn_major && get_tensor_map(&tmB, b, 2, 2, K, N, 0, (uint64_t)ldb * 2, 0, 64, 128, 0, 3)) return -1;
    cp.pull_target = epoch * static_cast<unsigned int>(grid & ~1);
    return b_mn_major ? launch_gemm_comm2<1, MODE_AG>(tmA, tmAl, tmB, shp, ep, cp, grid, s)
                      : launch_gemm_comm2<0, MODE_AG>(tmA, tmAl, tmB, shp, ep, cp, grid, s);
  }
  return b_mn_major ? launch_gemm_comm<256, 1, MODE_AG>(tmA, tmAl, tmB, shp, ep, cp, grid, s)
                    : launch_gemm_comm<256, 0, MODE_AG>(tmA, tmAl, tmB, shp, ep, cp, grid, s);
}
