// Fused multi-head attention backward for sm_100a (bf16, head dim 64 or 128; query length != key length,
// grouped-query attention and Philox dropout as in the forward kernel).
//
// One CTA owns a 128-key tile (K_j, V_j stay resident in shared memory) of one (batch, key/value head)
// and walks over the query tiles i that see it, for every query head of the group in turn (so dK and dV of a
// shared key/value head accumulate in TMEM and need no second reduction). Per (i, j) pair five tcgen05 products run,
// all fed from the same shared-memory tiles without any transposition pass:
//     S   = Q_i K_j^T            (K-major  x K-major)       -> TMEM
//     dP  = dO_i V_j^T           (K-major  x K-major)       -> TMEM
//     dV += P^T dO_i             (MN-major x MN-major)      -> TMEM accumulator
//     dK += dS^T Q_i             (MN-major x MN-major)      -> TMEM accumulator
//     dQ_i partial = dS K_j      (K-major  x MN-major)      -> TMEM, then staged in shared memory and added to HBM by TMA (cp.reduce.async.bulk)
// 256 compute threads (two warps per scheduler: one alone issued a fifth of the cycles), two per query row: warps
// 2..5 take key columns 0..63 of the tile, warps 6..9 columns 64..127 (a warp reaches the TMEM lanes of its own
// quarter only, so the work is split by columns). They rebuild P from S and the saved log-sum-exp, form
// dS = P * (dP - delta) * scale, and publish P / dS (bf16) through one shared buffer in the 128-byte swizzled
// layout that serves both as K-major and MN-major operand; the dQ drain and the dK / dV epilogue are split the
// same way. TMEM: S | dP (reused for the dQ partial) | dV | dK = 512 columns at D = 128.
//
// Reference counterpart: oneflow/user/kernels/scaled_dot_product_attention_grad_kernel.cu
// (flash-attention library call).
#include "../common/host_utils.h"
#include "../common/philox.cuh"
#include "../common/ptx.cuh"
#include "ofb_kernels.h"

namespace ofb {

int fmha_tensor_map(CUtensorMap* out, const void* ptr, int B, int S, int H, int D, long long row_stride);
int fmha_dropout_cfg(DropoutCfg* d, float p_dropout, unsigned long long seed, unsigned int offset);

struct FmhaBwdParams {
  const float* lse;     // [B, H, Sq]
  const float* delta;   // [B, H, Sq] rowsum(dO * O)
  float* dq_acc;        // [B, Sq, H, D] fp32, zero-initialised, receives red.add
  __nv_bfloat16* dk;    // element (b,s,hk,d) at ((b*Sk+s)*dkv_row_stride + hk*D + d)
  __nv_bfloat16* dv;
  long long dkv_row_stride;
  const int* kv_len;
  int B, H, Hk, Sq, Sk, D;
  int causal;
  int causal_off;       // Sk - Sq
  DropoutCfg drop;
  float scale;          // softmax scale
  float scale_log2e;
  int* status;
};

template <int D>
struct FmhaBwdCfg {
  static constexpr int T_BYTES = 128 * D * 2;       // one [128 x D] tile
  static constexpr int PDS_BYTES = 128 * 128 * 2;
  static constexpr int SMEM_BYTES = 6 * T_BYTES + PDS_BYTES + 256 + 1024;
};

__device__ __forceinline__ float fast_exp2_b(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// fp32 add-reduction of a shared-memory tile into global memory through TMA (one bulk operation instead of
// thousands of per-thread red instructions; L2 sees whole 128-byte lines).
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, const void* smem_src, int x, int y, int z, int w) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
// Rendezvous of the 128 compute threads on an mbarrier (bounded, unlike bar.sync: a thread that gave up on
// another wait can never leave its peers stuck here).
__device__ __forceinline__ bool compute_sync(uint64_t* bar, uint32_t& parity, volatile int* abort_flag) {
  mbar_arrive(bar);
  const bool ok = mbar_wait(bar, parity, abort_flag);
  parity ^= 1;
  return ok;
}

template <int D, bool DROP>
__global__ void __launch_bounds__(320, 1)
fmha_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const __grid_constant__ CUtensorMap tmdQ, FmhaBwdParams p) {
  using Cfg = FmhaBwdCfg<D>;
  constexpr int DCH = D / 64;
  constexpr int CH_BYTES = 128 * 128;
  constexpr uint32_t IDESC_S = make_idesc_bf16(128, 128, 0, 0);   // S, dP
  constexpr uint32_t IDESC_TT = make_idesc_bf16(128, D, 1, 1);    // dV, dK (both operands MN-major)
  constexpr uint32_t IDESC_DQ = make_idesc_bf16(128, D, 0, 1);    // dQ (A K-major, B MN-major)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::T_BYTES;
  uint8_t* sQ = sV + Cfg::T_BYTES;          // 2 stages
  uint8_t* sdO = sQ + 2 * Cfg::T_BYTES;     // 2 stages
  uint8_t* sPdS = sdO + 2 * Cfg::T_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sPdS + Cfg::PDS_BYTES);
  uint64_t* kv_full = bars;         // 1
  uint64_t* q_full = bars + 1;      // [2]
  uint64_t* q_empty = bars + 3;     // [2]
  uint64_t* do_full = bars + 5;     // [2]
  uint64_t* do_empty = bars + 7;    // [2]
  uint64_t* s_full = bars + 9;
  uint64_t* dp_full = bars + 10;
  uint64_t* p_ready = bars + 11;    // count 128
  uint64_t* dv_done = bars + 12;
  uint64_t* ds_ready = bars + 13;   // count 128
  uint64_t* dq_full = bars + 14;
  uint64_t* dq_drained = bars + 15; // count 128
  uint64_t* all_done = bars + 16;
  uint64_t* stg_bar = bars + 17;    // count 128: rendezvous of the compute threads around the dQ staging area
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int group = p.H / p.Hk;          // query heads per key/value head
  const int k0 = jt * 128;
  const int n_qt = (p.Sq + 127) / 128;
  int kv_limit = p.Sk;
  if (p.kv_len) kv_limit = min(kv_limit, p.kv_len[b]);
  // first query tile with a row that sees this key tile: row + causal_off >= k0
  const int i_start = p.causal ? max(0, k0 - p.causal_off) / 128 : 0;
  const bool tile_visible = k0 < kv_limit;
  const int n_i = tile_visible ? max(0, n_qt - i_start) : 0;   // query tiles per head
  const int n_iter = n_i * group;                               // iteration t: head hk*group + t / n_i, tile i_start + t % n_i

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
      mbar_init(&do_full[s], 1);
      mbar_init(&do_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_ready, 256);
    mbar_init(dv_done, 1);
    mbar_init(ds_ready, 256);
    mbar_init(dq_full, 1);
    mbar_init(dq_drained, 256);
    mbar_init(all_done, 1);
    mbar_init(stg_bar, 256);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;
  const uint32_t tdP = tmem_base + 128;   // also receives the dQ partial (first D columns)
  const uint32_t tdV = tmem_base + 256;
  const uint32_t tdK = tmem_base + 256 + D;

  if (warp == 0) {
    if (elect_one() && n_iter > 0) {
      mbar_arrive_expect_tx(kv_full, 2 * Cfg::T_BYTES);
#pragma unroll
      for (int c = 0; c < DCH; ++c) {
        tma_load_4d(sK + c * CH_BYTES, &tmK, kv_full, c * 64, hk, k0, b);
        tma_load_4d(sV + c * CH_BYTES, &tmV, kv_full, c * 64, hk, k0, b);
      }
      for (int t = 0; t < n_iter; ++t) {
        const int st = t & 1;
        const uint32_t ph = ((t >> 1) & 1) ^ 1;
        const int h = hk * group + t / n_i;
        const int qrow = (i_start + t % n_i) * 128;
        if (!mbar_wait(&q_empty[st], ph, abort_flag)) break;
        mbar_arrive_expect_tx(&q_full[st], Cfg::T_BYTES);
#pragma unroll
        for (int c = 0; c < DCH; ++c) tma_load_4d(sQ + st * Cfg::T_BYTES + c * CH_BYTES, &tmQ, &q_full[st], c * 64, h, qrow, b);
        if (!mbar_wait(&do_empty[st], ph, abort_flag)) break;
        mbar_arrive_expect_tx(&do_full[st], Cfg::T_BYTES);
#pragma unroll
        for (int c = 0; c < DCH; ++c) tma_load_4d(sdO + st * Cfg::T_BYTES + c * CH_BYTES, &tmdO, &do_full[st], c * 64, h, qrow, b);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one() && n_iter > 0) {
      bool ok = mbar_wait(kv_full, 0, abort_flag);
      const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV), pds_base = smem_u32(sPdS);
      for (int t = 0; t < n_iter && ok; ++t) {
        const int st = t & 1;
        const uint32_t ph2 = (t >> 1) & 1;  // phase of the 2-stage rings
        const uint32_t ph1 = t & 1;         // phase of the once-per-iteration barriers
        const uint32_t q_base = smem_u32(sQ + st * Cfg::T_BYTES);
        const uint32_t do_base = smem_u32(sdO + st * Cfg::T_BYTES);
        // S = Q_i K_j^T
        if (!mbar_wait(&q_full[st], ph2, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * CH_BYTES + (kk & 3) * 32;
          umma_bf16_ss(tS, make_smem_desc_sw128(q_base + off, 16, 1024), make_smem_desc_sw128(k_base + off, 16, 1024),
                       IDESC_S, kk != 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        // dP = dO_i V_j^T (its TMEM region held the previous dQ partial: wait until that was drained)
        if (!mbar_wait(&do_full[st], ph2, abort_flag)) { ok = false; break; }
        if (t > 0 && !mbar_wait(dq_drained, (t - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * CH_BYTES + (kk & 3) * 32;
          umma_bf16_ss(tdP, make_smem_desc_sw128(do_base + off, 16, 1024), make_smem_desc_sw128(v_base + off, 16, 1024),
                       IDESC_S, kk != 0 ? 1u : 0u);
        }
        umma_commit(dp_full);
        // dV += P^T dO_i : A = P as MN-major (M = keys, K = query rows), B = dO_i as MN-major (N = d)
        if (!mbar_wait(p_ready, ph1, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk) {
          umma_bf16_ss(tdV, make_smem_desc_sw128(pds_base + kk * 2048, CH_BYTES, 1024),
                       make_smem_desc_sw128(do_base + kk * 2048, CH_BYTES, 1024), IDESC_TT, (t | kk) != 0 ? 1u : 0u);
        }
        umma_commit(dv_done);
        umma_commit(&do_empty[st]);
        // dK += dS^T Q_i ; dQ partial = dS K_j
        if (!mbar_wait(ds_ready, ph1, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk) {
          umma_bf16_ss(tdK, make_smem_desc_sw128(pds_base + kk * 2048, CH_BYTES, 1024),
                       make_smem_desc_sw128(q_base + kk * 2048, CH_BYTES, 1024), IDESC_TT, (t | kk) != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk) {
          umma_bf16_ss(tdP, make_smem_desc_sw128(pds_base + (kk >> 2) * CH_BYTES + (kk & 3) * 32, 16, 1024),
                       make_smem_desc_sw128(k_base + kk * 2048, CH_BYTES, 1024), IDESC_DQ, kk != 0 ? 1u : 0u);
        }
        umma_commit(dq_full);
        umma_commit(&q_empty[st]);
      }
      if (ok) umma_commit(all_done);
    }
    __syncwarp();
  } else if (n_iter > 0) {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;          // which 64 key columns of the tile this thread takes
    const int r = quad * 32 + lane;
    const bool issuer = r == 0 && half == 0;   // the one thread that issues and awaits the dQ bulk reductions
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    uint8_t* pds_row = sPdS + half * CH_BYTES + r * 128;   // 64 columns = one swizzled chunk
    const int kc0 = k0 + half * 64;            // first key column of this half
    const float kLog2e = 1.4426950408889634f;
    bool ok = true;
    uint32_t stg_parity = 0;
    for (int t = 0; t < n_iter; ++t) {
      const uint32_t ph1 = t & 1;
      const int h = hk * group + t / n_i;
      const int q0 = (i_start + t % n_i) * 128;
      const int row_g = q0 + r;
      const bool row_ok = row_g < p.Sq;
      const long long stat_idx = (static_cast<long long>(b) * p.H + h) * p.Sq + row_g;
      const float lse = row_ok ? p.lse[stat_idx] : -INFINITY;
      const float delta = row_ok ? p.delta[stat_idx] : 0.f;
      const float lse2 = lse * kLog2e;
      const bool dead_row = !row_ok || lse == -INFINITY;
      const bool need_mask = (p.causal && k0 + 127 > q0 + p.causal_off) || (k0 + 128 > kv_limit);
      const int col_max = p.causal ? min(row_g + p.causal_off, kv_limit - 1) : kv_limit - 1;
      uint32_t pk[32];  // P, later dS, as packed bf16 pairs for this row's 64 columns
      uint32_t keep_bits[DROP ? 2 : 1];  // dropout: bit c of word w = column 32 * w + c of this half is kept
      if (!mbar_wait(s_full, ph1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      // the previous pair's dQ reduction must have finished reading the staging area (= this P buffer)
      if (t > 0) {
        if (issuer) tma_store_wait_read<0>();
        if (!compute_sync(stg_bar, stg_parity, abort_flag)) { ok = false; break; }
      }
      {
        uint32_t v[2][32];
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 2; ++c) tmem_ld_32x32(tS + lane_addr + half * 64 + c * 32, v[c]);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = fast_exp2_b(__uint_as_float(v[c][i]) * p.scale_log2e - lse2);
            float p1 = fast_exp2_b(__uint_as_float(v[c][i + 1]) * p.scale_log2e - lse2);
            if (dead_row || (need_mask && kc0 + c * 32 + i > col_max)) p0 = 0.f;
            if (dead_row || (need_mask && kc0 + c * 32 + i + 1 > col_max)) p1 = 0.f;
            pk[c * 16 + (i >> 1)] = pack_bf16x2(p0, p1);
          }
      }
      if constexpr (DROP) {
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          uint32_t bits = 0;
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4)
            bits |= dropout_keep4(p.drop, static_cast<uint32_t>(b * p.H + h), static_cast<uint32_t>(row_g),
                                  static_cast<uint32_t>((kc0 + w * 32 + q4 * 4) >> 2)) << (q4 * 4);
          keep_bits[w] = bits;
        }
      }
      // Publish P (with dropout: only the kept probabilities, which is what multiplied V in the forward; the factor
      // 1 / keep is applied to dV at the end). The buffer is free: the MMAs that read dS of the previous iteration
      // were covered by the dq_full wait below in that iteration.
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        uint32_t w4[4] = {pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]};
        if constexpr (DROP) {
          // pair q of this 16-byte group holds columns 8 * g + 2 * q and + 1 of this half
          const uint32_t bits = keep_bits[g >> 2] >> ((g & 3) * 8);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            w4[q] &= ((bits >> (2 * q)) & 1u ? 0x0000FFFFu : 0u) | ((bits >> (2 * q + 1)) & 1u ? 0xFFFF0000u : 0u);
        }
        *reinterpret_cast<uint4*>(pds_row + ((g ^ (r & 7)) << 4)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
      // dS = P * (dP - delta) * scale
      if (!mbar_wait(dp_full, ph1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t v[2][32];
        __syncwarp();
        tmem_ld_32x32(tdP + lane_addr + half * 64, v[0]);
        tmem_ld_32x32(tdP + lane_addr + half * 64 + 32, v[1]);
        tmem_wait_ld();
#pragma unroll
        for (int cc = 0; cc < 2; ++cc)
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int c = cc;
            float2 pp = unpack_bf16x2(pk[c * 16 + (i >> 1)]);
            float g0 = __uint_as_float(v[cc][i]), g1 = __uint_as_float(v[cc][i + 1]);
            if constexpr (DROP) {   // the gradient reaches P only through the kept entries, scaled by 1 / keep
              g0 = (keep_bits[c] >> i) & 1u ? g0 * p.drop.inv_keep : 0.f;
              g1 = (keep_bits[c] >> (i + 1)) & 1u ? g1 * p.drop.inv_keep : 0.f;
            }
            float d0 = pp.x * (g0 - delta) * p.scale;
            float d1 = pp.y * (g1 - delta) * p.scale;
            pk[c * 16 + (i >> 1)] = pack_bf16x2(d0, d1);
          }
      }
      tc_fence_before();
      if (!mbar_wait(dv_done, ph1, abort_flag)) { ok = false; break; }
#pragma unroll
      for (int g = 0; g < 8; ++g)
        *reinterpret_cast<uint4*>(pds_row + ((g ^ (r & 7)) << 4)) = make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(ds_ready);
      // Drain the dQ partial of this pair: TMEM -> swizzled fp32 staging in shared memory (the P/dS buffer,
      // idle until the next pair's P) -> one TMA add-reduction per 32-column slab into the fp32 accumulator.
      if (!mbar_wait(dq_full, ph1, abort_flag)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int hh = 0; hh < D / 64; ++hh) {
        if (hh > 0) {
          if (issuer) tma_store_wait_read<0>();
          if (!compute_sync(stg_bar, stg_parity, abort_flag)) { ok = false; break; }
        }
        uint32_t v[32];     // this half's 32 of the 64 columns of the slab
        __syncwarp();
        tmem_ld_32x32(tdP + lane_addr + hh * 64 + half * 32, v);
        tmem_wait_ld();
        if (hh == D / 64 - 1) {
          // every column of the dQ partial has left TMEM: the dP region may be overwritten
          tc_fence_before();
          mbar_arrive(dq_drained);
        }
        {
          uint8_t* st = sPdS + half * (128 * 128) + r * 128;
#pragma unroll
          for (int g = 0; g < 8; ++g)
            *reinterpret_cast<uint4*>(st + ((g ^ (r & 7)) << 4)) = make_uint4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
        }
        fence_proxy_async_smem();
        if (!compute_sync(stg_bar, stg_parity, abort_flag)) { ok = false; break; }
        if (issuer) {
          tma_reduce_add_4d(&tmdQ, sPdS, hh * 64, h, q0, b);
          tma_reduce_add_4d(&tmdQ, sPdS + 128 * 128, hh * 64 + 32, h, q0, b);
          tma_store_commit();
        }
      }
      if (!ok) break;
    }
    if (issuer) tma_store_wait<0>();
    // dK, dV of this key tile: TMEM lane = key row; each half writes its half of the D columns
    if (ok) ok = mbar_wait(all_done, 0, abort_flag);
    if (ok) {
      tc_fence_after();
      const int krow = k0 + r;
      __nv_bfloat16* dk_row = p.dk + (static_cast<long long>(b) * p.Sk + krow) * p.dkv_row_stride + hk * D;
      __nv_bfloat16* dv_row = p.dv + (static_cast<long long>(b) * p.Sk + krow) * p.dkv_row_stride + hk * D;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = which == 0 ? tdK : tdV;
        __nv_bfloat16* dst = which == 0 ? dk_row : dv_row;
        const float osc = (DROP && which == 1) ? p.drop.inv_keep : 1.f;
#pragma unroll
        for (int c0 = 0; c0 < D / 64; ++c0) {
          const int c = half * (D / 64) + c0;
          uint32_t v[32];
          __syncwarp();
          tmem_ld_32x32(src + lane_addr + c * 32, v);
          tmem_wait_ld();
          if (krow < p.Sk) {
#pragma unroll
            for (int g = 0; g < 4; ++g)
              *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = make_uint4(
                  pack_bf16x2(__uint_as_float(v[g * 8]) * osc, __uint_as_float(v[g * 8 + 1]) * osc),
                  pack_bf16x2(__uint_as_float(v[g * 8 + 2]) * osc, __uint_as_float(v[g * 8 + 3]) * osc),
                  pack_bf16x2(__uint_as_float(v[g * 8 + 4]) * osc, __uint_as_float(v[g * 8 + 5]) * osc),
                  pack_bf16x2(__uint_as_float(v[g * 8 + 6]) * osc, __uint_as_float(v[g * 8 + 7]) * osc));
          }
        }
      }
    }
  } else {
    // Key tile invisible to every query (beyond kv_len, or right of the causal diagonal for all rows): zero gradients.
    const int r = (warp & 3) * 32 + lane;
    const int krow = k0 + r;
    if (krow < p.Sk) {
      __nv_bfloat16* dk_row = p.dk + (static_cast<long long>(b) * p.Sk + krow) * p.dkv_row_stride + hk * D;
      __nv_bfloat16* dv_row = p.dv + (static_cast<long long>(b) * p.Sk + krow) * p.dkv_row_stride + hk * D;
      for (int i = 0; i < D; i += 8) {
        *reinterpret_cast<uint4*>(dk_row + i) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(dv_row + i) = make_uint4(0, 0, 0, 0);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, (int)kStatusMbarTimeout);
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// delta[b,h,s] = sum_d dO[b,s,h,d] * O[b,s,h,d]; one warp per (b,s,h) row.
__global__ void fmha_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ delta, int B, int S, int H, int D) {
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(B) * S * H;
  if (w >= total) return;
  const int h = static_cast<int>(w % H);
  const long long bs = w / H;
  const int s = static_cast<int>(bs % S);
  const int b = static_cast<int>(bs / S);
  const __nv_bfloat16* po = o + w * D;
  const __nv_bfloat16* pd = d_o + w * D;
  float acc = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(po + i));
    float2 c = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(pd + i));
    acc += a.x * c.x + a.y * c.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[(static_cast<long long>(b) * H + h) * S + s] = acc;
}

// dq (bf16, strided rows) = cast(dq_acc fp32 [B*S, H*D])
__global__ void fmha_dq_cast_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long rows, int hd,
                                    long long row_stride) {
  const int vec_per_row = hd >> 3;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    const float4 a = *reinterpret_cast<const float4*>(acc + row * hd + c);
    const float4 bb = *reinterpret_cast<const float4*>(acc + row * hd + c + 4);
    *reinterpret_cast<uint4*>(dq + row * row_stride + c) =
        make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(bb.x, bb.y), pack_bf16x2(bb.z, bb.w));
  }
}

template <int D, bool DROP>
static int launch_fmha_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                           const CUtensorMap& tdq, const FmhaBwdParams& p, cudaStream_t stream) {
  using Cfg = FmhaBwdCfg<D>;
  auto kern = fmha_bwd_kernel<D, DROP>;
  static bool configured = false;
  if (!configured) {
    OFB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    configured = true;
  }
  dim3 grid((p.Sk + 127) / 128, p.Hk, p.B);
  kern<<<grid, 320, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, tdo, tdq, p);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace ofb

using namespace ofb;

// Floats of scratch the backward needs: B*Sq*H*D for the fp32 dQ accumulator + B*H*Sq for delta.
OFB_API long long ofb_fmha_bwd_scratch_floats(int B, int S, int H, int D) {
  return static_cast<long long>(B) * S * H * D + static_cast<long long>(B) * H * S;
}

// q: [B,Sq,H,D] view (token stride q_row_stride); k, v: [B,Sk,Hk,D] views (kv_row_stride); o, d_o: contiguous
// [B,Sq,H,D]; dq: [B,Sq,H,D] view with token stride dq_row_stride; dk, dv: [B,Sk,Hk,D] views with token stride
// dkv_row_stride. scratch: ofb_fmha_bwd_scratch_floats(B, Sq, H, D) floats. Dropout arguments as in the forward call
// whose output is differentiated.
OFB_API int ofb_fmha_bwd_ex(const void* q, const void* k, const void* v, long long q_row_stride, long long kv_row_stride,
                            const void* o, const void* d_o, const float* lse, void* dq, void* dk, void* dv,
                            long long dq_row_stride, long long dkv_row_stride, float* scratch, const int* kv_len, int B,
                            int Sq, int Sk, int H, int Hk, int D, int causal, float scale, float p_dropout,
                            unsigned long long seed, unsigned int offset, void* stream) {
  if (D != 64 && D != 128) return fail("fmha_bwd: head dim must be 64 or 128");
  if (Hk <= 0 || H % Hk) return fail("fmha_bwd: the number of query heads must be a multiple of the key/value heads");
  if (dq_row_stride % 8 || dkv_row_stride % 8) return fail("fmha_bwd: gradient row strides must be multiples of 8");
  if (B <= 0 || Sq <= 0 || Sk <= 0) return fail("fmha_bwd: empty problem");
  auto s = reinterpret_cast<cudaStream_t>(stream);
  CUtensorMap tq, tk, tv, tdo;
  if (fmha_tensor_map(&tq, q, B, Sq, H, D, q_row_stride)) return -1;
  if (fmha_tensor_map(&tk, k, B, Sk, Hk, D, kv_row_stride)) return -1;
  if (fmha_tensor_map(&tv, v, B, Sk, Hk, D, kv_row_stride)) return -1;
  if (fmha_tensor_map(&tdo, d_o, B, Sq, H, D, static_cast<long long>(H) * D)) return -1;
  const long long n_acc = static_cast<long long>(B) * Sq * H * D;
  float* dq_acc = scratch;
  float* delta = scratch + n_acc;
  OFB_CUDA_OK(cudaMemsetAsync(dq_acc, 0, n_acc * sizeof(float), s));
  {
    const long long rows = static_cast<long long>(B) * Sq * H;
    const int threads = 256;
    const long long blocks = (rows * 32 + threads - 1) / threads;
    fmha_delta_kernel<<<static_cast<unsigned>(blocks), threads, 0, s>>>(
        reinterpret_cast<const __nv_bfloat16*>(o), reinterpret_cast<const __nv_bfloat16*>(d_o), delta, B, Sq, H, D);
    OFB_CUDA_OK(cudaGetLastError());
  }
  FmhaBwdParams p;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc;
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk); p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.dkv_row_stride = dkv_row_stride; p.kv_len = kv_len;
  p.B = B; p.H = H; p.Hk = Hk; p.Sq = Sq; p.Sk = Sk; p.D = D; p.causal = causal; p.causal_off = Sk - Sq;
  p.scale = scale; p.scale_log2e = scale * 1.4426950408889634f;
  p.status = device_status_ptr();
  if (fmha_dropout_cfg(&p.drop, p_dropout, seed, offset)) return -1;
  CUtensorMap tdq;
  {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail("cuTensorMapEncodeTiled is not available");
    cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)Sq, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)D * 4, (cuuint64_t)H * D * 4, (cuuint64_t)Sq * H * D * 4};
    cuuint32_t box[4] = {32, 1, 128, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(&tdq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dq_acc, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("fmha_bwd: cuTensorMapEncodeTiled(dq) failed with code " + std::to_string((int)r));
  }
  int rc;
  if (p_dropout > 0.f)
    rc = D == 64 ? launch_fmha_bwd<64, true>(tq, tk, tv, tdo, tdq, p, s) : launch_fmha_bwd<128, true>(tq, tk, tv, tdo, tdq, p, s);
  else
    rc = D == 64 ? launch_fmha_bwd<64, false>(tq, tk, tv, tdo, tdq, p, s) : launch_fmha_bwd<128, false>(tq, tk, tv, tdo, tdq, p, s);
  if (rc) return rc;
  {
    const long long rows = static_cast<long long>(B) * Sq;
    const long long total = rows * (H * D / 8);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    fmha_dq_cast_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(dq_acc, reinterpret_cast<__nv_bfloat16*>(dq), rows,
                                                                     H * D, dq_row_stride);
    OFB_CUDA_OK(cudaGetLastError());
  }
  return 0;
}

// Self-attention form: one length, one head count, dq / dk / dv slices of one packed buffer.
OFB_API int ofb_fmha_bwd(const void* q, const void* k, const void* v, long long q_row_stride, long long kv_row_stride,
                         const void* o, const void* d_o, const float* lse, void* dq, void* dk, void* dv,
                         long long dqkv_row_stride, float* scratch, const int* kv_len, int B, int S, int H, int D,
                         int causal, float scale, void* stream) {
  return ofb_fmha_bwd_ex(q, k, v, q_row_stride, kv_row_stride, o, d_o, lse, dq, dk, dv, dqkv_row_stride, dqkv_row_stride, scratch,
                         kv_len, B, S, S, H, H, D, causal, scale, 0.f, 0ull, 0u, stream);
}
