// Fused multi-head attention forward for sm_100a (bf16, head dim 64 or 128, causal or
// full, optional per-batch key length for padding, query length != key length with the causal
// diagonal aligned to the bottom-right corner, grouped-query attention: H query heads share
// Hk key/value heads, dropout on the probabilities from a Philox counter indexed by position).
//
// One CTA owns a 128-row query tile of one (batch, head). Roles:
//   warp 0      TMA producer: Q once, then K_j / V_j tiles through a 2-stage ring
//   warp 1      tcgen05 issuer: S_j = Q K_j^T and O_j = P_j V_j, accumulators in TMEM
//   warps 2..9  softmax, two warps per scheduler: query row r is shared by two threads (warps 2..5 take key columns
//               0..63 of every tile, warps 6..9 columns 64..127; a warp reaches the TMEM lanes of its own quarter
//               only, so the split is by columns). Each reads its half of the S row with tcgen05.ld, the two exchange
//               their row maxima through shared memory (one bounded rendezvous per tile), keep identical running
//               maxima and their own partial sums, and write their half of P_j (bf16) to shared memory in the
//               128-byte-swizzled K-major layout the second MMA consumes. One softmax warp per scheduler issued
//               only a third of the cycles (a single warp cannot hide the MUFU and TMEM-load latencies); two do.
// O accumulates in TMEM across all key tiles (the PV product runs with accumulate on); the exponent
// reference trails the true running maximum by up to 2^8, so O is only rescaled in TMEM
// (tcgen05.ld / st) on the rare tiles where a row maximum jumps. S is double-buffered in TMEM so the
// tensor core computes tile j+1 while the softmax warps work on tile j.
//
// Reference counterparts: oneflow/user/kernels/scaled_dot_product_attention_kernel.cu (flash
// attention library call), fused_attention_kernels.cu :710 (CUTLASS fMHA, no sm_100 path) and the
// unfused fused_tril_scale_softmax_mask_scale chain.
#include "../common/host_utils.h"
#include "../common/philox.cuh"
#include "../common/ptx.cuh"
#include "ofb_kernels.h"

namespace ofb {

struct FmhaFwdParams {
  __nv_bfloat16* out;   // [B, Sq, H, D] contiguous
  float* lse;           // [B, H, Sq] natural-log sum-exp of the scaled scores
  const int* kv_len;    // [B] number of valid keys per batch or null
  int B, H, Hk, Sq, Sk, D;   // H query heads, Hk key/value heads (H % Hk == 0)
  int causal;
  int causal_off;       // Sk - Sq: query row r sees key columns <= r + causal_off
  DropoutCfg drop;
  float scale_log2e;    // softmax scale * log2(e)
  int* status;
};

template <int D>
struct FmhaFwdCfg {
  static constexpr int BM = 128, BN = 128;
  static constexpr int Q_BYTES = BM * D * 2;
  static constexpr int KV_BYTES = BN * D * 2;
  static constexpr int P_BYTES = BM * BN * 2;
  static constexpr int BAR_BYTES = 128;                 // 14 mbarriers, the TMEM slot, the abort flag
  static constexpr int XCHG_BYTES = 2 * 2 * 128 * 4;    // row maxima of the two column halves, one buffer per tile parity
  // At D = 128 the tiles take 224 KiB of the 227 KiB a CTA may have: the dynamic shared memory is declared 1024-byte
  // aligned (the kernel has no static shared memory, so it starts the CTA's window) instead of being aligned by hand
  // with a kilobyte of slack; the kernel checks the alignment and reports a status instead of running if it is not there.
  static constexpr int SMEM_BYTES = Q_BYTES + 4 * KV_BYTES + 2 * P_BYTES + BAR_BYTES + XCHG_BYTES;
};

// ex2.approx: one MUFU op (inputs here are <= ~8, -inf gives 0)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D, bool DROP>
__global__ void __launch_bounds__(320, 1)
fmha_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, FmhaFwdParams p) {
  using Cfg = FmhaFwdCfg<D>;
  constexpr int BM = 128, BN = 128, DCH = D / 64;  // 64-element chunks along the head dimension
  constexpr uint32_t IDESC_S = make_idesc_bf16(BM, BN, 0, 0);
  constexpr uint32_t IDESC_O = make_idesc_bf16(BM, D, 0, 1);
  constexpr int CH_BYTES = 128 * 128;  // one [128 rows x 64 elements] swizzled chunk

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {   // uniform over the CTA: nobody has touched a barrier or TMEM yet
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, (int)kStatusBounds);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::Q_BYTES;            // 2 stages
  uint8_t* sV = sK + 2 * Cfg::KV_BYTES;       // 2 stages
  uint8_t* sP = sV + 2 * Cfg::KV_BYTES;       // 2 buffers
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * Cfg::P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;     // [2]
  uint64_t* v_full = bars + 3;     // [2]
  uint64_t* kv_empty = bars + 5;   // [2]
  uint64_t* s_full = bars + 7;     // [2]
  uint64_t* p_full = bars + 9;     // [2]
  uint64_t* pv_done = bars + 11;   // [2]
  uint64_t* pair_bar = bars + 13;  // rendezvous of the 256 softmax threads
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xchg = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + Cfg::BAR_BYTES);   // [2 parities][2 halves][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Heavier (later) causal tiles first.
  const int n_qt = (p.Sq + BM - 1) / BM;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x);
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hk);
  const int q0 = qt * BM;
  int kv_limit = p.Sk;
  if (p.kv_len) kv_limit = min(kv_limit, p.kv_len[b]);
  int kv_end = kv_limit;
  if (p.causal) kv_end = min(kv_end, q0 + BM + p.causal_off);
  const int n_kv = kv_end > 0 ? (kv_end + BN - 1) / BN : 0;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&kv_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 256);
      mbar_init(&pv_done[s], 1);
    }
    mbar_init(pair_bar, 256);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;            // S[0], S[1] at +0, +128
  const uint32_t tO = tmem_base + 256;      // running O accumulator, D columns

  if (warp == 0) {
    if (elect_one() && n_kv > 0) {
      mbar_arrive_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
      for (int c = 0; c < DCH; ++c) tma_load_4d(sQ + c * CH_BYTES, &tmQ, q_full, c * 64, h, q0, b);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) break;
        mbar_arrive_expect_tx(&k_full[s], Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < DCH; ++c) tma_load_4d(sK + s * Cfg::KV_BYTES + c * CH_BYTES, &tmK, &k_full[s], c * 64, hk, j * BN, b);
        mbar_arrive_expect_tx(&v_full[s], Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < DCH; ++c) tma_load_4d(sV + s * Cfg::KV_BYTES + c * CH_BYTES, &tmV, &v_full[s], c * 64, hk, j * BN, b);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one() && n_kv > 0) {
      bool ok = mbar_wait(q_full, 0, abort_flag);
      const uint32_t q_base = smem_u32(sQ);
      auto issue_s = [&](int j) {
        const int s = j & 1;
        const uint32_t k_base = smem_u32(sK + s * Cfg::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * CH_BYTES + (kk & 3) * 32;
          umma_bf16_ss(tS + s * BN, make_smem_desc_sw128(q_base + off, 16, 1024),
                       make_smem_desc_sw128(k_base + off, 16, 1024), IDESC_S, kk != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[s]);
      };
      if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag);
      if (ok) { tc_fence_after(); issue_s(0); }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < n_kv) {
          if (!mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_s(j + 1);
        }
        if (!mbar_wait(&p_full[s], ph, abort_flag)) { ok = false; break; }
        if (!mbar_wait(&v_full[s], ph, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t p_base = smem_u32(sP + s * Cfg::P_BYTES);
        const uint32_t v_base = smem_u32(sV + s * Cfg::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint64_t da = make_smem_desc_sw128(p_base + (kk >> 2) * CH_BYTES + (kk & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(v_base + kk * 2048, CH_BYTES, 1024);
          umma_bf16_ss(tO, da, db, IDESC_O, (j | kk) != 0 ? 1u : 0u);   // O accumulates in TMEM over all key tiles
        }
        umma_commit(&pv_done[s]);
        umma_commit(&kv_empty[s]);
      }
    }
    __syncwarp();
  } else if (n_kv > 0) {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;        // which 64 key columns of every tile this thread takes
    const int r = quad * 32 + lane;          // row inside the tile == TMEM lane
    const int row_g = q0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    // m_ref is the exponent reference actually used for P and l; it trails the true running maximum by at
    // most kLazy (log2 units) so that the TMEM-resident O only has to be rescaled when the maximum jumps.
    // Both threads of a row carry the same m_ref (they see the same joint maxima); l_run is this half's sum.
    constexpr float kLazy = 8.0f;
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;
    uint32_t pair_parity = 0;
    auto pair_sync = [&]() {   // bounded: a thread that gave up elsewhere can never leave the others stuck here
      mbar_arrive(pair_bar);
      const bool w = mbar_wait(pair_bar, pair_parity, abort_flag);
      pair_parity ^= 1;
      return w;
    };
    for (int j = 0; j < n_kv; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&s_full[s], ph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int col_base = j * BN + half * 64;
      const bool need_mask = (p.causal && j * BN + BN - 1 > q0 + p.causal_off) || (j * BN + BN > kv_limit);
      const int col_max = p.causal ? min(row_g + p.causal_off, kv_limit - 1) : kv_limit - 1;  // last visible column
      uint32_t sv[2][32];
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 2; ++c) tmem_ld_32x32(tS + lane_addr + s * BN + half * 64 + c * 32, sv[c]);
      tmem_wait_ld();
      // eight independent max chains: a dependent chain of 64 cannot be hidden
      float mxs[8] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY, -INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          // the scores stay unscaled here: the scale is positive, so the maximum commutes with it, and the exponent below
          // applies it inside one fused multiply-add (one instruction per element less)
          float e = __uint_as_float(sv[c][i]);
          if (need_mask && col_base + c * 32 + i > col_max) { e = -INFINITY; sv[c][i] = __float_as_uint(e); }
          mxs[i & 7] = fmaxf(mxs[i & 7], e);
        }
      float mx = fmaxf(fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])), fmaxf(fmaxf(mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7])));
      mx *= p.scale_log2e;   // -inf stays -inf
      // joint row maximum of the two halves (buffer = tile parity: the partner may be one tile behind, never two)
      xchg[(s * 2 + half) * 128 + r] = mx;
      if (!pair_sync()) { ok = false; break; }
      mx = fmaxf(mx, xchg[(s * 2 + (half ^ 1)) * 128 + r]);
      // Rescale O (and l) only when some row of the warp moved its maximum by more than kLazy.
      const bool jump = mx > m_ref + kLazy;
      if (__any_sync(0xffffffffu, jump)) {
        const float m_new = fmaxf(m_ref, mx);
        const float alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);  // m_new is finite here or equals m_ref
        if (j > 0) {
          if (!mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          // each half rescales its half of the O columns
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            const int cc = half * (D / 32) + c;
            uint32_t o[16];
            tmem_ld_32x16(tO + lane_addr + cc * 16, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x16(tO + lane_addr + cc * 16, o);
          }
          tmem_wait_st();
        }
        l_run *= alpha;
        m_ref = m_new;
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      if (j >= 2) {  // the P buffer of parity s was last read by the PV product of tile j-2
        if (!mbar_wait(&pv_done[s], ((j - 2) >> 1) & 1, abort_flag)) { ok = false; break; }
      }
      float rs[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      uint8_t* chunk = sP + s * Cfg::P_BYTES + half * CH_BYTES + r * 128;   // 64 columns = one swizzled chunk
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float pv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) pv[e] = fast_exp2(fmaf(__uint_as_float(sv[c][i + e]), p.scale_log2e, -m_use));  // masked entries are -inf -> 0
          rs[(i >> 2) & 7] += (pv[0] + pv[1]) + (pv[2] + pv[3]);
          if constexpr (DROP) {
            // the row sum keeps every probability; only what multiplies V is dropped (1 / keep is applied at the end)
            const uint32_t keep = dropout_keep4(p.drop, static_cast<uint32_t>(b * p.H + h), static_cast<uint32_t>(row_g),
                                                static_cast<uint32_t>((col_base + c * 32 + i) >> 2));
#pragma unroll
            for (int e = 0; e < 4; ++e) pv[e] = (keep >> e) & 1u ? pv[e] : 0.f;
          }
          packed[i >> 1] = pack_bf16x2(pv[0], pv[1]);
          packed[(i >> 1) + 1] = pack_bf16x2(pv[2], pv[3]);
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int grp = c * 4 + g;
          *reinterpret_cast<uint4*>(chunk + ((grp ^ (r & 7)) << 4)) =
              make_uint4(packed[4 * g], packed[4 * g + 1], packed[4 * g + 2], packed[4 * g + 3]);
        }
      }
      l_run += ((rs[0] + rs[1]) + (rs[2] + rs[3])) + ((rs[4] + rs[5]) + (rs[6] + rs[7]));
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&p_full[s]);
    }
    if (ok) {
      // The row sum is the sum of the two halves' sums. It travels through the maxima buffer of the OTHER parity than the
      // last tile's: every thread finished reading that one before it could pass the last tile's rendezvous.
      const int so = (n_kv - 1) & 1;
      xchg[(((so ^ 1) * 2) + half) * 128 + r] = l_run;
      ok = pair_sync();
      const float l_tot = ok ? l_run + xchg[(((so ^ 1) * 2) + (half ^ 1)) * 128 + r] : 0.f;
      if (ok) ok = mbar_wait(&pv_done[so], ((n_kv - 1) >> 1) & 1, abort_flag);
      if (ok) {
        tc_fence_after();
        const float inv = l_tot > 0.f ? (DROP ? p.drop.inv_keep : 1.f) / l_tot : 0.f;
        __nv_bfloat16* orow = p.out + ((static_cast<long long>(b) * p.Sq + row_g) * p.H + h) * D;
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          const int cc = half * (D / 64) + c;     // each half writes its half of the output columns
          uint32_t v[32];
          __syncwarp();
          tmem_ld_32x32(tO + lane_addr + cc * 32, v);
          tmem_wait_ld();
          if (row_g < p.Sq) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[g * 8 + i]) * inv;
              *reinterpret_cast<uint4*>(orow + cc * 32 + g * 8) =
                  make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                             pack_bf16x2(f[6], f[7]));
            }
          }
        }
        if (half == 0 && row_g < p.Sq && p.lse)
          p.lse[(static_cast<long long>(b) * p.H + h) * p.Sq + row_g] =
              l_tot > 0.f ? (m_ref + log2f(l_tot)) * 0.6931471805599453f : -INFINITY;
      }
    }
  } else {
    // No visible keys at all (kv_len == 0, or a causal tile above the shifted diagonal): the output rows are zero.
    const int r = (warp & 3) * 32 + lane;
    const int row_g = q0 + r;
    if (row_g < p.Sq) {
      __nv_bfloat16* orow = p.out + ((static_cast<long long>(b) * p.Sq + row_g) * p.H + h) * D;
      for (int i = 0; i < D; i += 8) *reinterpret_cast<uint4*>(orow + i) = make_uint4(0, 0, 0, 0);
      if (p.lse) p.lse[(static_cast<long long>(b) * p.H + h) * p.Sq + row_g] = -INFINITY;
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

template <int D, bool DROP>
static int launch_fmha_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FmhaFwdParams& p,
                           cudaStream_t stream) {
  using Cfg = FmhaFwdCfg<D>;
  auto kern = fmha_fwd_kernel<D, DROP>;
  static bool configured = false;
  if (!configured) {
    OFB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    configured = true;
  }
  dim3 grid((p.Sq + 127) / 128, p.H, p.B);
  kern<<<grid, 320, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// 4-D map over a [B, S, H, D] view with a token stride of `row_stride` elements.
int fmha_tensor_map(CUtensorMap* out, const void* ptr, int B, int S, int H, int D, long long row_stride) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail("cuTensorMapEncodeTiled is not available");
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (row_stride * 2) % 16) return fail("fmha: operands must be 16-byte aligned");
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)row_stride * 2, (cuuint64_t)row_stride * 2 * S};
  cuuint32_t box[4] = {64, 1, 128, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("fmha: cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return 0;
}

// Fills a DropoutCfg from a drop probability, a 64-bit seed and a per-call offset.
int fmha_dropout_cfg(DropoutCfg* d, float p_dropout, unsigned long long seed, unsigned int offset) {
  if (!(p_dropout >= 0.f) || p_dropout >= 1.f) return fail("fmha: dropout probability must be in [0, 1)");
  const double keep = 1.0 - static_cast<double>(p_dropout);
  const double t = keep * 4294967296.0;
  d->seed_lo = static_cast<uint32_t>(seed);
  d->seed_hi = static_cast<uint32_t>(seed >> 32);
  d->offset = offset;
  d->threshold = t >= 4294967295.0 ? 0xFFFFFFFFu : static_cast<uint32_t>(t);
  d->inv_keep = static_cast<float>(1.0 / keep);
  return 0;
}

__global__ void fmha_dropout_mask_kernel(DropoutCfg d, unsigned char* __restrict__ mask, int BH, int Sq, int Sk) {
  const long long groups = (Sk + 3) / 4;
  const long long total = static_cast<long long>(BH) * Sq * groups;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const uint32_t cg = static_cast<uint32_t>(i % groups);
    const uint32_t row = static_cast<uint32_t>((i / groups) % Sq);
    const uint32_t bh = static_cast<uint32_t>(i / (groups * Sq));
    const uint32_t keep = dropout_keep4(d, bh, row, cg);
    for (int e = 0; e < 4; ++e) {
      const long long col = 4ll * cg + e;
      if (col < Sk) mask[(static_cast<long long>(bh) * Sq + row) * Sk + col] = (keep >> e) & 1u;
    }
  }
}

}  // namespace ofb

using namespace ofb;

// q: bf16 view [B, Sq, H, D], element (b, s, h, d) at ((b*Sq + s) * q_row_stride + h*D + d); k, v: [B, Sk, Hk, D] views
// with token stride kv_row_stride. out: contiguous [B, Sq, H, D]; lse: [B, H, Sq]. With causal set, query row r sees
// key columns <= r + (Sk - Sq). p_dropout > 0 drops probabilities by the Philox stream (seed, offset).
OFB_API int ofb_fmha_fwd_ex(const void* q, const void* k, const void* v, long long q_row_stride, long long kv_row_stride,
                            void* out, float* lse, const int* kv_len, int B, int Sq, int Sk, int H, int Hk, int D, int causal,
                            float scale, float p_dropout, unsigned long long seed, unsigned int offset, void* stream) {
  if (D != 64 && D != 128) return fail("fmha: head dim must be 64 or 128");
  if (Hk <= 0 || H % Hk) return fail("fmha: the number of query heads must be a multiple of the key/value heads");
  if (B <= 0 || Sq <= 0 || Sk <= 0) return fail("fmha: empty problem");
  if (!(scale > 0.f)) return fail("fmha: the softmax scale must be positive");   // the kernel takes row maxima before scaling
  CUtensorMap tq, tk, tv;
  if (fmha_tensor_map(&tq, q, B, Sq, H, D, q_row_stride)) return -1;
  if (fmha_tensor_map(&tk, k, B, Sk, Hk, D, kv_row_stride)) return -1;
  if (fmha_tensor_map(&tv, v, B, Sk, Hk, D, kv_row_stride)) return -1;
  FmhaFwdParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse; p.kv_len = kv_len; p.B = B; p.H = H; p.Hk = Hk; p.Sq = Sq; p.Sk = Sk; p.D = D; p.causal = causal;
  p.causal_off = Sk - Sq;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.status = device_status_ptr();
  if (fmha_dropout_cfg(&p.drop, p_dropout, seed, offset)) return -1;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (p_dropout > 0.f) return D == 64 ? launch_fmha_fwd<64, true>(tq, tk, tv, p, s) : launch_fmha_fwd<128, true>(tq, tk, tv, p, s);
  return D == 64 ? launch_fmha_fwd<64, false>(tq, tk, tv, p, s) : launch_fmha_fwd<128, false>(tq, tk, tv, p, s);
}

OFB_API int ofb_fmha_fwd(const void* q, const void* k, const void* v, long long q_row_stride, long long kv_row_stride,
                         void* out, float* lse, const int* kv_len, int B, int S, int H, int D, int causal, float scale,
                         void* stream) {
  return ofb_fmha_fwd_ex(q, k, v, q_row_stride, kv_row_stride, out, lse, kv_len, B, S, S, H, H, D, causal, scale, 0.f, 0ull, 0u,
                         stream);
}

// mask[b*H + h, row, col] = 1 where the attention dropout of (seed, offset) keeps the probability: the mask the fused
// kernels regenerate on the fly, written out for tests and for the unfused fallback.
OFB_API int ofb_fmha_dropout_mask(unsigned char* mask, int BH, int Sq, int Sk, float p_dropout, unsigned long long seed,
                                  unsigned int offset, void* stream) {
  DropoutCfg d;
  if (fmha_dropout_cfg(&d, p_dropout, seed, offset)) return -1;
  const long long total = static_cast<long long>(BH) * Sq * ((Sk + 3) / 4);
  if (total <= 0) return 0;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  fmha_dropout_mask_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(d, mask, BH, Sq, Sk);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
