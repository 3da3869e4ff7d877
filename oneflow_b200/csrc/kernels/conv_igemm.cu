// Implicit-GEMM convolution for NHWC bf16 activations on tcgen05 (stride 1, "same" padding, odd R x S filters,
// channel counts that are multiples of 64): forward, input gradient and weight gradient.
//
// No im2col buffer exists anywhere. The activation operand of every MMA is fetched by a 4-D TMA box
// {64 channels, BW, BH, BN pixels} whose start coordinate is shifted by the filter tap, so the halo and the
// zero padding come from TMA's out-of-bounds fill, and the box lands in shared memory exactly as the
// 128-byte-swizzled operand tile that tcgen05.mma reads:
//   fprop  Y[pix, k]   = sum_{tap, c} X[pix + tap, c] W[k, tap, c]     A = X boxes (K-major),  B = W rows (K-major)
//   dgrad  dX[pix, c]  = sum_{tap, k} dY[pix - tap, k] W[k, tap, c]    A = dY boxes (K-major), B = W boxes (MN-major)
//   wgrad  dW[k, tap, c] = sum_pix dY[pix, k] X[pix + tap, c]          A = dY boxes (MN-major), B = X boxes (MN-major),
//                                                                      K loop over pixel boxes, split over the SMs
// A tile of 128 output pixels is BN images x BH rows x BW columns (powers of two chosen per layer so that the
// boxes tile the feature map with little or no waste). The kernel skeleton is the persistent warp-specialised
// one of the GEMM (TMA producer, single-thread MMA issuer, four epilogue warps, two TMEM accumulators); the
// epilogue maps accumulator rows back to NHWC pixels and stores through the swizzled staging tile.
//
// Reference: oneflow/user/kernels/conv_cudnn_kernels.cpp, conv_cutlass_kernels.cu (cuDNN / CUTLASS implicit GEMM).
#include <map>
#include <mutex>
#include <tuple>

#include "../common/host_utils.h"
#include "../common/ptx.cuh"
#include "gemm_tcgen05.cuh"
#include "ofb_kernels.h"

namespace ofb {

enum ConvMode : int { kConvFprop = 0, kConvDgrad = 1, kConvWgrad = 2 };

struct ConvGeom {
  int N, H, W;       // images and feature-map size (input = output: stride 1, same padding)
  int CA;            // channels of the activation operand (fprop: Cin, dgrad: Cout, wgrad: Cin)
  int CO;            // channels of the result rows (fprop: Cout, dgrad: Cin); wgrad: Cout (rows of dW)
  int R, S;          // filter size, padding (R - 1) / 2, (S - 1) / 2
  int lbw, lbh;      // log2 of the pixel box: BW, BH (BN = pixels per box / (BW * BH))
  int tiles_w, tiles_h, tiles_n;
  int splits;        // wgrad: pieces of the pixel loop
};

__device__ __forceinline__ void conv_tile_origin(const ConvGeom& g, int t, int pix_per_box, int& n0, int& h0, int& w0) {
  const int bn = pix_per_box >> (g.lbw + g.lbh);
  const int tw = t % g.tiles_w;
  const int th = (t / g.tiles_w) % g.tiles_h;
  const int tn = t / (g.tiles_w * g.tiles_h);
  w0 = tw << g.lbw;
  h0 = th << g.lbh;
  n0 = tn * bn;
}

template <int MODE, int BN, int ST = 0, int MINB = 1>
__global__ void __launch_bounds__(192, MINB)
conv_igemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, ConvGeom g, GemmEpilogue ep,
                  int* status) {
  using Cfg = GemmCfg<BN, ST>;
  constexpr int BM = 128, BK = 64, STAGES = Cfg::STAGES;
  constexpr int A_BYTES = Cfg::A_BYTES, B_BYTES = Cfg::B_BYTES;
  constexpr int A_MN = MODE == kConvWgrad ? 1 : 0;
  constexpr int B_MN = MODE == kConvFprop ? 0 : 1;
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
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

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

  const int pad_h = (g.R - 1) >> 1, pad_w = (g.S - 1) >> 1;
  const int pix_tiles = g.tiles_w * g.tiles_h * g.tiles_n;
  // GEMM view of the problem
  int tiles_m, tiles_n, kblocks;
  if (MODE == kConvWgrad) {
    tiles_m = (g.CO + BM - 1) / BM;
    tiles_n = (g.R * g.S * g.CA + BN - 1) / BN;
    kblocks = pix_tiles;  // boxes of 64 pixels
  } else {
    tiles_m = pix_tiles;  // boxes of 128 pixels
    tiles_n = (g.CO + BN - 1) / BN;
    kblocks = g.R * g.S * (g.CA / BK);
  }
  const int total_tiles = tiles_m * tiles_n;
  const int kb_per = (kblocks + max(g.splits, 1) - 1) / max(g.splits, 1);
  const int splits = (kblocks + kb_per - 1) / kb_per;
  const int total_units = total_tiles * splits;
  const int cpb = g.CA / BK;  // channel chunks per tap

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        const int t = u % total_tiles;
        // M tiles vary fastest so that CTAs running together share the weight (or dY) tile in L2
        const int tm = t % tiles_m, tn = t / tiles_m;
        const int kb0 = (u / total_tiles) * kb_per, kb1 = min(kblocks, kb0 + kb_per);
        int n0 = 0, h0 = 0, w0 = 0;
        if (MODE != kConvWgrad) conv_tile_origin(g, tm, 128, n0, h0, w0);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(&full[stage], A_BYTES + B_BYTES);
          uint8_t* a_dst = sA + stage * A_BYTES;
          uint8_t* b_dst = sB + stage * B_BYTES;
          if (MODE == kConvFprop) {
            const int tap = kb / cpb, c0 = (kb % cpb) * BK;
            const int r = tap / g.S, s = tap % g.S;
            tma_load_4d(a_dst, &tmA, &full[stage], c0, w0 + s - pad_w, h0 + r - pad_h, n0);
            tma_load_2d(b_dst, &tmB, &full[stage], kb * BK, tn * BN);                      // W[k rows][tap * C + c]
          } else if (MODE == kConvDgrad) {
            const int tap = kb / cpb, c0 = (kb % cpb) * BK;                                // c0: chunk of dY channels (= Cout)
            const int r = tap / g.S, s = tap % g.S;
            tma_load_4d(a_dst, &tmA, &full[stage], c0, w0 - s + pad_w, h0 - r + pad_h, n0);
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)                                              // W[k0.. rows][tap * Cin + cin chunk]
              tma_load_2d(b_dst + c * (BK * 128), &tmB, &full[stage], tap * g.CO + tn * BN + c * 64, c0);
          } else {
            conv_tile_origin(g, kb, 64, n0, h0, w0);
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_4d(a_dst + c * (BK * 128), &tmA, &full[stage], tm * BM + c * 64, w0, h0, n0);
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) {
              const int col = tn * BN + c * 64;  // column of dW: tap * Cin + channel
              const int tap = col / g.CA, c0 = col % g.CA;
              const int r = tap / g.S, s = tap % g.S;
              // columns past the last tap read out of bounds (tap >= R S): shifted far outside so that they come back as zeros
              tma_load_4d(b_dst + c * (BK * 128), &tmB, &full[stage], c0, tap < g.R * g.S ? w0 + s - pad_w : -(1 << 20),
                          h0 + r - pad_h, n0);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
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
          umma_commit(&empty[stage]);
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
    const int quad = warp & 3;
    const uint32_t stage_sm = smem_u32(epi_stage + quad * kEpiStageBytesPerWarp);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int u = blockIdx.x; u < total_units; u += gridDim.x) {
      const int t = u % total_tiles;
      const int tm = t % tiles_m, tn = t / tiles_m;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      if (MODE == kConvWgrad) {
        GemmShape shp{g.CO, g.R * g.S * g.CA, 0, splits};
        gemm_epilogue_warp<BN>(ep, shp, taddr, tm * BM + quad * 32, tn * BN, lane, stage_sm, splits > 1);
      } else {
        int n0, h0, w0;
        conv_tile_origin(g, tm, 128, n0, h0, w0);
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(ep.C);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = tn * BN + c * 32;
          if (col0 >= g.CO) break;
          uint32_t r[32];
          __syncwarp();
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 qv;
            qv.x = pack_bf16x2(__uint_as_float(r[ch * 8 + 0]), __uint_as_float(r[ch * 8 + 1]));
            qv.y = pack_bf16x2(__uint_as_float(r[ch * 8 + 2]), __uint_as_float(r[ch * 8 + 3]));
            qv.z = pack_bf16x2(__uint_as_float(r[ch * 8 + 4]), __uint_as_float(r[ch * 8 + 5]));
            qv.w = pack_bf16x2(__uint_as_float(r[ch * 8 + 6]), __uint_as_float(r[ch * 8 + 7]));
            epi_sts(epi_addr64(stage_sm, lane, ch), qv);
          }
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int rr = it * 8 + (lane >> 2), ch = lane & 3;
            const int row = quad * 32 + rr;  // pixel of the box: [bn][bh][bw]
            const int w = w0 + (row & ((1 << g.lbw) - 1));
            const int h = h0 + ((row >> g.lbw) & ((1 << g.lbh) - 1));
            const int n = n0 + (row >> (g.lbw + g.lbh));
            const uint4 qv = epi_lds(epi_addr64(stage_sm, rr, ch));
            if (w < g.W && h < g.H && n < g.N && col0 + ch * 8 < g.CO) {
              const long long pix = (static_cast<long long>(n) * g.H + h) * g.W + w;
              *reinterpret_cast<uint4*>(out + pix * ep.ldc + col0 + ch * 8) = qv;
            }
          }
          __syncwarp();
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
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace ofb

using namespace ofb;

// Rank-4 NHWC tensor map {C, W, H, N} with a box {64, bw, bh, bn}, 128-byte swizzle, zero fill outside.
static int conv_tensor_map(CUtensorMap* out, const void* ptr, int N, int H, int W, int C, int bw, int bh, int bn) {
  using Key = std::tuple<const void*, int, int, int, int, int, int, int>;
  static std::map<Key, CUtensorMap> cache;
  static std::mutex mu;
  const Key key{ptr, N, H, W, C, bw, bh, bn};
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
  }
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail("cuTensorMapEncodeTiled is not available");
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (C % 8) != 0) return fail("conv: tensors must be 16-byte aligned with C % 8 == 0");
  cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
  cuuint64_t strides[3] = {(cuuint64_t)C * 2, (cuuint64_t)W * C * 2, (cuuint64_t)H * W * C * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)bw, (cuuint32_t)bh, (cuuint32_t)bn};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("conv: cuTensorMapEncodeTiled failed for the activation tensor");
  std::lock_guard<std::mutex> lk(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

static int pow2_floor_log(int v) {
  int l = 0;
  while ((2 << l) <= v) ++l;
  return l;
}

// Splits `pixels` (a power of two) into a box bw x bh x bn over a W x H map: widths that divide W when possible.
static void conv_pick_box(int W, int H, int pixels, int* lbw, int* lbh) {
  auto pick = [](int extent, int cap_log) {
    int l = 0;
    while (l < cap_log && extent % (2 << l) == 0) ++l;  // largest power of two dividing the extent
    if ((1 << l) < 4 && extent > 4) {                   // tiny divisor: take a covering box instead, some lanes idle
      l = 0;
      while ((1 << l) < extent && l < cap_log) ++l;
      if (l > 3) l = 3;
    }
    return l;
  };
  const int total = pow2_floor_log(pixels);
  int w = pick(W, total < 4 ? total : 4);
  int h = pick(H, total - w < 3 ? total - w : 3);
  *lbw = w;
  *lbh = h;
}

template <int MODE, int BN, int ST = 0, int MINB = 1>
static int conv_launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const ConvGeom& g, const GemmEpilogue& ep, int units,
                       cudaStream_t stream) {
  using Cfg = GemmCfg<BN, ST>;
  auto kern = conv_igemm_kernel<MODE, BN, ST, MINB>;
  static bool configured = false;
  if (!configured) {
    OFB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    configured = true;
  }
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    OFB_CUDA_OK(cudaGetDevice(&dev));
    OFB_CUDA_OK(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  const int grid = units < sm_count * MINB ? units : sm_count * MINB;
  kern<<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, g, ep, device_status_ptr());
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

static int conv_check(int N, int H, int W, int Cin, int Cout, int R, int S) {
  if (N < 1 || H < 1 || W < 1) return fail("conv: empty problem");
  if (Cin % 64 || Cout % 64) return fail("conv: channel counts must be multiples of 64");
  if (!(R & 1) || !(S & 1) || R > 7 || S > 7) return fail("conv: odd filter sizes up to 7");
  return 0;
}

// y[N, H, W, Cout] = conv(x[N, H, W, Cin], w[Cout, R, S, Cin]), stride 1, padding (R-1)/2, (S-1)/2. bf16.
OFB_API int ofb_conv_fprop(const void* x, const void* w, void* y, int N, int H, int W, int Cin, int Cout, int R, int S, void* stream_) {
  if (conv_check(N, H, W, Cin, Cout, R, S)) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  ConvGeom g{};
  g.N = N; g.H = H; g.W = W; g.CA = Cin; g.CO = Cout; g.R = R; g.S = S; g.splits = 1;
  conv_pick_box(W, H, 128, &g.lbw, &g.lbh);
  const int bw = 1 << g.lbw, bh = 1 << g.lbh, bn = 128 / (bw * bh);
  g.tiles_w = (W + bw - 1) / bw; g.tiles_h = (H + bh - 1) / bh; g.tiles_n = (N + bn - 1) / bn;
  CUtensorMap tmA, tmB;
  if (conv_tensor_map(&tmA, x, N, H, W, Cin, bw, bh, bn)) return -1;
  const int bnt = Cout >= 256 ? 256 : 128;
  if (get_tensor_map(&tmB, w, 2, 2, static_cast<uint64_t>(R) * S * Cin, Cout, 0, static_cast<uint64_t>(R) * S * Cin * 2, 0, 64, bnt, 0, 3))
    return -1;
  GemmEpilogue ep;
  std::memset(&ep, 0, sizeof(ep));
  ep.C = y; ep.ldc = Cout; ep.alpha = 1.f;
  const int units = g.tiles_w * g.tiles_h * g.tiles_n * ((Cout + bnt - 1) / bnt);
  // few K blocks: the accumulator drain bounds the tile rate, two CTAs per SM (short ring) double it
  if (bnt == 128 && R * S * (Cin / 64) <= 18 && units >= 4 * 148) return conv_launch<kConvFprop, 128, 2, 2>(tmA, tmB, g, ep, units, stream);
  return bnt == 256 ? conv_launch<kConvFprop, 256>(tmA, tmB, g, ep, units, stream) : conv_launch<kConvFprop, 128>(tmA, tmB, g, ep, units, stream);
}

// dx[N, H, W, Cin] = gradient of ofb_conv_fprop wrt x, from dy[N, H, W, Cout] and w[Cout, R, S, Cin].
OFB_API int ofb_conv_dgrad(const void* dy, const void* w, void* dx, int N, int H, int W, int Cin, int Cout, int R, int S, void* stream_) {
  if (conv_check(N, H, W, Cin, Cout, R, S)) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  ConvGeom g{};
  g.N = N; g.H = H; g.W = W; g.CA = Cout; g.CO = Cin; g.R = R; g.S = S; g.splits = 1;
  conv_pick_box(W, H, 128, &g.lbw, &g.lbh);
  const int bw = 1 << g.lbw, bh = 1 << g.lbh, bn = 128 / (bw * bh);
  g.tiles_w = (W + bw - 1) / bw; g.tiles_h = (H + bh - 1) / bh; g.tiles_n = (N + bn - 1) / bn;
  CUtensorMap tmA, tmB;
  if (conv_tensor_map(&tmA, dy, N, H, W, Cout, bw, bh, bn)) return -1;
  // weights as a matrix [Cout rows][R S Cin columns]; a B tile is a set of {64 columns, 64 rows} boxes
  if (get_tensor_map(&tmB, w, 2, 2, static_cast<uint64_t>(R) * S * Cin, Cout, 0, static_cast<uint64_t>(R) * S * Cin * 2, 0, 64, 64, 0, 3))
    return -1;
  GemmEpilogue ep;
  std::memset(&ep, 0, sizeof(ep));
  ep.C = dx; ep.ldc = Cin; ep.alpha = 1.f;
  const int bnt = Cin >= 256 ? 256 : 128;
  const int units = g.tiles_w * g.tiles_h * g.tiles_n * ((Cin + bnt - 1) / bnt);
  if (bnt == 128 && R * S * (Cout / 64) <= 18 && units >= 4 * 148) return conv_launch<kConvDgrad, 128, 2, 2>(tmA, tmB, g, ep, units, stream);
  return bnt == 256 ? conv_launch<kConvDgrad, 256>(tmA, tmB, g, ep, units, stream) : conv_launch<kConvDgrad, 128>(tmA, tmB, g, ep, units, stream);
}

// dw[Cout, R, S, Cin] (fp32) (+)= gradient of ofb_conv_fprop wrt w, from x and dy.
OFB_API int ofb_conv_wgrad(const void* x, const void* dy, float* dw, int N, int H, int W, int Cin, int Cout, int R, int S,
                           int accumulate, void* stream_) {
  if (conv_check(N, H, W, Cin, Cout, R, S)) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  ConvGeom g{};
  g.N = N; g.H = H; g.W = W; g.CA = Cin; g.CO = Cout; g.R = R; g.S = S;
  conv_pick_box(W, H, 64, &g.lbw, &g.lbh);
  const int bw = 1 << g.lbw, bh = 1 << g.lbh, bn = 64 / (bw * bh);
  g.tiles_w = (W + bw - 1) / bw; g.tiles_h = (H + bh - 1) / bh; g.tiles_n = (N + bn - 1) / bn;
  CUtensorMap tmA, tmB;
  if (conv_tensor_map(&tmA, dy, N, H, W, Cout, bw, bh, bn)) return -1;
  if (conv_tensor_map(&tmB, x, N, H, W, Cin, bw, bh, bn)) return -1;
  const int ncols = R * S * Cin;
  const int bnt = ncols >= 256 ? 256 : 128;
  const int tiles = ((Cout + 127) / 128) * ((ncols + bnt - 1) / bnt);
  const int kblocks = g.tiles_w * g.tiles_h * g.tiles_n;
  int sm_count = 148;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  int splits = (2 * sm_count + tiles - 1) / tiles;  // about two work units per SM
  if (splits > kblocks / 4) splits = kblocks / 4;
  if (splits < 1) splits = 1;
  g.splits = splits;
  GemmEpilogue ep;
  std::memset(&ep, 0, sizeof(ep));
  ep.C = dw; ep.ldc = ncols; ep.alpha = 1.f; ep.out_fp32 = 1; ep.accumulate = accumulate;
  if (splits > 1 && !accumulate) OFB_CUDA_OK(cudaMemsetAsync(dw, 0, static_cast<size_t>(Cout) * ncols * 4, stream));
  const int units = tiles * splits;
  return bnt == 256 ? conv_launch<kConvWgrad, 256>(tmA, tmB, g, ep, units, stream) : conv_launch<kConvWgrad, 128>(tmA, tmB, g, ep, units, stream);
}
