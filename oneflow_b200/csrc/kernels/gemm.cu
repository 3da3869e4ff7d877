// C entry points of the tcgen05 GEMM (see gemm_tcgen05.cuh for the kernel).
#include <cstdlib>

#include "../common/host_utils.h"
#include "gemm_tcgen05.cuh"
#include "gemm_2cta.cuh"
#include "ofb_kernels.h"

namespace ofb {

// Whether shapes that fill the machine use the two-SM kernel unless told otherwise.
constexpr bool kDefault2Cta = true;

template <int BN, int A_MN, int B_MN, int ST = 0, int MINB = 1>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmShape& shp, const GemmEpilogue& ep,
                       int* status, int max_ctas, cudaStream_t stream) {
  using Cfg = GemmCfg<BN, ST>;
  auto kern = gemm_bf16_tcgen05_kernel<BN, A_MN, B_MN, ST, MINB>;
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
  const int tiles = ((shp.M + 127) / 128) * ((shp.N + BN - 1) / BN) * (shp.splits > 1 ? shp.splits : 1);
  int grid = tiles < sm_count * MINB ? tiles : sm_count * MINB;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  kern<<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, shp, ep, status);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

template <int A_MN, int B_MN>
static int launch_gemm_2cta(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmShape& shp, const GemmEpilogue& ep,
                            int* status, int max_ctas, cudaStream_t stream) {
  auto kern = gemm_bf16_2cta_kernel<A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    OFB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Gemm2Cfg::SMEM_BYTES));
    configured = true;
  }
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    OFB_CUDA_OK(cudaGetDevice(&dev));
    OFB_CUDA_OK(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  const int tiles = ((shp.M + 255) / 256) * ((shp.N + 255) / 256);
  int grid = 2 * tiles < sm_count ? 2 * tiles : (sm_count & ~1);
  if (max_ctas > 1 && grid > (max_ctas & ~1)) grid = max_ctas & ~1;
  kern<<<grid, 192, Gemm2Cfg::SMEM_BYTES, stream>>>(tmA, tmB, shp, ep, status);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

static int gemm_mode_2cta() {
  // OFB_GEMM_2CTA=0 turns the two-SM kernel off, =1 forces it for every shape it supports.
  static int mode = -2;
  if (mode == -2) {
    const char* e = std::getenv("OFB_GEMM_2CTA");
    mode = e ? std::atoi(e) : -1;
  }
  return mode;
}

int gemm_dispatch(const OfbGemmArgs* a, const GemmEpilogue& ep, cudaStream_t stream) {
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return fail("gemm: empty problem");
  if (a->N % 8 != 0) return fail("gemm: N must be a multiple of 8");
  const int a_mn = a->a_mn_major, b_mn = a->b_mn_major;
  // K-major: dims {K, rows}, row stride ld*2 bytes. MN-major: dims {rows, K}.
  CUtensorMap tmA, tmB;
  int bn = a->bn;
  const int mode2 = gemm_mode_2cta();
  bool two = bn == 512 || (mode2 == 1 && bn == 0);
  if (mode2 == -1 && bn == 0) {
    // default: the two-SM kernel for problems that fill the machine with 256 x 256 tiles
    const long long tiles2 = (long long)((a->M + 255) / 256) * ((a->N + 255) / 256);
    two = kDefault2Cta && tiles2 >= 74 && a->N >= 256 && a->M >= 256;
  }
  if (mode2 == 0) two = bn == 512;
  // Few K blocks and many tiles: the epilogue is the bottleneck, so run two one-SM CTAs per SM (short ring) instead.
  const bool short_k = a->K <= 1024 && bn == 0 && !a_mn && (long long)((a->M + 127) / 128) * ((a->N + 127) / 128) >= 2 * 148 &&
                       std::getenv("OFB_GEMM_SHORTK_OFF") == nullptr;
  if (short_k) two = false;
  if (two) {
    if (!a_mn) {
      if (get_tensor_map(&tmA, a->A, 2, 2, a->K, a->M, 0, (uint64_t)a->lda * 2, 0, 64, 128, 0, 3)) return -1;
    } else {
      if (get_tensor_map(&tmA, a->A, 2, 2, a->M, a->K, 0, (uint64_t)a->lda * 2, 0, 64, 64, 0, 3)) return -1;
    }
    if (!b_mn) {
      if (get_tensor_map(&tmB, a->B, 2, 2, a->K, a->N, 0, (uint64_t)a->ldb * 2, 0, 64, 128, 0, 3)) return -1;
    } else {
      if (get_tensor_map(&tmB, a->B, 2, 2, a->N, a->K, 0, (uint64_t)a->ldb * 2, 0, 64, 64, 0, 3)) return -1;
    }
    GemmShape shp2{a->M, a->N, a->K, 1};
    int* st2 = device_status_ptr();
    if (!a_mn && !b_mn) return launch_gemm_2cta<0, 0>(tmA, tmB, shp2, ep, st2, a->max_ctas, stream);
    if (!a_mn && b_mn) return launch_gemm_2cta<0, 1>(tmA, tmB, shp2, ep, st2, a->max_ctas, stream);
    if (a_mn && !b_mn) return launch_gemm_2cta<1, 0>(tmA, tmB, shp2, ep, st2, a->max_ctas, stream);
    return launch_gemm_2cta<1, 1>(tmA, tmB, shp2, ep, st2, a->max_ctas, stream);
  }
  if (short_k) bn = 128;
  if (bn != 128 && bn != 256) {
    // Small problems: prefer more, smaller tiles so that all SMs get work.
    long long tiles256 = (long long)((a->M + 127) / 128) * ((a->N + 255) / 256);
    bn = (tiles256 >= 120 && a->N >= 256) ? 256 : 128;
  }
  if (!a_mn) {
    if (get_tensor_map(&tmA, a->A, 2, 2, a->K, a->M, 0, (uint64_t)a->lda * 2, 0, 64, 128, 0, 3)) return -1;
  } else {
    if (get_tensor_map(&tmA, a->A, 2, 2, a->M, a->K, 0, (uint64_t)a->lda * 2, 0, 64, 64, 0, 3)) return -1;
  }
  if (!b_mn) {
    if (get_tensor_map(&tmB, a->B, 2, 2, a->K, a->N, 0, (uint64_t)a->ldb * 2, 0, 64, bn, 0, 3)) return -1;
  } else {
    if (get_tensor_map(&tmB, a->B, 2, 2, a->N, a->K, 0, (uint64_t)a->ldb * 2, 0, 64, 64, 0, 3)) return -1;
  }
  GemmShape shp{a->M, a->N, a->K, 1};
  // Split-K: few output tiles but a long K (weight gradients: [out, in] = dY^T X over all tokens) would leave most
  // SMs idle. The K range is cut so that about one work unit per SM exists; partial sums are added atomically into
  // the fp32 output, which is cleared first unless the call accumulates anyway.
  {
    static int sm_count = 0, allow = -1;
    if (sm_count == 0) {
      int dev = 0;
      OFB_CUDA_OK(cudaGetDevice(&dev));
      OFB_CUDA_OK(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
    }
    if (allow < 0) {
      const char* e = std::getenv("OFB_GEMM_SPLITK");
      allow = e ? std::atoi(e) : 1;
    }
    const bool plain = !ep.bias && !ep.aux_in && !ep.aux_out && !ep.residual && ep.act == 0 && ep.out_fp32;
    const int tiles = ((a->M + 127) / 128) * ((a->N + bn - 1) / bn);
    const int kblocks = (a->K + 63) / 64;
    int cap = a->max_ctas > 0 && a->max_ctas < sm_count ? a->max_ctas : sm_count;
    if (allow && plain && tiles * 2 <= cap && kblocks >= 16) {
      int splits = cap / tiles;
      if (splits > kblocks / 4) splits = kblocks / 4;
      if (splits > 1) {
        shp.splits = splits;
        if (!ep.accumulate)
          OFB_CUDA_OK(cudaMemset2DAsync(ep.C, static_cast<size_t>(ep.ldc) * 4, 0, static_cast<size_t>(a->N) * 4, a->M, stream));
      }
    }
  }
  int* status = device_status_ptr();
  if (short_k && shp.splits <= 1) {
    if (!b_mn) return launch_gemm<128, 0, 0, 2, 2>(tmA, tmB, shp, ep, status, a->max_ctas, stream);
    return launch_gemm<128, 0, 1, 2, 2>(tmA, tmB, shp, ep, status, a->max_ctas, stream);
  }
#define OFB_GEMM_CASE(BN_, AM_, BM_) \
  if (bn == BN_ && a_mn == AM_ && b_mn == BM_) return launch_gemm<BN_, AM_, BM_>(tmA, tmB, shp, ep, status, a->max_ctas, stream);
  OFB_GEMM_CASE(256, 0, 0)
  OFB_GEMM_CASE(256, 0, 1)
  OFB_GEMM_CASE(256, 1, 0)
  OFB_GEMM_CASE(256, 1, 1)
  OFB_GEMM_CASE(128, 0, 0)
  OFB_GEMM_CASE(128, 0, 1)
  OFB_GEMM_CASE(128, 1, 0)
  OFB_GEMM_CASE(128, 1, 1)
#undef OFB_GEMM_CASE
  return fail("gemm: unsupported configuration");
}

}  // namespace ofb

OFB_API int ofb_gemm_bf16(const OfbGemmArgs* a, void* stream) {
  using namespace ofb;
  GemmEpilogue ep;
  std::memset(&ep, 0, sizeof(ep));
  ep.C = a->C;
  ep.ldc = a->ldc;
  ep.bias = reinterpret_cast<const __nv_bfloat16*>(a->bias);
  ep.residual = reinterpret_cast<const __nv_bfloat16*>(a->residual);
  ep.ldr = a->ldr;
  ep.aux_in = reinterpret_cast<const __nv_bfloat16*>(a->aux_in);
  ep.aux_out = reinterpret_cast<__nv_bfloat16*>(a->aux_out);
  ep.ld_aux = a->ld_aux;
  ep.alpha = a->alpha;
  ep.act = a->act;
  ep.out_fp32 = a->out_fp32;
  ep.accumulate = a->accumulate;
  return gemm_dispatch(a, ep, reinterpret_cast<cudaStream_t>(stream));
}

OFB_API const char* ofb_last_error() { return ofb::last_error().c_str(); }

// Reads (and optionally clears) the device status block written by kernels whose bounded
// waits gave up. Synchronises the device: call it at step boundaries, not per kernel.
OFB_API int ofb_read_status(int clear, int* out_code, int* out_detail) {
  int* p = ofb::device_status_ptr();
  if (!p) return ofb::fail("no status block");
  int h[2] = {0, 0};
  OFB_CUDA_OK(cudaMemcpy(h, p, sizeof(h), cudaMemcpyDeviceToHost));
  if (out_code) *out_code = h[0];
  if (out_detail) *out_detail = h[1];
  if (clear && (h[0] || h[1])) OFB_CUDA_OK(cudaMemset(p, 0, 64 * sizeof(int)));
  return 0;
}
