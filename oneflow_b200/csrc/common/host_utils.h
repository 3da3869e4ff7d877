// Host-side helpers shared by the kernel libraries: error reporting through a C API
// (no exceptions cross the ctypes boundary), the device status word that kernels
// with bounded waits write on failure, and a cache of TMA tensor maps.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>

#define OFB_API extern "C" __attribute__((visibility("default")))

namespace ofb {

inline std::string& last_error() {
  static thread_local std::string s;
  return s;
}
inline int fail(const std::string& msg) {
  last_error() = msg;
  return -1;
}

#define OFB_CUDA_OK(expr)                                                                      \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess)                                                                     \
      return ::ofb::fail(std::string(#expr) + ": " + cudaGetErrorString(_e));                  \
  } while (0)

// One 64-int status block per device, allocated on first use. Slot 0 holds the first
// non-zero StatusCode any kernel recorded; slot 1 a kernel-specific detail value.
inline int* device_status_ptr() {
  static int* ptrs[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> g(mu);
  if (!ptrs[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 64 * sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 64 * sizeof(int));
    ptrs[dev] = p;
  }
  return ptrs[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  // The encoder is a driver entry point and needs a current context on the CALLING thread. A thread that has only run this
  // library's code so far (autograd's device thread whose first work item is one of these kernels) has none bound yet:
  // the first runtime call that needs one binds the primary context of the thread's device. That call may come while a
  // stream capture is open (a thread that records a graph after other threads ran the same kernels eagerly), where
  // cudaFree counts as unsafe and would invalidate the capture: the thread's capture mode is relaxed around it.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
    cudaThreadExchangeStreamCaptureMode(&mode);
    cudaFree(nullptr);
    cudaThreadExchangeStreamCaptureMode(&mode);
    context_bound = true;
  }
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct TmapKey {
  const void* ptr;
  uint64_t d0, d1, d2, stride1, stride2;
  uint32_t b0, b1, b2, elem, swz;
  bool operator==(const TmapKey& o) const { return std::memcmp(this, &o, sizeof(TmapKey)) == 0; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
    size_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(TmapKey) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
    return h;
  }
};

// Rank-2 or rank-3 tiled tensor map over 2-byte (bf16/fp16) or 4-byte elements, 128-byte swizzle
// (swz=3) or no swizzle (swz=0). Dimension 0 is the contiguous one. Strides in bytes.
inline int get_tensor_map(CUtensorMap* out, const void* ptr, int elem_bytes, int rank, uint64_t d0, uint64_t d1,
                          uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1,
                          uint32_t b2, int swz) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  static std::mutex mu;
  TmapKey key;
  std::memset(&key, 0, sizeof(key));
  key.ptr = ptr; key.d0 = d0; key.d1 = d1; key.d2 = (rank == 3 ? d2 : 0);
  key.stride1 = stride1_bytes; key.stride2 = (rank == 3 ? stride2_bytes : 0);
  key.b0 = b0; key.b1 = b1; key.b2 = (rank == 3 ? b2 : 0); key.elem = elem_bytes; key.swz = swz;
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
  }
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail("cuTensorMapEncodeTiled is not available (no CUDA driver?)");
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return fail("TMA base address must be 16-byte aligned");
  if ((stride1_bytes & 15) != 0 || (rank == 3 && (stride2_bytes & 15) != 0))
    return fail("TMA strides must be multiples of 16 bytes");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUtensorMapSwizzle sw = swz == 3 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = fn(out, dt, rank, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    snprintf(buf, sizeof(buf),
             "cuTensorMapEncodeTiled failed (%d): rank=%d dims=(%llu,%llu,%llu) strides=(%llu,%llu) box=(%u,%u,%u)",
             (int)r, rank, (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2,
             (unsigned long long)stride1_bytes, (unsigned long long)stride2_bytes, b0, b1, b2);
    return fail(buf);
  }
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

}  // namespace ofb
