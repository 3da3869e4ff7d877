// C ABI of libofb_kernels.so. Python binds these with ctypes
// (oneflow_b200/ops/_native.py); every function returns 0 on success and -1 on failure with the
// message available from ofb_last_error(). All pointers are device pointers unless noted;
// `stream` is a cudaStream_t passed as void*.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct OfbGemmArgs {
  const void* A;  // bf16. K-major: [M, lda]; MN-major: [K, lda]
  const void* B;  // bf16. K-major: [N, ldb]; MN-major: [K, ldb]
  void* C;        // bf16 [M, ldc] (fp32 when out_fp32)
  const void* bias;      // bf16 [N] or null
  const void* residual;  // bf16 [M, ldr] or null
  const void* aux_in;    // bf16 [M, ld_aux] or null
  void* aux_out;         // bf16 [M, ld_aux] or null
  long long lda, ldb, ldc, ldr, ld_aux;  // leading dimensions in elements
  int M, N, K;
  int a_mn_major, b_mn_major;
  int act;         // 0 none, 1 gelu(erf), 2 gelu(tanh), 3 relu
  int out_fp32;
  int accumulate;  // C += result
  int bn;          // tile width override: 0 auto, 128 or 256
  int max_ctas;    // 0 = one CTA per SM
  float alpha;
} OfbGemmArgs;

// Set-associative LRU cache of fp32 rows (lru_cache.cu): 32 ways per set, storage provided by the caller.
typedef struct OfbLruCache {
  void* keys;     // int64  [n_sets * 32]
  void* ticks;    // uint32 [n_sets * 32], zero-initialised (0 = empty way)
  void* lines;    // fp32   [n_sets * 32 * line]
  void* locks;    // uint32 [n_sets], zero-initialised
  long long n_sets;
  int line;       // floats per row, multiple of 4
} OfbLruCache;
int ofb_lru_get(const OfbLruCache* c, const long long* keys, long long n, float* out, unsigned int tick, int* n_miss, int* miss_index,
                long long* miss_keys, unsigned char* hit_mask, void* stream);
int ofb_lru_put(const OfbLruCache* c, const long long* keys, const float* rows, long long n, unsigned int tick, int* n_evicted,
                long long* evicted_keys, float* evicted_rows, void* stream);
int ofb_lru_dump(const OfbLruCache* c, int* n_out, long long* keys_out, float* rows_out, long long cap, void* stream);

int ofb_gemm_bf16(const OfbGemmArgs* args, void* stream);
const char* ofb_last_error(void);
int ofb_read_status(int clear, int* out_code, int* out_detail);

#ifdef __cplusplus
}
#endif
