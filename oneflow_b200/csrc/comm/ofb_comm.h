// C ABI of the communication part of libofb_kernels.so (symmetric memory, stand-alone collectives,
// GEMM fused with reduce-scatter / all-gather). Bound from Python in oneflow_b200/comm/symmetric.py.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct OfbCommCtx {
  int rank;
  int n;
  void* arena[8];    // arena base of every rank as mapped into this process
  void* signals[8];  // SignalBlock of every rank as mapped into this process
} OfbCommCtx;

int ofb_symm_alloc(long long bytes, void** ptr, unsigned char* handle64);
int ofb_symm_open(const unsigned char* handle64, void** ptr);
int ofb_symm_close(void* ptr);
int ofb_symm_free(void* ptr);
int ofb_comm_collective(const OfbCommCtx* ctx, int mode, long long in_off, long long stage_off, int in_dtype, void* out,
                        int out_dtype, long long count, float scale, unsigned int epoch, int ctas, void* stream);
int ofb_comm_all_to_all(const OfbCommCtx* ctx, long long in_off, int dtype, void* out, long long outer, long long I,
                        long long mid, long long J, long long inner, unsigned int epoch, int ctas, void* stream);

#ifdef __cplusplus
}
#endif
