// LayerNorm backward that allocates nothing. This entry point has no counterpart in the reference
// framework; it exists for users of this library who cannot obtain device memory at call time.
//
// Who needs it: a caller that is not allowed to call cudaMalloc (or any allocating library routine) when
// it needs the gradient - for example an inference/training server that froze its memory pool after
// start-up so that latency stays flat, a plug-in that only receives raw device pointers from its host
// application and must leave the host's allocator alone, or a job whose memory budget is fully assigned.
// The regular ofb_layer_norm_bwd() asks such a caller for a scratch buffer it has no way to provide.
//
// What it does instead: the partial-sum scratch is a static device array inside libofb_kernels.so
// (9.25 MiB, held by every GPU that loads the library until the process ends). The caller passes only
// the inputs and outputs of the operation, exactly as for ofb_layer_norm_bwd() minus `scratch`.
//
// Limits and rules
//   * cols must be <= ofb_layer_norm_bwd_noalloc_max_cols() (4096) and a multiple of 8; larger problems
//     are refused with an error (returns -1, message from ofb_last_error()). rows is unlimited.
//   * The first call on each device looks up the device address of the static array (with that device
//     current). Make that first call outside any CUDA stream capture; later calls only launch kernels.
//   * This function itself calls no cudaMalloc / cudaFree / allocating library routine, on any call. The
//     CUDA runtime may still load the library's module image (which contains the 9.25 MiB array) lazily
//     at the first call on a device, and that load needs device memory: make the first call before the
//     memory is frozen or exhausted, or run with CUDA_MODULE_LOADING=EAGER.
//   * dgamma and dbeta are given together or not at all; one without the other is refused (-1).
//   * All calls share the same array, which keeps the previous call's contents. The kernels overwrite
//     every value they later read, so nothing has to be cleared between calls; but calls that overlap on
//     the GPU (several streams or threads) race on it. Serialise them on one stream or with events.
//   * Results are the same as ofb_layer_norm_bwd() for the same inputs.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest `cols` the built-in scratch supports.
int ofb_layer_norm_bwd_noalloc_max_cols(void);

// dy, x, add_to_dx (optional), dx: bf16 [rows, cols]; gamma (optional): bf16 [cols]; mean, rstd: fp32 [rows]
// as produced by ofb_layer_norm_fwd(); dgamma, dbeta (optional, both or neither): fp32 [cols], overwritten
// or accumulated into when accumulate_param_grads != 0. stream: cudaStream_t. Returns 0 or -1.
int ofb_layer_norm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                               const void* add_to_dx, void* dx, float* dgamma, float* dbeta, int accumulate_param_grads,
                               int rows, int cols, void* stream);

#ifdef __cplusplus
}
#endif
