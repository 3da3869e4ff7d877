// NVLink / NVSwitch bandwidth of plain SM accesses to a peer's symmetric arena, as seen by the fused kernels of this
// library: the figures that set the roofline of a fused compute+collective kernel and tell which access pattern its
// epilogue or copier warps should use. One kernel, no synchronisation with the peer (the peer only lends memory):
//   mode 0  pull, wide:    ld 16 B per lane from the peer, 512 contiguous bytes per warp instruction, st locally
//   mode 1  push, wide:    ld locally, st 16 B per lane to the peer, 512 contiguous bytes per warp instruction
//   mode 2  push, 64-byte row segments: every warp instruction writes 8 pieces of 64 B that lie `pitch` bytes apart
//           (the pattern of a GEMM epilogue that drains 32-column chunks of an accumulator tile)
//   mode 3  push, 256-byte row segments: 2 pieces of 256 B per warp instruction, `pitch` bytes apart
// The caller times the launch with CUDA events.
#include "../common/host_utils.h"
#include "comm_common.cuh"
#include "ofb_comm.h"

namespace ofb {

__global__ void __launch_bounds__(256) p2p_bandwidth_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long vecs,
                                                           int mode, long long pitch_vecs) {
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  if (mode <= 1) {
    long long i = tid;
    for (; i + 3 * nth < vecs; i += 4 * nth) {
      uint4 t0 = src[i], t1 = src[i + nth], t2 = src[i + 2 * nth], t3 = src[i + 3 * nth];
      dst[i] = t0; dst[i + nth] = t1; dst[i + 2 * nth] = t2; dst[i + 3 * nth] = t3;
    }
    for (; i < vecs; i += nth) dst[i] = src[i];
    return;
  }
  // strided segments: the matrix is [rows][pitch_vecs]; a warp covers `seg` vectors of `32 / seg` consecutive rows
  const int seg = mode == 2 ? 4 : 16;             // 16-byte vectors per segment (64 B or 256 B)
  const int rows_per_instr = 32 / seg;
  const int lane = threadIdx.x & 31;
  const long long warp = tid >> 5, nwarps = nth >> 5;
  const long long rows = vecs / pitch_vecs;
  const long long col_groups = pitch_vecs / seg;
  const long long units = (rows / rows_per_instr) * col_groups;
  for (long long u = warp; u < units; u += nwarps) {
    const long long rg = u / col_groups, cg = u % col_groups;
    const long long r = rg * rows_per_instr + lane / seg;
    const long long idx = r * pitch_vecs + cg * seg + lane % seg;
    dst[idx] = src[idx];
  }
}

}  // namespace ofb

// Copies `bytes` (multiple of 16) between this rank's arena (offset local_off) and the arena of `peer` (offset peer_off).
OFB_API int ofb_comm_p2p_bandwidth(const OfbCommCtx* ctx, int peer, int mode, long long local_off, long long peer_off,
                                   long long bytes, long long pitch_bytes, int ctas, void* stream) {
  using namespace ofb;
  if (peer < 0 || peer >= ctx->n) return fail("p2p_bandwidth: bad peer");
  if (bytes % 16 || pitch_bytes % 256 || mode < 0 || mode > 3) return fail("p2p_bandwidth: bad arguments");
  auto* local = reinterpret_cast<unsigned char*>(ctx->arena[ctx->rank]) + local_off;
  auto* remote = reinterpret_cast<unsigned char*>(ctx->arena[peer]) + peer_off;
  const uint4* src = reinterpret_cast<const uint4*>(mode == 0 ? remote : local);
  uint4* dst = reinterpret_cast<uint4*>(mode == 0 ? local : remote);
  p2p_bandwidth_kernel<<<ctas, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(src, dst, bytes / 16, mode,
                                                                               pitch_bytes > 0 ? pitch_bytes / 16 : 512);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
