// All-reduce through the NVSwitch's in-fabric reduction (NVLS): `multimem.ld_reduce` reads one address of a multicast
// mapping and gets the SUM of that address over every GPU of the group, formed inside the switch; `multimem.st` writes
// one value to all of them. An all-reduce of `count` elements therefore moves count/n elements in and count/n out per
// GPU (each rank reduces and re-broadcasts one slice), half the traffic of the two-shot P2P form in symm.cu and one
// pass instead of n reads per element.
//
// The buffer is a symmetric allocation bound to a multicast object (created by the caller: comm/symmetric.py takes it
// from torch's symmetric memory, which owns the cuMulticast* plumbing); `mc` is the multicast address of it, `local`
// this rank's own unicast address. Cross-rank ordering uses the same signal-block barrier as the P2P collectives
// (plain flags in the arena, bounded waits). Partial sums are accumulated in fp32 (`.acc::f32` for bf16).
//
// The reference has no counterpart: its all-reduce is one ncclAllReduce (oneflow/user/kernels/collective_communication/
// cuda/cuda_all_reduce.cpp); NCCL's own NVLS algorithm is the library-side equivalent.
#include "../common/host_utils.h"
#include "comm_common.cuh"
#include "ofb_comm.h"

namespace ofb {

struct McCtx {
  int rank, n;
  SignalBlock* sig[kMaxPeers];
  int* status;
};

// same protocol as grid_peer_barrier of symm.cu (kept here so that this file stands alone)
__device__ bool mc_grid_peer_barrier(const McCtx& c, unsigned int epoch, int slot) {
  __shared__ int ok_s;
  __syncthreads();
  if (threadIdx.x == 0) {
    ok_s = 1;
    SignalBlock* me = c.sig[c.rank];
    __threadfence_system();
    const unsigned int arrived = atomicAdd(&me->local_cnt[slot], 1u) + 1u;
    const unsigned int target = epoch * gridDim.x;
    if (arrived == target) {
      for (int p = 0; p < c.n; ++p) st_release_sys(&c.sig[p]->barrier[c.rank], epoch);
      bool ok = true;
      for (int p = 0; p < c.n && ok; ++p) ok = wait_flag_ge(&me->barrier[p], epoch, c.status, 900 + p);
      __threadfence_system();
      atomicExch(&me->local_cnt[slot + 1], ok ? epoch : 0x7fffffffu);
      if (!ok) ok_s = 0;
    } else {
      if (!wait_local_ge(&me->local_cnt[slot + 1], epoch, c.status, 920)) ok_s = 0;
      if (ld_acquire_gpu(&me->local_cnt[slot + 1]) == 0x7fffffffu) ok_s = 0;
    }
    __threadfence_system();
  }
  __syncthreads();
  return ok_s != 0;
}

__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const void* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_b32x4(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(mc_addr), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// In place: after the call every rank's buffer holds scale * sum over ranks. vecs = number of 16-byte vectors, a multiple
// of n (the host pads). dtype 0 = fp32, 1 = bf16.
__global__ void __launch_bounds__(512) multimem_all_reduce_kernel(McCtx c, unsigned char* mc, long long vecs, int dtype, float scale,
                                                                 unsigned int epoch, int slot) {
  // every rank's input is in its buffer
  if (!mc_grid_peer_barrier(c, 2 * epoch - 1, slot)) return;
  const long long slice = vecs / c.n;
  const long long base = slice * c.rank;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  for (long long i = tid; i < slice; i += nth) {
    unsigned char* addr = mc + (base + i) * 16;
    uint4 out;
    if (dtype == 1) {
      uint4 v = multimem_ld_reduce_bf16x8(addr);
      if (scale != 1.f) {
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(w[j]);
          w[j] = pack_bf16x2(f.x * scale, f.y * scale);
        }
        v = make_uint4(w[0], w[1], w[2], w[3]);
      }
      out = v;
    } else {
      float4 v = multimem_ld_reduce_f32x4(addr);
      out = make_uint4(__float_as_uint(v.x * scale), __float_as_uint(v.y * scale), __float_as_uint(v.z * scale), __float_as_uint(v.w * scale));
    }
    multimem_st_b32x4(addr, out);
  }
  // the reduced slices of all ranks have landed everywhere
  mc_grid_peer_barrier(c, 2 * epoch, slot);
}

}  // namespace ofb

// ctx: the P2P arena whose signal blocks carry the barrier; mc: multicast address of the (torch symmetric-memory) buffer.
OFB_API int ofb_comm_multimem_all_reduce(const OfbCommCtx* ctx, void* mc, long long count, int dtype, float scale, unsigned int epoch,
                                         int slot, int ctas, void* stream) {
  using namespace ofb;
  if (!mc) return fail("multimem_all_reduce: no multicast address (NVLS is not available for this group)");
  const int esz = dtype == 1 ? 2 : 4;
  if (dtype != 0 && dtype != 1) return fail("multimem_all_reduce: dtype must be fp32 (0) or bf16 (1)");
  const long long bytes = count * esz;
  if (bytes % (16ll * ctx->n)) return fail("multimem_all_reduce: byte size must be a multiple of 16 * group size");
  int dev = 0, sms = 0;
  OFB_CUDA_OK(cudaGetDevice(&dev));
  OFB_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (ctas <= 0 || ctas > sms) ctas = sms;      // the grid barrier needs every CTA resident
  McCtx c;
  c.rank = ctx->rank; c.n = ctx->n; c.status = device_status_ptr();
  for (int i = 0; i < kMaxPeers; ++i) c.sig[i] = reinterpret_cast<SignalBlock*>(ctx->signals[i]);
  multimem_all_reduce_kernel<<<ctas, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(c, reinterpret_cast<unsigned char*>(mc), bytes / 16,
                                                                                     dtype, scale, epoch, slot);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
