// Self-test of the bounded waits that every kernel of this library uses (mbarrier waits inside a CTA, waits on
// flags written by a peer GPU, waits on counters advanced by other CTAs): a one-block kernel waits, with a caller
// chosen limit of a few milliseconds, for an event that never happens -- an mbarrier nobody arrives on, a flag word
// nobody writes -- and must come back by itself with the matching status code, leaving the context usable.
// This is how failure detection of the device-side waits is tested: nothing faults, traps or hangs; the wait
// simply runs out (reference behaviour being replaced: the reference's p2p kernels spin without a limit,
// oneflow/user/kernels/one_embedding_embedding_shuffle_p2p_kernel.cu).
#include "../common/host_utils.h"
#include "comm_common.cuh"
#include "ofb_comm.h"

namespace ofb {

__device__ unsigned int g_probe_flag[4];  // stays zero: nothing ever writes it

__global__ void wait_probe_kernel(int kind, unsigned long long timeout_ns, int* status, unsigned int* elapsed_us) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  const unsigned long long t0 = global_timer_ns();
  bool ok = true;
  if (kind == 0) {
    // every thread polls; the first one whose limit runs out raises the CTA's abort flag, the others follow
    ok = mbar_wait(&bar, 0, &abort_flag, timeout_ns);
    if (!ok && threadIdx.x == 0 && status) {
      if (atomicCAS(status, 0, (int)kStatusMbarTimeout) == 0) status[1] = 7001;
    }
  } else if (threadIdx.x == 0) {
    ok = kind == 1 ? wait_flag_ge(&g_probe_flag[0], 1u, status, 7002, timeout_ns)
                   : wait_local_ge(&g_probe_flag[1], 1u, status, 7003, timeout_ns);
  }
  __syncthreads();
  if (threadIdx.x == 0 && elapsed_us) *elapsed_us = static_cast<unsigned int>((global_timer_ns() - t0) / 1000ull);
}

}  // namespace ofb

// kind 0: mbarrier wait, 1: peer-flag wait (system scope), 2: local-counter wait (gpu scope). The wait gives up after
// timeout_ns (clamped to [1 ms, 1 s]) and records kStatusMbarTimeout / kStatusPeerTimeout in the device status block
// (read it with ofb_read_status). elapsed_us_out (device pointer, optional) receives how long the kernel waited.
OFB_API int ofb_wait_probe(int kind, long long timeout_ns, unsigned int* elapsed_us_out, void* stream) {
  using namespace ofb;
  if (kind < 0 || kind > 2) return fail("wait_probe: kind must be 0, 1 or 2");
  if (timeout_ns < 1000000ll) timeout_ns = 1000000ll;
  if (timeout_ns > 1000000000ll) timeout_ns = 1000000000ll;
  wait_probe_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(kind, static_cast<unsigned long long>(timeout_ns),
                                                                          device_status_ptr(), elapsed_us_out);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
