// Device-side building blocks for kernels that talk to peer GPUs over NVLink / NVSwitch through
// peer-mapped ("symmetric") buffers: release/acquire flag accesses at system scope and waits that
// give up after a wall-clock limit, recording a status code instead of hanging.
#pragma once
#include "../common/ptx.cuh"

namespace ofb {

constexpr int kMaxPeers = 8;

#ifndef OFB_PEER_TIMEOUT_NS
#define OFB_PEER_TIMEOUT_NS 10000000000ull
#endif

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_relaxed_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Waits until *flag >= target (wrap-safe signed comparison). Returns false after the time limit,
// after writing kStatusPeerTimeout to `status` (first failure wins) with `detail` beside it.
__device__ __forceinline__ bool wait_flag_ge(const unsigned int* flag, unsigned int target, int* status, int detail,
                                             unsigned long long timeout_ns = OFB_PEER_TIMEOUT_NS) {
  if (static_cast<int>(ld_acquire_sys(flag) - target) >= 0) return true;
  const unsigned long long t0 = global_timer_ns();
  unsigned int spins = 0;
  while (static_cast<int>(ld_acquire_sys(flag) - target) < 0) {
    if ((++spins & 0xff) == 0) {
      if (global_timer_ns() - t0 > timeout_ns) {
        if (status) {
          if (atomicCAS(status, 0, (int)kStatusPeerTimeout) == 0) status[1] = detail;
        }
        return false;
      }
      __nanosleep(64);
    }
  }
  return true;
}

// Same, for a counter that lives in this GPU's own memory and is advanced by other CTAs of this kernel.
__device__ __forceinline__ bool wait_local_ge(const unsigned int* flag, unsigned int target, int* status, int detail,
                                              unsigned long long timeout_ns = OFB_PEER_TIMEOUT_NS) {
  if (static_cast<int>(ld_acquire_gpu(flag) - target) >= 0) return true;
  const unsigned long long t0 = global_timer_ns();
  unsigned int spins = 0;
  while (static_cast<int>(ld_acquire_gpu(flag) - target) < 0) {
    if ((++spins & 0xff) == 0) {
      if (global_timer_ns() - t0 > timeout_ns) {
        if (status) {
          if (atomicCAS(status, 0, (int)kStatusPeerTimeout) == 0) status[1] = detail;
        }
        return false;
      }
      __nanosleep(64);
    }
  }
  return true;
}

// Per-rank signal block living in symmetric memory (every rank maps every peer's block).
// All counters are monotonic "epochs": nobody ever resets them, so a late reader never misses a value.
struct SignalBlock {
  unsigned int barrier[kMaxPeers];       // barrier[r] = last barrier epoch rank r announced to me
  unsigned int rs_consumed[kMaxPeers];   // rs_consumed[r] = last gemm_rs epoch whose partials rank r finished reducing
  unsigned int ag_ready[kMaxPeers];      // ag_ready[r] = last all-gather epoch for which rank r's shard is readable
  unsigned int ag_pulled[kMaxPeers];     // ag_pulled[r] = last all-gather epoch whose shard rank r finished pulling from me
  unsigned int local_cnt[32];            // scratch counters used only by this GPU's own CTAs
  unsigned int emb_ids[kMaxPeers];       // emb_ids[r] = last embedding step whose unique ids rank r stored into my key buffer
  unsigned int emb_rows[kMaxPeers];      // emb_rows[r] = last embedding step whose rows owner r stored into my row buffer
  unsigned int emb_grads[kMaxPeers];     // emb_grads[r] = last embedding step whose gradients rank r stored into my buffer
};

}  // namespace ofb
