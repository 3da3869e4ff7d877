// Set-associative LRU cache of embedding rows in device memory: the device tier in front of the host-memory and SSD
// stores of OneEmbedding (what the reference builds in oneflow/core/embedding/lru_cache.cu:309-470 and uses from
// cached_key_value_store.cu: Get -> misses go to the next tier -> Put, evicted rows are written back).
//
// Geometry: `n_sets` sets of 32 ways; a key lives in set mix64(key) % n_sets. One warp serves one key at a time, lane =
// way: a lookup is one coalesced 256-byte read of the set's keys plus a ballot. Every way carries the tick of its last
// use (0 = empty); the least recently used way of a full set is the lane holding the smallest tick (warp min-reduction).
// A `put` takes the set's spin lock (one word per set, bounded spin) because several warps may insert into one set;
// a `get` does not lock: gets and puts are different launches on one stream, and concurrent gets only race on ticks.
//
//   ofb_lru_get   keys -> rows of the hits (copied to out[i]), and the list of misses (index into the batch + key)
//   ofb_lru_put   keys (unique within the call) + rows -> cache; rows pushed out come back as (key, row) pairs
//   ofb_lru_dump  every resident (key, row): snapshots and flushes
//
// Rows are fp32 lines of `line` floats (embedding + optimizer state), `line` a multiple of 4.
#include <cuda_runtime.h>

#include "../common/host_utils.h"
#include "../common/ptx.cuh"
#include "ofb_kernels.h"

namespace ofb {

constexpr int kLruWays = 32;

struct LruCache {
  long long* keys;        // [n_sets][32]
  unsigned int* ticks;    // [n_sets][32], 0 = empty way
  float* lines;           // [n_sets][32][line]
  unsigned int* locks;    // [n_sets]
  long long n_sets;
  int line;
};

__device__ __forceinline__ unsigned long long lru_mix64(unsigned long long k) {
  k ^= k >> 30; k *= 0xBF58476D1CE4E5B9ull;
  k ^= k >> 27; k *= 0x94D049BB133111EBull;
  return k ^ (k >> 31);
}

__device__ __forceinline__ void lru_copy_line(float* dst, const float* src, int line, int lane) {
  const float4* s = reinterpret_cast<const float4*>(src);
  float4* d = reinterpret_cast<float4*>(dst);
  for (int q = lane; q < line / 4; q += 32) d[q] = s[q];
}

// Warp-wide lock of one set. Returns false (and records the status) when the spin limit runs out.
__device__ __forceinline__ bool lru_lock(unsigned int* lock, int lane, int* status) {
  int ok = 1;
  if (lane == 0) {
    unsigned int spins = 0;
    while (atomicCAS(lock, 0u, 1u) != 0u) {
      if (++spins > (1u << 22)) {
        if (status && atomicCAS(status, 0, (int)kStatusPeerTimeout) == 0) status[1] = 8100;
        ok = 0;
        break;
      }
      __nanosleep(32);
    }
    __threadfence();
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void lru_unlock(unsigned int* lock, int lane) {
  __syncwarp();
  if (lane == 0) {
    __threadfence();
    atomicExch(lock, 0u);
  }
}

__global__ void __launch_bounds__(256) lru_get_kernel(LruCache c, const long long* __restrict__ keys, long long n, float* __restrict__ out,
                                                      unsigned int tick, int* __restrict__ n_miss, int* __restrict__ miss_index,
                                                      long long* __restrict__ miss_keys, unsigned char* __restrict__ hit_mask) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i = warp; i < n; i += nwarps) {
    const long long key = keys[i];
    const long long set = static_cast<long long>(lru_mix64(static_cast<unsigned long long>(key)) % static_cast<unsigned long long>(c.n_sets));
    const long long base = set * kLruWays;
    const bool mine = c.ticks[base + lane] != 0u && c.keys[base + lane] == key;
    const unsigned int hit = __ballot_sync(0xffffffffu, mine);
    if (hit) {
      const int way = __ffs(hit) - 1;
      if (lane == way) c.ticks[base + way] = tick;
      if (out) lru_copy_line(out + i * c.line, c.lines + (base + way) * c.line, c.line, lane);
      if (hit_mask && lane == 0) hit_mask[i] = 1;
    } else if (lane == 0) {
      const int m = atomicAdd(n_miss, 1);
      miss_index[m] = static_cast<int>(i);
      miss_keys[m] = key;
      if (hit_mask) hit_mask[i] = 0;
    }
  }
}

__global__ void __launch_bounds__(256) lru_put_kernel(LruCache c, const long long* __restrict__ keys, const float* __restrict__ rows,
                                                      long long n, unsigned int tick, int* __restrict__ n_evicted,
                                                      long long* __restrict__ evicted_keys, float* __restrict__ evicted_rows, int* status) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i = warp; i < n; i += nwarps) {
    const long long key = keys[i];
    const long long set = static_cast<long long>(lru_mix64(static_cast<unsigned long long>(key)) % static_cast<unsigned long long>(c.n_sets));
    const long long base = set * kLruWays;
    if (!lru_lock(c.locks + set, lane, status)) continue;
    // another SM may have changed this set under the lock a moment ago: read it through L2, not a stale L1 line
    const unsigned int t = __ldcg(c.ticks + base + lane);
    const bool mine = t != 0u && __ldcg(c.keys + base + lane) == key;
    const unsigned int hit = __ballot_sync(0xffffffffu, mine);
    int way;
    if (hit) {
      way = __ffs(hit) - 1;
    } else {
      const unsigned int empty = __ballot_sync(0xffffffffu, t == 0u);
      if (empty) {
        way = __ffs(empty) - 1;
      } else {
        // least recently used way: smallest tick, ties to the lowest way
        unsigned long long best = (static_cast<unsigned long long>(t) << 5) | static_cast<unsigned int>(lane);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
          best = other < best ? other : best;
        }
        way = static_cast<int>(best & 31u);
        int slot = 0;
        if (lane == 0) slot = atomicAdd(n_evicted, 1);
        slot = __shfl_sync(0xffffffffu, slot, 0);
        if (lane == 0) evicted_keys[slot] = __ldcg(c.keys + base + way);
        {
          const float4* sv = reinterpret_cast<const float4*>(c.lines + (base + way) * c.line);
          float4* dv = reinterpret_cast<float4*>(evicted_rows + static_cast<long long>(slot) * c.line);
          for (int q = lane; q < c.line / 4; q += 32) dv[q] = __ldcg(sv + q);
        }
        __syncwarp();
      }
    }
    lru_copy_line(c.lines + (base + way) * c.line, rows + i * c.line, c.line, lane);
    if (lane == way) {
      c.keys[base + way] = key;
      c.ticks[base + way] = tick;
    }
    lru_unlock(c.locks + set, lane);
  }
}

__global__ void __launch_bounds__(256) lru_dump_kernel(LruCache c, int* __restrict__ n_out, long long* __restrict__ keys_out,
                                                       float* __restrict__ rows_out, long long cap) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long set = warp; set < c.n_sets; set += nwarps) {
    const long long base = set * kLruWays;
    const unsigned int valid = __ballot_sync(0xffffffffu, c.ticks[base + lane] != 0u);
    if (!valid) continue;
    int start = 0;
    if (lane == 0) start = atomicAdd(n_out, __popc(valid));
    start = __shfl_sync(0xffffffffu, start, 0);
    unsigned int rest = valid;
    int k = 0;
    while (rest) {
      const int way = __ffs(rest) - 1;
      rest &= rest - 1;
      const long long slot = start + k++;
      if (slot < cap) {
        if (lane == 0) keys_out[slot] = c.keys[base + way];
        if (rows_out) lru_copy_line(rows_out + slot * c.line, c.lines + (base + way) * c.line, c.line, lane);
      }
    }
  }
}

static int lru_grid(long long n) {
  long long blocks = (n * 32 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return blocks < 1 ? 1 : static_cast<int>(blocks);
}

}  // namespace ofb

using namespace ofb;

static int lru_check(const OfbLruCache* c) {
  if (!c || !c->keys || !c->ticks || !c->lines || !c->locks) return fail("lru cache: null storage");
  if (c->n_sets <= 0 || c->line <= 0 || c->line % 4) return fail("lru cache: n_sets must be positive and line a positive multiple of 4");
  return 0;
}
static LruCache to_dev(const OfbLruCache* c) {
  LruCache d;
  d.keys = reinterpret_cast<long long*>(c->keys); d.ticks = reinterpret_cast<unsigned int*>(c->ticks);
  d.lines = reinterpret_cast<float*>(c->lines); d.locks = reinterpret_cast<unsigned int*>(c->locks);
  d.n_sets = c->n_sets; d.line = c->line;
  return d;
}

// out: [n, line] or null (test only). n_miss: device int, zeroed by the caller. miss_index / miss_keys: capacity n.
OFB_API int ofb_lru_get(const OfbLruCache* c, const long long* keys, long long n, float* out, unsigned int tick, int* n_miss,
                        int* miss_index, long long* miss_keys, unsigned char* hit_mask, void* stream) {
  if (lru_check(c)) return -1;
  if (n <= 0) return 0;
  if (tick == 0) return fail("lru cache: tick 0 marks an empty way");
  lru_get_kernel<<<lru_grid(n), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(to_dev(c), keys, n, out, tick, n_miss, miss_index,
                                                                                  miss_keys, hit_mask);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// keys must be unique within the call. n_evicted: device int, zeroed by the caller; evicted_*: capacity n rows.
OFB_API int ofb_lru_put(const OfbLruCache* c, const long long* keys, const float* rows, long long n, unsigned int tick, int* n_evicted,
                        long long* evicted_keys, float* evicted_rows, void* stream) {
  if (lru_check(c)) return -1;
  if (n <= 0) return 0;
  if (tick == 0) return fail("lru cache: tick 0 marks an empty way");
  lru_put_kernel<<<lru_grid(n), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(to_dev(c), keys, rows, n, tick, n_evicted, evicted_keys,
                                                                                  evicted_rows, device_status_ptr());
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// n_out: device int, zeroed by the caller. Writes at most cap entries; *n_out is the number of resident rows.
OFB_API int ofb_lru_dump(const OfbLruCache* c, int* n_out, long long* keys_out, float* rows_out, long long cap, void* stream) {
  if (lru_check(c)) return -1;
  lru_dump_kernel<<<lru_grid(c->n_sets), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(to_dev(c), n_out, keys_out, rows_out, cap);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
