// OneEmbedding on device: the id shuffle, the table lookup fused with the embedding shuffle, and the
// gradient shuffle fused with the sparse row update, all over peer-mapped memory (no NCCL, no host sync).
//
// One training step of a model-parallel embedding with N ranks (every rank owns the keys whose hash maps to it):
//
//   forward  (requester)  partition : dedupe this rank's ids in a per-step hash table, number the unique keys per
//                                     owner, and store every unique key straight into the owner's receive buffer
//                         publish   : translate every id position to (owner, index), push the per-owner counts,
//                                     raise the "ids ready" flag at every owner
//            (owner)      resolve   : wait for the flags, find-or-insert every received key in the persistent
//                                     table (new rows are initialised in place from a counter-based generator,
//                                     so a row's initial value depends only on its key and the seed)
//                         serve     : read each row (fp32), convert, and store it into the requester's receive
//                                     buffer; raise "rows ready" at every requester
//            (requester)  gather    : wait for the flags, expand unique rows to [ids, dim] by the inverse index
//   backward (requester)  reduce    : segment-sum the output gradient per unique key (fp32 vector atomics in L2)
//                         push      : convert each summed row and store it into the owner's gradient buffer,
//                                     clear the sum, raise "grads ready" at every owner
//            (owner)      combine   : wait for the flags, add the rows of all requesters per touched table row
//                         update    : apply SGD / momentum / Adam / Adagrad / FTRL to each touched row once
//
// All capacities are worst case (every id of a rank unique and owned by one peer), so no count ever has to
// reach the host. Flags are monotonic step numbers; every wait is bounded and reports through the status
// block. Buffer reuse across steps is safe without extra flags: a requester cannot publish step t+1 before it
// gathered step t, which needs every owner's serve(t), and the counts are double-buffered by step parity
// because the owner still reads them in combine(t) while a fast requester publishes step t+1.
//
// Reference counterparts: oneflow/user/kernels/one_embedding_kernels.cu (lookup / put),
// one_embedding_id_shuffle_p2p_kernel.cu, one_embedding_embedding_shuffle_p2p_kernel.cu,
// one_embedding_embedding_gradient_shuffle_p2p_kernel.cu, one_embedding_update_kernels.cu:60-110,
// oneflow/core/embedding/hash_functions.cuh, full_cache.cu.
#include <cuda_fp16.h>

#include "../common/host_utils.h"
#include "comm_common.cuh"
#include "ofb_comm.h"

namespace ofb {

constexpr unsigned long long kEmptyKey = ~0ull;
constexpr int kOwnerShift = 28;
constexpr unsigned int kIndexMask = (1u << kOwnerShift) - 1u;

struct EmbCtx {
  int rank, n;
  unsigned char* arena[kMaxPeers];
  SignalBlock* sig[kMaxPeers];
  int* status;
};

static EmbCtx to_emb_ctx(const OfbCommCtx* c) {
  EmbCtx x;
  x.rank = c->rank;
  x.n = c->n;
  for (int i = 0; i < kMaxPeers; ++i) {
    x.arena[i] = reinterpret_cast<unsigned char*>(c->arena[i]);
    x.sig[i] = reinterpret_cast<SignalBlock*>(c->signals[i]);
  }
  x.status = device_status_ptr();
  return x;
}

// splitmix64 finaliser on a signed value with arithmetic shifts: bit-identical to the int64 tensor version
// that the host side uses to compute owners.
__device__ __forceinline__ long long mix64s(long long k) {
  k = k ^ (k >> 30);
  k = k * static_cast<long long>(0xBF58476D1CE4E5B9ull);
  k = k ^ (k >> 27);
  k = k * static_cast<long long>(0x94D049BB133111EBull);
  return k ^ (k >> 31);
}
__device__ __forceinline__ int owner_of(long long key, int world) {
  return static_cast<int>((mix64s(key) & 0x7FFFFFFFll) % world);
}
// table position: a second, independent mix (the owner hash fixes some bits of the first one)
__device__ __forceinline__ unsigned long long slot_hash(long long key) {
  return static_cast<unsigned long long>(mix64s(key + static_cast<long long>(0x9E3779B97F4A7C15ull))) >> 17;
}
__device__ __forceinline__ float unit_uniform(unsigned long long key, unsigned int c, unsigned long long seed) {
  const unsigned long long h =
      static_cast<unsigned long long>(mix64s(static_cast<long long>(key * 0x9E3779B97F4A7C15ull + c * 0xD6E8FEB86659FD93ull + seed)));
  // bits 8..31: the arithmetic shifts of the signed mix leave the top bit constant
  return (static_cast<float>((h >> 8) & 0xFFFFFFull) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
}

__device__ __forceinline__ void record(int* status, int code, int detail) {
  if (status && atomicCAS(status, 0, code) == 0) status[1] = detail;
}

// --------------------------------------------------------------------------------------------- requester: ids
// Lanes of `mask` (all of them call this) that hold the same `bucket` share one atomicAdd on counter[bucket]:
// returns each lane's own index. Same-address atomics from every thread would serialise in L2.
__device__ __forceinline__ int grouped_count(unsigned int mask, int bucket, int* counters) {
  const unsigned int lane = threadIdx.x & 31;
  const unsigned int peers = __match_any_sync(mask, bucket);
  const int leader = __ffs(peers) - 1;
  int base = 0;
  if (static_cast<int>(lane) == leader) base = atomicAdd(&counters[bucket], __popc(peers));
  base = __shfl_sync(peers, base, leader);
  return base + __popc(peers & ((1u << lane) - 1u));
}

__global__ void __launch_bounds__(256)
emb_partition_kernel(const long long* __restrict__ ids, const int* __restrict__ tids, long long n, int num_tables, int columns,
                     unsigned long long* dkeys, unsigned int* dval, long long dmask, int* cnt, unsigned int* inv, EmbCtx c,
                     long long keys_off, long long cap) {
  for (long long base = blockIdx.x * (long long)blockDim.x; base < n; base += (long long)gridDim.x * blockDim.x) {
    const long long p = base + threadIdx.x;
    const bool active = p < n;
    unsigned int found = 0xFFFFFFFFu;
    bool first = false;
    long long key = 0;
    if (active) {
      const int t = tids ? tids[p] : static_cast<int>(p % columns) % num_tables;
      key = ids[p] * num_tables + t;
      const unsigned long long ukey = static_cast<unsigned long long>(key);
      long long s = static_cast<long long>(slot_hash(key)) & dmask;
      for (long long probe = 0; probe <= dmask; ++probe) {
        // plain read first: repeated ids (the head of a Zipf distribution) never reach the atomic
        unsigned long long cur = *reinterpret_cast<volatile unsigned long long*>(&dkeys[s]);
        if (cur == kEmptyKey) {
          cur = atomicCAS(&dkeys[s], kEmptyKey, ukey);
          if (cur == kEmptyKey) {
            first = true;
            cur = ukey;
          }
        }
        if (cur == ukey) {
          found = static_cast<unsigned int>(s);
          break;
        }
        s = (s + 1) & dmask;
      }
      if (found == 0xFFFFFFFFu) record(c.status, kStatusHashTableFull, 1);
    }
    const unsigned int fmask = __ballot_sync(0xffffffffu, first);
    if (first) {
      const int owner = owner_of(key, c.n);
      const int idx = grouped_count(fmask, owner, cnt);
      dval[found] = (static_cast<unsigned int>(owner) << kOwnerShift) | static_cast<unsigned int>(idx);
      if (idx < cap)
        reinterpret_cast<unsigned long long*>(c.arena[owner] + keys_off)[c.rank * cap + idx] = static_cast<unsigned long long>(key);
    }
    if (active) inv[p] = found;
  }
}

__global__ void __launch_bounds__(256)
emb_publish_kernel(long long n, const unsigned int* __restrict__ dval, const int* __restrict__ cnt, unsigned int* inv, EmbCtx c,
                   long long cnt_off, unsigned int epoch) {
  if (blockIdx.x == 0 && threadIdx.x < c.n) {
    const int r = threadIdx.x;
    int* peer_cnt = reinterpret_cast<int*>(c.arena[r] + cnt_off) + (epoch & 1u) * kMaxPeers;
    peer_cnt[c.rank] = cnt[r];
    __threadfence_system();
    st_release_sys(&c.sig[r]->emb_ids[c.rank], epoch);
  }
  for (long long p = blockIdx.x * (long long)blockDim.x + threadIdx.x; p < n; p += (long long)gridDim.x * blockDim.x) {
    const unsigned int s = inv[p];
    inv[p] = s == 0xFFFFFFFFu ? s : dval[s];
  }
}

// Waits (thread r for peer r) until every peer's flag reached `epoch`, then loads the per-source counts into
// shared memory as an exclusive prefix. Returns false for the whole block when a wait ran out.
__device__ bool wait_and_prefix(const unsigned int* flags, const int* counts, int n, long long cap, unsigned int epoch, int* status,
                                int detail, long long* pre /* [kMaxPeers + 1] shared */) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < n) {
    if (!wait_flag_ge(&flags[threadIdx.x], epoch, status, detail + threadIdx.x)) ok_s = 0;
  }
  __syncthreads();
  if (threadIdx.x == 0 && ok_s) {
    long long acc = 0;
    for (int r = 0; r < n; ++r) {
      pre[r] = acc;
      long long v = counts ? reinterpret_cast<const volatile int*>(counts)[r] : 0;
      if (v < 0) v = 0;
      if (v > cap) v = cap;
      acc += v;
    }
    pre[n] = acc;
  }
  __syncthreads();
  return ok_s != 0;
}

__device__ __forceinline__ void locate(const long long* pre, int n, long long w, int* r, long long* idx) {
  int q = 0;
  while (q + 1 < n && w >= pre[q + 1]) ++q;
  *r = q;
  *idx = w - pre[q];
}

// Raises `flag[c.rank] = epoch` at every peer once all CTAs of the grid have finished their stores.
__device__ void signal_when_grid_done(const EmbCtx& c, int* done_cnt, unsigned int epoch, int which) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int old = atomicAdd(done_cnt, 1);
    if (old == static_cast<int>(gridDim.x) - 1) {
      *done_cnt = 0;
      __threadfence_system();
      for (int r = 0; r < c.n; ++r) {
        unsigned int* f = which == 0 ? &c.sig[r]->emb_rows[c.rank] : &c.sig[r]->emb_grads[c.rank];
        st_release_sys(f, epoch);
      }
    }
  }
}

// --------------------------------------------------------------------------------------------- owner: lookup
__global__ void __launch_bounds__(256)
emb_resolve_kernel(OfbEmbStore st, EmbCtx c, long long keys_off, long long cnt_off, long long cap, int* slot_tmp, int* n_uo,
                   unsigned int epoch, int insert) {
  __shared__ long long pre[kMaxPeers + 1];
  const int* counts = reinterpret_cast<const int*>(c.arena[c.rank] + cnt_off) + (epoch & 1u) * kMaxPeers;
  if (!wait_and_prefix(c.sig[c.rank]->emb_ids, counts, c.n, cap, epoch, c.status, 200, pre)) return;
  const unsigned long long* keys = reinterpret_cast<const unsigned long long*>(c.arena[c.rank] + keys_off);
  const long long tmask = st.tcap - 1;
  const int lane = threadIdx.x & 31;
  const long long total = pre[c.n];
  // one key per thread for the probe (32 independent probes per warp in flight), then the warp fills new rows together
  for (long long base = blockIdx.x * (long long)blockDim.x; base < total; base += (long long)gridDim.x * blockDim.x) {
    const long long w = base + threadIdx.x;
    const bool active = w < total;
    int s_found = -1;
    bool is_new = false;
    unsigned long long ukey = 0;
    long long where = 0;
    if (active) {
      int r;
      long long idx;
      locate(pre, c.n, w, &r, &idx);
      where = r * cap + idx;
      ukey = keys[where];
      long long s = static_cast<long long>(slot_hash(static_cast<long long>(ukey))) & tmask;
      for (long long probe = 0; probe <= tmask; ++probe) {
        unsigned long long cur = *reinterpret_cast<volatile unsigned long long*>(&st.slots[s].key);
        if (cur == kEmptyKey) {
          if (!insert) break;  // absent and not inserting: the row reads as zeros
          cur = atomicCAS(&st.slots[s].key, kEmptyKey, ukey);
          if (cur == kEmptyKey) {
            is_new = true;
            cur = ukey;
          }
        }
        if (cur == ukey) {
          s_found = static_cast<int>(s);
          break;
        }
        s = (s + 1) & tmask;
      }
      if (s_found < 0 && insert) record(c.status, kStatusHashTableFull, 3);
    }
    // rows for the new keys: one atomic per warp
    const unsigned int nmask = __ballot_sync(0xffffffffu, is_new);
    int new_row = -1;
    if (is_new) {
      new_row = grouped_count(nmask, 0, st.counters);
      if (new_row < st.row_cap) {
        st.slots[s_found].row = new_row;
        st.row_key[new_row] = ukey;
      } else {
        st.slots[s_found].row = -1;
        new_row = -1;
        record(c.status, kStatusHashTableFull, 2);
      }
    }
    // number the rows touched in this step (a key can arrive from several ranks: the first stamp wins)
    const bool fresh = s_found >= 0 && atomicExch(&st.slots[s_found].stamp, epoch) != epoch;
    const unsigned int umask = __ballot_sync(0xffffffffu, fresh);
    if (fresh) st.slots[s_found].uo = grouped_count(umask, 0, n_uo);
    if (active) slot_tmp[where] = s_found;
    // initialise the new rows, one row per warp pass
    unsigned int todo = __ballot_sync(0xffffffffu, new_row >= 0);
    while (todo) {
      const int src = __ffs(todo) - 1;
      todo &= todo - 1;
      const int row_i = __shfl_sync(0xffffffffu, new_row, src);
      const unsigned long long k = __shfl_sync(0xffffffffu, ukey, src);
      const int table = static_cast<int>(k % static_cast<unsigned long long>(st.num_tables));
      const int kind = st.init_kind[table];
      const float a = st.init_a[table], b = st.init_b[table];
      float* row = st.rows + static_cast<long long>(row_i) * st.line;
      for (int col = lane; col < st.line; col += 32) {
        float v;
        if (col >= st.dim) {
          v = col < 2 * st.dim ? st.state_init : 0.f;  // first state vector (accumulator) only
        } else if (kind == 0) {  // uniform(a, b)
          v = a + (b - a) * unit_uniform(k, col, st.seed);
        } else if (kind == 1) {  // normal(mean a, std b), Box-Muller on a column pair
          const float u1 = unit_uniform(k, 2 * (col >> 1), st.seed);
          const float u2 = unit_uniform(k, 2 * (col >> 1) + 1, st.seed ^ 0x5851F42D4C957F2Dull);
          const float rad = sqrtf(-2.f * __logf(u1));
          float sn, cs;
          __sincosf(6.283185307179586f * u2, &sn, &cs);
          v = a + b * rad * ((col & 1) ? sn : cs);
        } else {  // constant a
          v = a;
        }
        row[col] = v;
      }
    }
  }
}

template <bool kHalf>
__device__ __forceinline__ uint2 pack4(float4 v) {
  uint2 o;
  if (kHalf) {
    const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
    o.x = *reinterpret_cast<const unsigned int*>(&lo);
    o.y = *reinterpret_cast<const unsigned int*>(&hi);
  } else {
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
  }
  return o;
}
template <bool kHalf>
__device__ __forceinline__ float4 unpack4(uint2 q) {
  if (kHalf) {
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&q.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&q.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
  }
  const float2 lo = unpack_bf16x2(q.x), hi = unpack_bf16x2(q.y);
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

template <bool kHalf>
__global__ void __launch_bounds__(256)
emb_serve_kernel(OfbEmbStore st, EmbCtx c, long long cnt_off, long long emb_off, long long cap, const int* __restrict__ slot_tmp,
                 int* rowidx, int* uoidx, int* u_row, int* done_cnt, unsigned int epoch) {
  __shared__ long long pre[kMaxPeers + 1];
  const int* counts = reinterpret_cast<const int*>(c.arena[c.rank] + cnt_off) + (epoch & 1u) * kMaxPeers;
  const bool ok = wait_and_prefix(c.sig[c.rank]->emb_ids, counts, c.n, cap, epoch, c.status, 210, pre);
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int D = st.dim;
  constexpr int UNR = 4;  // rows per warp and pass: their dependent index loads and row loads overlap
  const long long total = ok ? pre[c.n] : 0;
  for (long long w0 = warp * UNR; w0 < total; w0 += nwarps * UNR) {
    int rr[UNR], row[UNR], sl[UNR];
    long long where[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      rr[u] = 0;
      where[u] = -1;
      sl[u] = -1;
      if (w0 + u < total) {
        long long idx;
        locate(pre, c.n, w0 + u, &rr[u], &idx);
        where[u] = rr[u] * cap + idx;
        sl[u] = slot_tmp[where[u]];
      }
    }
#pragma unroll
    int uov[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      row[u] = uov[u] = -1;
      if (sl[u] >= 0) {  // row and touch number sit side by side in the slot: one 8-byte read
        const int2 q = *reinterpret_cast<const int2*>(&st.slots[sl[u]].row);
        row[u] = q.x;
        uov[u] = q.y;
      }
    }
    if (lane < UNR) {
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        if (lane == u && where[u] >= 0) {
          const int uo = uov[u];
          rowidx[where[u]] = row[u];
          uoidx[where[u]] = uo;
          if (uo >= 0) u_row[uo] = row[u];
        }
      }
    }
    for (int q = lane; q < (D >> 2); q += 32) {
      float4 v[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row[u] >= 0) v[u] = reinterpret_cast<const float4*>(st.rows + static_cast<long long>(row[u]) * st.line)[q];
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        if (where[u] < 0) continue;
        const long long idx = where[u] - rr[u] * cap;
        uint2* dst = reinterpret_cast<uint2*>(c.arena[rr[u]] + emb_off) + (c.rank * cap + idx) * (D >> 2);
        dst[q] = pack4<kHalf>(v[u]);
      }
    }
  }
  signal_when_grid_done(c, done_cnt, epoch, 0);
}

// --------------------------------------------------------------------------------------------- requester: gather
__global__ void __launch_bounds__(256)
emb_gather_kernel(EmbCtx c, long long emb_off, long long cap, const unsigned int* __restrict__ inv, long long n, int D, uint2* out,
                  unsigned int epoch) {
  __shared__ long long pre[kMaxPeers + 1];
  if (!wait_and_prefix(c.sig[c.rank]->emb_rows, nullptr, c.n, cap, epoch, c.status, 220, pre)) return;
  const uint2* src = reinterpret_cast<const uint2*>(c.arena[c.rank] + emb_off);
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int vec = D >> 2;
  constexpr int UNR = 4;
  for (long long p0 = warp * UNR; p0 < n; p0 += nwarps * UNR) {
    long long u[UNR];
#pragma unroll
    for (int k = 0; k < UNR; ++k) {
      u[k] = -1;
      if (p0 + k < n) {
        const unsigned int v = inv[p0 + k];
        if (v != 0xFFFFFFFFu) u[k] = (long long)(v >> kOwnerShift) * cap + (v & kIndexMask);
      }
    }
    for (int q = lane; q < vec; q += 32) {
      uint2 t[UNR];
#pragma unroll
      for (int k = 0; k < UNR; ++k) t[k] = u[k] >= 0 ? src[u[k] * vec + q] : make_uint2(0u, 0u);
#pragma unroll
      for (int k = 0; k < UNR; ++k)
        if (p0 + k < n) out[(p0 + k) * vec + q] = t[k];
    }
  }
}

// --------------------------------------------------------------------------------------------- requester: gradients
template <bool kHalf>
__global__ void __launch_bounds__(256)
emb_grad_reduce_kernel(const uint2* __restrict__ grad, const unsigned int* __restrict__ inv, long long n, int D, long long cap,
                       float* gsum) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int vec = D >> 2;
  constexpr int UNR = 4;
  for (long long p0 = warp * UNR; p0 < n; p0 += nwarps * UNR) {
    long long u[UNR];
#pragma unroll
    for (int k = 0; k < UNR; ++k) {
      u[k] = -1;
      if (p0 + k < n) {
        const unsigned int v = inv[p0 + k];
        if (v != 0xFFFFFFFFu) u[k] = (long long)(v >> kOwnerShift) * cap + (v & kIndexMask);
      }
    }
    for (int q = lane; q < vec; q += 32) {
      uint2 t[UNR];
#pragma unroll
      for (int k = 0; k < UNR; ++k) t[k] = u[k] >= 0 ? grad[(p0 + k) * vec + q] : make_uint2(0u, 0u);
#pragma unroll
      for (int k = 0; k < UNR; ++k)
        if (u[k] >= 0) atomicAdd(reinterpret_cast<float4*>(gsum + u[k] * D) + q, unpack4<kHalf>(t[k]));
    }
  }
}

template <bool kHalf>
__global__ void __launch_bounds__(256)
emb_grad_push_kernel(EmbCtx c, const int* __restrict__ cnt, long long grad_off, long long cap, int D, float* gsum, int* done_cnt,
                     unsigned int epoch) {
  __shared__ long long pre[kMaxPeers + 1];
  if (threadIdx.x == 0) {
    long long acc = 0;
    for (int r = 0; r < c.n; ++r) {
      pre[r] = acc;
      long long v = cnt[r];
      acc += v > cap ? cap : v;
    }
    pre[c.n] = acc;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int vec = D >> 2;
  for (long long w = warp; w < pre[c.n]; w += nwarps) {
    int o;
    long long idx;
    locate(pre, c.n, w, &o, &idx);
    float4* src = reinterpret_cast<float4*>(gsum + (o * cap + idx) * D);
    uint2* dst = reinterpret_cast<uint2*>(c.arena[o] + grad_off) + (c.rank * cap + idx) * vec;
    for (int q = lane; q < vec; q += 32) {
      dst[q] = pack4<kHalf>(src[q]);
      src[q] = make_float4(0.f, 0.f, 0.f, 0.f);  // the sums stay zero between steps
    }
  }
  signal_when_grid_done(c, done_cnt, epoch, 1);
}

// Records the step of the update in every row the step touched (smart-decay Adam), after the update kernel has read
// the previous value.
__global__ void emb_stamp_step_kernel(OfbEmbStore st, const int* __restrict__ u_row, const int* __restrict__ n_uo, int step) {
  const int total = *n_uo;
  for (long long u = blockIdx.x * (long long)blockDim.x + threadIdx.x; u < total; u += (long long)gridDim.x * blockDim.x) {
    const int row = u_row[u];
    if (row >= 0) *reinterpret_cast<int*>(st.rows + static_cast<long long>(row) * st.line + 3 * st.dim) = step;
  }
}

// --------------------------------------------------------------------------------------------- owner: update
template <bool kHalf>
__global__ void __launch_bounds__(256)
emb_grad_combine_kernel(EmbCtx c, long long cnt_off, long long grad_off, long long cap, int D, const int* __restrict__ uoidx,
                        float* gacc, unsigned int epoch) {
  __shared__ long long pre[kMaxPeers + 1];
  const int* counts = reinterpret_cast<const int*>(c.arena[c.rank] + cnt_off) + (epoch & 1u) * kMaxPeers;
  if (!wait_and_prefix(c.sig[c.rank]->emb_grads, counts, c.n, cap, epoch, c.status, 230, pre)) return;
  const uint2* src = reinterpret_cast<const uint2*>(c.arena[c.rank] + grad_off);
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int vec = D >> 2;
  constexpr int UNR = 4;
  const long long total = pre[c.n];
  for (long long w0 = warp * UNR; w0 < total; w0 += nwarps * UNR) {
    long long where[UNR];
    int uo[UNR];
#pragma unroll
    for (int k = 0; k < UNR; ++k) {
      where[k] = -1;
      uo[k] = -1;
      if (w0 + k < total) {
        int r;
        long long idx;
        locate(pre, c.n, w0 + k, &r, &idx);
        where[k] = r * cap + idx;
        uo[k] = uoidx[where[k]];
      }
    }
    for (int q = lane; q < vec; q += 32) {
      uint2 t[UNR];
#pragma unroll
      for (int k = 0; k < UNR; ++k) t[k] = uo[k] >= 0 ? src[where[k] * vec + q] : make_uint2(0u, 0u);
#pragma unroll
      for (int k = 0; k < UNR; ++k)
        if (uo[k] >= 0) atomicAdd(reinterpret_cast<float4*>(gacc + static_cast<long long>(uo[k]) * D) + q, unpack4<kHalf>(t[k]));
    }
  }
}

// One element of the row update. Row layout: [w (D) | state 1 (D) | state 2 (D)] as far as the optimizer needs.
template <int KIND>
__device__ __forceinline__ void update_one(float& x, float g, float& s1, float& s2, const OfbEmbUpdate& h) {
  g *= h.scale;
  if (h.l2 != 0.f) g += h.l2 * x;
  if (KIND == 0) {  // sgd
    x -= h.lr * (g + h.weight_decay * x);
  } else if (KIND == 1) {  // momentum
    s1 = h.momentum * s1 + g;
    x -= h.lr * (s1 + h.weight_decay * x);
  } else if (KIND == 2) {  // adam
    s1 = h.beta1 * s1 + (1.f - h.beta1) * g;
    s2 = h.beta2 * s2 + (1.f - h.beta2) * g * g;
    x -= (h.lr / h.bias_corr1) * s1 / (sqrtf(s2) / sqrtf(h.bias_corr2) + h.eps) + h.lr * h.weight_decay * x;
  } else if (KIND == 5) {  // smart-decay adam: the caller put beta^skipped into bias_corr1/2 and the catch-up factor into lr_eff
    const float catchup = s1 * h.lr_eff;
    s1 = h.bias_corr1 * s1 + (1.f - h.beta1) * g;
    s2 = h.bias_corr2 * s2 + (1.f - h.beta2) * g * g;
    x -= h.lr * (s1 + catchup) / (sqrtf(s2) + h.eps);
  } else if (KIND == 3) {  // adagrad
    s1 += g * g;
    x -= h.lr_eff * g / (sqrtf(s1) + h.eps) + h.lr * h.weight_decay * x;
  } else {  // ftrl: s1 = accumulator, s2 = z
    const float nacc = s1 + g * g;
    const float sigma = (powf(nacc, -h.lr_power) - powf(s1, -h.lr_power)) / h.lr;
    s2 += g - sigma * x;
    s1 = nacc;
    const float denom = (h.beta + powf(nacc, -h.lr_power)) / h.lr + h.lambda2;
    x = fabsf(s2) > h.lambda1 ? -(s2 - copysignf(h.lambda1, s2)) / denom : 0.f;
  }
}

// One warp per touched row, 16 bytes per lane and access: reads the summed gradient (and clears it, so the
// accumulators stay zero between steps), the weights and the state, writes them back.
template <int KIND>
__global__ void __launch_bounds__(256)
emb_update_kernel(OfbEmbStore st, const int* __restrict__ u_row, const int* __restrict__ n_uo, float* __restrict__ gacc,
                  OfbEmbUpdate h) {
  constexpr int kStates = KIND == 0 ? 0 : (KIND == 1 || KIND == 3) ? 1 : 2;
  // KIND 5 (smart-decay Adam, reference: one_embedding_update_kernels.cu:140-186): a row also remembers the step of its
  // last update (first word after the two moments). Moments decay by beta^(steps since then), and the steps in
  // between, in which the row would have kept moving along its first moment, are caught up in one go.
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int vec = st.dim >> 2;
  const int total = *n_uo;
  constexpr int UNR = 4;  // rows per warp and pass
  for (long long u0 = warp * UNR; u0 < total; u0 += nwarps * UNR) {
    int row[UNR];
#pragma unroll
    for (int k = 0; k < UNR; ++k) row[k] = u0 + k < total ? u_row[u0 + k] : -2;
    for (int q = lane; q < vec; q += 32) {
      float4 g[UNR], x[UNR], a[UNR], b[UNR];
#pragma unroll
      for (int k = 0; k < UNR; ++k) {
        g[k] = x[k] = a[k] = b[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row[k] == -2) continue;
        g[k] = reinterpret_cast<const float4*>(gacc + (u0 + k) * st.dim)[q];
        if (row[k] < 0) continue;
        const float4* w4 = reinterpret_cast<const float4*>(st.rows + static_cast<long long>(row[k]) * st.line);
        x[k] = w4[q];
        if (kStates >= 1) a[k] = w4[vec + q];
        if (kStates >= 2) b[k] = w4[2 * vec + q];
      }
#pragma unroll
      for (int k = 0; k < UNR; ++k) {
        if (row[k] == -2) continue;
        reinterpret_cast<float4*>(gacc + (u0 + k) * st.dim)[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row[k] < 0) continue;
        OfbEmbUpdate hk = h;
        if (KIND == 5) {
          const int prev = *reinterpret_cast<const int*>(st.rows + static_cast<long long>(row[k]) * st.line + 3 * st.dim);
          const float skip = static_cast<float>(h.step - prev);
          hk.bias_corr1 = powf(h.beta1, skip);
          hk.bias_corr2 = powf(h.beta2, skip);
          hk.lr_eff = skip > 1.f ? h.beta1 * (1.f - powf(h.beta1, skip - 1.f)) / (1.f - h.beta1) : 0.f;
        }
        const OfbEmbUpdate& h = hk;
        update_one<KIND>(x[k].x, g[k].x, a[k].x, b[k].x, h);
        update_one<KIND>(x[k].y, g[k].y, a[k].y, b[k].y, h);
        update_one<KIND>(x[k].z, g[k].z, a[k].z, b[k].z, h);
        update_one<KIND>(x[k].w, g[k].w, a[k].w, b[k].w, h);
        float4* w4 = reinterpret_cast<float4*>(st.rows + static_cast<long long>(row[k]) * st.line);
        w4[q] = x[k];
        if (kStates >= 1) w4[vec + q] = a[k];
        if (kStates >= 2) w4[2 * vec + q] = b[k];
      }
    }
  }
}

// Finds (optionally inserts, without initialising) keys in the table of one rank: rows[i] = row index or -1.
__global__ void __launch_bounds__(256)
emb_find_kernel(OfbEmbStore st, const long long* __restrict__ keys, long long n, int insert, int* rows, int* status) {
  const long long tmask = st.tcap - 1;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long key = keys[i];
    const unsigned long long ukey = static_cast<unsigned long long>(key);
    long long s = static_cast<long long>(slot_hash(key)) & tmask;
    int row = -1;
    for (long long probe = 0; probe <= tmask; ++probe) {
      unsigned long long prev = st.slots[s].key;
      if (prev == kEmptyKey && insert) prev = atomicCAS(&st.slots[s].key, kEmptyKey, ukey);
      if (prev == kEmptyKey) {
        if (insert) {
          row = atomicAdd(&st.counters[0], 1);
          if (row < st.row_cap) {
            st.row_key[row] = ukey;
          } else {
            row = -1;
            record(status, kStatusHashTableFull, 4);
          }
          st.slots[s].row = row;
        }
        break;
      }
      if (prev == ukey) {
        // a concurrent inserter of the same key may not have published the row yet: callers pass unique keys
        row = st.slots[s].row;
        break;
      }
      s = (s + 1) & tmask;
    }
    rows[i] = row;
  }
}

}  // namespace ofb

using namespace ofb;

static int emb_grid(long long items, int per_block) {
  long long b = (items + per_block - 1) / per_block;
  if (b < 1) b = 1;
  if (b > 148 * 8) b = 148 * 8;
  return static_cast<int>(b);
}

static int emb_check(const OfbCommCtx* ctx, const OfbEmbStore* st, const OfbEmbShuffle* sh, long long n) {
  if (!ctx || !st || !sh) return fail("embedding: null argument");
  if (ctx->n < 1 || ctx->n > kMaxPeers) return fail("embedding: 1..8 ranks");
  if (st->dim % 4 || st->line < st->dim || st->line % 4) return fail("embedding: dim and row length must be multiples of 4, dim <= row length");
  if (n > sh->cap || sh->cap > (1ll << kOwnerShift)) return fail("embedding: more ids than the exchange buffers hold");
  if (sh->dcap & (sh->dcap - 1) || st->tcap & (st->tcap - 1)) return fail("embedding: table sizes must be powers of two");
  if (sh->dcap < 2 * n || sh->dcap > (1ll << 32) - 2) return fail("embedding: dedupe table too small for this many ids");
  if (st->tcap > (1ll << 31)) return fail("embedding: table too large");
  return 0;
}

// Forward: ids [n] (row-major [batch, columns]) -> out [n, dim] in `out_half ? fp16 : bf16`. `epoch` is this
// arena's embedding step number (same on every rank, starting at 1).
OFB_API int ofb_emb_forward(const OfbCommCtx* cctx, const OfbEmbStore* st, const OfbEmbShuffle* sh, const long long* ids,
                            const int* tids, long long n, int columns, int insert, unsigned int epoch, void* out, int out_half,
                            void* stream_) {
  if (emb_check(cctx, st, sh, n)) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  EmbCtx c = to_emb_ctx(cctx);
  OFB_CUDA_OK(cudaMemsetAsync(sh->dkeys, 0xFF, sh->dcap * sizeof(unsigned long long), stream));
  OFB_CUDA_OK(cudaMemsetAsync(sh->cnt, 0, kMaxPeers * sizeof(int), stream));
  OFB_CUDA_OK(cudaMemsetAsync(sh->n_uo, 0, sizeof(int), stream));
  emb_partition_kernel<<<emb_grid(n, 256), 256, 0, stream>>>(ids, tids, n, st->num_tables, columns < 1 ? 1 : columns, sh->dkeys, sh->dval,
                                                            sh->dcap - 1, sh->cnt, sh->inv, c, sh->keys_off, sh->cap);
  emb_publish_kernel<<<emb_grid(n, 256), 256, 0, stream>>>(n, sh->dval, sh->cnt, sh->inv, c, sh->cnt_off, epoch);
  const long long worst = sh->cap * c.n;
  emb_resolve_kernel<<<emb_grid(worst, 256), 256, 0, stream>>>(*st, c, sh->keys_off, sh->cnt_off, sh->cap, sh->slot_tmp, sh->n_uo, epoch,
                                                            insert);
  if (out_half)
    emb_serve_kernel<true><<<emb_grid(worst, 8), 256, 0, stream>>>(*st, c, sh->cnt_off, sh->emb_off, sh->cap, sh->slot_tmp, sh->rowidx,
                                                                   sh->uoidx, sh->u_row, sh->done + 0, epoch);
  else
    emb_serve_kernel<false><<<emb_grid(worst, 8), 256, 0, stream>>>(*st, c, sh->cnt_off, sh->emb_off, sh->cap, sh->slot_tmp, sh->rowidx,
                                                                    sh->uoidx, sh->u_row, sh->done + 0, epoch);
  emb_gather_kernel<<<emb_grid(n, 8), 256, 0, stream>>>(c, sh->emb_off, sh->cap, sh->inv, n, st->dim, reinterpret_cast<uint2*>(out), epoch);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// Backward of the forward with the same `epoch`: grad [n, dim] (same 16-bit type as the forward output).
OFB_API int ofb_emb_backward(const OfbCommCtx* cctx, const OfbEmbStore* st, const OfbEmbShuffle* sh, const void* grad, long long n,
                             int grad_half, unsigned int epoch, const OfbEmbUpdate* upd, void* stream_) {
  if (emb_check(cctx, st, sh, n)) return -1;
  if (!upd) return fail("embedding: no update rule");
  const int need = upd->kind == 0 ? 1 : (upd->kind == 1 || upd->kind == 3) ? 2 : 3;
  if (st->line < need * st->dim + (upd->kind == 5 ? 4 : 0)) return fail("embedding: rows too short for this optimizer's state");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  EmbCtx c = to_emb_ctx(cctx);
  const long long worst = sh->cap * c.n;
  const uint2* g = reinterpret_cast<const uint2*>(grad);
  if (grad_half) {
    emb_grad_reduce_kernel<true><<<emb_grid(n, 8), 256, 0, stream>>>(g, sh->inv, n, st->dim, sh->cap, sh->gsum);
    emb_grad_push_kernel<true><<<emb_grid(n, 8), 256, 0, stream>>>(c, sh->cnt, sh->grad_off, sh->cap, st->dim, sh->gsum, sh->done + 1, epoch);
    emb_grad_combine_kernel<true><<<emb_grid(worst, 8), 256, 0, stream>>>(c, sh->cnt_off, sh->grad_off, sh->cap, st->dim, sh->uoidx, sh->gacc,
                                                                          epoch);
  } else {
    emb_grad_reduce_kernel<false><<<emb_grid(n, 8), 256, 0, stream>>>(g, sh->inv, n, st->dim, sh->cap, sh->gsum);
    emb_grad_push_kernel<false><<<emb_grid(n, 8), 256, 0, stream>>>(c, sh->cnt, sh->grad_off, sh->cap, st->dim, sh->gsum, sh->done + 1, epoch);
    emb_grad_combine_kernel<false><<<emb_grid(worst, 8), 256, 0, stream>>>(c, sh->cnt_off, sh->grad_off, sh->cap, st->dim, sh->uoidx,
                                                                           sh->gacc, epoch);
  }
  const int ug = emb_grid(worst, 8);
  switch (upd->kind) {
    case 0: emb_update_kernel<0><<<ug, 256, 0, stream>>>(*st, sh->u_row, sh->n_uo, sh->gacc, *upd); break;
    case 1: emb_update_kernel<1><<<ug, 256, 0, stream>>>(*st, sh->u_row, sh->n_uo, sh->gacc, *upd); break;
    case 2: emb_update_kernel<2><<<ug, 256, 0, stream>>>(*st, sh->u_row, sh->n_uo, sh->gacc, *upd); break;
    case 3: emb_update_kernel<3><<<ug, 256, 0, stream>>>(*st, sh->u_row, sh->n_uo, sh->gacc, *upd); break;
    case 5: emb_update_kernel<5><<<ug, 256, 0, stream>>>(*st, sh->u_row, sh->n_uo, sh->gacc, *upd); break;
    default: emb_update_kernel<4><<<ug, 256, 0, stream>>>(*st, sh->u_row, sh->n_uo, sh->gacc, *upd); break;
  }
  OFB_CUDA_OK(cudaGetLastError());
  if (upd->kind == 5) {
    emb_stamp_step_kernel<<<emb_grid(worst, 256), 256, 0, stream>>>(*st, sh->u_row, sh->n_uo, upd->step);
  }
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

// rows[i] = row index of keys[i] in this rank's table (-1 when absent and not inserting). Keys must be unique
// when inserting. Used by snapshot loading and by tests.
OFB_API int ofb_emb_find(const OfbEmbStore* st, const long long* keys, long long n, int insert, int* rows, void* stream_) {
  if (!st || (st->tcap & (st->tcap - 1))) return fail("embedding: bad table");
  if (n == 0) return 0;
  emb_find_kernel<<<emb_grid(n, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(*st, keys, n, insert, rows, device_status_ptr());
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
