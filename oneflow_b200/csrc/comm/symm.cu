// Symmetric (peer-mapped) memory plumbing and the stand-alone collectives of the comm library.
//
// Every rank of a group allocates an arena with cudaMalloc, exports it as a CUDA IPC handle, and maps
// the arenas of all peers; kernels then read and write peer memory directly over NVLink / NVSwitch.
// The collectives below are the "boxing" primitives of the SBP layer:
//     all_reduce      P -> B      (two-shot: reduce own slice from all peers, push it to all peers)
//     reduce_scatter  P -> S(0)   (reduce own slice from all peers)
//     all_gather      S(0) -> B   (pull every peer's shard)
//     all_to_all      S(i) -> S(j) (pull the sub-blocks addressed to this rank, transposition folded
//                                   into the addressing)
// each optionally fused with a cast and a scale (gradient path: bf16/fp32 in, fp32/bf16 out, * 1/N or
// 1/loss_scale), so no separate pack / cast pass runs. Cross-rank synchronisation uses monotonic epoch
// flags with bounded spins (comm_common.cuh); no NCCL call is involved.
//
// Reference counterparts: oneflow/user/kernels/collective_communication/cuda/*.cpp (one NCCL call each),
// nccl_logical_kernels.cpp (pack/unpack permutes around them), fused_cast_scale_kernel.cu, and the IPC
// handle exchange in one_embedding_id_shuffle_p2p_kernel.cu:344-357.
#include <cuda_fp16.h>

#include "../common/host_utils.h"
#include "comm_common.cuh"
#include "ofb_comm.h"

namespace ofb {

struct CommCtx {
  int rank, n;
  unsigned char* arena[kMaxPeers];   // base of every rank's arena (arena[rank] is local)
  SignalBlock* sig[kMaxPeers];       // signal block of every rank
  int* status;
};

static CommCtx to_ctx(const OfbCommCtx* c) {
  CommCtx x;
  x.rank = c->rank;
  x.n = c->n;
  for (int i = 0; i < kMaxPeers; ++i) {
    x.arena[i] = reinterpret_cast<unsigned char*>(c->arena[i]);
    x.sig[i] = reinterpret_cast<SignalBlock*>(c->signals[i]);
  }
  x.status = device_status_ptr();
  return x;
}

// Grid-wide + cross-rank barrier. `slot` selects one of the local scratch counters, `epoch` is the
// per-context barrier epoch (same value on every rank for the same barrier). All CTAs of the grid must
// be co-resident (the launchers below never start more CTAs than SMs).
__device__ bool grid_peer_barrier(const CommCtx& c, unsigned int epoch, int slot) {
  __shared__ int ok_s;
  __syncthreads();
  if (threadIdx.x == 0) {
    ok_s = 1;
    SignalBlock* me = c.sig[c.rank];
    __threadfence_system();
    const unsigned int arrived = atomicAdd(&me->local_cnt[slot], 1u) + 1u;
    const unsigned int target = epoch * gridDim.x;
    if (arrived == target) {
      // last CTA of this GPU: announce to every peer, wait for every peer, then release the others
      for (int p = 0; p < c.n; ++p) st_release_sys(&c.sig[p]->barrier[c.rank], epoch);
      bool ok = true;
      for (int p = 0; p < c.n && ok; ++p) ok = wait_flag_ge(&me->barrier[p], epoch, c.status, 100 + p);
      __threadfence_system();
      atomicExch(&me->local_cnt[slot + 1], ok ? epoch : 0x7fffffffu);
      if (!ok) ok_s = 0;
    } else {
      if (!wait_local_ge(&me->local_cnt[slot + 1], epoch, c.status, 120)) ok_s = 0;
      if (ld_acquire_gpu(&me->local_cnt[slot + 1]) == 0x7fffffffu) ok_s = 0;
    }
    __threadfence_system();
  }
  __syncthreads();
  return ok_s != 0;
}

template <typename T>
__device__ __forceinline__ float to_f(T v) { return static_cast<float>(v); }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v) { return static_cast<T>(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) Pack {
  T v[VEC];
};


// dst[0..VEC) = v as TOut, written with the widest aligned stores (dst is aligned to VEC * sizeof(TOut) bytes).
template <typename TOut, int VEC>
__device__ __forceinline__ void store_vec(TOut* dst, const float (&v)[VEC]) {
  if constexpr (sizeof(TOut) == 4) {
#pragma unroll
    for (int j = 0; j < VEC; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
  } else {
    uint32_t w[VEC / 2];
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) w[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
    if constexpr (VEC == 8) {
      *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
    }
  }
}

// mode 0: all-reduce, 1: reduce-scatter, 2: all-gather.
// Input of every rank sits in its arena at `in_off` (count elements of TIn for reduce modes, count/n for
// all-gather); the result goes to `out` (local memory, TOut), count elements for all-reduce / all-gather,
// count/n for reduce-scatter. `stage_off` is arena scratch of count elements of float used by all-reduce.
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(512) collective_kernel(CommCtx c, int mode, long long in_off, long long stage_off,
                                                         TOut* __restrict__ out, long long count, float scale,
                                                         unsigned int epoch, long long gather_src_stride) {
  constexpr int VEC = 16 / sizeof(TIn);
  using PIn = Pack<TIn, VEC>;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  // inputs of all ranks are in place
  if (!grid_peer_barrier(c, 2 * epoch - 1, 0)) return;
  const long long slice = count / c.n;  // host guarantees divisibility by n * VEC
  if (mode == 3) {  // pure barrier
    grid_peer_barrier(c, 2 * epoch, 0);
    return;
  }
  constexpr int UNR = 4;  // independent 16-byte accesses per thread and pass: NVLink latency needs megabytes in flight
  if (mode == 0 || mode == 1) {
    const long long base = slice * c.rank;
    for (long long i0 = tid * VEC; i0 < slice; i0 += nth * VEC * UNR) {
      float acc[UNR][VEC];
#pragma unroll
      for (int u = 0; u < UNR; ++u)
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[u][j] = 0.f;
#pragma unroll 1
      for (int k = 0; k < c.n; ++k) {
        const int p = (c.rank + k) % c.n;  // spread the peers' load
        PIn v[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const long long i = i0 + u * nth * VEC;
          if (i < slice) v[u] = *reinterpret_cast<const PIn*>(c.arena[p] + in_off + (base + i) * sizeof(TIn));
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          if (i0 + u * nth * VEC < slice) {
#pragma unroll
            for (int j = 0; j < VEC; ++j) acc[u][j] += to_f<TIn>(v[u].v[j]);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const long long i = i0 + u * nth * VEC;
        if (i >= slice) continue;
        if (mode == 1) {
          float o[VEC];
#pragma unroll
          for (int j = 0; j < VEC; ++j) o[j] = acc[u][j] * scale;
          store_vec<TOut, VEC>(out + i, o);
        } else {
          // push the reduced slice (fp32) into every rank's staging area
#pragma unroll 1
          for (int k = 0; k < c.n; ++k) {
            const int p = (c.rank + k) % c.n;
            float* dst = reinterpret_cast<float*>(c.arena[p] + stage_off) + base + i;
#pragma unroll
            for (int j = 0; j < VEC; j += 4)
              *reinterpret_cast<float4*>(dst + j) =
                  make_float4(acc[u][j] * scale, acc[u][j + 1] * scale, acc[u][j + 2] * scale, acc[u][j + 3] * scale);
          }
        }
      }
    }
    if (mode == 0) {
      if (!grid_peer_barrier(c, 2 * epoch, 0)) return;
      const float* st = reinterpret_cast<const float*>(c.arena[c.rank] + stage_off);
      for (long long i = tid * 4; i < count; i += nth * 4) {
        const float4 v = *reinterpret_cast<const float4*>(st + i);
        const float o[4] = {v.x, v.y, v.z, v.w};
        store_vec<TOut, 4>(out + i, o);
      }
      return;  // the staging area is rewritten only after the next call's first barrier
    }
  } else {
    for (int k = 0; k < c.n; ++k) {
      const int p = (c.rank + k) % c.n;
      // gather_src_stride != 0: every rank keeps the WHOLE buffer in its arena and contributes the slice at its own
      // offset (in-place all-gather of a flat parameter buffer); 0: every rank's shard sits at in_off
      const TIn* src = reinterpret_cast<const TIn*>(c.arena[p] + in_off + p * gather_src_stride);
      for (long long i0 = tid * VEC; i0 < slice; i0 += nth * VEC * UNR) {
        PIn v[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const long long i = i0 + u * nth * VEC;
          if (i < slice) v[u] = *reinterpret_cast<const PIn*>(src + i);
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const long long i = i0 + u * nth * VEC;
          if (i >= slice) continue;
          float o[VEC];
#pragma unroll
          for (int j = 0; j < VEC; ++j) o[j] = to_f<TIn>(v[u].v[j]) * scale;
          store_vec<TOut, VEC>(out + slice * p + i, o);
        }
      }
    }
  }
  // nobody may overwrite its input before every peer finished reading it
  grid_peer_barrier(c, 2 * epoch, 0);
}

// S(i) -> S(j) all-to-all on a logical tensor viewed as [outer, I, mid, J, inner] where the input is split
// along I (local I/n) and the output along J (local J/n): out[o, i_full, m, j_local, x] pulls from the peer
// owning i_full. `inner` is a multiple of the vector width.
template <typename T>
__global__ void __launch_bounds__(512) all_to_all_kernel(CommCtx c, long long in_off, T* __restrict__ out, long long outer,
                                                         long long I, long long mid, long long J, long long inner,
                                                         unsigned int epoch) {
  constexpr int VEC = 16 / sizeof(T);
  using P = Pack<T, VEC>;
  if (!grid_peer_barrier(c, 2 * epoch - 1, 0)) return;
  const long long Il = I / c.n, Jl = J / c.n;
  const long long vin = inner / VEC;
  const long long total = outer * I * mid * Jl * vin;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  for (long long e = tid; e < total; e += nth) {
    long long r = e;
    const long long x = r % vin; r /= vin;
    const long long jl = r % Jl; r /= Jl;
    const long long m = r % mid; r /= mid;
    const long long i = r % I; r /= I;
    const long long o = r;
    const int p = static_cast<int>(i / Il);
    const long long il = i - p * Il;
    // peer p holds [outer, Il, mid, J, inner]
    const long long src = (((o * Il + il) * mid + m) * J + (c.rank * Jl + jl)) * inner + x * VEC;
    const P v = *reinterpret_cast<const P*>(reinterpret_cast<const T*>(c.arena[p] + in_off) + src);
    *reinterpret_cast<P*>(out + ((((o * I + i) * mid + m) * Jl + jl) * inner + x * VEC)) = v;
  }
  grid_peer_barrier(c, 2 * epoch, 0);
}

}  // namespace ofb

using namespace ofb;

// ------------------------------------------------------------------------------------------------ IPC
OFB_API int ofb_symm_alloc(long long bytes, void** ptr, unsigned char* handle64) {
  void* p = nullptr;
  OFB_CUDA_OK(cudaMalloc(&p, static_cast<size_t>(bytes)));
  OFB_CUDA_OK(cudaMemset(p, 0, static_cast<size_t>(bytes)));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
  }
  static_assert(sizeof(h) == 64, "IPC handle size");
  std::memcpy(handle64, &h, 64);
  *ptr = p;
  return 0;
}
OFB_API int ofb_symm_open(const unsigned char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  OFB_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}
OFB_API int ofb_symm_close(void* ptr) {
  OFB_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return 0;
}
OFB_API int ofb_symm_free(void* ptr) {
  OFB_CUDA_OK(cudaFree(ptr));
  return 0;
}

static int comm_grid(long long work, int threads, int max_ctas) {
  long long b = (work + threads - 1) / threads;
  int cap = max_ctas > 0 ? max_ctas : 64;
  if (cap > 132) cap = 132;  // strictly co-resident on a 148-SM part
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

// mode: 0 all-reduce, 1 reduce-scatter, 2 all-gather, 3 barrier only. dtype codes: 0 fp32, 1 bf16.
// Every launch of a collective on one context must use the same grid size (the barrier counts CTAs):
// the launcher therefore always uses `ctas` CTAs (default 64).
static int comm_collective_impl(const OfbCommCtx* ctx, int mode, long long in_off, long long stage_off, int in_dtype, void* out,
                                int out_dtype, long long count, float scale, unsigned int epoch, int ctas, long long gather_src_stride,
                                void* stream) {
  if (ctx->n < 1 || ctx->n > kMaxPeers) return fail("comm: group size must be 1..8");
  const int vec = in_dtype == 0 ? 4 : 8;
  if (count % (static_cast<long long>(ctx->n) * vec)) return fail("comm: element count must be a multiple of n * 16 bytes");
  CommCtx c = to_ctx(ctx);
  auto s = (cudaStream_t)stream;
  const int grid = ctas > 0 ? (ctas > 132 ? 132 : ctas) : 64;
#define OFB_COLL(TI, TO) \
  collective_kernel<TI, TO><<<grid, 512, 0, s>>>(c, mode, in_off, stage_off, (TO*)out, count, scale, epoch, gather_src_stride)
  if (in_dtype == 0 && out_dtype == 0) OFB_COLL(float, float);
  else if (in_dtype == 0 && out_dtype == 1) OFB_COLL(float, __nv_bfloat16);
  else if (in_dtype == 1 && out_dtype == 0) OFB_COLL(__nv_bfloat16, float);
  else if (in_dtype == 1 && out_dtype == 1) OFB_COLL(__nv_bfloat16, __nv_bfloat16);
  else return fail("comm: unsupported dtype pair");
#undef OFB_COLL
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}

OFB_API int ofb_comm_collective(const OfbCommCtx* ctx, int mode, long long in_off, long long stage_off, int in_dtype,
                                void* out, int out_dtype, long long count, float scale, unsigned int epoch, int ctas,
                                void* stream) {
  return comm_collective_impl(ctx, mode, in_off, stage_off, in_dtype, out, out_dtype, count, scale, epoch, ctas, 0, stream);
}

// In-place all-gather of a flat buffer that every rank holds whole in its arena at in_off: rank p's slice (count / n
// elements at byte offset p * slice bytes) is copied into `out` (normally this rank's own copy of the buffer) at the
// same position. No staging copy on either side.
OFB_API int ofb_comm_all_gather_inplace(const OfbCommCtx* ctx, long long in_off, int dtype, void* out, long long count,
                                        unsigned int epoch, int ctas, void* stream) {
  const long long esz = dtype == 0 ? 4 : 2;
  if (ctx->n < 1 || count % ctx->n) return fail("comm: element count must be a multiple of the group size");
  return comm_collective_impl(ctx, 2, in_off, in_off, dtype, out, dtype, count, 1.f, epoch, ctas, (count / ctx->n) * esz, stream);
}

OFB_API int ofb_comm_all_to_all(const OfbCommCtx* ctx, long long in_off, int dtype, void* out, long long outer, long long I,
                                long long mid, long long J, long long inner, unsigned int epoch, int ctas, void* stream) {
  if (ctx->n < 1 || ctx->n > kMaxPeers) return fail("comm: group size must be 1..8");
  const int vec = dtype == 0 ? 4 : 8;
  if (I % ctx->n || J % ctx->n || inner % vec) return fail("all_to_all: split axes must divide by n and inner by the vector width");
  CommCtx c = to_ctx(ctx);
  const int grid = ctas > 0 ? (ctas > 132 ? 132 : ctas) : 64;
  auto s = (cudaStream_t)stream;
  if (dtype == 0) all_to_all_kernel<float><<<grid, 512, 0, s>>>(c, in_off, (float*)out, outer, I, mid, J, inner, epoch);
  else all_to_all_kernel<__nv_bfloat16><<<grid, 512, 0, s>>>(c, in_off, (__nv_bfloat16*)out, outer, I, mid, J, inner, epoch);
  OFB_CUDA_OK(cudaGetLastError());
  return 0;
}
