// Fused GEMM epilogue shared by the one-SM and the two-SM tcgen05 kernels.
//
// An epilogue warp owns 32 accumulator rows (its TMEM lane quadrant). It walks the tile in chunks of
// 32 columns: tcgen05.ld brings the chunk into registers (thread = row), the elementwise part runs in fp32
// (alpha, bias, pre-activation output, activation or activation gradient, residual), and the result goes to
// global memory through a warp-private shared-memory staging tile, so that every global access of the
// epilogue -- the stores and the loads of aux_in / residual / the accumulate read -- is a full, aligned 16-byte
// piece of a row segment that the neighbouring lanes complete to 64 or 128 contiguous bytes. Writing the
// accumulator rows directly (one row per thread) would issue 32 scattered half-sector writes per instruction.
//
// Staging tile: 32 rows x 64 bytes (bf16) or x 128 bytes (fp32), 16-byte chunks XOR-swizzled by the row so
// that both the row-wise (thread = row) and the coalesced (several lanes per row) access patterns are free
// of bank conflicts. The activation is selected by a warp-uniform switch around the element loops: only the
// selected function's instructions are issued.
#pragma once
#include "../common/ptx.cuh"

namespace ofb {

constexpr int kEpiStageBytesPerWarp = 32 * 128;

__device__ __forceinline__ uint32_t epi_addr64(uint32_t base, int row, int chunk) {
  return base + row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4);
}
__device__ __forceinline__ uint32_t epi_addr128(uint32_t base, int row, int chunk) {
  return base + row * 128 + ((chunk ^ (row & 7)) << 4);
}
__device__ __forceinline__ void epi_sts(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 epi_lds(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}

// v[0..31] = bf16 tile src[row = lane][0..31] as fp32, loaded with coalesced 16-byte accesses (4 lanes per row).
// L2_ONLY: bypass L1 (ld.global.cg) for memory that a peer GPU writes while this kernel runs.
template <bool L2_ONLY = false>
__device__ __forceinline__ void epi_load_bf16(uint32_t stage, int lane, const __nv_bfloat16* src, long long ld, int rows_valid,
                                              int cols_valid, float (&v)[32]) {
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int r = it * 8 + (lane >> 2), ch = lane & 3;
    uint4 q = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows_valid && ch * 8 < cols_valid) {
      const uint4* p = reinterpret_cast<const uint4*>(src + r * ld + ch * 8);
      q = L2_ONLY ? __ldcg(p) : __ldg(p);
    }
    epi_sts(epi_addr64(stage, r, ch), q);
  }
  __syncwarp();
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    const uint4 q = epi_lds(epi_addr64(stage, lane, ch));
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(w[j]);
      v[ch * 8 + 2 * j] = f.x;
      v[ch * 8 + 2 * j + 1] = f.y;
    }
  }
  __syncwarp();
}

__device__ __forceinline__ uint32_t epi_bf16x2_add(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hadd2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}

// v[0..31] = sum over several bf16 tiles of the same shape: sources s = 0..nsrc-1 except `skip` at
// base + s * src_stride (row pitch ld, read through L2 only: peers write them), plus one more tile `extra`
// (row pitch ld_extra) when it is not null. The tiles are added as packed bf16 pairs in the coalesced layout (what a
// bf16 reduce-scatter does on the wire as well), all loads of a group of four sources are issued before the first is
// consumed, and only the sum goes through the staging tile, whatever the number of sources.
__device__ __forceinline__ void epi_load_sum_bf16(uint32_t stage, int lane, const __nv_bfloat16* base, long long src_stride, int nsrc, int skip,
                                                  long long ld, const __nv_bfloat16* extra, long long ld_extra, int rows_valid, int cols_valid,
                                                  float (&v)[32]) {
  uint4 sum[4];
#pragma unroll
  for (int it = 0; it < 4; ++it) sum[it] = make_uint4(0u, 0u, 0u, 0u);
  const int ch = lane & 3;
  const bool col_ok = ch * 8 < cols_valid;
  const int total = nsrc + (extra ? 1 : 0);
  for (int s0 = 0; s0 < total; s0 += 4) {
    uint4 q[4][4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int s = s0 + k;
      const __nv_bfloat16* src = nullptr;
      long long pitch = ld;
      if (s < nsrc && s != skip) src = base + s * src_stride;
      if (s == nsrc) { src = extra; pitch = ld_extra; }
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int r = it * 8 + (lane >> 2);
        q[k][it] = make_uint4(0u, 0u, 0u, 0u);
        if (src && col_ok && r < rows_valid) q[k][it] = __ldcg(reinterpret_cast<const uint4*>(src + r * pitch + ch * 8));
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k)
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        sum[it].x = epi_bf16x2_add(sum[it].x, q[k][it].x);
        sum[it].y = epi_bf16x2_add(sum[it].y, q[k][it].y);
        sum[it].z = epi_bf16x2_add(sum[it].z, q[k][it].z);
        sum[it].w = epi_bf16x2_add(sum[it].w, q[k][it].w);
      }
  }
#pragma unroll
  for (int it = 0; it < 4; ++it) epi_sts(epi_addr64(stage, it * 8 + (lane >> 2), ch), sum[it]);
  __syncwarp();
#pragma unroll
  for (int c16 = 0; c16 < 4; ++c16) {
    const uint4 q = epi_lds(epi_addr64(stage, lane, c16));
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(w[j]);
      v[c16 * 8 + 2 * j] = f.x;
      v[c16 * 8 + 2 * j + 1] = f.y;
    }
  }
  __syncwarp();
}

// dst[row][0..31] (bf16) = v of the thread that owns the row (+ old contents when `accumulate`).
__device__ __forceinline__ void epi_store_bf16(uint32_t stage, int lane, const float (&v)[32], __nv_bfloat16* dst, long long ld,
                                               int rows_valid, int cols_valid, bool accumulate) {
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    uint4 q;
    q.x = pack_bf16x2(v[ch * 8 + 0], v[ch * 8 + 1]);
    q.y = pack_bf16x2(v[ch * 8 + 2], v[ch * 8 + 3]);
    q.z = pack_bf16x2(v[ch * 8 + 4], v[ch * 8 + 5]);
    q.w = pack_bf16x2(v[ch * 8 + 6], v[ch * 8 + 7]);
    epi_sts(epi_addr64(stage, lane, ch), q);
  }
  __syncwarp();
  // the old values are all read before the first store (see epi_store_f32)
  uint4 olds[4];
  if (accumulate) {
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int r = it * 8 + (lane >> 2), ch = lane & 3;
      olds[it] = (r < rows_valid && ch * 8 < cols_valid) ? *reinterpret_cast<const uint4*>(dst + r * ld + ch * 8) : make_uint4(0u, 0u, 0u, 0u);
    }
  }
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int r = it * 8 + (lane >> 2), ch = lane & 3;
    uint4 q = epi_lds(epi_addr64(stage, r, ch));
    if (r < rows_valid && ch * 8 < cols_valid) {
      uint4* p = reinterpret_cast<uint4*>(dst + r * ld + ch * 8);
      if (accumulate) {
        const uint4 old = olds[it];
        const uint32_t a[4] = {q.x, q.y, q.z, q.w}, b[4] = {old.x, old.y, old.z, old.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 x = unpack_bf16x2(a[j]), y = unpack_bf16x2(b[j]);
          o[j] = pack_bf16x2(x.x + y.x, x.y + y.y);
        }
        q = make_uint4(o[0], o[1], o[2], o[3]);
      }
      *p = q;
    }
  }
  __syncwarp();
}

// fp32 destination. mode 0: store, 1: read-add-write, 2: atomic add (split-K partial sums).
__device__ __forceinline__ void epi_store_f32(uint32_t stage, int lane, const float (&v)[32], float* dst, long long ld, int rows_valid,
                                              int cols_valid, int mode) {
#pragma unroll
  for (int ch = 0; ch < 8; ++ch) {
    uint4 q;
    q.x = __float_as_uint(v[ch * 4 + 0]);
    q.y = __float_as_uint(v[ch * 4 + 1]);
    q.z = __float_as_uint(v[ch * 4 + 2]);
    q.w = __float_as_uint(v[ch * 4 + 3]);
    epi_sts(epi_addr128(stage, lane, ch), q);
  }
  __syncwarp();
  // read-add-write: all eight reads of the old values are issued before the first store. Inside one loop the compiler has
  // to keep every load behind the previous iteration's store (the pointers may alias for all it knows), which makes eight
  // dependent round trips to memory per chunk; with one output tile per CTA nothing hides them.
  float4 old[8];
  if (mode == 1) {
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int r = it * 4 + (lane >> 3), ch = lane & 7;
      old[it] = (r < rows_valid && ch * 4 < cols_valid) ? *reinterpret_cast<const float4*>(dst + r * ld + ch * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 4 + (lane >> 3), ch = lane & 7;
    const uint4 q = epi_lds(epi_addr128(stage, r, ch));
    if (r < rows_valid && ch * 4 < cols_valid) {
      float4 x = make_float4(__uint_as_float(q.x), __uint_as_float(q.y), __uint_as_float(q.z), __uint_as_float(q.w));
      float4* p = reinterpret_cast<float4*>(dst + r * ld + ch * 4);
      if (mode == 2) {
        atomicAdd(p, x);
      } else {
        if (mode == 1) {
          x.x += old[it].x; x.y += old[it].y; x.z += old[it].z; x.w += old[it].w;
        }
        *p = x;
      }
    }
  }
  __syncwarp();
}

// Elementwise part and stores of one 32-column chunk whose accumulator values are already in `r`.
__device__ __forceinline__ void gemm_epilogue_chunk(const GemmEpilogue& ep, const uint32_t (&r)[32], int row0, int col0, int rows_valid,
                                                    int cols_valid, int lane, uint32_t stage, bool atomic_out) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * ep.alpha;
  if (ep.bias) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (g * 8 < cols_valid) {
        const uint4 bb = __ldg(reinterpret_cast<const uint4*>(ep.bias + col0 + g * 8));  // same address in every lane
        const uint32_t bw[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(bw[j]);
          v[g * 8 + 2 * j] += f.x;
          v[g * 8 + 2 * j + 1] += f.y;
        }
      }
    }
  }
  const long long tile_off_aux = static_cast<long long>(row0) * ep.ld_aux + col0;
  if (ep.aux_out) epi_store_bf16(stage, lane, v, ep.aux_out + tile_off_aux, ep.ld_aux, rows_valid, cols_valid, false);
  if (ep.aux_in) {
    float h[32];
    epi_load_bf16(stage, lane, ep.aux_in + tile_off_aux, ep.ld_aux, rows_valid, cols_valid, h);
    switch (ep.act) {
      case kActGeluErf:
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= gelu_erf_grad(h[j]);
        break;
      case kActGeluTanh:
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= gelu_tanh_grad(h[j]);
        break;
      case kActRelu:
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = h[j] > 0.f ? v[j] : 0.f;
        break;
      default:
        break;
    }
  } else {
    switch (ep.act) {
      case kActGeluErf:
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
        break;
      case kActGeluTanh:
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
        break;
      case kActRelu:
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
        break;
      default:
        break;
    }
  }
  if (ep.residual) {
    float h[32];
    epi_load_bf16(stage, lane, ep.residual + static_cast<long long>(row0) * ep.ldr + col0, ep.ldr, rows_valid, cols_valid, h);
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] += h[j];
  }
  const long long tile_off = static_cast<long long>(row0) * ep.ldc + col0;
  if (ep.out_fp32) {
    epi_store_f32(stage, lane, v, reinterpret_cast<float*>(ep.C) + tile_off, ep.ldc, rows_valid, cols_valid,
                  atomic_out ? 2 : (ep.accumulate ? 1 : 0));
  } else {
    epi_store_bf16(stage, lane, v, reinterpret_cast<__nv_bfloat16*>(ep.C) + tile_off, ep.ldc, rows_valid, cols_valid,
                   ep.accumulate != 0);
  }
}

// Epilogue of one accumulator tile for one warp: rows [row0, row0 + 32) x columns [n0, n0 + BN) of the problem,
// accumulator at TMEM address `taddr` (lane quadrant and column base already applied). `atomic_out` selects
// atomic accumulation into an fp32 C (split-K); the fused elementwise options are not combined with it.
template <int BN>
__device__ __forceinline__ void gemm_epilogue_warp(const GemmEpilogue& ep, const GemmShape& shp, uint32_t taddr, int row0, int n0,
                                                   int lane, uint32_t stage, bool atomic_out, int c_begin = 0, int c_end = BN / 32) {
  const int rows_valid = shp.M - row0;
  int nchunks = (shp.N - n0 + 31) / 32;
  if (nchunks > c_end) nchunks = c_end;
  if (nchunks <= c_begin) return;
#pragma unroll 1
  for (int c = c_begin; c < nchunks; ++c) {
    uint32_t r[32];
    __syncwarp();  // tcgen05.ld is warp-collective
    tmem_ld_32x32(taddr + c * 32, r);
    tmem_wait_ld();
    if (rows_valid > 0) gemm_epilogue_chunk(ep, r, row0, n0 + c * 32, rows_valid, shp.N - (n0 + c * 32), lane, stage, atomic_out);
  }
}

}  // namespace ofb
