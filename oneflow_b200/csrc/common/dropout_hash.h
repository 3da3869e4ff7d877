// Counter-based keep/drop decision of the graph runtime's dropout operator, shared by its CUDA kernel and its host
// implementation so that both drop exactly the same elements. Nothing is stored: the forward operator and the backward
// operator (the same operator applied to the gradient) evaluate the same function of (seed, call counter, operator index,
// element index). One 64-bit draw decides four elements (16 bits each, so p has a resolution of 1/65536).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define OFB_HD __host__ __device__ __forceinline__
#else
#define OFB_HD inline
#endif

namespace ofb {

OFB_HD uint64_t dropout_mix(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
// one value per (seed, call, operator)
OFB_HD uint64_t dropout_base(uint64_t seed, uint64_t call_counter, uint32_t op_index) {
  return dropout_mix(seed ^ dropout_mix(call_counter * 0xD1B54A32D192ED03ull + op_index));
}
// the draw for elements 4 * group .. 4 * group + 3
OFB_HD uint64_t dropout_draw(uint64_t base, uint64_t group) { return dropout_mix(base + group * 0x9E3779B97F4A7C15ull); }
OFB_HD uint32_t dropout_threshold(float p) {
  const float c = p < 0.f ? 0.f : (p > 1.f ? 1.f : p);
  return static_cast<uint32_t>(c * 65536.0f);
}
// lane = element index & 3
OFB_HD bool dropout_keep(uint64_t draw, int lane, uint32_t threshold) { return ((draw >> (16 * lane)) & 0xffffull) >= threshold; }

}  // namespace ofb
