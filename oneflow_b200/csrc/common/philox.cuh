// Philox4x32-10 counter-based random numbers (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3").
// A (key, counter) pair always gives the same four 32-bit words, so a forward and a backward kernel that index the
// counter by the element's position regenerate the same dropout mask without storing it.
#pragma once
#include <cstdint>

namespace ofb {

struct Philox4 {
  uint32_t x, y, z, w;
};

__host__ __device__ __forceinline__ void philox_mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
#ifdef __CUDA_ARCH__
  hi = __umulhi(a, b);
  lo = a * b;
#else
  const unsigned long long p = static_cast<unsigned long long>(a) * b;
  hi = static_cast<uint32_t>(p >> 32);
  lo = static_cast<uint32_t>(p);
#endif
}

__host__ __device__ __forceinline__ Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                                          uint32_t k1) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    philox_mulhilo(M0, c0, hi0, lo0);
    philox_mulhilo(M1, c2, hi1, lo1);
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0; k1 += W1;
  }
  return Philox4{c0, c1, c2, c3};
}

// Attention dropout: the four keep decisions of score columns 4*cg .. 4*cg+3 of query row `row` of (batch*heads + head)
// `bh`. A word below `threshold` (= keep probability * 2^32, saturated) keeps the element.
struct DropoutCfg {
  uint32_t seed_lo, seed_hi;   // philox key
  uint32_t offset;             // philox counter word 3: advanced by the caller per launch pair (forward + its backward)
  uint32_t threshold;          // keep when word < threshold
  float inv_keep;              // 1 / keep probability
};

__device__ __forceinline__ uint32_t dropout_keep4(const DropoutCfg& d, uint32_t bh, uint32_t row, uint32_t cg) {
  const Philox4 r = philox4x32_10(cg, row, bh, d.offset, d.seed_lo, d.seed_hi);
  return (r.x < d.threshold ? 1u : 0u) | (r.y < d.threshold ? 2u : 0u) | (r.z < d.threshold ? 4u : 0u) |
         (r.w < d.threshold ? 8u : 0u);
}

}  // namespace ofb
