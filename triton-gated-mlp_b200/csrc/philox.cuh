// Counter-based dropout mask shared by every kernel that applies or re-creates
// the mask. The contract (restated on the CPU by oracle/philox.py):
//
//   e      = global_row * N_global + global_col        (element index in the
//            un-sharded hidden state H[M_global, N_global])
//   r[0:4] = Philox4x32-10(counter = (lo32(e>>3), hi32(e>>3), lo32(offset),
//            hi32(offset)), key = (lo32(seed), hi32(seed)))
//   u16    = the (e & 1)-th 16-bit half (0 = low) of word r[(e & 7) >> 1]
//   keep   = u16 >= floor(p * 2^16);   kept values are scaled by 1/(1-p)
//
// One Philox call serves 8 consecutive elements (sixteen random bits each, so p is
// honoured to within 2^-16). The mask depends only on (seed, offset, e): not on
// tiling, not on forward versus backward, not on how tokens or intermediate columns
// are sharded.
#pragma once
#include <stdint.h>

namespace gmlp {

struct Philox4 {
  uint32_t x, y, z, w;
};

__host__ __device__ __forceinline__ Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2,
                                                          uint32_t c3, uint32_t k0,
                                                          uint32_t k1) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  constexpr uint32_t W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    // one 32 x 32 -> 64-bit multiply per product (a single IMAD.WIDE on the GPU)
    const uint64_t p0 = static_cast<uint64_t>(M0) * c0, p1 = static_cast<uint64_t>(M1) * c2;
    const uint32_t hi0 = static_cast<uint32_t>(p0 >> 32), lo0 = static_cast<uint32_t>(p0);
    const uint32_t hi1 = static_cast<uint32_t>(p1 >> 32), lo1 = static_cast<uint32_t>(p1);
    const uint32_t n0 = hi1 ^ c1 ^ k0;
    const uint32_t n2 = hi0 ^ c3 ^ k1;
    c0 = n0;
    c1 = lo1;
    c2 = n2;
    c3 = lo0;
    k0 += W0;
    k1 += W1;
  }
  return Philox4{c0, c1, c2, c3};
}

struct DropoutParams {
  uint32_t thresh;      // floor(p * 2^16); 0 disables dropout
  float scale;          // 1 / (1 - p)
  uint32_t seed_lo, seed_hi, off_lo, off_hi;
  long long row0_global;   // global row of local row 0
  long long col0_global;   // global column of local column 0
  long long ncols_global;  // N_global
};

// Four random words (eight 16-bit lanes) for the 8 consecutive elements starting at
// element index e8 * 8 (e8 = e >> 3).
__device__ __forceinline__ Philox4 dropout_words(const DropoutParams& d, unsigned long long e8) {
  return philox4x32_10(static_cast<uint32_t>(e8), static_cast<uint32_t>(e8 >> 32), d.off_lo,
                       d.off_hi, d.seed_lo, d.seed_hi);
}

}  // namespace gmlp
