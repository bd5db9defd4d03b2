// Counter-based RNG (Philox4x32, 7 rounds) used by the element-wise dropouts of
// this library.  A dropout site is identified by (seed, offset); the 8 elements
// [8k, 8k + 8) of the site read the eight 16-bit halves of counter block k.  Forward and backward regenerate the same
// bits, so no mask tensor is stored, and a recomputed forward (activation
// checkpointing) reproduces the original mask as long as it is given the same
// (seed, offset) pair.
#pragma once
#include <stdint.h>

namespace rb {

struct Philox4 {
    uint32_t v[4];
};

__device__ __forceinline__ Philox4 philox4x32(uint64_t seed, uint64_t offset, uint64_t block) {
    uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
    uint32_t c0 = static_cast<uint32_t>(block), c1 = static_cast<uint32_t>(block >> 32);
    uint32_t c2 = static_cast<uint32_t>(offset), c3 = static_cast<uint32_t>(offset >> 32);
#pragma unroll
    for (int r = 0; r < 7; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0;
        const uint32_t n2 = hi0 ^ c3 ^ k1;
        c0 = n0;
        c1 = lo1;
        c2 = n2;
        c3 = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    Philox4 o;
    o.v[0] = c0;
    o.v[1] = c1;
    o.v[2] = c2;
    o.v[3] = c3;
    return o;
}

// keep-threshold for probability p of dropping, on 16-bit draws: keep iff bits >= thr
__host__ __device__ inline uint32_t drop_threshold(float p) {
    double t = static_cast<double>(p) * 65536.0 + 0.5;
    if (t < 0) t = 0;
    if (t > 65535.0) t = 65535.0;
    return static_cast<uint32_t>(t);
}
// keep flags of the 8 consecutive elements starting at linear index idx (idx % 8 == 0)
__device__ __forceinline__ void keep8(uint64_t seed, uint64_t offset, uint64_t idx, uint32_t thr,
                                      bool (&k)[8]) {
    const Philox4 a = philox4x32(seed, offset, idx >> 3);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        k[2 * j] = (a.v[j] & 0xffffu) >= thr;
        k[2 * j + 1] = (a.v[j] >> 16) >= thr;
    }
}

}  // namespace rb
