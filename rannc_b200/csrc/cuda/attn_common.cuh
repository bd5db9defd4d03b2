// Helpers shared by the attention forward and backward kernels.
#pragma once
#include <stdint.h>

#include "tc_common.cuh"

namespace rb {

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        :
        : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)),
          "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// barrier among `count` threads of the CTA (count % 32 == 0); id 0 is __syncthreads
__device__ __forceinline__ void bar_sync_named(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// ---- attention dropout -----------------------------------------------------
// The keep decision of element (b, h, q, key) is a pure function of the dropout
// site's seed and the element's coordinates, so the backward regenerates it.
// One 32-bit hash serves the key pair (2k, 2k + 1): low half = even key.
__host__ __device__ inline uint32_t drop_seed(uint64_t seed, uint64_t offset) {
    uint64_t z = seed * 0x9E3779B97F4A7C15ull + offset * 0xBF58476D1CE4E5B9ull + 0x94D049BB133111EBull;
    z ^= z >> 31;
    z *= 0xD6E8FEB86659FD93ull;
    z ^= z >> 32;
    return static_cast<uint32_t>(z);
}
__device__ __forceinline__ uint32_t hash32(uint32_t x) {
    x ^= x >> 16;
    x *= 0x7FEB352Du;
    x ^= x >> 15;
    x *= 0x846CA68Bu;
    x ^= x >> 16;
    return x;
}
__device__ __forceinline__ uint32_t drop_row_hash(uint32_t seed, int b, int h, int q, int H, int S) {
    const uint32_t row = (static_cast<uint32_t>(b) * H + h) * static_cast<uint32_t>(S) + q;
    return hash32(row ^ seed) + seed;
}
__device__ __forceinline__ uint32_t drop_bits(uint32_t row_hash, int key_pair) {
    return hash32(row_hash + static_cast<uint32_t>(key_pair) * 0x9E3779B1u);
}

}  // namespace rb
