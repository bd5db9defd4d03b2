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

// Adds a [32 x 128] fp32 tile of this CTA's shared memory (128-byte swizzled rows) into global memory
// through the tensor map: one bulk reduction instead of per-thread atomics; rows past the tensor's
// extent are dropped by the copy engine.  Completion is tracked by the bulk async-group.
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, const void* smem_src, int c0, int c1,
                                                  int c2, int c3) {
    asm volatile(
        "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
        :
        : "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// ---- packed fp32 arithmetic (two lanes per instruction) and the three-input maximum of sm_100 ----
// The softmax threads are bound by instruction issue, so every element-wise step that has a two-wide
// form uses it.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ uint64_t f2_pack_bits(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// barrier among `count` threads of the CTA (count % 32 == 0); id 0 is __syncthreads
__device__ __forceinline__ void bar_sync_named(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// ---- attention dropout -----------------------------------------------------
// The keep decision of element (b, h, q, key) is a pure function of the dropout
// site's seed and the element's coordinates, so the backward regenerates it.
// It is separable: a well-mixed hash per query row and one per key are computed
// once each (per thread, or staged in shared memory), and an element costs one
// XOR, one multiply and one compare against the 32-bit threshold p * 2^32 -- in
// the forward kernel (thread = query row) and in the backward (thread = key) alike.
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
__device__ __forceinline__ uint32_t drop_key_hash(uint32_t seed, int key) {
    return hash32(static_cast<uint32_t>(key) * 0x9E3779B1u + (seed ^ 0x85EBCA6Bu));
}
__device__ __forceinline__ bool drop_keep(uint32_t row_hash, uint32_t key_hash, uint32_t thr32) {
    return (row_hash ^ key_hash) * 0x9E3779B1u >= thr32;
}
__host__ inline uint32_t drop_threshold(float p_drop) {
    if (!(p_drop > 0.f)) return 0u;
    const double t = static_cast<double>(p_drop) * 4294967296.0;
    return t >= 4294967295.0 ? 4294967295u : static_cast<uint32_t>(t);
}

}  // namespace rb
