// Fused  y = LayerNorm( dropout(x) + residual )  forward and backward.
//
// One warp owns one row; a lane holds NCHUNK groups of 8 consecutive elements
// (16-byte loads), so a row of H = 256 * NCHUNK elements is read exactly once
// and kept in registers.  The forward also writes z = dropout(x) + residual
// (the LayerNorm input, needed by the backward) and the per-row mean / rstd.
// The backward produces dz (gradient of the residual branch), dx (dz through
// the dropout mask, regenerated from the Philox counter) and per-CTA partial
// sums of dgamma / dbeta in a scratch buffer that a second kernel reduces.
//
// These take the place of aten::layer_norm / aten::dropout / aten::add nodes of
// the traced graph that the reference executes one by one
// (src/torch/TorchDriver.cpp:566; dropout train flag: src/graph/ConvertGraph.cpp:469-484).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdlib>
#include <stdint.h>

#include "philox.cuh"
#include "tc_common.cuh"

namespace rb {

constexpr int LN_WARPS = 8;
constexpr int LN_THREADS = LN_WARPS * 32;

template <typename T>
__device__ __forceinline__ void ld8(const T* p, float (&v)[8]) {
    uint4 q = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = to_f32<T>(e[j]);
}
template <typename T>
__device__ __forceinline__ void st8(T* p, const float (&v)[8]) {
    uint4 q;
    T* e = reinterpret_cast<T*>(&q);
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = from_f32<T>(v[j]);
    *reinterpret_cast<uint4*>(p) = q;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// sum over the WPR warps that share a row (warps [slot*WPR, slot*WPR+WPR))
template <int WPR>
__device__ __forceinline__ float group_sum(float v, float* sm, int warp, int lane) {
    v = warp_sum(v);
    if constexpr (WPR == 1) {
        return v;
    } else {
        __syncthreads();
        if (lane == 0) sm[warp] = v;
        __syncthreads();
        const int base = (warp / WPR) * WPR;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < WPR; ++i) s += sm[base + i];
        return s;
    }
}

// A row of H = 256 * NCHUNK * WPR elements is shared by WPR warps.
template <typename T, int NCHUNK, int WPR>
__global__ void __launch_bounds__(LN_THREADS, 3)
    ln_fwd_kernel(const T* __restrict__ x, const T* __restrict__ residual,
                  const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
                  T* __restrict__ z_out, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                  int rows, float eps, uint32_t thr, float scale, uint64_t seed, uint64_t offset) {
    constexpr int H = NCHUNK * 256 * WPR;
    constexpr int RPB = LN_WARPS / WPR;  // rows per CTA per iteration
    __shared__ float sm[LN_WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slot = warp / WPR, part = warp % WPR;
    // gamma / beta are re-read per row (they stay in L1): keeping them in registers costs 16 * NCHUNK
    // registers and with them a third of the warps that could be in flight, which is what bounds a kernel
    // whose rows are one dependent load -> reduce -> store chain each
    for (int r0 = blockIdx.x * RPB; r0 < rows; r0 += gridDim.x * RPB) {
        const int row = r0 + slot;
        const bool live = row < rows;
        const size_t base = static_cast<size_t>(live ? row : 0) * H;
        float v[NCHUNK][8];
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < NCHUNK; ++c) {
            const int col = ((part * NCHUNK + c) * 32 + lane) * 8;
            ld8(x + base + col, v[c]);
            if (thr) {
                bool k[8];
                keep8(seed, offset, base + col, thr, k);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[c][j] = k[j] ? v[c][j] * scale : 0.f;
            }
            if (residual) {
                float r[8];
                ld8(residual + base + col, r);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[c][j] += r[j];
            }
            if (z_out) {
                if (live) st8(z_out + base + col, v[c]);
                // the backward reads z in storage precision: normalise the same values
#pragma unroll
                for (int j = 0; j < 8; ++j) v[c][j] = to_f32<T>(from_f32<T>(v[c][j]));
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) s += v[c][j];
        }
        const float mean = group_sum<WPR>(s, sm, warp, lane) * (1.f / H);
        float sq = 0.f;
#pragma unroll
        for (int c = 0; c < NCHUNK; ++c)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float d = v[c][j] - mean;
                sq += d * d;
            }
        const float rstd = rsqrtf(group_sum<WPR>(sq, sm, warp, lane) * (1.f / H) + eps);
        if (!live) continue;
        if (lane == 0 && part == 0) {
            mean_out[row] = mean;
            rstd_out[row] = rstd;
        }
#pragma unroll
        for (int c = 0; c < NCHUNK; ++c) {
            float o[8], g[8], b[8];
            ld8(gamma + ((part * NCHUNK + c) * 32 + lane) * 8, g);
            ld8(beta + ((part * NCHUNK + c) * 32 + lane) * 8, b);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = (v[c][j] - mean) * rstd * g[j] + b[j];
            st8(y + base + ((part * NCHUNK + c) * 32 + lane) * 8, o);
        }
    }
}

// scratch layout: partial[blockIdx][0][H] = dgamma, partial[blockIdx][1][H] = dbeta
template <typename T, int NCHUNK, int WPR>
__global__ void __launch_bounds__(LN_THREADS)
    ln_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ z, const T* __restrict__ gamma,
                  const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                  T* __restrict__ dz_out, T* __restrict__ dx_out, float* __restrict__ partial,
                  int rows, uint32_t thr, float scale, uint64_t seed, uint64_t offset) {
    constexpr int H = NCHUNK * 256 * WPR;
    constexpr int RPB = LN_WARPS / WPR;
    __shared__ float red[LN_WARPS][256 + 8];
    __shared__ float sm1[LN_WARPS], sm2[LN_WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slot = warp / WPR, part = warp % WPR;
    float g[NCHUNK][8], dg[NCHUNK][8], db[NCHUNK][8];
#pragma unroll
    for (int c = 0; c < NCHUNK; ++c) {
        ld8(gamma + ((part * NCHUNK + c) * 32 + lane) * 8, g[c]);
#pragma unroll
        for (int j = 0; j < 8; ++j) dg[c][j] = db[c][j] = 0.f;
    }
    for (int r0 = blockIdx.x * RPB; r0 < rows; r0 += gridDim.x * RPB) {
        const int row = r0 + slot;
        const bool live = row < rows;
        const size_t base = static_cast<size_t>(live ? row : 0) * H;
        const float mean = mean_in[live ? row : 0], rstd = rstd_in[live ? row : 0];
        float xh[NCHUNK][8], wdy[NCHUNK][8];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int c = 0; c < NCHUNK; ++c) {
            const int col = ((part * NCHUNK + c) * 32 + lane) * 8;
            float d[8], zz[8];
            ld8(dy + base + col, d);
            ld8(z + base + col, zz);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (!live) d[j] = 0.f;
                xh[c][j] = (zz[j] - mean) * rstd;
                wdy[c][j] = d[j] * g[c][j];
                s1 += wdy[c][j];
                s2 += wdy[c][j] * xh[c][j];
                dg[c][j] += d[j] * xh[c][j];
                db[c][j] += d[j];
            }
        }
        s1 = group_sum<WPR>(s1, sm1, warp, lane) * (1.f / H);
        s2 = group_sum<WPR>(s2, sm2, warp, lane) * (1.f / H);
        if (!live) continue;
#pragma unroll
        for (int c = 0; c < NCHUNK; ++c) {
            const int col = ((part * NCHUNK + c) * 32 + lane) * 8;
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = rstd * (wdy[c][j] - s1 - xh[c][j] * s2);
            st8(dz_out + base + col, o);
            if (dx_out) {
                bool k[8];
                keep8(seed, offset, base + col, thr, k);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = k[j] ? o[j] * scale : 0.f;
                st8(dx_out + base + col, o);
            }
        }
    }
    // reduce the per-warp partials across the CTA, one 256-column slab at a time
    float* out_g = partial + static_cast<size_t>(blockIdx.x) * 2 * H;
    float* out_b = out_g + H;
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
        for (int c = 0; c < NCHUNK; ++c) {
            __syncthreads();
#pragma unroll
            for (int j = 0; j < 8; ++j) red[warp][lane * 8 + j] = pass == 0 ? dg[c][j] : db[c][j];
            __syncthreads();
            const int t = threadIdx.x;  // 256 threads, 256 columns
#pragma unroll
            for (int pt = 0; pt < WPR; ++pt) {
                float s = 0.f;
#pragma unroll
                for (int sl = 0; sl < RPB; ++sl) s += red[sl * WPR + pt][t];
                (pass == 0 ? out_g : out_b)[(pt * NCHUNK + c) * 256 + t] = s;
            }
        }
    }
}

// dgamma[h] (+)= sum_blocks partial[b][0][h]; dbeta likewise.  grid = 2H/32 blocks of (32, 8).
__global__ void ln_bwd_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dgamma,
                                     float* __restrict__ dbeta, int nblocks, int H,
                                     int accumulate) {
    __shared__ float red[8][33];
    const int col2 = blockIdx.x * 32 + threadIdx.x;  // in [0, 2H)
    float s = 0.f;
    for (int b = threadIdx.y; b < nblocks; b += 8) s += partial[static_cast<size_t>(b) * 2 * H + col2];
    red[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0) {
#pragma unroll
        for (int w = 1; w < 8; ++w) s += red[w][threadIdx.x];
        float* dst = col2 < H ? dgamma + col2 : dbeta + (col2 - H);
        *dst = accumulate ? *dst + s : s;
    }
}

template <typename T, int NCHUNK, int WPR>
static int launch_fwd(const void* x, const void* res, const void* g, const void* b, void* y,
                      void* z, float* mean, float* rstd, int rows, float eps, float p,
                      uint64_t seed, uint64_t offset, cudaStream_t st) {
    const uint32_t thr = p > 0.f ? drop_threshold(p) : 0u;
    const float scale = p > 0.f ? 1.f / (1.f - p) : 1.f;
    constexpr int RPB = LN_WARPS / WPR;
    int grid = (rows + RPB - 1) / RPB;
    const int cap = 148 * 12;
    if (grid > cap) grid = cap;
    ln_fwd_kernel<T, NCHUNK, WPR><<<grid, LN_THREADS, 0, st>>>(
        static_cast<const T*>(x), static_cast<const T*>(res), static_cast<const T*>(g),
        static_cast<const T*>(b), static_cast<T*>(y), static_cast<T*>(z), mean, rstd, rows, eps,
        thr, scale, seed, offset);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

template <typename T, int NCHUNK, int WPR>
static int launch_bwd(const void* dy, const void* z, const void* g, const float* mean,
                      const float* rstd, void* dz, void* dx, float* partial, int grid, int rows,
                      float p, uint64_t seed, uint64_t offset, cudaStream_t st) {
    const uint32_t thr = p > 0.f ? drop_threshold(p) : 0u;
    const float scale = p > 0.f ? 1.f / (1.f - p) : 1.f;
    ln_bwd_kernel<T, NCHUNK, WPR><<<grid, LN_THREADS, 0, st>>>(
        static_cast<const T*>(dy), static_cast<const T*>(z), static_cast<const T*>(g), mean, rstd,
        static_cast<T*>(dz), static_cast<T*>(p > 0.f ? dx : nullptr), partial, rows, thr, scale,
        seed, offset);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace rb

#define RB_LN_DISPATCH(T, FN, ...)                      \
    switch (H / 256) {                                  \
        case 1: return rb::FN<T, 1, 1>(__VA_ARGS__);    \
        case 2: return rb::FN<T, 2, 1>(__VA_ARGS__);    \
        case 3: return rb::FN<T, 3, 1>(__VA_ARGS__);    \
        case 4: return rb::FN<T, 2, 2>(__VA_ARGS__);    \
        case 6: return rb::FN<T, 3, 2>(__VA_ARGS__);    \
        case 8: return rb::FN<T, 2, 4>(__VA_ARGS__);    \
        case 12: return rb::FN<T, 3, 4>(__VA_ARGS__);   \
        case 16: return rb::FN<T, 4, 4>(__VA_ARGS__);   \
        default: return -2;                             \
    }

// The forward kernel prefers fewer elements per thread (more warps per row): fewer registers, more CTAs
// per SM, more loads in flight (measured at H = 1024: 0.69 of the copy bandwidth against 0.63).
#define RB_LN_DISPATCH_FWD(T, FN, ...)                  \
    switch (H / 256) {                                  \
        case 1: return rb::FN<T, 1, 1>(__VA_ARGS__);    \
        case 2: return rb::FN<T, 2, 1>(__VA_ARGS__);    \
        case 3: return rb::FN<T, 3, 1>(__VA_ARGS__);    \
        case 4: return rb::FN<T, 2, 2>(__VA_ARGS__);    \
        case 6: return rb::FN<T, 3, 2>(__VA_ARGS__);    \
        case 8: return rb::FN<T, 2, 4>(__VA_ARGS__);    \
        case 12: return rb::FN<T, 3, 4>(__VA_ARGS__);   \
        case 16: return rb::FN<T, 4, 4>(__VA_ARGS__);   \
        default: return -2;                             \
    }

// 1 when H is a width the register-resident kernels cover
extern "C" int rb_ln_supported(int H) {
    if (H % 256) return 0;
    switch (H / 256) {
        case 1: case 2: case 3: case 4: case 6: case 8: case 12: case 16: return 1;
        default: return 0;
    }
}

// number of CTAs (= rows of the scratch buffer) the backward uses for `rows`
extern "C" int rb_ln_bwd_grid(int rows) {
    int grid = (rows + 1) / 2;
    const int cap = 148 * 2;
    return grid > cap ? cap : (grid < 1 ? 1 : grid);
}

// dtype: 0 fp16, 1 bf16.  residual / z may be null (z == x then).
extern "C" int rb_ln_fwd(const void* x, const void* residual, const void* gamma, const void* beta,
                         void* y, void* z, float* mean, float* rstd, int rows, int H, float eps,
                         float p, uint64_t seed, uint64_t offset, int dtype, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows <= 0) return 0;
    if (dtype == 1) {
        RB_LN_DISPATCH_FWD(__nv_bfloat16, launch_fwd, x, residual, gamma, beta, y, z, mean, rstd, rows,
                       eps, p, seed, offset, st)
    } else {
        RB_LN_DISPATCH_FWD(__half, launch_fwd, x, residual, gamma, beta, y, z, mean, rstd, rows, eps, p,
                       seed, offset, st)
    }
}

// `partial` is scratch of rb_ln_bwd_grid(rows) * 2 * H floats.  dgamma / dbeta are
// fp32 [H]; accumulate != 0 adds to them.
extern "C" int rb_ln_bwd(const void* dy, const void* z, const void* gamma, const float* mean,
                         const float* rstd, void* dz, void* dx, float* dgamma, float* dbeta,
                         float* partial, int rows, int H, float p, uint64_t seed, uint64_t offset,
                         int accumulate, int dtype, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows <= 0) return 0;
    const int grid = rb_ln_bwd_grid(rows);
    int rc;
    auto run = [&]() -> int {
        if (dtype == 1) {
            RB_LN_DISPATCH(__nv_bfloat16, launch_bwd, dy, z, gamma, mean, rstd, dz, dx, partial,
                           grid, rows, p, seed, offset, st)
        } else {
            RB_LN_DISPATCH(__half, launch_bwd, dy, z, gamma, mean, rstd, dz, dx, partial, grid,
                           rows, p, seed, offset, st)
        }
    };
    rc = run();
    if (rc) return rc;
    rb::ln_bwd_reduce_kernel<<<2 * H / 32, dim3(32, 8), 0, st>>>(partial, dgamma, dbeta, grid, H,
                                                                 accumulate);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// ---------------------------------------------------------------------------
// Allocation-free variant of rb_ln_bwd (declared and documented in norm_noalloc.h)
// ---------------------------------------------------------------------------
#include <atomic>

#include "norm_noalloc.h"

// Scratch for the per-CTA partial sums of dgamma / dbeta.  In host code this name is only a
// stand-in for the symbol: kernels must be given the address cudaGetSymbolAddress returns.
static __device__ __align__(256) float g_ln_noalloc_scratch[RB_LN_NOALLOC_MAX_FLOATS];

// One cached address per device.  The slots are atomics: two host threads that make their first call on a
// device at the same time both resolve the symbol and store the same value, which is harmless.
static float* ln_noalloc_scratch_ptr() {
    static std::atomic<float*> ptrs[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    float* p = ptrs[dev].load(std::memory_order_acquire);
    if (!p) {
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_ln_noalloc_scratch) != cudaSuccess) return nullptr;
        ptrs[dev].store(p, std::memory_order_release);
    }
    return p;
}

extern "C" const char* rb_ln_bwd_noalloc_strerror(int code) {
    switch (code) {
        case RB_LN_NOALLOC_OK: return "ok";
        case RB_LN_NOALLOC_LAUNCH_FAILED: return "kernel launch failed";
        case RB_LN_NOALLOC_BAD_WIDTH: return "unsupported row width H (supported: 256, 512, 768, 1024, 1536, 2048, 3072, 4096)";
        case RB_LN_NOALLOC_NO_SYMBOL: return "could not resolve the device address of the built-in scratch array";
        case RB_LN_NOALLOC_TOO_LARGE: return "rows x H needs more scratch than the built-in array holds (RB_LN_NOALLOC_MAX_FLOATS)";
        default: return "unknown error";
    }
}

extern "C" int rb_ln_bwd_noalloc(const void* dy, const void* z, const void* gamma, const float* mean,
                                 const float* rstd, void* dz, void* dx, float* dgamma, float* dbeta, int rows,
                                 int H, float p, uint64_t seed, uint64_t offset, int accumulate, int dtype,
                                 void* stream) {
    if (rows <= 0) return RB_LN_NOALLOC_OK;
    if (!rb_ln_supported(H)) return RB_LN_NOALLOC_BAD_WIDTH;
    const long long need = static_cast<long long>(rb_ln_bwd_grid(rows)) * 2 * H;
    if (need > RB_LN_NOALLOC_MAX_FLOATS) return RB_LN_NOALLOC_TOO_LARGE;
    float* scratch = ln_noalloc_scratch_ptr();
    if (!scratch) return RB_LN_NOALLOC_NO_SYMBOL;
    const int rc = rb_ln_bwd(dy, z, gamma, mean, rstd, dz, dx, dgamma, dbeta, scratch, rows, H, p, seed, offset,
                             accumulate, dtype, stream);
    return rc == 0 ? RB_LN_NOALLOC_OK : (rc == -2 ? RB_LN_NOALLOC_BAD_WIDTH : RB_LN_NOALLOC_LAUNCH_FAILED);
}
