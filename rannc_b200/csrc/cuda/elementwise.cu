// Memory-bound element-wise and reduction kernels: GELU forward/backward,
// dropout (Philox counter, mask regenerated in the backward), bias gradient
// (column sum), 16-bit -> fp32 gradient accumulation, embedding gather and its
// scatter-add backward, micro-batch row pack/unpack.
//
// They take the place of the ATen element-wise kernels the reference launches
// one node at a time from its interpreter (src/torch/TorchDriver.cpp:566) and of
// the pad / slice / cat helpers of src/torch/TorchUtil.cpp:785-843,1091-1136.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "debug_check.cuh"
#include "philox.cuh"
#include "tc_common.cuh"

namespace rb {

template <typename T>
__device__ __forceinline__ void ld8e(const T* p, float (&v)[8]) {
    uint4 q = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = to_f32<T>(e[j]);
}
template <typename T>
__device__ __forceinline__ void st8e(T* p, const float (&v)[8]) {
    uint4 q;
    T* e = reinterpret_cast<T*>(&q);
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = from_f32<T>(v[j]);
    *reinterpret_cast<uint4*>(p) = q;
}

// mode 0: y = gelu(x); mode 1: y = dy * gelu'(x)
template <typename T>
__global__ void gelu_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ y,
                            size_t n, int mode) {
    const size_t nv = n / 8;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nv;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float a[8], o[8];
        ld8e(x + i * 8, a);
        if (mode == 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = gelu_erf(a[j]);
        } else {
            float d[8];
            ld8e(dy + i * 8, d);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = d[j] * gelu_erf_grad(a[j]);
        }
        st8e(y + i * 8, o);
    }
    if (blockIdx.x == 0 && threadIdx.x < n % 8) {
        const size_t i = nv * 8 + threadIdx.x;
        const float a = to_f32<T>(x[i]);
        y[i] = from_f32<T>(mode == 0 ? gelu_erf(a) : to_f32<T>(dy[i]) * gelu_erf_grad(a));
    }
}

// y = keep ? x * scale : 0, mask from (seed, offset, linear index)
template <typename T>
__global__ void dropout_kernel(const T* __restrict__ x, T* __restrict__ y, size_t n, uint32_t thr,
                               float scale, uint64_t seed, uint64_t offset) {
    const size_t nv = n / 8;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nv;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float a[8];
        ld8e(x + i * 8, a);
        bool k[8];
        keep8(seed, offset, i * 8, thr, k);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = k[j] ? a[j] * scale : 0.f;
        st8e(y + i * 8, a);
    }
    if (blockIdx.x == 0 && threadIdx.x < n % 8) {
        const size_t i = nv * 8 + threadIdx.x;
        const Philox4 r = philox4x32(seed, offset, i >> 3);
        const uint32_t w = r.v[(i & 7) >> 1];
        const uint32_t bits = (i & 1) ? (w >> 16) : (w & 0xffffu);
        y[i] = from_f32<T>(bits >= thr ? to_f32<T>(x[i]) * scale : 0.f);
    }
}

// out[n] (+)= sum_m x[m, n]; x is [M, N] row-major 16-bit, out fp32.
// grid (ceil(N/64), SPLIT); block (32, 8): thread handles 2 columns.
template <typename T>
__global__ void colsum_kernel(const T* __restrict__ x, float* __restrict__ out, int M, int N,
                              long long ld) {
    __shared__ float red[8][65];
    const int col = blockIdx.x * 64 + threadIdx.x * 2;
    float s0 = 0.f, s1 = 0.f;
    if (col < N) {
        for (int m = blockIdx.y * 8 + threadIdx.y; m < M; m += gridDim.y * 8) {
            const T* p = x + static_cast<long long>(m) * ld + col;
            if (col + 1 < N) {
                s0 += to_f32<T>(p[0]);
                s1 += to_f32<T>(p[1]);
            } else {
                s0 += to_f32<T>(p[0]);
            }
        }
    }
    red[threadIdx.y][threadIdx.x * 2] = s0;
    red[threadIdx.y][threadIdx.x * 2 + 1] = s1;
    __syncthreads();
    if (threadIdx.y == 0) {
#pragma unroll
        for (int w = 1; w < 8; ++w) {
            s0 += red[w][threadIdx.x * 2];
            s1 += red[w][threadIdx.x * 2 + 1];
        }
        if (col < N) atomicAdd(out + col, s0);
        if (col + 1 < N) atomicAdd(out + col + 1, s1);
    }
}

// Vector variant: a thread owns 8 adjacent columns (one 16-byte load per row), a block of (32, 8)
// covers 256 columns; rows are strided over threadIdx.y and blockIdx.y.  Needs N % 8 == 0,
// ld % 8 == 0 and a 16-byte aligned base.
template <typename T>
__global__ void colsum_vec_kernel(const T* __restrict__ x, float* __restrict__ out, int M, int N,
                                  long long ld) {
    __shared__ float red[8][256 + 8];
    const int col = blockIdx.x * 256 + threadIdx.x * 8;
    float s[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j] = 0.f;
    if (col < N) {
        const int step = gridDim.y * 8;
        int m = blockIdx.y * 8 + threadIdx.y;
        // two rows in flight per iteration
        for (; m + step < M; m += 2 * step) {
            float a[8], b[8];
            ld8e(x + static_cast<long long>(m) * ld + col, a);
            ld8e(x + static_cast<long long>(m + step) * ld + col, b);
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j] += a[j] + b[j];
        }
        if (m < M) {
            float a[8];
            ld8e(x + static_cast<long long>(m) * ld + col, a);
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j] += a[j];
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) red[threadIdx.y][threadIdx.x * 8 + j] = s[j];
    __syncthreads();
    const int t = threadIdx.y * 32 + threadIdx.x;  // 256 threads, one column each
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) acc += red[w][t];
    const int c = blockIdx.x * 256 + t;
    if (c < N) atomicAdd(out + c, acc);
}

// dst(fp32) += src(16-bit) * scale
template <typename T>
__global__ void accum_kernel(float* __restrict__ dst, const T* __restrict__ src, size_t n,
                             float scale) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
        dst[i] += to_f32<T>(src[i]) * scale;
}

// dst(16-bit) = src(fp32) * scale
template <typename T>
__global__ void cast_kernel(T* __restrict__ dst, const float* __restrict__ src, size_t n,
                            float scale) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
        dst[i] = from_f32<T>(src[i] * scale);
}

// out[r, :] = table[ids[r], :]  (H % 8 == 0); one warp per row
template <typename T>
__global__ void embed_fwd_kernel(const long long* __restrict__ ids, const T* __restrict__ table,
                                 T* __restrict__ out, int rows, int H, long long vocab) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows) return;
    long long id = ids[warp];
    const bool ok = id >= 0 && id < vocab;
    const uint4* src = reinterpret_cast<const uint4*>(table + (ok ? id : 0) * H);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(warp) * H);
    for (int i = lane; i < H / 8; i += 32) dst[i] = ok ? src[i] : make_uint4(0, 0, 0, 0);
}

// dtable(fp32)[ids[r], :] += dout[r, :] ; rows with id == padding_idx are skipped
template <typename T>
__global__ void embed_bwd_kernel(const long long* __restrict__ ids, const T* __restrict__ dout,
                                 float* __restrict__ dtable, int rows, int H, long long vocab,
                                 long long padding_idx) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows) return;
    const long long id = ids[warp];
    if (id < 0 || id >= vocab || id == padding_idx) return;
    const T* src = dout + static_cast<long long>(warp) * H;
    float* dst = dtable + id * H;
    for (int i = lane; i < H; i += 32) atomicAdd(dst + i, to_f32<T>(src[i]));
}

// Row copy between two row-major buffers with different row offsets; used to
// pack micro-batch slices and pipeline send buffers.  bytes_per_row % 16 == 0.
__global__ void rowcopy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                               long long rows, long long vec_per_row, long long src_ld,
                               long long dst_ld) {
    const long long total = rows * vec_per_row;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = i / vec_per_row, c = i - r * vec_per_row;
        dst[r * dst_ld + c] = src[r * src_ld + c];
    }
}

static inline int grid_for(size_t work, int threads) {
    size_t g = (work + threads - 1) / threads;
    const size_t cap = 148 * 16;
    return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace rb

using namespace rb;

extern "C" int rb_gelu(const void* x, const void* dy, void* y, long long n, int mode, int dtype,
                       void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (n <= 0) return 0;
    const int g = grid_for(n / 8 + 1, 256);
    if (dtype == 1)
        gelu_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                     static_cast<const __nv_bfloat16*>(dy),
                                                     static_cast<__nv_bfloat16*>(y), n, mode);
    else
        gelu_kernel<__half><<<g, 256, 0, st>>>(static_cast<const __half*>(x),
                                              static_cast<const __half*>(dy),
                                              static_cast<__half*>(y), n, mode);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int rb_dropout(const void* x, void* y, long long n, float p, uint64_t seed,
                          uint64_t offset, int dtype, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (n <= 0) return 0;
    const uint32_t thr = drop_threshold(p);
    const float scale = 1.f / (1.f - p);
    const int g = grid_for(n / 8 + 1, 256);
    if (dtype == 1)
        dropout_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                        static_cast<__nv_bfloat16*>(y), n, thr,
                                                        scale, seed, offset);
    else
        dropout_kernel<__half><<<g, 256, 0, st>>>(static_cast<const __half*>(x),
                                                 static_cast<__half*>(y), n, thr, scale, seed,
                                                 offset);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// out must be zeroed by the caller unless it accumulates on purpose
extern "C" int rb_colsum(const void* x, float* out, int M, int N, long long ld, int dtype,
                         void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (M <= 0 || N <= 0) return 0;
    if (N % 8 == 0 && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        const int cols = (N + 255) / 256;
        int split = (148 * 6 + cols - 1) / cols;  // about six blocks per SM in total
        const int max_split = (M + 15) / 16;
        if (split > max_split) split = max_split;
        if (split < 1) split = 1;
        dim3 grid(cols, split), block(32, 8);
        if (dtype == 1)
            colsum_vec_kernel<__nv_bfloat16><<<grid, block, 0, st>>>(static_cast<const __nv_bfloat16*>(x), out, M,
                                                                    N, ld);
        else
            colsum_vec_kernel<__half><<<grid, block, 0, st>>>(static_cast<const __half*>(x), out, M, N, ld);
        return cudaGetLastError() == cudaSuccess ? 0 : -1;
    }
    int split = (M + 255) / 256;
    if (split > 64) split = 64;
    dim3 grid((N + 63) / 64, split), block(32, 8);
    if (dtype == 1)
        colsum_kernel<__nv_bfloat16><<<grid, block, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                            out, M, N, ld);
    else
        colsum_kernel<__half><<<grid, block, 0, st>>>(static_cast<const __half*>(x), out, M, N, ld);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int rb_accum_f32(float* dst, const void* src, long long n, float scale, int dtype,
                            void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (n <= 0) return 0;
    const int g = grid_for(n, 256);
    if (dtype == 1)
        accum_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(dst, static_cast<const __nv_bfloat16*>(src),
                                                      n, scale);
    else
        accum_kernel<__half><<<g, 256, 0, st>>>(dst, static_cast<const __half*>(src), n, scale);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int rb_cast_from_f32(void* dst, const float* src, long long n, float scale, int dtype,
                                void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (n <= 0) return 0;
    const int g = grid_for(n, 256);
    if (dtype == 1)
        cast_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<__nv_bfloat16*>(dst), src, n,
                                                     scale);
    else
        cast_kernel<__half><<<g, 256, 0, st>>>(static_cast<__half*>(dst), src, n, scale);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int rb_embed_fwd(const long long* ids, const void* table, void* out, int rows, int H,
                            long long vocab, int dtype, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows <= 0) return 0;
    RB_DEBUG_ARG(H % 8 == 0, "rb_embed_fwd: H must be a multiple of 8");
    if (H % 8) return -2;
    RB_DEBUG_RANGE(ids, rows, 0, vocab, -1 - vocab, st);
    const int g = (rows * 32 + 255) / 256;
    if (dtype == 1)
        embed_fwd_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(
            ids, static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), rows,
            H, vocab);
    else
        embed_fwd_kernel<__half><<<g, 256, 0, st>>>(ids, static_cast<const __half*>(table),
                                                   static_cast<__half*>(out), rows, H, vocab);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int rb_embed_bwd(const long long* ids, const void* dout, float* dtable, int rows, int H,
                            long long vocab, long long padding_idx, int dtype, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows <= 0) return 0;
    RB_DEBUG_RANGE(ids, rows, 0, vocab, padding_idx, st);
    const int g = (rows * 32 + 255) / 256;
    if (dtype == 1)
        embed_bwd_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(
            ids, static_cast<const __nv_bfloat16*>(dout), dtable, rows, H, vocab, padding_idx);
    else
        embed_bwd_kernel<__half><<<g, 256, 0, st>>>(ids, static_cast<const __half*>(dout), dtable,
                                                   rows, H, vocab, padding_idx);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// src/dst row strides in bytes; bytes_per_row, strides and both bases 16 B aligned
extern "C" int rb_rowcopy(const void* src, void* dst, long long rows, long long bytes_per_row,
                          long long src_stride_bytes, long long dst_stride_bytes, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows <= 0 || bytes_per_row <= 0) return 0;
    RB_DEBUG_ARG(((bytes_per_row | src_stride_bytes | dst_stride_bytes) & 15) == 0,
                 "rb_rowcopy: row length and strides must be multiples of 16 bytes");
    RB_DEBUG_ARG(((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0,
                 "rb_rowcopy: both buffers must be 16-byte aligned");
    RB_DEBUG_ARG(src_stride_bytes >= bytes_per_row && dst_stride_bytes >= bytes_per_row,
                 "rb_rowcopy: a row stride shorter than the row makes rows overlap");
    if ((bytes_per_row | src_stride_bytes | dst_stride_bytes) & 15) return -2;
    if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) return -2;
    const long long vpr = bytes_per_row / 16;
    const int g = grid_for(static_cast<size_t>(rows * vpr), 256);
    rowcopy_kernel<<<g, 256, 0, st>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst),
                                      rows, vpr, src_stride_bytes / 16, dst_stride_bytes / 16);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
