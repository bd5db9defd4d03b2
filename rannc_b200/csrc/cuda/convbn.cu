// Convolution support kernels and batch normalisation for channels-last (NHWC) activations.
//
// A convolution runs as a tcgen05 GEMM (gemm_tcgen05.cu): a 1x1 convolution IS a GEMM over the
// [N*H*W, C] view of an NHWC tensor, and a k x k convolution becomes one after `im2col` lays the k*k
// shifted windows of every output pixel side by side ([N*Ho*Wo, k*k*C], tap-major).  For the wide
// ResNets this framework is benchmarked on (C >= 512) the gathered matrix is read at more than 1000
// FLOP per byte, so the gather is a small fraction of the GEMM time.  `col2im` is the adjoint (input
// gradient), written as a gather so that no atomics are needed.
//
// Batch normalisation over [R = N*H*W, C]: per-channel sums in fp32 (one pass, 16-byte loads, 8 channels
// per thread), then one element-wise pass that normalises, optionally adds a residual and applies ReLU.
// Backward: one reduction pass (sum dy, sum dy * xhat, with the ReLU mask taken from the saved output),
// one element-wise pass.  Running statistics are updated by the finalising kernel, per replica (no
// cross-rank synchronisation), like the reference, which runs aten::batch_norm inside each replica's
// TorchScript interpreter (src/torch/TorchDriver.cpp:566) and treats the statistics as non-gradient
// parameters (src/comp/ParamStorage.cpp:209-211).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tc_common.cuh"

namespace rb {

template <typename T>
__device__ __forceinline__ void ld8(const T* p, float (&v)[8]) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = to_f32<T>(e[j]);
}
template <typename T>
__device__ __forceinline__ void st8(T* p, const float (&v)[8]) {
    uint4 q;
    q.x = pack2<T>(v[0], v[1]);
    q.y = pack2<T>(v[2], v[3]);
    q.z = pack2<T>(v[4], v[5]);
    q.w = pack2<T>(v[6], v[7]);
    *reinterpret_cast<uint4*>(p) = q;
}

// ---------------------------------------------------------------------------------------------------
// im2col / col2im, NHWC, square kernel k, stride s, padding pad.  C % 8 == 0.
// cols[(n, ho, wo), (ky, kx, c)] = x[n, ho*s - pad + ky, wo*s - pad + kx, c]  (0 outside)
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void im2col_kernel(const T* __restrict__ x, T* __restrict__ cols, int N, int H, int W, int C, int Ho,
                              int Wo, int k, int s, int pad) {
    // one thread per (output pixel, 8 channels): the pixel coordinates are decoded once, the taps are a loop
    const int cv = C / 8;
    const long long total = static_cast<long long>(N) * Ho * Wo * cv;
    const long long row_len = static_cast<long long>(k) * k * C;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c8 = static_cast<int>(i % cv);
        const long long pix = i / cv;
        const int wo = static_cast<int>(pix % Wo);
        const int ho = static_cast<int>((pix / Wo) % Ho);
        const int n = static_cast<int>(pix / (static_cast<long long>(Wo) * Ho));
        const T* xin = x + static_cast<long long>(n) * H * W * C + c8 * 8;
        T* out = cols + pix * row_len + c8 * 8;
        for (int ky = 0; ky < k; ++ky) {
            const int h = ho * s - pad + ky;
            const bool hin = h >= 0 && h < H;
#pragma unroll 3
            for (int kx = 0; kx < k; ++kx) {
                const int w = wo * s - pad + kx;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (hin && w >= 0 && w < W)
                    v = *reinterpret_cast<const uint4*>(xin + (static_cast<long long>(h) * W + w) * C);
                *reinterpret_cast<uint4*>(out + static_cast<long long>(ky * k + kx) * C) = v;
            }
        }
    }
}

// dx[n, h, w, c] = sum over the taps (ky, kx) and output pixels that read (h, w) of dcols
template <typename T>
__global__ void col2im_kernel(const T* __restrict__ dcols, T* __restrict__ dx, int N, int H, int W, int C, int Ho,
                              int Wo, int k, int s, int pad) {
    const int cv = C / 8;
    const long long total = static_cast<long long>(N) * H * W * cv;
    const long long row_len = static_cast<long long>(k) * k * C;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c8 = static_cast<int>(i % cv);
        long long r = i / cv;
        const int w = static_cast<int>(r % W);
        r /= W;
        const int h = static_cast<int>(r % H);
        const int n = static_cast<int>(r / H);
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int ky = 0; ky < k; ++ky) {
            const int hn = h + pad - ky;
            if (hn < 0 || hn % s) continue;
            const int ho = hn / s;
            if (ho >= Ho) continue;
            for (int kx = 0; kx < k; ++kx) {
                const int wn = w + pad - kx;
                if (wn < 0 || wn % s) continue;
                const int wo = wn / s;
                if (wo >= Wo) continue;
                float v[8];
                ld8(dcols + ((static_cast<long long>(n) * Ho + ho) * Wo + wo) * row_len +
                        (static_cast<long long>(ky) * k + kx) * C + c8 * 8,
                    v);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += v[j];
            }
        }
        st8(dx + i * 8, acc);
    }
}

// ---------------------------------------------------------------------------------------------------
// batch norm
// ---------------------------------------------------------------------------------------------------
// part[0][c] += sum_r a(r, c), part[1][c] += sum_r a(r, c) * b(r, c); a thread owns 8 adjacent channels,
// a block of (32, 8) covers 256 channels, rows are strided over threadIdx.y and blockIdx.y.
//   MODE 0 (statistics):  a = x,                 b = x
//   MODE 1 (backward):    a = dy masked by relu, b = xhat = (x - mean) * rstd
template <typename T, int MODE>
__global__ void bn_reduce_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ y,
                                 const float* __restrict__ mean, const float* __restrict__ rstd,
                                 float* __restrict__ part, long long R, int C, int relu) {
    __shared__ float red[2][8][256 + 8];
    const int col = blockIdx.x * 256 + threadIdx.x * 8;
    float s0[8], s1[8], mu[8], rs[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) s0[j] = s1[j] = 0.f, mu[j] = 0.f, rs[j] = 1.f;
    if (col < C) {
        if (MODE == 1) {
#pragma unroll
            for (int j = 0; j < 8; ++j) mu[j] = mean[col + j], rs[j] = rstd[col + j];
        }
        for (long long r = blockIdx.y * 8 + threadIdx.y; r < R; r += static_cast<long long>(gridDim.y) * 8) {
            float a[8];
            ld8(x + r * C + col, a);
            if (MODE == 0) {
#pragma unroll
                for (int j = 0; j < 8; ++j) s0[j] += a[j], s1[j] = fmaf(a[j], a[j], s1[j]);
            } else {
                float g[8];
                ld8(dy + r * C + col, g);
                if (relu) {
                    float o[8];
                    ld8(y + r * C + col, o);
#pragma unroll
                    for (int j = 0; j < 8; ++j) g[j] = o[j] > 0.f ? g[j] : 0.f;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) s0[j] += g[j], s1[j] = fmaf(g[j], (a[j] - mu[j]) * rs[j], s1[j]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        red[0][threadIdx.y][threadIdx.x * 8 + j] = s0[j];
        red[1][threadIdx.y][threadIdx.x * 8 + j] = s1[j];
    }
    __syncthreads();
    const int t = threadIdx.y * 32 + threadIdx.x;
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) a0 += red[0][w][t], a1 += red[1][w][t];
    const int c = blockIdx.x * 256 + t;
    if (c < C) {
        atomicAdd(part + c, a0);
        atomicAdd(part + C + c, a1);
    }
}

// mean / rstd from the sums, running statistics (momentum, unbiased variance); the per-channel scale and shift
// of the element-wise pass replace the sums in `part`: y = x * part[0][c] + part[1][c]
__global__ void bn_finalize_kernel(float* __restrict__ part, float* __restrict__ mean, float* __restrict__ rstd,
                                   const float* __restrict__ gamma, const float* __restrict__ beta,
                                   float* __restrict__ run_mean, float* __restrict__ run_var, long long R, int C,
                                   float eps, float momentum) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const float inv = 1.f / static_cast<float>(R);
    const float m = part[c] * inv;
    const float var = fmaxf(part[C + c] * inv - m * m, 0.f);
    const float rs = rsqrtf(var + eps);
    mean[c] = m;
    rstd[c] = rs;
    const float sc = rs * gamma[c];
    part[c] = sc;
    part[C + c] = beta[c] - m * sc;
    if (run_mean) {
        const float unbiased = R > 1 ? var * static_cast<float>(R) / static_cast<float>(R - 1) : var;
        run_mean[c] = (1.f - momentum) * run_mean[c] + momentum * m;
        run_var[c] = (1.f - momentum) * run_var[c] + momentum * unbiased;
    }
}

// backward coefficients: dx = A g + B x + Cc with A = gamma rstd, B = -gamma rstd^2 sum(g xhat) / R,
// Cc = -A sum(g) / R - B mean; written behind the two sums: part[2..4][C]
__global__ void bn_bwd_coef_kernel(float* __restrict__ part, const float* __restrict__ mean,
                                   const float* __restrict__ rstd, const float* __restrict__ gamma, long long R,
                                   int C) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const float inv = 1.f / static_cast<float>(R);
    const float A = gamma[c] * rstd[c];
    const float B = -A * rstd[c] * part[C + c] * inv;
    part[2 * C + c] = A;
    part[3 * C + c] = B;
    part[4 * C + c] = -A * part[c] * inv - B * mean[c];
}

__device__ __forceinline__ void ldf8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}

// y = act(x * scale + shift (+ residual)); scale / shift per channel, 8 channels = two 16-byte loads each
template <typename T>
__global__ void bn_apply_kernel(const T* __restrict__ x, const T* __restrict__ res, const float* __restrict__ scale,
                                const float* __restrict__ shift, T* __restrict__ y, long long R, int C, int relu) {
    const int cv = C / 8;
    const long long total = R * cv;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(i % cv) * 8;
        float v[8], o[8], sc[8], sh[8];
        ld8(x + i * 8, v);
        ldf8(scale + c, sc);
        ldf8(shift + c, sh);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = fmaf(v[j], sc[j], sh[j]);
        if (res) {
            float rr[8];
            ld8(res + i * 8, rr);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] += rr[j];
        }
        if (relu) {
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = fmaxf(o[j], 0.f);
        }
        st8(y + i * 8, o);
    }
}

// dx = A g + B x + Cc, g = dy masked by relu; dres = g (optional).  coef = [A, B, Cc][C]
template <typename T>
__global__ void bn_bwd_apply_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ y,
                                    const float* __restrict__ coef, T* __restrict__ dx, T* __restrict__ dres,
                                    long long R, int C, int relu) {
    const int cv = C / 8;
    const long long total = R * cv;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(i % cv) * 8;
        float v[8], g[8], o[8], A[8], B[8], Cc[8];
        ld8(x + i * 8, v);
        ld8(dy + i * 8, g);
        if (relu) {
            float yy[8];
            ld8(y + i * 8, yy);
#pragma unroll
            for (int j = 0; j < 8; ++j) g[j] = yy[j] > 0.f ? g[j] : 0.f;
        }
        ldf8(coef + c, A);
        ldf8(coef + C + c, B);
        ldf8(coef + 2 * C + c, Cc);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = fmaf(A[j], g[j], fmaf(B[j], v[j], Cc[j]));
        st8(dx + i * 8, o);
        if (dres) st8(dres + i * 8, g);
    }
}

static inline int ew_grid(long long n) {
    long long g = (n + 255) / 256;
    const long long cap = 148LL * 16;
    return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace rb

// dtype: 1 = bf16, 0 = fp16
extern "C" int rb_im2col(const void* x, void* cols, int N, int H, int W, int C, int k, int s, int pad, int dtype,
                         void* stream) {
    using namespace rb;
    if (C % 8 || k < 1 || s < 1) return -2;
    const int Ho = (H + 2 * pad - k) / s + 1, Wo = (W + 2 * pad - k) / s + 1;
    if (Ho <= 0 || Wo <= 0) return -2;
    const long long total = static_cast<long long>(N) * Ho * Wo * k * k * (C / 8);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == 1)
        im2col_kernel<__nv_bfloat16><<<ew_grid(total), 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(cols), N, H, W, C, Ho, Wo, k, s, pad);
    else
        im2col_kernel<__half><<<ew_grid(total), 256, 0, st>>>(static_cast<const __half*>(x),
                                                             static_cast<__half*>(cols), N, H, W, C, Ho, Wo, k, s, pad);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int rb_col2im(const void* dcols, void* dx, int N, int H, int W, int C, int k, int s, int pad, int dtype,
                         void* stream) {
    using namespace rb;
    if (C % 8 || k < 1 || s < 1) return -2;
    const int Ho = (H + 2 * pad - k) / s + 1, Wo = (W + 2 * pad - k) / s + 1;
    if (Ho <= 0 || Wo <= 0) return -2;
    const long long total = static_cast<long long>(N) * H * W * (C / 8);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == 1)
        col2im_kernel<__nv_bfloat16><<<ew_grid(total), 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(dcols), static_cast<__nv_bfloat16*>(dx), N, H, W, C, Ho, Wo, k, s, pad);
    else
        col2im_kernel<__half><<<ew_grid(total), 256, 0, st>>>(static_cast<const __half*>(dcols),
                                                             static_cast<__half*>(dx), N, H, W, C, Ho, Wo, k, s, pad);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Forward statistics + normalisation.  part: fp32 [2, C] scratch (zeroed here); mean / rstd: fp32 [C] outputs;
// run_mean / run_var may be null (evaluation of a frozen layer is not handled here: pass training only).
extern "C" int rb_bn_fwd(const void* x, const void* res, const float* gamma, const float* beta, void* y, float* part,
                         float* mean, float* rstd, float* run_mean, float* run_var, long long R, int C, float eps,
                         float momentum, int relu, int dtype, void* stream) {
    using namespace rb;
    if (C % 8 || R <= 0) return -2;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaMemsetAsync(part, 0, 2 * sizeof(float) * C, st);
    int split = static_cast<int>((R + 63) / 64);
    const int colblocks = (C + 255) / 256;
    const int want = (148 * 4 + colblocks - 1) / colblocks;
    if (split > want) split = want;
    if (split < 1) split = 1;
    dim3 grid(colblocks, split), block(32, 8);
    if (dtype == 1)
        bn_reduce_kernel<__nv_bfloat16, 0><<<grid, block, 0, st>>>(static_cast<const __nv_bfloat16*>(x), nullptr, nullptr,
                                                                  nullptr, nullptr, part, R, C, 0);
    else
        bn_reduce_kernel<__half, 0><<<grid, block, 0, st>>>(static_cast<const __half*>(x), nullptr, nullptr, nullptr,
                                                           nullptr, part, R, C, 0);
    bn_finalize_kernel<<<(C + 255) / 256, 256, 0, st>>>(part, mean, rstd, gamma, beta, run_mean, run_var, R, C, eps,
                                                        momentum);
    const long long total = R * (C / 8);
    if (dtype == 1)
        bn_apply_kernel<__nv_bfloat16><<<ew_grid(total), 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(res), part, part + C,
            static_cast<__nv_bfloat16*>(y), R, C, relu);
    else
        bn_apply_kernel<__half><<<ew_grid(total), 256, 0, st>>>(static_cast<const __half*>(x),
                                                               static_cast<const __half*>(res), part, part + C,
                                                               static_cast<__half*>(y), R, C, relu);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Backward.  part: fp32 [5, C] scratch; on return part[0] = d beta, part[1] = d gamma (part[2..4]: coefficients).
extern "C" int rb_bn_bwd(const void* x, const void* dy, const void* y, const float* mean, const float* rstd,
                         const float* gamma, float* part, void* dx, void* dres, long long R, int C, int relu, int dtype,
                         void* stream) {
    using namespace rb;
    if (C % 8 || R <= 0) return -2;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaMemsetAsync(part, 0, 2 * sizeof(float) * C, st);
    int split = static_cast<int>((R + 63) / 64);
    const int colblocks = (C + 255) / 256;
    const int want = (148 * 4 + colblocks - 1) / colblocks;
    if (split > want) split = want;
    if (split < 1) split = 1;
    dim3 grid(colblocks, split), block(32, 8);
    const long long total = R * (C / 8);
    if (dtype == 1) {
        bn_reduce_kernel<__nv_bfloat16, 1><<<grid, block, 0, st>>>(
            static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy),
            static_cast<const __nv_bfloat16*>(y), mean, rstd, part, R, C, relu);
        bn_bwd_coef_kernel<<<(C + 255) / 256, 256, 0, st>>>(part, mean, rstd, gamma, R, C);
        bn_bwd_apply_kernel<__nv_bfloat16><<<ew_grid(total), 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy),
            static_cast<const __nv_bfloat16*>(y), part + 2 * C, static_cast<__nv_bfloat16*>(dx),
            static_cast<__nv_bfloat16*>(dres), R, C, relu);
    } else {
        bn_reduce_kernel<__half, 1><<<grid, block, 0, st>>>(static_cast<const __half*>(x),
                                                           static_cast<const __half*>(dy),
                                                           static_cast<const __half*>(y), mean, rstd, part, R, C, relu);
        bn_bwd_coef_kernel<<<(C + 255) / 256, 256, 0, st>>>(part, mean, rstd, gamma, R, C);
        bn_bwd_apply_kernel<__half><<<ew_grid(total), 256, 0, st>>>(
            static_cast<const __half*>(x), static_cast<const __half*>(dy), static_cast<const __half*>(y),
            part + 2 * C, static_cast<__half*>(dx), static_cast<__half*>(dres), R, C, relu);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
