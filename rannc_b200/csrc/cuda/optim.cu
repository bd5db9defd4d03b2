// Fused optimizer kernels over flat buffers.
//
// All parameters of a rank live in one flat fp32 master buffer with a matching
// flat fp32 gradient buffer, Adam moments and a 16-bit model copy, so a step
// is ONE launch: un-scale (loss scale, clip factor), skip on overflow, Adam or
// SGD-momentum update, and write-back of the 16-bit parameters.  The norm
// kernel yields the global L2 norm and the overflow flag in one pass (a
// non-finite gradient makes the sum non-finite), so no per-parameter
// `.item()` is needed.
//
// Takes the place of the stock / Apex optimizers stepping over the patched
// parameter lists (pyrannc/opt.py:205-312), the Apex unscale + overflow check
// (pyrannc/amp/__init__.py:44-65) and the per-parameter norm loop of
// src/comp/ParamStorage.cpp:721-819.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tc_common.cuh"

namespace rb {

struct AdamHyper {
    float lr, beta1, beta2, eps, weight_decay;
    float bias_corr1, bias_corr2;  // 1 - beta^t
    int adamw;                     // 1: decoupled weight decay
};

// ctrl[0] = gradient multiplier (1/loss_scale * clip), ctrl[1] != 0 -> skip step
template <typename T16>
__global__ void adam_flat_kernel(float* __restrict__ master, const float* __restrict__ grad,
                                 float* __restrict__ m, float* __restrict__ v,
                                 T16* __restrict__ model16, size_t n, AdamHyper h,
                                 const float* __restrict__ ctrl) {
    const float gmul = ctrl ? ctrl[0] : 1.f;
    if (ctrl && ctrl[1] != 0.f) return;
    const size_t nv = n / 4;
    const float4* g4 = reinterpret_cast<const float4*>(grad);
    float4* p4 = reinterpret_cast<float4*>(master);
    float4* m4 = reinterpret_cast<float4*>(m);
    float4* v4 = reinterpret_cast<float4*>(v);
    auto upd = [&](float& p, float g, float& mm, float& vv) {
        g *= gmul;
        if (!h.adamw && h.weight_decay != 0.f) g += h.weight_decay * p;
        mm = h.beta1 * mm + (1.f - h.beta1) * g;
        vv = h.beta2 * vv + (1.f - h.beta2) * g * g;
        const float mh = mm / h.bias_corr1;
        const float vh = vv / h.bias_corr2;
        float u = mh / (sqrtf(vh) + h.eps);
        if (h.adamw && h.weight_decay != 0.f) u += h.weight_decay * p;
        p -= h.lr * u;
    };
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nv;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float4 p = p4[i], g = g4[i], mm = m4[i], vv = v4[i];
        upd(p.x, g.x, mm.x, vv.x);
        upd(p.y, g.y, mm.y, vv.y);
        upd(p.z, g.z, mm.z, vv.z);
        upd(p.w, g.w, mm.w, vv.w);
        p4[i] = p;
        m4[i] = mm;
        v4[i] = vv;
        if (model16) {
            T16 o[4] = {from_f32<T16>(p.x), from_f32<T16>(p.y), from_f32<T16>(p.z),
                        from_f32<T16>(p.w)};
            *reinterpret_cast<uint2*>(model16 + i * 4) = *reinterpret_cast<uint2*>(o);
        }
    }
    if (blockIdx.x == 0 && threadIdx.x < n % 4) {
        const size_t i = nv * 4 + threadIdx.x;
        float p = master[i], mm = m[i], vv = v[i];
        upd(p, grad[i], mm, vv);
        master[i] = p;
        m[i] = mm;
        v[i] = vv;
        if (model16) model16[i] = from_f32<T16>(p);
    }
}

struct SgdHyper {
    float lr, momentum, dampening, weight_decay;
    int nesterov, first_step;
};

template <typename T16>
__global__ void sgd_flat_kernel(float* __restrict__ master, const float* __restrict__ grad,
                                float* __restrict__ mom, T16* __restrict__ model16, size_t n,
                                SgdHyper h, const float* __restrict__ ctrl) {
    const float gmul = ctrl ? ctrl[0] : 1.f;
    if (ctrl && ctrl[1] != 0.f) return;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float p = master[i];
        float g = grad[i] * gmul + h.weight_decay * p;
        if (h.momentum != 0.f) {
            float b = h.first_step ? g : h.momentum * mom[i] + (1.f - h.dampening) * g;
            mom[i] = b;
            g = h.nesterov ? g + h.momentum * b : b;
        }
        p -= h.lr * g;
        master[i] = p;
        if (model16) model16[i] = from_f32<T16>(p);
    }
}

// out[0] += sum x^2 (fp32 accumulate)
template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ x, size_t n, float* __restrict__ out) {
    __shared__ float red[32];
    float s = 0.f;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float a = to_f32<T>(x[i]);
        s += a * a;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
        s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (threadIdx.x == 0) atomicAdd(out, s);
    }
}

// ctrl[0] = inv_scale * min(1, max_norm / (sqrt(sumsq) * inv_scale + 1e-6));
// ctrl[1] = 1 if sumsq is not finite.  max_norm <= 0 disables clipping.
__global__ void finalize_ctrl_kernel(const float* __restrict__ sumsq, float inv_scale,
                                     float max_norm, float* __restrict__ ctrl,
                                     float* __restrict__ norm_out) {
    const float s = sumsq[0];
    const bool bad = !isfinite(s);
    const float norm = sqrtf(s) * inv_scale;
    float mul = inv_scale;
    if (max_norm > 0.f && !bad) {
        const float c = max_norm / (norm + 1e-6f);
        if (c < 1.f) mul *= c;
    }
    ctrl[0] = mul;
    ctrl[1] = bad ? 1.f : 0.f;
    if (norm_out) norm_out[0] = norm;
}

template <typename T>
__global__ void scale_kernel(T* __restrict__ x, size_t n, float s) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
        x[i] = from_f32<T>(to_f32<T>(x[i]) * s);
}

static inline int grid_for(size_t work, int threads) {
    size_t g = (work + threads - 1) / threads;
    const size_t cap = 148 * 16;
    return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace rb

using namespace rb;

// dtype16: 0 fp16, 1 bf16 (type of model16; ignored when model16 is null)
extern "C" int rb_adam_flat(float* master, const float* grad, float* m, float* v, void* model16,
                            long long n, float lr, float beta1, float beta2, float eps,
                            float weight_decay, float bias_corr1, float bias_corr2, int adamw,
                            const float* ctrl, int dtype16, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (n <= 0) return 0;
    AdamHyper h{lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, adamw};
    const int g = grid_for(n / 4 + 1, 256);
    if (dtype16 == 1)
        adam_flat_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(
            master, grad, m, v, static_cast<__nv_bfloat16*>(model16), n, h, ctrl);
    else
        adam_flat_kernel<__half><<<g, 256, 0, st>>>(master, grad, m, v,
                                                    static_cast<__half*>(model16), n, h, ctrl);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int rb_sgd_flat(float* master, const float* grad, float* mom, void* model16,
                           long long n, float lr, float momentum, float dampening,
                           float weight_decay, int nesterov, int first_step, const float* ctrl,
                           int dtype16, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (n <= 0) return 0;
    SgdHyper h{lr, momentum, dampening, weight_decay, nesterov, first_step};
    const int g = grid_for(n, 256);
    if (dtype16 == 1)
        sgd_flat_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(
            master, grad, mom, static_cast<__nv_bfloat16*>(model16), n, h, ctrl);
    else
        sgd_flat_kernel<__half><<<g, 256, 0, st>>>(master, grad, mom,
                                                   static_cast<__half*>(model16), n, h, ctrl);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// dtype: 0 fp16, 1 bf16, 2 fp32.  Adds to out[0].
extern "C" int rb_sumsq(const void* x, long long n, float* out, int dtype, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (n <= 0) return 0;
    const int g = grid_for(n, 256) > 148 * 4 ? 148 * 4 : grid_for(n, 256);
    if (dtype == 2)
        sumsq_kernel<float><<<g, 256, 0, st>>>(static_cast<const float*>(x), n, out);
    else if (dtype == 1)
        sumsq_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), n, out);
    else
        sumsq_kernel<__half><<<g, 256, 0, st>>>(static_cast<const __half*>(x), n, out);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int rb_finalize_ctrl(const float* sumsq, float inv_scale, float max_norm, float* ctrl,
                                float* norm_out, void* stream) {
    finalize_ctrl_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(sumsq, inv_scale, max_norm,
                                                                        ctrl, norm_out);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int rb_scale(void* x, long long n, float s, int dtype, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (n <= 0) return 0;
    const int g = grid_for(n, 256);
    if (dtype == 2)
        scale_kernel<float><<<g, 256, 0, st>>>(static_cast<float*>(x), n, s);
    else if (dtype == 1)
        scale_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<__nv_bfloat16*>(x), n, s);
    else
        scale_kernel<__half><<<g, 256, 0, st>>>(static_cast<__half*>(x), n, s);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
