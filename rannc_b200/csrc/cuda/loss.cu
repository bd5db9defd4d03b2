// Fused softmax + cross-entropy (mean over non-ignored rows) forward/backward.
//
// Forward: one CTA per row, single pass with an online (max, sum) pair; rows
// whose label is `ignore_index` are not read at all (85 % of the rows in
// masked-LM pre-training).  It accumulates the loss sum and the row count in
// `acc[0..1]`; `rb_xent_finalize` turns them into the mean.  Backward writes
// (softmax - onehot) * gout / count, optionally in place over the logits.
//
// Takes the place of the aten::log_softmax + aten::nll_loss nodes of the traced
// criterion; the batch-share weighting of a replica's loss
// (src/comm/SComm.cpp:526-578) is folded into `weight`.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "debug_check.cuh"
#include "tc_common.cuh"

namespace rb {

constexpr int XT = 256;

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
    const float nm = fmaxf(m, m2);
    if (nm == -INFINITY) return;  // both sides empty
    s = s * __expf(m - nm) + s2 * __expf(m2 - nm);
    m = nm;
}

template <typename T>
__global__ void __launch_bounds__(XT)
    xent_fwd_kernel(const T* __restrict__ logits, const long long* __restrict__ labels,
                    float* __restrict__ lse_out, float* __restrict__ acc, int V, long long ld,
                    long long ignore_index) {
    __shared__ float sm_m[XT / 32], sm_s[XT / 32];
    const int row = blockIdx.x;
    const long long label = labels[row];
    if (label == ignore_index || label < 0 || label >= V) {
        if (threadIdx.x == 0) lse_out[row] = 0.f;
        return;
    }
    const T* x = logits + static_cast<long long>(row) * ld;
    float m = -INFINITY, s = 0.f;
    const bool vec = (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
    if (vec) {
        const int nv = V / 8;
        for (int i = threadIdx.x; i < nv; i += XT) {
            uint4 q = *reinterpret_cast<const uint4*>(x + i * 8);
            const T* e = reinterpret_cast<const T*>(&q);
            float v[8], lm = -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = to_f32<T>(e[j]);
                lm = fmaxf(lm, v[j]);
            }
            const float nm = fmaxf(m, lm);
            float ls = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) ls += __expf(v[j] - nm);
            s = s * __expf(m - nm) + ls;
            m = nm;
        }
        for (int i = nv * 8 + threadIdx.x; i < V; i += XT) online_merge(m, s, to_f32<T>(x[i]), 1.f);
    } else {
        for (int i = threadIdx.x; i < V; i += XT) online_merge(m, s, to_f32<T>(x[i]), 1.f);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
        const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
        online_merge(m, s, m2, s2);
    }
    if ((threadIdx.x & 31) == 0) {
        sm_m[threadIdx.x >> 5] = m;
        sm_s[threadIdx.x >> 5] = s;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        m = sm_m[0];
        s = sm_s[0];
#pragma unroll
        for (int w = 1; w < XT / 32; ++w) online_merge(m, s, sm_m[w], sm_s[w]);
        const float lse = m + __logf(s);
        lse_out[row] = lse;
        atomicAdd(acc, lse - to_f32<T>(x[label]));
        atomicAdd(acc + 1, 1.f);
    }
}

// loss[0] = weight * acc[0] / max(acc[1], 1)
__global__ void xent_finalize_kernel(const float* __restrict__ acc, float* __restrict__ loss,
                                     float weight) {
    loss[0] = weight * acc[0] / fmaxf(acc[1], 1.f);
}

template <typename T>
__global__ void __launch_bounds__(XT)
    xent_bwd_kernel(const T* __restrict__ logits, const long long* __restrict__ labels,
                    const float* __restrict__ lse_in, const float* __restrict__ acc,
                    const float* __restrict__ gout, T* __restrict__ dlogits, int V, long long ld,
                    long long ignore_index, float weight) {
    const int row = blockIdx.x;
    const long long label = labels[row];
    const bool live = !(label == ignore_index || label < 0 || label >= V);
    const T* x = logits + static_cast<long long>(row) * ld;
    T* d = dlogits + static_cast<long long>(row) * ld;
    const float g = live ? gout[0] * weight / fmaxf(acc[1], 1.f) : 0.f;
    const float lse = lse_in[row];
    const bool vec = (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(dlogits) & 15) == 0);
    const int width = static_cast<int>(ld);  // also clears padding columns [V, ld)
    if (vec) {
        for (int i = threadIdx.x; i < width / 8; i += XT) {
            uint4 q = make_uint4(0, 0, 0, 0);
            if (live) {
                q = *reinterpret_cast<const uint4*>(x + i * 8);
                T* e = reinterpret_cast<T*>(&q);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int c = i * 8 + j;
                    float v = c < V ? __expf(to_f32<T>(e[j]) - lse) : 0.f;
                    if (c == label) v -= 1.f;
                    e[j] = from_f32<T>(v * g);
                }
            }
            *reinterpret_cast<uint4*>(d + i * 8) = q;
        }
    } else {
        for (int c = threadIdx.x; c < width; c += XT) {
            float v = 0.f;
            if (live && c < V) {
                v = __expf(to_f32<T>(x[c]) - lse);
                if (c == label) v -= 1.f;
            }
            d[c] = from_f32<T>(v * g);
        }
    }
}

}  // namespace rb

using namespace rb;

// acc: 2 floats, zeroed by the caller.  lse: [rows].
extern "C" int rb_xent_fwd(const void* logits, const long long* labels, float* lse, float* acc,
                           float* loss, int rows, int V, long long ld, long long ignore_index,
                           float weight, int dtype, void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RB_DEBUG_RANGE(labels, rows, 0, V, ignore_index, st);
    if (rows > 0) {
        if (dtype == 1)
            xent_fwd_kernel<__nv_bfloat16><<<rows, XT, 0, st>>>(
                static_cast<const __nv_bfloat16*>(logits), labels, lse, acc, V, ld, ignore_index);
        else
            xent_fwd_kernel<__half><<<rows, XT, 0, st>>>(static_cast<const __half*>(logits), labels,
                                                        lse, acc, V, ld, ignore_index);
    }
    xent_finalize_kernel<<<1, 1, 0, st>>>(acc, loss, weight);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int rb_xent_bwd(const void* logits, const long long* labels, const float* lse,
                           const float* acc, const float* gout, void* dlogits, int rows, int V,
                           long long ld, long long ignore_index, float weight, int dtype,
                           void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows <= 0) return 0;
    if (dtype == 1)
        xent_bwd_kernel<__nv_bfloat16><<<rows, XT, 0, st>>>(
            static_cast<const __nv_bfloat16*>(logits), labels, lse, acc, gout,
            static_cast<__nv_bfloat16*>(dlogits), V, ld, ignore_index, weight);
    else
        xent_bwd_kernel<__half><<<rows, XT, 0, st>>>(static_cast<const __half*>(logits), labels,
                                                     lse, acc, gout, static_cast<__half*>(dlogits),
                                                     V, ld, ignore_index, weight);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
