// Fused data-parallel gradient step over NVLink / NVSwitch peer memory:
//
//   reduce-scatter(fp32 grads over the owner set) * 1/world * unscale
//     -> Adam on this rank's fp32 master shard
//     -> all-gather of the updated 16-bit parameters
//
// in ONE kernel per rank.  Each rank owns the contiguous shard [lo, lo+len) of
// the flat gradient / parameter buffers, which live in symmetric memory: every
// rank holds the peers' base pointers.  The kernel
//   0. tells every peer "my gradients are complete" (flag store, release.sys)
//      and waits for the same word from every peer (acquire.sys, bounded);
//   1. for every 16-byte group of its shard: loads the group from every peer's
//      gradient buffer (plain peer loads, or ONE multimem.ld_reduce through the
//      switch when a multicast mapping exists), scales, runs Adam on the local
//      master / moments, and stores the bf16 result into every peer's parameter
//      buffer (peer stores, or one multimem.st);
//   2. the last CTA to finish publishes "my writes are done" and waits for the
//      peers' words, so that on return every rank's parameters are complete.
// No TMA and no cluster multicast is involved: remote data moves with ordinary
// ld/st/multimem instructions issued by the SMs.
//
// Replaces, per owner rank set, the reference's per-parameter ncclAllReduce /
// bucketed ncclReduceScatter + pack/unpack copies + mul_ scaling + Apex Adam +
// per-forward ncclAllGather (src/comp/ParamStorage.cpp:347-596,
// src/comm/NCCLWrapper.cpp:324-437, pyrannc/opt.py:205-312).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "rs_adam.h"
#include "tc_common.cuh"

namespace rb {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc) {
    float4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
}
__device__ __forceinline__ void multimem_st_b128(void* mc, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc),
                 "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
                 "f"(__uint_as_float(v.w))
                 : "memory");
}

// Waits until *flag >= expected.  Returns false when `max_polls` ran out or after RB_PEER_WAIT_LIMIT_NS of
// wall-clock time (peers may reach the kernel late, so this cap is longer than the one for on-chip waits).
#ifndef RB_PEER_WAIT_LIMIT_NS
#define RB_PEER_WAIT_LIMIT_NS 20000000000ull
#endif
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t expected,
                                          unsigned long long max_polls) {
    const uint64_t t0 = globaltimer_ns();
    for (unsigned long long i = 0; i < max_polls; ++i) {
        const uint32_t v = ld_acquire_sys(flag);
        if (static_cast<int32_t>(v - expected) >= 0) return true;
        if ((i & 0xff) == 0xff && globaltimer_ns() - t0 > RB_PEER_WAIT_LIMIT_NS) return false;
        __nanosleep(100);
    }
    return false;
}

struct RsAdamParams {
    const float* peer_grad[RB_MAX_PEERS];   // each rank's flat fp32 gradient buffer
    void* peer_param[RB_MAX_PEERS];         // each rank's flat 16-bit parameter buffer
    uint32_t* peer_flags[RB_MAX_PEERS];     // each rank's flag block: [2][RB_MAX_PEERS] words
    const float* mc_grad;                   // multicast alias of the gradient buffers (or null)
    void* mc_param;                         // multicast alias of the parameter buffers (or null)
    float* master;                          // local: fp32 master shard [len]
    float* m;
    float* v;
    unsigned int* done_counter;             // local scratch word, zero on entry, zero on exit
    long long lo, len;                      // shard in flat coordinates (elements, multiples of 8)
    int nranks, my_idx;
    uint32_t epoch;
    float grad_mul;                         // 1/world * 1/loss_scale
    float lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2;
    int adamw;
    const float* ctrl;                      // optional [mul, skip]
    unsigned long long max_polls;
    int* err;
    int mode;                               // RB_RS_* bits
    float* own_grad;                        // this rank's gradient buffer (writable)
    float* sumsq;                           // optional accumulator of the squared reduced gradients
};

// What happens to one group of 8 reduced gradient elements (index i within this rank's slice): either the
// scaled sum goes back into this rank's own gradient buffer (reduction-only launch; returns its sum of
// squares), or the optimizer updates master / moments and the 16-bit result is written to every rank.
template <typename T16>
__device__ __forceinline__ float apply_group(const RsAdamParams& p, long long i, float (&g)[8], float gmul,
                                             bool update) {
    const long long e = p.lo + i * 8;
    if (p.mode & RB_RS_STORE_GRAD) {
        float ssq = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            g[j] *= gmul;
            ssq += g[j] * g[j];
        }
        *reinterpret_cast<float4*>(p.own_grad + e) = make_float4(g[0], g[1], g[2], g[3]);
        *reinterpret_cast<float4*>(p.own_grad + e + 4) = make_float4(g[4], g[5], g[6], g[7]);
        return ssq;
    }
    if (!update) return 0.f;
    float w[8], mm[8], vv[8];
    const bool sgd = p.adamw == 2;
    *reinterpret_cast<float4*>(w) = *reinterpret_cast<const float4*>(p.master + i * 8);
    *reinterpret_cast<float4*>(w + 4) = *reinterpret_cast<const float4*>(p.master + i * 8 + 4);
    *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(p.m + i * 8);
    *reinterpret_cast<float4*>(mm + 4) = *reinterpret_cast<const float4*>(p.m + i * 8 + 4);
    if (!sgd) {
        *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(p.v + i * 8);
        *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(p.v + i * 8 + 4);
    }
    uint4 packed;
    T16* o = reinterpret_cast<T16*>(&packed);
    if (sgd) {
        // SGD with momentum (torch.optim.SGD): beta1 = momentum, beta2 = dampening, eps > 0.5 = Nesterov,
        // bias_corr1 == 0 marks the first step (the buffer starts as the gradient)
        const bool first = p.bias_corr1 == 0.f, nesterov = p.eps > 0.5f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float gg = g[j] * gmul;
            if (p.weight_decay != 0.f) gg += p.weight_decay * w[j];
            mm[j] = first ? gg : p.beta1 * mm[j] + (1.f - p.beta2) * gg;
            const float u = nesterov ? gg + p.beta1 * mm[j] : mm[j];
            w[j] -= p.lr * u;
            o[j] = from_f32<T16>(w[j]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float gg = g[j] * gmul;
            if (!p.adamw && p.weight_decay != 0.f) gg += p.weight_decay * w[j];
            mm[j] = p.beta1 * mm[j] + (1.f - p.beta1) * gg;
            vv[j] = p.beta2 * vv[j] + (1.f - p.beta2) * gg * gg;
            float u = (mm[j] / p.bias_corr1) / (sqrtf(vv[j] / p.bias_corr2) + p.eps);
            if (p.adamw && p.weight_decay != 0.f) u += p.weight_decay * w[j];
            w[j] -= p.lr * u;
            o[j] = from_f32<T16>(w[j]);
        }
    }
    *reinterpret_cast<float4*>(p.master + i * 8) = *reinterpret_cast<float4*>(w);
    *reinterpret_cast<float4*>(p.master + i * 8 + 4) = *reinterpret_cast<float4*>(w + 4);
    *reinterpret_cast<float4*>(p.m + i * 8) = *reinterpret_cast<float4*>(mm);
    *reinterpret_cast<float4*>(p.m + i * 8 + 4) = *reinterpret_cast<float4*>(mm + 4);
    if (!sgd) {
        *reinterpret_cast<float4*>(p.v + i * 8) = *reinterpret_cast<float4*>(vv);
        *reinterpret_cast<float4*>(p.v + i * 8 + 4) = *reinterpret_cast<float4*>(vv + 4);
    }
    if (p.mc_param) {
        multimem_st_b128(reinterpret_cast<T16*>(p.mc_param) + e, packed);
    } else {
#pragma unroll 1
        for (int r = 0; r < p.nranks; ++r) {
            int dst = p.my_idx + r;
            if (dst >= p.nranks) dst -= p.nranks;
            *reinterpret_cast<uint4*>(reinterpret_cast<T16*>(p.peer_param[dst]) + e) = packed;
        }
    }
    return 0.f;
}

template <typename T16>
__global__ void __launch_bounds__(512)
    rs_adam_ag_kernel(const RsAdamParams p) {
    __shared__ int s_ok;
    __shared__ int s_last;
    __shared__ float s_red[16];
    // ---- phase 0: everyone's gradients are complete
    if ((p.mode & RB_RS_BEGIN) && blockIdx.x == 0 && threadIdx.x < p.nranks) {
        __threadfence_system();
        st_release_sys(p.peer_flags[threadIdx.x] + 0 * RB_MAX_PEERS + p.my_idx, p.epoch);
    }
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if ((p.mode & RB_RS_BEGIN) && threadIdx.x < p.nranks) {
        if (!wait_flag(p.peer_flags[p.my_idx] + 0 * RB_MAX_PEERS + threadIdx.x, p.epoch, p.max_polls)) {
            s_ok = 0;
            atomicExch(p.err, ERR_PEER_TIMEOUT);
        }
    }
    __syncthreads();
    const bool ok = s_ok != 0;
    const bool pull = (p.mode & RB_RS_PULL) != 0, update = (p.mode & RB_RS_UPDATE) != 0;
    const bool skip = update && p.ctrl && p.ctrl[1] != 0.f;
    const float gmul = p.grad_mul * ((update && p.ctrl) ? p.ctrl[0] : 1.f);
    float ssq = 0.f;

    // ---- phase 1: reduce -> Adam -> scatter the 16-bit result (8 elements = one 16-byte store per step)
    if (ok && !skip) {
        const long long nvec = p.len / 8;
        const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
        const long long first = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
        if (pull && p.mc_grad) {
            // In-switch reduction: one multimem.ld_reduce returns the sum over all ranks.  Its round trip through
            // the switch is long, so every thread keeps UNROLL groups (2 x 16 bytes each) in flight.
            constexpr int UNROLL = 4;
            for (long long i0 = first; i0 < nvec; i0 += stride * UNROLL) {
                float4 ga[UNROLL], gb[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const long long i = i0 + u * stride;
                    if (i < nvec) {
                        ga[u] = multimem_ld_reduce_f32x4(p.mc_grad + p.lo + i * 8);
                        gb[u] = multimem_ld_reduce_f32x4(p.mc_grad + p.lo + i * 8 + 4);
                    }
                }
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const long long i = i0 + u * stride;
                    if (i < nvec) {
                        float g[8] = {ga[u].x, ga[u].y, ga[u].z, ga[u].w, gb[u].x, gb[u].y, gb[u].z, gb[u].w};
                        ssq += apply_group<T16>(p, i, g, gmul, update);
                    }
                }
            }
        } else {
            for (long long i = first; i < nvec; i += stride) {
                const long long e = p.lo + i * 8;
                float g[8];
                if (!pull) {
                    const float4 a = *reinterpret_cast<const float4*>(p.own_grad + e);
                    const float4 b = *reinterpret_cast<const float4*>(p.own_grad + e + 4);
                    g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w;
                    g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
                } else {
                    // every peer's 32 bytes are requested before any of them is used, so that the NVLink round
                    // trips overlap; own buffer first, then the peers in a per-rank rotated order
                    float4 a[RB_MAX_PEERS], b[RB_MAX_PEERS];
#pragma unroll
                    for (int r = 0; r < RB_MAX_PEERS; ++r) {
                        if (r < p.nranks) {
                            int src = p.my_idx + r;
                            if (src >= p.nranks) src -= p.nranks;
                            a[r] = *reinterpret_cast<const float4*>(p.peer_grad[src] + e);
                            b[r] = *reinterpret_cast<const float4*>(p.peer_grad[src] + e + 4);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) g[j] = 0.f;
#pragma unroll
                    for (int r = 0; r < RB_MAX_PEERS; ++r) {
                        if (r < p.nranks) {
                            g[0] += a[r].x; g[1] += a[r].y; g[2] += a[r].z; g[3] += a[r].w;
                            g[4] += b[r].x; g[5] += b[r].y; g[6] += b[r].z; g[7] += b[r].w;
                        }
                    }
                }
                ssq += apply_group<T16>(p, i, g, gmul, update);
            }
        }
    }

    if (p.sumsq && (p.mode & RB_RS_STORE_GRAD)) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
        if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ssq;
        __syncthreads();
        if (threadIdx.x < 32) {
            float t = threadIdx.x < (blockDim.x >> 5) ? s_red[threadIdx.x] : 0.f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            if (threadIdx.x == 0) atomicAdd(p.sumsq, t);
        }
    }
    if (!(p.mode & RB_RS_END)) return;   // uniform over the grid: the caller runs rb_peer_barrier instead
    // ---- phase 2: the last CTA publishes completion and waits for the peers
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(p.done_counter, 1u);
        s_last = (prev == gridDim.x - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
        if (threadIdx.x == 0) *p.done_counter = 0;  // ready for the next launch
        __threadfence_system();
        if (threadIdx.x < p.nranks)
            st_release_sys(p.peer_flags[threadIdx.x] + 1 * RB_MAX_PEERS + p.my_idx, p.epoch);
        if (threadIdx.x < p.nranks && ok) {
            if (!wait_flag(p.peer_flags[p.my_idx] + 1 * RB_MAX_PEERS + threadIdx.x, p.epoch, p.max_polls))
                atomicExch(p.err, ERR_PEER_TIMEOUT);
        }
    }
}

// Single-GPU check of the bounded wait: polls a flag nobody sets.
__global__ void wait_flag_probe_kernel(const uint32_t* flag, uint32_t expected,
                                       unsigned long long max_polls, int* err) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        if (!wait_flag(flag, expected, max_polls)) atomicExch(err, ERR_PEER_TIMEOUT);
    }
}

int* error_word_ptr();

}  // namespace rb

extern "C" int rb_rs_adam_ag(const RbRsAdamArgs* a, void* stream) {
    using namespace rb;
    if (a->nranks < 1 || a->nranks > RB_MAX_PEERS) return -2;
    if ((a->lo % 8) || (a->len % 8)) return -2;
    if (a->len <= 0) return 0;
    RsAdamParams p;
    for (int r = 0; r < RB_MAX_PEERS; ++r) {
        p.peer_grad[r] = r < a->nranks ? static_cast<const float*>(a->peer_grad[r]) : nullptr;
        p.peer_param[r] = r < a->nranks ? a->peer_param[r] : nullptr;
        p.peer_flags[r] = r < a->nranks ? static_cast<uint32_t*>(a->peer_flags[r]) : nullptr;
    }
    p.mc_grad = static_cast<const float*>(a->mc_grad);
    p.mc_param = a->mc_param;
    p.master = a->master;
    p.m = a->m;
    p.v = a->v;
    p.done_counter = static_cast<unsigned int*>(a->done_counter);
    p.lo = a->lo;
    p.len = a->len;
    p.nranks = a->nranks;
    p.my_idx = a->my_idx;
    p.epoch = a->epoch;
    p.grad_mul = a->grad_mul;
    p.lr = a->lr;
    p.beta1 = a->beta1;
    p.beta2 = a->beta2;
    p.eps = a->eps;
    p.weight_decay = a->weight_decay;
    p.bias_corr1 = a->bias_corr1;
    p.bias_corr2 = a->bias_corr2;
    p.adamw = a->adamw;
    p.ctrl = a->ctrl;
    p.max_polls = a->max_polls ? a->max_polls : (1ull << 26);
    p.err = error_word_ptr();
    if (!p.err) return -3;
    p.mode = a->mode ? a->mode : (RB_RS_BEGIN | RB_RS_END | RB_RS_PULL | RB_RS_UPDATE);
    if ((p.mode & RB_RS_STORE_GRAD) && (p.mode & RB_RS_UPDATE)) return -2;
    p.own_grad = const_cast<float*>(p.peer_grad[a->my_idx]);
    p.sumsq = a->sumsq;
    int grid = a->num_ctas > 0 ? a->num_ctas : 148;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (a->dtype16 == 1)
        rs_adam_ag_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(p);
    else
        rs_adam_ag_kernel<__half><<<grid, 512, 0, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int rb_wait_flag_probe(const void* flag, unsigned int expected, unsigned long long max_polls,
                                  void* stream) {
    int* err = rb::error_word_ptr();
    if (!err) return -3;
    rb::wait_flag_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint32_t*>(flag), expected, max_polls, err);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

namespace rb {
// Barrier among the ranks of a group through flags in symmetric memory: every rank stores `epoch`
// into slot [row][my_idx] of every peer's flag block and waits for all slots of its own block.
__global__ void peer_barrier_kernel(uint32_t* const* peer_flags_dev, uint32_t* f0, uint32_t* f1, uint32_t* f2,
                                    uint32_t* f3, uint32_t* f4, uint32_t* f5, uint32_t* f6, uint32_t* f7, int nranks,
                                    int my_idx, int row, uint32_t epoch, unsigned long long max_polls, int* err) {
    uint32_t* flags[8] = {f0, f1, f2, f3, f4, f5, f6, f7};
    const int t = threadIdx.x;
    if (t < nranks) {
        __threadfence_system();
        st_release_sys(flags[t] + row * RB_MAX_PEERS + my_idx, epoch);
        if (!wait_flag(flags[my_idx] + row * RB_MAX_PEERS + t, epoch, max_polls)) atomicExch(err, ERR_PEER_TIMEOUT);
    }
}
}  // namespace rb

// Stream-ordered barrier over a rank set: work enqueued before it on every rank is complete (and visible
// system-wide) on all ranks once it returns on this rank's stream.  peer_flags[r]: rank r's flag block
// (uint32 [2][RB_MAX_PEERS], zero-initialised, symmetric memory); `row` selects one of its two rows.
extern "C" int rb_peer_barrier(void* const* peer_flags, int nranks, int my_idx, int row, unsigned int epoch,
                               unsigned long long max_polls, void* stream) {
    using namespace rb;
    if (nranks < 1 || nranks > RB_MAX_PEERS || row < 0 || row > 1) return -2;
    int* err = error_word_ptr();
    if (!err) return -3;
    uint32_t* f[8];
    for (int r = 0; r < 8; ++r) f[r] = r < nranks ? static_cast<uint32_t*>(peer_flags[r]) : nullptr;
    peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        nullptr, f[0], f[1], f[2], f[3], f[4], f[5], f[6], f[7], nranks, my_idx, row, epoch,
        max_polls ? max_polls : (1ull << 26), err);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
