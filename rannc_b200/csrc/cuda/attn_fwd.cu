// Fused multi-head attention forward (flash style) on tcgen05 tensor cores.
//
//   O = dropout(softmax(Q K^T * scale + key_bias)) V        head dim D = 64
//
// One CTA handles 128 query rows of one (batch, head).  Keys/values stream
// through a 2-stage TMA ring in chunks of 128.  S = Q K^T is accumulated in
// TMEM (128 lanes x 128 columns); each of the 128 softmax threads owns one
// query row (= one TMEM lane), so row max / sum need no shuffles.  P is written
// as bf16 into shared memory in the 128-byte-swizzled K-major layout and fed
// back to the tensor core as the A operand of O += P V, with V consumed as an
// MN-major B operand straight from its [key, d] layout.  The S^2 score matrix
// never reaches HBM.  Warps 0..3 = softmax, warp 4 = TMA + MMA issue.
//
// Takes the place of the matmul -> div -> add(mask) -> softmax -> dropout ->
// matmul chain of the traced BERT attention, which the reference runs as
// separate cuBLAS / ATen kernels (src/torch/TorchDriver.cpp:566).
#include "attn.h"

#include "tc_common.cuh"

namespace rb {

constexpr int AQ = 128;   // query rows per CTA
constexpr int AK = 128;   // keys per chunk
constexpr int AD = 64;    // head dim
constexpr int TILE_B = AQ * AD * 2;  // 16 KiB: one [128 x 64] 16-bit tile
constexpr int P_BYTES = AQ * AK * 2; // 32 KiB
constexpr int ATT_THREADS = 160;
constexpr int ATT_TMEM_COLS = 256;
constexpr int COL_S = 0, COL_O = 128;
constexpr int ATT_SMEM = TILE_B /*Q*/ + 4 * TILE_B /*K,V x2*/ + P_BYTES + 1024 + 256;

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

// 32-bit mix of (seed, offset, index); two 16-bit dropout decisions per call
__device__ __forceinline__ uint32_t mix32(uint64_t seed, uint64_t idx) {
    uint64_t z = idx * 0x9E3779B97F4A7C15ull + seed;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return static_cast<uint32_t>(z ^ (z >> 31));
}

struct AttnFwdParams {
    int B, H, S;
    float scale_log2;
    const float* key_bias;  // [B, S] additive, natural-log units; may be null
    void* O;
    long long o_sb, o_ss, o_sh;
    float* lse;  // [B, H, S]
    uint32_t thr16;
    float inv_keep;
    uint64_t seed;
    int* err;
};

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    uint8_t* sQ = smem;
    uint8_t* sK = smem + TILE_B;               // [2][TILE_B]
    uint8_t* sV = smem + 3 * TILE_B;           // [2][TILE_B]
    uint8_t* sP = smem + 5 * TILE_B;           // [2 col blocks][128 rows x 128 B]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 5 * TILE_B + P_BYTES);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;  // [2]
    uint64_t* s_full = bars + 3;
    uint64_t* s_free = bars + 4;
    uint64_t* p_ready = bars + 5;
    uint64_t* o_done = bars + 6;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q0 = blockIdx.x * AQ, h = blockIdx.y, b = blockIdx.z;
    const int nchunks = (p.S + AK - 1) / AK;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(&kv_full[0], 1);
        mbar_init(&kv_full[1], 1);
        mbar_init(s_full, 1);
        mbar_init(s_free, 128);
        mbar_init(p_ready, 128);
        mbar_init(o_done, 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 4) {
        tmem_alloc(tmem_slot, ATT_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;

    if (warp == 4) {
        if (lane == 0) {
            const uint32_t idesc_s = make_idesc_f16(fmt, 0, 0, AQ, AK);
            const uint32_t idesc_o = make_idesc_f16(fmt, 0, 1, AQ, AD);
            auto load_kv = [&](int j) {
                const int st = j & 1;
                mbar_arrive_expect_tx(&kv_full[st], 2 * TILE_B);
                tma_load_4d(sK + st * TILE_B, &tmK, &kv_full[st], 0, j * AK, h, b);
                tma_load_4d(sV + st * TILE_B, &tmV, &kv_full[st], 0, j * AK, h, b);
            };
            auto issue_s = [&](int j) {
                const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + (j & 1) * TILE_B);
#pragma unroll
                for (int k = 0; k < AD / 16; ++k)
                    umma_f16(tmem + COL_S, make_smem_desc_sw128(qa + k * 32, 16, 1024),
                             make_smem_desc_sw128(ka + k * 32, 16, 1024), idesc_s, k != 0);
                umma_commit(s_full);
            };
            mbar_arrive_expect_tx(q_full, TILE_B);
            tma_load_4d(sQ, &tmQ, q_full, 0, q0, h, b);
            load_kv(0);
            if (nchunks > 1) load_kv(1);
            bool ok = mbar_wait(q_full, 0, abort_flag) && mbar_wait(&kv_full[0], 0, abort_flag);
            if (ok) {
                tc_fence_after();
                issue_s(0);
            }
            for (int j = 0; j < nchunks && ok; ++j) {
                if (j + 1 < nchunks) {
                    ok = mbar_wait(&kv_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag) &&
                         mbar_wait(s_free, j & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(j + 1);
                }
                if (!mbar_wait(p_ready, j & 1, abort_flag)) break;
                tc_fence_after();
                const uint32_t pa = smem_u32(sP), va = smem_u32(sV + (j & 1) * TILE_B);
#pragma unroll
                for (int k = 0; k < AK / 16; ++k)
                    umma_f16(tmem + COL_O,
                             make_smem_desc_sw128(pa + (k >> 2) * (P_BYTES / 2) + (k & 3) * 32, 16, 1024),
                             make_smem_desc_sw128(va + k * 2048, 8192, 1024), idesc_o,
                             (j | k) != 0);
                umma_commit(o_done);
                if (j + 2 < nchunks) {
                    if (!mbar_wait(o_done, j & 1, abort_flag)) break;
                    load_kv(j + 2);
                }
            }
        }
    } else {
        // ------------- softmax threads: one query row each -------------
        const int r = threadIdx.x;  // row in tile == TMEM lane
        const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
        const int q = q0 + r;
        const float* kb = p.key_bias ? p.key_bias + static_cast<long long>(b) * p.S : nullptr;
        const uint64_t drop_row =
            ((static_cast<uint64_t>(b) * p.H + h) * p.S + static_cast<uint64_t>(q)) *
            static_cast<uint64_t>((p.S + 1) / 2);
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        const uint32_t sw = r & 7;
        uint8_t* prow = sP + (r >> 3) * 1024 + sw * 128;
        for (int j = 0; j < nchunks; ++j) {
            if (!mbar_wait(s_full, j & 1, abort_flag)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const int key0 = j * AK;
            // pass 1: row max of the scaled, biased scores
            float cm = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem + lane_addr + COL_S + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int key = key0 + c * 32 + i;
                    float s = __uint_as_float(v[i]) * p.scale_log2;
                    if (kb) s += (key < p.S ? kb[key] : 0.f) * 1.4426950408889634f;
                    if (key >= p.S) s = -INFINITY;
                    cm = fmaxf(cm, s);
                }
            }
            const float m_new = fmaxf(m, cm);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = exp2f(m - m_use);
            // the previous P V product must be complete before P is overwritten and O rescaled
            if (j > 0) {
                if (!mbar_wait(o_done, (j - 1) & 1, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
                    for (int c = 0; c < 2; ++c) {
                        uint32_t v[32];
                        tmem_ld32(tmem + lane_addr + COL_O + c * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        tmem_st32(tmem + lane_addr + COL_O + c * 32, v);
                    }
                    tmem_st_wait();
                }
            }
            // pass 2: probabilities -> shared memory (bf16, swizzled K-major)
            float rs = 0.f;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem + lane_addr + COL_S + c * 32, v);
                tmem_ld_wait();
                float pr[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int key = key0 + c * 32 + i;
                    float s = __uint_as_float(v[i]) * p.scale_log2;
                    if (kb) s += (key < p.S ? kb[key] : 0.f) * 1.4426950408889634f;
                    const float e = key < p.S ? exp2f(s - m_use) : 0.f;
                    rs += e;
                    pr[i] = e;
                }
                if (p.thr16) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const int key = key0 + c * 32 + i;
                        const uint32_t bits = mix32(p.seed, drop_row + (key >> 1));
                        pr[i] = (bits & 0xffffu) >= p.thr16 ? pr[i] * p.inv_keep : 0.f;
                        pr[i + 1] = (bits >> 16) >= p.thr16 ? pr[i + 1] * p.inv_keep : 0.f;
                    }
                }
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint4 qv;
                    T* e = reinterpret_cast<T*>(&qv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) e[i] = from_f32<T>(pr[g * 8 + i]);
                    const int kk = c * 32 + g * 8;
                    const uint32_t c16 = (kk & 63) >> 3;
                    *reinterpret_cast<uint4*>(prow + (kk >> 6) * (P_BYTES / 2) + ((c16 ^ sw) << 4)) = qv;
                }
            }
            tc_fence_before();
            mbar_arrive(s_free);
            l = l * alpha + rs;
            m = m_new;
            fence_proxy_async();
            mbar_arrive(p_ready);
        }
        if (ok && mbar_wait(o_done, (nchunks - 1) & 1, abort_flag)) {
            tc_fence_after();
            const float inv_l = l > 0.f ? 1.f / l : 0.f;
            T* orow = reinterpret_cast<T*>(p.O) + b * p.o_sb + static_cast<long long>(q) * p.o_ss +
                      h * p.o_sh;
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem + lane_addr + COL_O + c * 32, v);
                tmem_ld_wait();
                if (q < p.S) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 qv;
                        T* e = reinterpret_cast<T*>(&qv);
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            e[i] = from_f32<T>(__uint_as_float(v[g * 8 + i]) * inv_l);
                        *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = qv;
                    }
                }
            }
            if (q < p.S)
                p.lse[(static_cast<long long>(b) * p.H + h) * p.S + q] =
                    (m == -INFINITY ? 0.f : m) * 0.6931471805599453f + __logf(fmaxf(l, 1e-30f));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            atomicExch(p.err, ERR_MBAR_TIMEOUT);
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000) {
            }
        }
        __syncthreads();
    }
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem, ATT_TMEM_COLS);
    }
}

template <typename T>
static int launch_fwd(const RbAttnArgs& a, cudaStream_t st) {
    CUtensorMap tq, tk, tv;
    int rc;
    const uint64_t D = a.D, S = a.S, H = a.H, B = a.B;
    if ((rc = make_tmap_4d(&tq, a.Q, a.dtype, D, S, H, B, a.q_ss * 2, a.q_sh * 2, a.q_sb * 2, 64, AQ))) return rc;
    if ((rc = make_tmap_4d(&tk, a.K, a.dtype, D, S, H, B, a.k_ss * 2, a.k_sh * 2, a.k_sb * 2, 64, AK))) return rc;
    if ((rc = make_tmap_4d(&tv, a.V, a.dtype, D, S, H, B, a.v_ss * 2, a.v_sh * 2, a.v_sb * 2, 64, AK))) return rc;
    AttnFwdParams p;
    p.B = a.B;
    p.H = a.H;
    p.S = a.S;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.key_bias = a.key_bias;
    p.O = a.O;
    p.o_sb = a.o_sb;
    p.o_ss = a.o_ss;
    p.o_sh = a.o_sh;
    p.lse = a.lse;
    p.thr16 = a.p_drop > 0.f ? static_cast<uint32_t>(a.p_drop * 65536.f + 0.5f) : 0u;
    p.inv_keep = a.p_drop > 0.f ? 1.f / (1.f - a.p_drop) : 1.f;
    p.seed = a.seed * 0x2545F4914F6CDD1Dull + a.offset;
    p.err = error_word_ptr();
    if (!p.err) return -3;
    auto kern = attn_fwd_kernel<T>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) != cudaSuccess)
            return -4;
        attr_set[dev & 63] = true;
    }
    dim3 grid((a.S + AQ - 1) / AQ, a.H, a.B);
    kern<<<grid, ATT_THREADS, ATT_SMEM, st>>>(tq, tk, tv, p);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace rb

extern "C" int rb_attn_fwd(const RbAttnArgs* a, void* stream) {
    if (a->D != 64) return -2;
    if (a->B <= 0 || a->H <= 0 || a->S <= 0) return 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return a->dtype == 1 ? rb::launch_fwd<__nv_bfloat16>(*a, st) : rb::launch_fwd<__half>(*a, st);
}
