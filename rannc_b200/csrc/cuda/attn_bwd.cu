// Fused multi-head attention backward on tcgen05 tensor cores (head dim 64).
//
// One CTA owns 128 keys of one (batch, head) and sweeps the query blocks.  Per
// query block i it recomputes, with the keys on the TMEM lanes,
//     St  = K_j Q_i^T          dPt = V_j dO_i^T                (TMEM, 2 x 128 cols)
//     Pt  = exp(St*scale + bias - lse_i)      dSt = Pt * (dPt - delta_i)
// writes Pt / dSt as 16-bit tiles into swizzled shared memory (one thread per
// key row) and feeds them back to the tensor core:
//     dV_j += Pt  dO_i        dK_j += dSt Q_i                  (TMEM accumulators)
//     dQ_i  = dSt^T K_j  -- the same dSt tile read as an MN-major A operand --
// dQ_i is drained from TMEM into a swizzled fp32 staging tile and added to an
// fp32 scratch buffer by ONE bulk tensor reduction per half tile (the copy
// engine does the read-modify-write; the math threads do not wait for it); a
// last kernel converts the scratch to the 16-bit dQ.  Q_i / dO_i stream
// through a 2-stage TMA ring; lse / delta of the next query block are fetched
// while the current one is processed.  Warps 0..7 = element math, warp 8 = TMA + MMA issue, warps
// 9..12 = dQ drain: the math warps' chain per query block is then only "S / dP -> P / dS", and the
// drain of block i runs beside the math of block i + 1.
//
// Takes the place of the autograd graph the reference runs for the traced
// attention chain (src/torch/TorchDriver.cpp:642-847).
#include "attn.h"
#include "attn_common.cuh"
#include "tc_common.cuh"

namespace rb {

constexpr int BQ = 128, BKEYS = 128;
constexpr int TILE = 128 * 64 * 2;       // 16 KiB
constexpr int SQ_BYTES = 128 * 128 * 2;  // 32 KiB
constexpr int BWD_MATH = 256;
constexpr int BWD_DRAIN = 128;                 // warps 9..12: move dQ out of tensor memory
constexpr int BWD_THREADS = BWD_MATH + 32 + BWD_DRAIN;
constexpr int BWD_TMEM_COLS = 512;
constexpr int C_ST = 0, C_DPT = 128, C_DV = 256, C_DK = 320, C_DQ = 384;
constexpr int DQ_STAGE = 128 * 64 * 4;   // 32 KiB: [2 column halves][128 rows x 128 B]
constexpr int QD_STAGES = 3;             // Q / dO ring: block i + 2 is loaded while blocks i and i + 1 are in use
// K, V + (Q, dO) x 3 stages + Pt, dSt + dQ staging + per-step (lse, delta, row hash) + barriers
constexpr int BWD_SMEM = 2 * TILE + 2 * QD_STAGES * TILE + 2 * SQ_BYTES + DQ_STAGE + 3 * 128 * 4 + 128;

struct AttnBwdParams {
    int B, H, S;
    float scale, scale_log2;
    const float* key_bias;
    const float* lse;
    const float* delta;
    float* dq_accum;  // [B, S, H, 64] fp32
    void* dK;
    void* dV;
    long long dk_sb, dk_ss, dk_sh, dv_sb, dv_ss, dv_sh;
    uint32_t thr32;   // keep an element when its 32-bit hash >= thr32 (0: no dropout)
    float inv_keep;
    uint32_t seed;
    int* err;
};

template <typename T>
__global__ void __launch_bounds__(BWD_THREADS, 1)
    attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const __grid_constant__ CUtensorMap tmDQ, const AttnBwdParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sK = smem;
    uint8_t* sV = smem + TILE;
    uint8_t* sQ = smem + 2 * TILE;                     // [QD_STAGES]
    uint8_t* sdO = smem + (2 + QD_STAGES) * TILE;      // [QD_STAGES]
    uint8_t* sPt = smem + (2 + 2 * QD_STAGES) * TILE;
    uint8_t* sdSt = sPt + SQ_BYTES;
    uint8_t* sDQ = sdSt + SQ_BYTES;
    float* s_lse = reinterpret_cast<float*>(sDQ + DQ_STAGE);        // [128], rewritten every step
    float* s_delta = s_lse + 128;                                   // [128]
    uint32_t* s_rhash = reinterpret_cast<uint32_t*>(s_delta + 128);  // [128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_rhash + 128);
    uint64_t* kv_full = bars;
    uint64_t* qd_full = bars + 1;  // [QD_STAGES]
    uint64_t* s_full = bars + 4;
    uint64_t* s_free = bars + 5;
    uint64_t* pds_ready = bars + 6;
    uint64_t* mma_done = bars + 7;
    uint64_t* dq_free = bars + 8;    // the previous bulk reduction has read the staging tile
    uint64_t* dq_ready = bars + 9;   // every drain thread has written its part of the staging tile
    uint64_t* dq_taken = bars + 10;  // dQ of the last step is out of tensor memory: the next may overwrite it
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int key0 = blockIdx.x * BKEYS, h = blockIdx.y, b = blockIdx.z;
    const int nq = (p.S + BQ - 1) / BQ;

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1);
        for (int st = 0; st < QD_STAGES; ++st) mbar_init(&qd_full[st], 1);
        mbar_init(s_full, 1);
        mbar_init(s_free, BWD_MATH);
        mbar_init(pds_ready, BWD_MATH);
        mbar_init(mma_done, 1);
        mbar_init(dq_free, 1);
        mbar_init(dq_ready, BWD_DRAIN);
        mbar_init(dq_taken, BWD_DRAIN);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 8) {
        tmem_alloc(tmem_slot, BWD_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;

    if (warp == 8) {
        if (lane == 0) {
            const uint32_t id_s = make_idesc_f16(fmt, 0, 0, 128, 128);
            const uint32_t id_kn = make_idesc_f16(fmt, 0, 1, 128, 64);  // A K-major, B MN-major
            const uint32_t id_nn = make_idesc_f16(fmt, 1, 1, 128, 64);  // A MN-major, B MN-major
            auto load_qd = [&](int i) {
                const int st = i % QD_STAGES;
                mbar_arrive_expect_tx(&qd_full[st], 2 * TILE);
                tma_load_4d(sQ + st * TILE, &tmQ, &qd_full[st], 0, i * BQ, h, b);
                tma_load_4d(sdO + st * TILE, &tmdO, &qd_full[st], 0, i * BQ, h, b);
            };
            auto issue_s = [&](int i) {
                const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
                const uint32_t qa = smem_u32(sQ + (i % QD_STAGES) * TILE), da = smem_u32(sdO + (i % QD_STAGES) * TILE);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_f16(tmem + C_ST, make_smem_desc_sw128(ka + k * 32, 16, 1024),
                             make_smem_desc_sw128(qa + k * 32, 16, 1024), id_s, k != 0);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_f16(tmem + C_DPT, make_smem_desc_sw128(va + k * 32, 16, 1024),
                             make_smem_desc_sw128(da + k * 32, 16, 1024), id_s, k != 0);
                umma_commit(s_full);
            };
            mbar_arrive_expect_tx(kv_full, 2 * TILE);
            tma_load_4d(sK, &tmK, kv_full, 0, key0, h, b);
            tma_load_4d(sV, &tmV, kv_full, 0, key0, h, b);
            for (int i = 0; i < QD_STAGES && i < nq; ++i) load_qd(i);
            bool ok = mbar_wait(kv_full, 0, abort_flag) && mbar_wait(&qd_full[0], 0, abort_flag);
            if (ok) {
                tc_fence_after();
                issue_s(0);
            }
            for (int i = 0; i < nq && ok; ++i) {
                // S / dP of the next block go to the tensor core as soon as the math warps have read this
                // block's: they run behind the previous block's products, while this block's math is busy
                if (i + 1 < nq) {
                    ok = mbar_wait(&qd_full[(i + 1) % QD_STAGES], ((i + 1) / QD_STAGES) & 1, abort_flag) &&
                         mbar_wait(s_free, i & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(i + 1);
                }
                // the stage block i - 1 used is free once its products are done: fetch block i + 2 into it,
                // a whole step before its S / dP products are issued
                if (i >= 1 && i + 2 < nq) {
                    if (!mbar_wait(mma_done, (i - 1) & 1, abort_flag)) break;
                    load_qd(i + 2);
                }
                if (!mbar_wait(pds_ready, i & 1, abort_flag)) break;
                tc_fence_after();
                const uint32_t pa = smem_u32(sPt), sa = smem_u32(sdSt), ka = smem_u32(sK);
                const uint32_t qa = smem_u32(sQ + (i % QD_STAGES) * TILE), da = smem_u32(sdO + (i % QD_STAGES) * TILE);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint32_t koff = (k >> 2) * (SQ_BYTES / 2) + (k & 3) * 32;
                    umma_f16(tmem + C_DV, make_smem_desc_sw128(pa + koff, 16, 1024),
                             make_smem_desc_sw128(da + k * 2048, 8192, 1024), id_kn, (i | k) != 0);
                }
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint32_t koff = (k >> 2) * (SQ_BYTES / 2) + (k & 3) * 32;
                    umma_f16(tmem + C_DK, make_smem_desc_sw128(sa + koff, 16, 1024),
                             make_smem_desc_sw128(qa + k * 2048, 8192, 1024), id_kn, (i | k) != 0);
                }
                // dQ of the previous step must have left tensor memory before this step's product replaces it
                if (i > 0) {
                    if (!mbar_wait(dq_taken, (i - 1) & 1, abort_flag)) break;
                    tc_fence_after();
                }
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    umma_f16(tmem + C_DQ, make_smem_desc_sw128(sa + k * 2048, SQ_BYTES / 2, 1024),
                             make_smem_desc_sw128(ka + k * 2048, 8192, 1024), id_nn, k != 0);
                umma_commit(mma_done);
            }
        }
    } else if (warp > 8) {
        // ------------- dQ drain: thread r owns query row r of the block (TMEM lane r), all 64 columns -------------
        const int r = (warp & 3) * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t sw = r & 7;
        const bool issuer = threadIdx.x == BWD_MATH + 32;
        for (int i = 0; i < nq; ++i) {
            if (!mbar_wait(mma_done, i & 1, abort_flag)) break;
            tc_fence_after();
            uint32_t v0[32], v1[32];
            tmem_ld32(tmem + lane_addr + C_DQ, v0);
            tmem_ld32(tmem + lane_addr + C_DQ + 32, v1);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(dq_taken);
            if (issuer) {
                tma_store_wait_read<0>();   // the previous reduction no longer reads the staging tile
                mbar_arrive(dq_free);
            }
            if (!mbar_wait(dq_free, i & 1, abort_flag)) break;
            uint8_t* row = sDQ + (r >> 3) * 1024 + sw * 128;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                const uint32_t off = (static_cast<uint32_t>(g) ^ sw) << 4;
                *reinterpret_cast<float4*>(row + off) =
                    make_float4(__uint_as_float(v0[g * 4]) * p.scale, __uint_as_float(v0[g * 4 + 1]) * p.scale,
                                __uint_as_float(v0[g * 4 + 2]) * p.scale, __uint_as_float(v0[g * 4 + 3]) * p.scale);
                *reinterpret_cast<float4*>(row + DQ_STAGE / 2 + off) =
                    make_float4(__uint_as_float(v1[g * 4]) * p.scale, __uint_as_float(v1[g * 4 + 1]) * p.scale,
                                __uint_as_float(v1[g * 4 + 2]) * p.scale, __uint_as_float(v1[g * 4 + 3]) * p.scale);
            }
            fence_proxy_async();
            mbar_arrive(dq_ready);
            if (issuer) {
                if (!mbar_wait(dq_ready, i & 1, abort_flag)) break;
                tma_reduce_add_4d(&tmDQ, sDQ, 0, i * BQ, h, b);
                tma_reduce_add_4d(&tmDQ, sDQ + DQ_STAGE / 2, 32, i * BQ, h, b);
                tma_store_commit();
            }
        }
        if (issuer) tma_store_wait<0>();   // the last reduction has landed
    } else {
        // thread pair (r, r + 128): TMEM lane r = key row for St/dPt/dV/dK;
        // `half` selects 64 of the 128 query columns of St/dPt and 32 of the 64 columns of dQ/dK/dV
        const int r = threadIdx.x & 127;
        const int half = threadIdx.x >> 7;
        const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const int key = key0 + r;
        const bool key_ok = key < p.S;
        // -inf for keys past the end of the sequence: their probabilities come out as exp2(-inf) = 0
        const float kbias =
            key_ok ? (p.key_bias ? p.key_bias[static_cast<long long>(b) * p.S + key] * 1.4426950408889634f : 0.f)
                   : -INFINITY;
        const uint32_t key_hash = drop_key_hash(p.seed, key);
        const long long bh = static_cast<long long>(b) * p.H + h;
        const uint32_t sw = r & 7;
        const uint32_t row_off = half * (SQ_BYTES / 2) + (r >> 3) * 1024 + sw * 128;
        uint8_t* prow = sPt + row_off;
        uint8_t* drow = sdSt + row_off;
        bool ok = true;

        // lse / delta of the first query block; later blocks are fetched one step ahead
        float n_lse = 0.f, n_delta = 0.f;
        bool n_lse_raw = false;   // n_lse still in natural-log units (as loaded)
        if (half == 0) {
            n_lse = r < p.S ? p.lse[bh * p.S + r] * 1.4426950408889634f : INFINITY;
            n_delta = r < p.S ? p.delta[bh * p.S + r] : 0.f;
        }
        for (int i = 0; i < nq; ++i) {
            const int q0 = i * BQ;
            // every thread is done reading the previous step's row statistics before they are replaced
            bar_sync_named(1, BWD_MATH);
            if (half == 0) {
                // +inf for rows past the end of the sequence: their probabilities come out as exp2(-inf) = 0
                s_lse[r] = n_lse_raw ? n_lse * 1.4426950408889634f : n_lse;
                s_delta[r] = n_delta;
                s_rhash[r] = drop_row_hash(p.seed, b, h, q0 + r, p.H, p.S);
                // issued here (volatile: not sunk to the use), consumed at the top of the next step
                const int qn = q0 + BQ + r;
                if (i + 1 < nq && qn < p.S) {
                    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(n_lse) : "l"(p.lse + bh * p.S + qn));
                    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(n_delta) : "l"(p.delta + bh * p.S + qn));
                    n_lse_raw = true;
                } else {
                    n_lse = INFINITY;
                    n_delta = 0.f;
                    n_lse_raw = false;
                }
            }
            bar_sync_named(1, BWD_MATH);
            // after a failed wait the loop keeps running (every later wait fails at once) so that all threads
            // still meet at the named barriers
            if (!mbar_wait(s_full, i & 1, abort_flag)) {
                ok = false;
                continue;
            }
            tc_fence_after();
            // Pt / dSt of this thread's 64 columns, packed to 16 bits, held in registers: the whole
            // computation overlaps the tensor-core work of the previous step, whose operands still
            // occupy the shared-memory tiles.  Pt carries the dropout mask without its 1 / (1 - p)
            // factor (dV is scaled once at the end); dSt = P (mask dP / (1 - p) - delta).
            uint4 pk[2][4], dk4[2][4];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t sv[32], dv[32];
                tmem_ld32(tmem + lane_addr + C_ST + half * 64 + c * 32, sv);
                tmem_ld32(tmem + lane_addr + C_DPT + half * 64 + c * 32, dv);
                tmem_ld_wait();
                if (c == 1) {
                    // both TMEM tiles are in registers: the next step's MMAs may overwrite them
                    tc_fence_before();
                    mbar_arrive(s_free);
                }
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    float pd[8], ds[8];
#pragma unroll
                    for (int hq = 0; hq < 2; ++hq) {
                        const int qb = half * 64 + c * 32 + g * 8 + hq * 4;
                        const float4 ls4 = *reinterpret_cast<const float4*>(s_lse + qb);
                        const float4 dl4 = *reinterpret_cast<const float4*>(s_delta + qb);
                        const float lsv[4] = {ls4.x, ls4.y, ls4.z, ls4.w};
                        const float dlv[4] = {dl4.x, dl4.y, dl4.z, dl4.w};
                        uint32_t rhv[4] = {0, 0, 0, 0};
                        if (p.thr32) {
                            const uint4 rh4 = *reinterpret_cast<const uint4*>(s_rhash + qb);
                            rhv[0] = rh4.x, rhv[1] = rh4.y, rhv[2] = rh4.z, rhv[3] = rh4.w;
                        }
#pragma unroll
                        for (int x = 0; x < 4; ++x) {
                            const int e = g * 8 + hq * 4 + x;
                            const float pr = exp2f(fmaf(__uint_as_float(sv[e]), p.scale_log2, kbias) - lsv[x]);
                            const float dp = __uint_as_float(dv[e]);
                            if (p.thr32) {
                                const bool keep = drop_keep(rhv[x], key_hash, p.thr32);
                                pd[hq * 4 + x] = keep ? pr : 0.f;
                                ds[hq * 4 + x] = pr * fmaf(keep ? dp : 0.f, p.inv_keep, -dlv[x]);
                            } else {
                                pd[hq * 4 + x] = pr;
                                ds[hq * 4 + x] = pr * (dp - dlv[x]);
                            }
                        }
                    }
                    pk[c][g] = make_uint4(pack2<T>(pd[0], pd[1]), pack2<T>(pd[2], pd[3]), pack2<T>(pd[4], pd[5]),
                                          pack2<T>(pd[6], pd[7]));
                    dk4[c][g] = make_uint4(pack2<T>(ds[0], ds[1]), pack2<T>(ds[2], ds[3]), pack2<T>(ds[4], ds[5]),
                                           pack2<T>(ds[6], ds[7]));
                }
            }
            if (i > 0) {
                // the previous step's dV / dK / dQ products read Pt / dSt: wait, then overwrite
                if (!mbar_wait(mma_done, (i - 1) & 1, abort_flag)) {
                    ok = false;
                    continue;
                }
                tc_fence_after();
            }
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const uint32_t off = (static_cast<uint32_t>(c * 4 + g) ^ sw) << 4;
                    *reinterpret_cast<uint4*>(prow + off) = pk[c][g];
                    *reinterpret_cast<uint4*>(drow + off) = dk4[c][g];
                }
            tc_fence_before();
            fence_proxy_async();
            mbar_arrive(pds_ready);
        }
        if (ok && mbar_wait(mma_done, (nq - 1) & 1, abort_flag)) {
            tc_fence_after();
            T* dk = reinterpret_cast<T*>(p.dK) + b * p.dk_sb + static_cast<long long>(key) * p.dk_ss + h * p.dk_sh +
                    half * 32;
            T* dvp = reinterpret_cast<T*>(p.dV) + b * p.dv_sb + static_cast<long long>(key) * p.dv_ss + h * p.dv_sh +
                     half * 32;
            uint32_t a[32], d[32];
            tmem_ld32(tmem + lane_addr + C_DV + half * 32, a);
            tmem_ld32(tmem + lane_addr + C_DK + half * 32, d);
            tmem_ld_wait();
            if (key_ok) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint4 qa, qd;
                    T* ea = reinterpret_cast<T*>(&qa);
                    T* ed = reinterpret_cast<T*>(&qd);
#pragma unroll
                    for (int x = 0; x < 8; ++x) {
                        ea[x] = from_f32<T>(__uint_as_float(a[g * 8 + x]) * p.inv_keep);
                        ed[x] = from_f32<T>(__uint_as_float(d[g * 8 + x]) * p.scale);
                    }
                    *reinterpret_cast<uint4*>(dvp + g * 8) = qa;
                    *reinterpret_cast<uint4*>(dk + g * 8) = qd;
                }
            }
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
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, BWD_TMEM_COLS);
    }
}

// delta[b,h,q] = sum_d dO[b,q,h,d] * O[b,q,h,d], D = 64.  Rows are taken in memory order ((b, q, h): h is
// the fastest index of a [B, S, H, D] tensor), 8 lanes x 16 bytes per row, so a warp reads 512 contiguous
// bytes of each tensor per step.
template <typename T>
__global__ void attn_delta_kernel(const T* __restrict__ O, const T* __restrict__ dO,
                                  float* __restrict__ delta, int B, int H, int S, long long o_sb,
                                  long long o_ss, long long o_sh, long long d_sb, long long d_ss,
                                  long long d_sh) {
    const long long rows = static_cast<long long>(B) * S * H;
    const int sub = threadIdx.x & 7;
    const long long step = (static_cast<long long>(gridDim.x) * blockDim.x) >> 3;
    // warp-uniform trip count: every lane takes part in the shuffles
    long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 3;
    const long long first = (blockIdx.x * static_cast<long long>(blockDim.x) + (threadIdx.x & ~31)) >> 3;
    for (long long base = first; base < rows; base += step, row += step) {
        float s = 0.f;
        int h = 0, q = 0, b = 0;
        if (row < rows) {
            h = static_cast<int>(row % H);
            q = static_cast<int>((row / H) % S);
            b = static_cast<int>(row / (static_cast<long long>(H) * S));
            const uint4 ov = *reinterpret_cast<const uint4*>(O + b * o_sb + q * o_ss + h * o_sh + sub * 8);
            const uint4 dv = *reinterpret_cast<const uint4*>(dO + b * d_sb + q * d_ss + h * d_sh + sub * 8);
            const T* oe = reinterpret_cast<const T*>(&ov);
            const T* de = reinterpret_cast<const T*>(&dv);
#pragma unroll
            for (int j = 0; j < 8; ++j) s = fmaf(to_f32<T>(oe[j]), to_f32<T>(de[j]), s);
        }
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        if (sub == 0 && row < rows) delta[(static_cast<long long>(b) * H + h) * S + q] = s;
    }
}

// dQ[b,q,h,:] = (T) acc[b,q,h,:]
template <typename T>
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, T* __restrict__ dQ, int B,
                                       int H, int S, long long sb, long long ss, long long sh) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;  // 8-element group
    const long long total = static_cast<long long>(B) * S * H * 8;
    if (i >= total) return;
    const int g = i & 7;
    const long long row = i >> 3;  // (b*S + q)*H + h
    const int h = row % H;
    const int q = (row / H) % S;
    const int b = row / (static_cast<long long>(H) * S);
    const float4 a = *reinterpret_cast<const float4*>(acc + row * 64 + g * 8);
    const float4 c = *reinterpret_cast<const float4*>(acc + row * 64 + g * 8 + 4);
    uint4 o;
    T* e = reinterpret_cast<T*>(&o);
    e[0] = from_f32<T>(a.x); e[1] = from_f32<T>(a.y); e[2] = from_f32<T>(a.z); e[3] = from_f32<T>(a.w);
    e[4] = from_f32<T>(c.x); e[5] = from_f32<T>(c.y); e[6] = from_f32<T>(c.z); e[7] = from_f32<T>(c.w);
    *reinterpret_cast<uint4*>(dQ + b * sb + q * ss + h * sh + g * 8) = o;
}

template <typename T>
static int launch_bwd(const RbAttnArgs& a, cudaStream_t st) {
    CUtensorMap tq, tk, tv, tdo;
    int rc;
    const uint64_t D = a.D, S = a.S, H = a.H, B = a.B;
    if ((rc = make_tmap_4d(&tq, a.Q, a.dtype, D, S, H, B, a.q_ss * 2, a.q_sh * 2, a.q_sb * 2, 64, 128))) return rc;
    if ((rc = make_tmap_4d(&tk, a.K, a.dtype, D, S, H, B, a.k_ss * 2, a.k_sh * 2, a.k_sb * 2, 64, 128))) return rc;
    if ((rc = make_tmap_4d(&tv, a.V, a.dtype, D, S, H, B, a.v_ss * 2, a.v_sh * 2, a.v_sb * 2, 64, 128))) return rc;
    if ((rc = make_tmap_4d(&tdo, a.dO, a.dtype, D, S, H, B, a.do_ss * 2, a.do_sh * 2, a.do_sb * 2, 64, 128))) return rc;
    const long long rows = static_cast<long long>(a.B) * a.H * a.S;
    unsigned rb_delta_grid = 1;
    {
        // 8 lanes per row; the grid is sized so that every thread handles a few rows
        long long blocks = (rows * 8 + 255) / 256;
        const long long cap = 148LL * 32;
        if (blocks > cap) blocks = cap;
        if (blocks < 1) blocks = 1;
        rb_delta_grid = static_cast<unsigned>(blocks);
    }
    attn_delta_kernel<T><<<rb_delta_grid, 256, 0, st>>>(
        static_cast<const T*>(a.O), static_cast<const T*>(a.dO), a.delta, a.B, a.H, a.S, a.o_sb,
        a.o_ss, a.o_sh, a.do_sb, a.do_ss, a.do_sh);
    cudaMemsetAsync(a.dq_accum, 0, static_cast<size_t>(rows) * 64 * sizeof(float), st);
    AttnBwdParams p;
    p.B = a.B; p.H = a.H; p.S = a.S;
    p.scale = a.scale;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.key_bias = a.key_bias;
    p.lse = a.lse;
    p.delta = a.delta;
    p.dq_accum = a.dq_accum;
    p.dK = a.dK; p.dV = a.dV;
    p.dk_sb = a.dk_sb; p.dk_ss = a.dk_ss; p.dk_sh = a.dk_sh;
    p.dv_sb = a.dv_sb; p.dv_ss = a.dv_ss; p.dv_sh = a.dv_sh;
    p.thr32 = drop_threshold(a.p_drop);
    p.inv_keep = a.p_drop > 0.f ? 1.f / (1.f - a.p_drop) : 1.f;
    p.seed = drop_seed(a.seed, a.offset);
    p.err = error_word_ptr();
    if (!p.err) return -3;
    auto kern = attn_bwd_kernel<T>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM) != cudaSuccess)
            return -4;
        attr_set[dev & 63] = true;
    }
    dim3 grid((a.S + BKEYS - 1) / BKEYS, a.H, a.B);
    CUtensorMap tdq;
    if ((rc = make_tmap_4d_f32(&tdq, a.dq_accum, 64, S, H, B, H * 64 * 4, 64 * 4, S * H * 64 * 4, 32, 128))) return rc;
    kern<<<grid, BWD_THREADS, BWD_SMEM, st>>>(tq, tk, tv, tdo, tdq, p);
    const long long groups = rows * 8;
    attn_dq_convert_kernel<T><<<static_cast<unsigned>((groups + 255) / 256), 256, 0, st>>>(
        a.dq_accum, static_cast<T*>(a.dQ), a.B, a.H, a.S, a.dq_sb, a.dq_ss, a.dq_sh);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace rb

extern "C" int rb_attn_bwd(const RbAttnArgs* a, void* stream) {
    if (a->D != 64) return -2;
    if (a->B <= 0 || a->H <= 0 || a->S <= 0) return 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return a->dtype == 1 ? rb::launch_bwd<__nv_bfloat16>(*a, st) : rb::launch_bwd<__half>(*a, st);
}
