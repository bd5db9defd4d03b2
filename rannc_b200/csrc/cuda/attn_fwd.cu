// Fused multi-head attention forward (flash style) on tcgen05 tensor cores.
//
//   O = dropout(softmax(Q K^T * scale + key_bias)) V        head dim D = 64
//
// One CTA per SM (a CTA that holds tensor memory does not share its SM), so the
// CTA keeps the tensor core busy by itself: it owns TWO 128-row query tiles of
// one (batch, head) and interleaves their dependency chains -- while one tile's
// softmax runs, the other tile's Q K^T or P V is on the tensor core.  Keys and
// values stream through a 2-stage TMA ring in chunks of 128 and are shared by
// both tiles.  Per tile: S = Q K^T accumulates in TMEM (128 lanes x 128
// columns); 256 softmax threads, the pair (t, t + 128) owns query row t
// (= TMEM lane t) and splits the chunk's columns in halves, so row max / sum
// need one shared-memory exchange and no shuffles; P goes to shared memory as
// 16-bit in the 128-byte-swizzled K-major layout and returns to the tensor
// core as the A operand of O += P V, with V read as an MN-major B operand
// straight from its [key, d] layout.  The S^2 score matrix never reaches HBM.
// Warps 0..7 = tile 0, warps 8..15 = tile 1, warps 16 / 17 = MMA issue for tile 0 / 1 (one warp each, so
// neither tile's chain waits on the other's barriers), warp 18 = TMA loads.
//
// Takes the place of the matmul -> div -> add(mask) -> softmax -> dropout ->
// matmul chain of the traced BERT attention, which the reference runs as
// separate cuBLAS / ATen kernels (src/torch/TorchDriver.cpp:566).
#include <cstdlib>

#include "attn.h"
#include "attn_common.cuh"
#include "tc_common.cuh"

namespace rb {

constexpr int AQ = 128;   // query rows per tile
constexpr int AK = 128;   // keys per chunk
constexpr int AD = 64;    // head dim
constexpr int TILE_B = AQ * AD * 2;   // 16 KiB: one [128 x 64] 16-bit tile
constexpr int P_BYTES = AQ * AK * 2;  // 32 KiB
constexpr int GROUP = 256;            // softmax threads per query tile
constexpr int ATT_THREADS = 2 * GROUP + 96;   // + one MMA-issue warp per tile + the K / V loader
constexpr int ATT_TMEM_COLS = 512;
constexpr int TILE_COLS = 192;        // S (128) + O (64) per tile
constexpr int KB_MAX = 1024;          // key-bias entries staged in shared memory
// Q (2 tiles) + K, V (2 stages each) + P (2 tiles) + row-stat exchange [tile][parity][half][128] + barriers
constexpr int ATT_SMEM = 2 * TILE_B + 4 * TILE_B + 2 * P_BYTES + 2 * 2 * 2 * 128 * 4 + 256;

struct AttnFwdParams {
    int B, H, S;
    float scale_log2;
    const float* key_bias;  // [B, S] additive, natural-log units; may be null
    void* O;
    long long o_sb, o_ss, o_sh;
    float* lse;  // [B, H, S]
    uint32_t thr32;   // keep an element when its 32-bit hash >= thr32 (0: no dropout)
    float inv_keep;
    uint32_t seed;
    int* err;
};

// FAST: the sequence fits the staged per-key tables (bias and dropout hash in shared memory)
template <typename T, bool FAST>
__global__ void __launch_bounds__(ATT_THREADS, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(16) float s_kb[KB_MAX];
    __shared__ __align__(16) uint32_t s_kh[KB_MAX];
    uint8_t* sQ = smem;               // [2 tiles][TILE_B]
    uint8_t* sK = smem + 2 * TILE_B;  // [2 stages][TILE_B]
    uint8_t* sV = smem + 4 * TILE_B;  // [2 stages][TILE_B]
    uint8_t* sP = smem + 6 * TILE_B;  // [2 tiles][2 column blocks][128 rows x 128 B]
    float* s_xch = reinterpret_cast<float*>(smem + 6 * TILE_B + 2 * P_BYTES);  // [2][2][2][128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_xch + 1024);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;    // [2 stages]
    uint64_t* v_full = bars + 3;    // [2 stages]
    uint64_t* s_full = bars + 5;    // [2 tiles]
    uint64_t* s_free = bars + 7;    // [2 tiles]
    uint64_t* p_ready = bars + 9;   // [2 tiles]
    uint64_t* o_done = bars + 11;   // [2 tiles]
    uint64_t* kv_free = bars + 13;  // [2 stages]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_base = blockIdx.x * 2 * AQ, h = blockIdx.y, b = blockIdx.z;
    const int nchunks = (p.S + AK - 1) / AK;
    const int ntiles = (q_base + AQ < p.S) ? 2 : 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&s_free[i], GROUP);
            mbar_init(&p_ready[i], GROUP);
            mbar_init(&o_done[i], 1);
            mbar_init(&kv_free[i], ntiles);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    int any_bias = FAST ? 0 : 1;
    if (FAST) {
        // per-key tables for the whole (padded) sequence: -inf bias masks the keys past its end
        const float* kb = p.key_bias ? p.key_bias + static_cast<long long>(b) * p.S : nullptr;
        for (int i = threadIdx.x; i < nchunks * AK; i += ATT_THREADS) {
            const float v = i < p.S ? (kb ? kb[i] * 1.4426950408889634f : 0.f) : -INFINITY;
            any_bias |= (v != 0.f);
            s_kb[i] = v;
            s_kh[i] = drop_key_hash(p.seed, i);
        }
    }
    if (warp == 16) {
        tmem_alloc(tmem_slot, ATT_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    // an all-zero bias (no padding in this batch row, sequence a multiple of the chunk) takes the loops
    // without the per-key add: the row maximum is then taken over the raw scores
    const bool has_bias = __syncthreads_or(any_bias) != 0 || !(p.scale_log2 > 0.f);
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;

    if (warp == 18) {
        // ------------- K / V loader: stage (j & 1) is refilled once every tile's P V of chunk j is done -------------
        if (lane == 0) {
            auto load_kv = [&](int j) {
                const int st = j & 1;
                mbar_arrive_expect_tx(&k_full[st], TILE_B);
                tma_load_4d(sK + st * TILE_B, &tmK, &k_full[st], 0, j * AK, h, b);
                mbar_arrive_expect_tx(&v_full[st], TILE_B);
                tma_load_4d(sV + st * TILE_B, &tmV, &v_full[st], 0, j * AK, h, b);
            };
            mbar_arrive_expect_tx(q_full, ntiles * TILE_B);
            for (int t = 0; t < ntiles; ++t) tma_load_4d(sQ + t * TILE_B, &tmQ, q_full, 0, q_base + t * AQ, h, b);
            load_kv(0);
            if (nchunks > 1) load_kv(1);
            for (int j = 0; j + 2 < nchunks; ++j) {
                if (!mbar_wait(&kv_free[j & 1], (j >> 1) & 1, abort_flag)) break;
                load_kv(j + 2);
            }
        }
    } else if (warp >= 16) {
        // ------------- MMA issue, one warp per query tile: the two tiles' chains advance independently -------------
        const int t = warp - 16;
        if (lane == 0 && t < ntiles) {
            const uint32_t idesc_s = make_idesc_f16(fmt, 0, 0, AQ, AK);
            const uint32_t idesc_o = make_idesc_f16(fmt, 0, 1, AQ, AD);
            auto issue_s = [&](int j) {
                const uint32_t qa = smem_u32(sQ + t * TILE_B), ka = smem_u32(sK + (j & 1) * TILE_B);
#pragma unroll
                for (int k = 0; k < AD / 16; ++k)
                    umma_f16(tmem + t * TILE_COLS, make_smem_desc_sw128(qa + k * 32, 16, 1024),
                             make_smem_desc_sw128(ka + k * 32, 16, 1024), idesc_s, k != 0);
                umma_commit(&s_full[t]);
            };
            bool ok = mbar_wait(q_full, 0, abort_flag) && mbar_wait(&k_full[0], 0, abort_flag);
            if (ok) {
                tc_fence_after();
                issue_s(0);
            }
            for (int j = 0; j < nchunks && ok; ++j) {
                const uint32_t kv_phase = (j >> 1) & 1, nkv_phase = ((j + 1) >> 1) & 1;
                if (j + 1 < nchunks) {
                    ok = mbar_wait(&k_full[(j + 1) & 1], nkv_phase, abort_flag) &&
                         mbar_wait(&s_free[t], j & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(j + 1);
                }
                ok = mbar_wait(&p_ready[t], j & 1, abort_flag) && mbar_wait(&v_full[j & 1], kv_phase, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t pa = smem_u32(sP + t * P_BYTES), va = smem_u32(sV + (j & 1) * TILE_B);
#pragma unroll
                for (int k = 0; k < AK / 16; ++k)
                    umma_f16(tmem + t * TILE_COLS + 128,
                             make_smem_desc_sw128(pa + (k >> 2) * (P_BYTES / 2) + (k & 3) * 32, 16, 1024),
                             make_smem_desc_sw128(va + k * 2048, 8192, 1024), idesc_o, (j | k) != 0);
                umma_commit(&o_done[t]);
                umma_commit(&kv_free[j & 1]);
            }
        }
    } else if ((warp >> 3) < ntiles) {
        // ------------- softmax: in tile t the thread pair (r, r + 128) owns query row r -------------
        const int t = warp >> 3;
        const int idx = threadIdx.x & (GROUP - 1);
        const int r = idx & 127;     // row in tile == TMEM lane
        const int half = idx >> 7;   // which 64 columns of a chunk / 32 columns of O
        const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t col_s = tmem + t * TILE_COLS, col_o = col_s + 128;
        const int q = q_base + t * AQ + r;
        const float* kbg = p.key_bias ? p.key_bias + static_cast<long long>(b) * p.S : nullptr;
        const uint32_t row_hash = drop_row_hash(p.seed, b, h, q, p.H, p.S);
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        const uint32_t sw = r & 7;
        uint8_t* prow = sP + t * P_BYTES + half * (P_BYTES / 2) + (r >> 3) * 1024 + sw * 128;
        float* xbase = s_xch + t * 512;
        // bias (log2 units, -inf past the end of the sequence) and dropout hash of 4 consecutive keys
        auto cols4 = [&](int key, float4& kb, uint4& kh) {
            if (FAST) {
                kb = *reinterpret_cast<const float4*>(s_kb + key);
                if (p.thr32) kh = *reinterpret_cast<const uint4*>(s_kh + key);
            } else {
                float kbv[4];
                uint32_t khv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int kk = key + i;
                    kbv[i] = kk < p.S ? (kbg ? kbg[kk] * 1.4426950408889634f : 0.f) : -INFINITY;
                    khv[i] = drop_key_hash(p.seed, kk);
                }
                kb = make_float4(kbv[0], kbv[1], kbv[2], kbv[3]);
                kh = make_uint4(khv[0], khv[1], khv[2], khv[3]);
            }
        };
        for (int j = 0; j < nchunks; ++j) {
            // after a failed wait the loop keeps running (every later wait fails at once) so that the pair of
            // threads sharing a row still meets at the named barrier below
            if (!mbar_wait(&s_full[t], j & 1, abort_flag)) {
                ok = false;
            }
            tc_fence_after();
            const int key0 = j * AK + half * 64;
            // pass 1: maximum over this thread's 64 columns of the scaled, biased scores (log2 units).
            // Tensor-memory reads are pipelined in 16-column pieces: the next piece is in flight while
            // the current one is processed.
            float cm = -INFINITY;
            const uint32_t s_addr = col_s + lane_addr + half * 64;
            const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2);
            {
                uint32_t va[16], vb[16];
                auto max16 = [&](const uint32_t(&v)[16], int colbase) {
                    if (has_bias) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            float4 kb;
                            uint4 kh = make_uint4(0, 0, 0, 0);
                            cols4(key0 + colbase + g * 4, kb, kh);
                            float s0, s1, s2, s3;
                            f2_unpack(f2_fma(f2_pack_bits(v[g * 4], v[g * 4 + 1]), scale2, f2_pack(kb.x, kb.y)), s0, s1);
                            f2_unpack(f2_fma(f2_pack_bits(v[g * 4 + 2], v[g * 4 + 3]), scale2, f2_pack(kb.z, kb.w)), s2,
                                      s3);
                            cm = fmax3(cm, s0, s1);
                            cm = fmax3(cm, s2, s3);
                        }
                    } else {
#pragma unroll
                        for (int g = 0; g < 8; ++g)
                            cm = fmax3(cm, __uint_as_float(v[g * 2]), __uint_as_float(v[g * 2 + 1]));
                    }
                };
                tmem_ld16(s_addr, va);
                tmem_ld_wait();
                tmem_ld16(s_addr + 16, vb);
                max16(va, 0);
                tmem_ld_wait();
                tmem_ld16(s_addr + 32, va);
                max16(vb, 16);
                tmem_ld_wait();
                tmem_ld16(s_addr + 48, vb);
                max16(va, 32);
                tmem_ld_wait();
                max16(vb, 48);
            }
            if (!has_bias) cm *= p.scale_log2;   // scale > 0: the maximum of the raw scores, scaled
            float* xch = xbase + (j & 1) * 256;
            xch[half * 128 + r] = cm;
            bar_sync_named(1 + t, GROUP);
            cm = fmaxf(cm, xch[(half ^ 1) * 128 + r]);
            // Lazy rescaling: the running reference m only moves when the row maximum grew by more than
            // 2^8 since it was set; until then probabilities are taken relative to the old reference
            // (at most 256, exact in the final normalisation), and the accumulator round trip through
            // tensor memory is skipped for the whole warp.
            const float m_new = fmaxf(m, cm);
            float m_use;
            if (m_new - m <= 8.f)
                m_use = m;
            else
                m_use = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = exp2f(m - m_use);
            // the previous P V product must be complete before P is overwritten and O rescaled
            if (j > 0) {
                if (!mbar_wait(&o_done[t], (j - 1) & 1, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (__any_sync(0xffffffffu, alpha != 1.f)) {
                    uint32_t v[32];
                    tmem_ld32(col_o + lane_addr + half * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    tmem_st32(col_o + lane_addr + half * 32, v);
                    tmem_st_wait();
                }
            }
            // pass 2: probabilities -> shared memory (16-bit, swizzled K-major).  Dropped entries are
            // zeroed here; the 1 / (1 - p) factor is applied once to the finished row.
            uint64_t rs2 = f2_pack(0.f, 0.f);
            {
                uint32_t va[16], vb[16];
                const uint64_t negm2 = f2_pack(-m_use, -m_use);
                auto prob16 = [&](const uint32_t(&v)[16], int colbase) {
#pragma unroll
                    for (int g = 0; g < 2; ++g) {
                        float pr[8];
#pragma unroll
                        for (int hq = 0; hq < 2; ++hq) {
                            float4 kb = make_float4(0.f, 0.f, 0.f, 0.f);
                            uint4 kh = make_uint4(0, 0, 0, 0);
                            if (has_bias) {
                                cols4(key0 + colbase + g * 8 + hq * 4, kb, kh);
                            } else if (p.thr32) {
                                if (FAST) {
                                    kh = *reinterpret_cast<const uint4*>(s_kh + key0 + colbase + g * 8 + hq * 4);
                                } else {
                                    cols4(key0 + colbase + g * 8 + hq * 4, kb, kh);
                                }
                            }
                            const uint32_t khv[4] = {kh.x, kh.y, kh.z, kh.w};
                            const int e0 = g * 8 + hq * 4;
                            uint64_t x01, x23;
                            if (has_bias) {
                                x01 = f2_add(f2_fma(f2_pack_bits(v[e0], v[e0 + 1]), scale2, f2_pack(kb.x, kb.y)), negm2);
                                x23 = f2_add(f2_fma(f2_pack_bits(v[e0 + 2], v[e0 + 3]), scale2, f2_pack(kb.z, kb.w)),
                                             negm2);
                            } else {
                                x01 = f2_fma(f2_pack_bits(v[e0], v[e0 + 1]), scale2, negm2);
                                x23 = f2_fma(f2_pack_bits(v[e0 + 2], v[e0 + 3]), scale2, negm2);
                            }
                            float x[4];
                            f2_unpack(x01, x[0], x[1]);
                            f2_unpack(x23, x[2], x[3]);
                            float e[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) e[i] = ex2_approx(x[i]);
                            rs2 = f2_add(rs2, f2_pack(e[0], e[1]));
                            rs2 = f2_add(rs2, f2_pack(e[2], e[3]));
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                pr[hq * 4 + i] = (!p.thr32 || drop_keep(row_hash, khv[i], p.thr32)) ? e[i] : 0.f;
                        }
                        uint4 qv;
                        qv.x = pack2<T>(pr[0], pr[1]);
                        qv.y = pack2<T>(pr[2], pr[3]);
                        qv.z = pack2<T>(pr[4], pr[5]);
                        qv.w = pack2<T>(pr[6], pr[7]);
                        *reinterpret_cast<uint4*>(prow + ((static_cast<uint32_t>(colbase / 8 + g) ^ sw) << 4)) = qv;
                    }
                };
                tmem_ld16(s_addr, va);
                tmem_ld_wait();
                tmem_ld16(s_addr + 16, vb);
                prob16(va, 0);
                tmem_ld_wait();
                tmem_ld16(s_addr + 32, va);
                prob16(vb, 16);
                tmem_ld_wait();
                tmem_ld16(s_addr + 48, vb);
                prob16(va, 32);
                tmem_ld_wait();
                // last read of S: the next Q K^T may overwrite it
                tc_fence_before();
                mbar_arrive(&s_free[t]);
                prob16(vb, 48);
            }
            float rs_lo, rs_hi;
            f2_unpack(rs2, rs_lo, rs_hi);
            const float rs = rs_lo + rs_hi;
            l = l * alpha + rs;
            m = m_new == -INFINITY ? -INFINITY : m_use;
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(&p_ready[t]);
        }
        if (ok && mbar_wait(&o_done[t], (nchunks - 1) & 1, abort_flag)) {
            tc_fence_after();
            // the pair's partial row sums
            float* xch = xbase + (nchunks & 1) * 256;
            xch[half * 128 + r] = l;
            bar_sync_named(1 + t, GROUP);
            l += xch[(half ^ 1) * 128 + r];
            const float inv_l = l > 0.f ? p.inv_keep / l : 0.f;
            T* orow = reinterpret_cast<T*>(p.O) + b * p.o_sb + static_cast<long long>(q) * p.o_ss + h * p.o_sh +
                      half * 32;
            uint32_t v[32];
            tmem_ld32(col_o + lane_addr + half * 32, v);
            tmem_ld_wait();
            if (q < p.S) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint4 qv;
                    qv.x = pack2<T>(__uint_as_float(v[g * 8]) * inv_l, __uint_as_float(v[g * 8 + 1]) * inv_l);
                    qv.y = pack2<T>(__uint_as_float(v[g * 8 + 2]) * inv_l, __uint_as_float(v[g * 8 + 3]) * inv_l);
                    qv.z = pack2<T>(__uint_as_float(v[g * 8 + 4]) * inv_l, __uint_as_float(v[g * 8 + 5]) * inv_l);
                    qv.w = pack2<T>(__uint_as_float(v[g * 8 + 6]) * inv_l, __uint_as_float(v[g * 8 + 7]) * inv_l);
                    *reinterpret_cast<uint4*>(orow + g * 8) = qv;
                }
                if (half == 0)
                    p.lse[(static_cast<long long>(b) * p.H + h) * p.S + q] =
                        (m == -INFINITY ? 0.f : m) * 0.6931471805599453f + __logf(fmaxf(l, 1e-30f));
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
    if (warp == 16) {
        tc_fence_after();
        tmem_dealloc(tmem, ATT_TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------------------
// Persistent variant.  With sequences of a few hundred tokens a CTA of the kernel above lives for only a few
// chunks, and what it spends outside its steady state -- tensor-memory allocation, barrier set-up, the first
// loads, the last store, the launch of its successor -- is a third of its life (measured: 6 us of 18 us at
// S = 512).  Here one CTA per SM walks a list of work items (batch, head, pair of query tiles) and every role
// runs ahead on its own: the loader fetches the next item's Q (second buffer) and streams K / V through the
// same two-stage ring across item boundaries, the MMA warps issue the next item's first Q K^T while the
// softmax threads still write the previous item's output, so the fill and drain of consecutive items overlap.
// Used when the whole (padded) sequence fits the per-key tables and every item has two full query tiles.
// ---------------------------------------------------------------------------------------------------------
constexpr int PQ_BUFS = 2;
// Q (2 buffers x 2 tiles) + K, V (2 stages each) + P (2 tiles) + row-stat exchange [tile][3 slots][half][128]
// + key bias (2 buffers) + key hashes + flags / barriers
constexpr int ATTP_SMEM = PQ_BUFS * 2 * TILE_B + 4 * TILE_B + 2 * P_BYTES + 2 * 3 * 2 * 128 * 4 + 2 * KB_MAX * 4 +
                          KB_MAX * 4 + 512;

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS, 1)
    attn_fwd_persist_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                            const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p, const int nitems) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;                                 // [2 bufs][2 tiles][TILE_B]
    uint8_t* sK = smem + PQ_BUFS * 2 * TILE_B;          // [2 stages][TILE_B]
    uint8_t* sV = sK + 2 * TILE_B;                      // [2 stages][TILE_B]
    uint8_t* sP = sV + 2 * TILE_B;                      // [2 tiles][P_BYTES]
    float* s_xch = reinterpret_cast<float*>(sP + 2 * P_BYTES);   // [2 tiles][3][2][128]
    float* s_kb = s_xch + 2 * 3 * 2 * 128;              // [2 bufs][KB_MAX]
    uint32_t* s_kh = reinterpret_cast<uint32_t*>(s_kb + 2 * KB_MAX);   // [KB_MAX]
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_kh + KB_MAX);
    uint64_t* q_full = bars;          // [2 bufs]
    uint64_t* item_done = bars + 2;   // [2 bufs]
    uint64_t* k_full = bars + 4;      // [2 stages]
    uint64_t* v_full = bars + 6;      // [2 stages]
    uint64_t* kv_free = bars + 8;     // [2 stages]
    uint64_t* s_full = bars + 10;     // [2 tiles]
    uint64_t* s_free = bars + 12;     // [2 tiles]
    uint64_t* p_ready = bars + 14;    // [2 tiles]
    uint64_t* o_done = bars + 16;     // [2 tiles]
    uint64_t* o_free = bars + 18;     // [2 tiles]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* s_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [2 bufs]: any non-zero key bias

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nchunks = p.S / AK;
    const int nqp = p.S / (2 * AQ);
    const int my_items = blockIdx.x < nitems ? (nitems - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    const int total_chunks = my_items * nchunks;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&q_full[i], 1);
            mbar_init(&item_done[i], 2 * GROUP);
            mbar_init(&k_full[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&kv_free[i], 2);
            mbar_init(&s_full[i], 1);
            mbar_init(&s_free[i], GROUP);
            mbar_init(&p_ready[i], GROUP);
            mbar_init(&o_done[i], 1);
            mbar_init(&o_free[i], GROUP);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    for (int i = threadIdx.x; i < p.S; i += ATT_THREADS) s_kh[i] = drop_key_hash(p.seed, i);
    if (warp == 16) {
        tmem_alloc(tmem_slot, ATT_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
    auto decode = [&](int item, int& b, int& h, int& q_base) {
        const int qp = item % nqp;
        const int bh = item / nqp;
        h = bh % p.H;
        b = bh / p.H;
        q_base = qp * 2 * AQ;
    };

    if (warp == 18) {
        // ------------- loader: per item the key-bias table and Q, then K / V chunk by chunk -------------
        bool ok = true;
        int k = 0;
        for (int item = blockIdx.x; item < nitems; item += gridDim.x, ++k) {
            const int buf = k & 1;
            int b, h, q_base;
            decode(item, b, h, q_base);
            // the buffer's previous item (k - 2) must be finished by every softmax thread
            if (k >= 2 && !mbar_wait(&item_done[buf], ((k >> 1) - 1) & 1, abort_flag)) ok = false;
            const float* kb = p.key_bias ? p.key_bias + static_cast<long long>(b) * p.S : nullptr;
            int any = 0;
            for (int i = lane; i < p.S; i += 32) {
                const float v = kb ? kb[i] * 1.4426950408889634f : 0.f;
                any |= (v != 0.f);
                s_kb[buf * KB_MAX + i] = v;
            }
            any = __any_sync(0xffffffffu, any);
            if (lane == 0) s_flag[buf] = any;
            __syncwarp();
            if (lane == 0 && ok) {
                mbar_arrive_expect_tx(&q_full[buf], 2 * TILE_B);
                tma_load_4d(sQ + (buf * 2 + 0) * TILE_B, &tmQ, &q_full[buf], 0, q_base, h, b);
                tma_load_4d(sQ + (buf * 2 + 1) * TILE_B, &tmQ, &q_full[buf], 0, q_base + AQ, h, b);
            }
            for (int j = 0; j < nchunks; ++j) {
                const int c = k * nchunks + j, st = c & 1;
                if (c >= 2 && !mbar_wait(&kv_free[st], ((c >> 1) - 1) & 1, abort_flag)) ok = false;
                if (lane == 0 && ok) {
                    mbar_arrive_expect_tx(&k_full[st], TILE_B);
                    tma_load_4d(sK + st * TILE_B, &tmK, &k_full[st], 0, j * AK, h, b);
                    mbar_arrive_expect_tx(&v_full[st], TILE_B);
                    tma_load_4d(sV + st * TILE_B, &tmV, &v_full[st], 0, j * AK, h, b);
                }
            }
        }
    } else if (warp >= 16) {
        // ------------- MMA issue, one warp per query tile, running over all items of this CTA -------------
        const int t = warp - 16;
        if (lane == 0 && total_chunks > 0) {
            const uint32_t idesc_s = make_idesc_f16(fmt, 0, 0, AQ, AK);
            const uint32_t idesc_o = make_idesc_f16(fmt, 0, 1, AQ, AD);
            auto issue_s = [&](int c) {
                const int buf = (c / nchunks) & 1;
                const uint32_t qa = smem_u32(sQ + (buf * 2 + t) * TILE_B), ka = smem_u32(sK + (c & 1) * TILE_B);
#pragma unroll
                for (int kk = 0; kk < AD / 16; ++kk)
                    umma_f16(tmem + t * TILE_COLS, make_smem_desc_sw128(qa + kk * 32, 16, 1024),
                             make_smem_desc_sw128(ka + kk * 32, 16, 1024), idesc_s, kk != 0);
                umma_commit(&s_full[t]);
            };
            bool ok = mbar_wait(&q_full[0], 0, abort_flag) && mbar_wait(&k_full[0], 0, abort_flag);
            if (ok) {
                tc_fence_after();
                issue_s(0);
            }
            for (int c = 0; c < total_chunks && ok; ++c) {
                const int j = c % nchunks, k = c / nchunks;
                if (c + 1 < total_chunks) {
                    const int kn = (c + 1) / nchunks;
                    if ((c + 1) % nchunks == 0) ok = mbar_wait(&q_full[kn & 1], (kn >> 1) & 1, abort_flag);
                    ok = ok && mbar_wait(&k_full[(c + 1) & 1], ((c + 1) >> 1) & 1, abort_flag) &&
                         mbar_wait(&s_free[t], c & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(c + 1);
                }
                ok = mbar_wait(&p_ready[t], c & 1, abort_flag) && mbar_wait(&v_full[c & 1], (c >> 1) & 1, abort_flag);
                // the first product of an item overwrites O: the previous item's output must have been read
                if (ok && j == 0 && k > 0) ok = mbar_wait(&o_free[t], (k - 1) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t pa = smem_u32(sP + t * P_BYTES), va = smem_u32(sV + (c & 1) * TILE_B);
#pragma unroll
                for (int kk = 0; kk < AK / 16; ++kk)
                    umma_f16(tmem + t * TILE_COLS + 128,
                             make_smem_desc_sw128(pa + (kk >> 2) * (P_BYTES / 2) + (kk & 3) * 32, 16, 1024),
                             make_smem_desc_sw128(va + kk * 2048, 8192, 1024), idesc_o, (j | kk) != 0);
                umma_commit(&o_done[t]);
                umma_commit(&kv_free[c & 1]);
            }
        }
    } else {
        // ------------- softmax: in tile t the thread pair (r, r + 128) owns query row r -------------
        const int t = warp >> 3;
        const int idx = threadIdx.x & (GROUP - 1);
        const int r = idx & 127;
        const int half = idx >> 7;
        const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t col_s = tmem + t * TILE_COLS, col_o = col_s + 128;
        const uint32_t sw = r & 7;
        uint8_t* prow = sP + t * P_BYTES + half * (P_BYTES / 2) + (r >> 3) * 1024 + sw * 128;
        float* xbase = s_xch + t * (3 * 256);
        const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2);
        const uint32_t s_addr = col_s + lane_addr + half * 64;
        bool ok = true;
        int k = 0;
        for (int item = blockIdx.x; item < nitems; item += gridDim.x, ++k) {
            const int buf = k & 1;
            int b, h, q_base;
            decode(item, b, h, q_base);
            const int q = q_base + t * AQ + r;
            const uint32_t row_hash = drop_row_hash(p.seed, b, h, q, p.H, p.S);
            // the item's key-bias table (and Q) have landed
            if (!mbar_wait(&q_full[buf], (k >> 1) & 1, abort_flag)) ok = false;
            const bool has_bias = s_flag[buf] != 0 || !(p.scale_log2 > 0.f);
            const float* kbt = s_kb + buf * KB_MAX;
            float m = -INFINITY, l = 0.f;
            for (int j = 0; j < nchunks; ++j) {
                const int c = k * nchunks + j;
                if (!mbar_wait(&s_full[t], c & 1, abort_flag)) ok = false;
                tc_fence_after();
                const int key0 = j * AK + half * 64;
                float cm = -INFINITY;
                {
                    uint32_t va[16], vb[16];
                    auto max16 = [&](const uint32_t(&v)[16], int colbase) {
                        if (has_bias) {
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                const float4 kb = *reinterpret_cast<const float4*>(kbt + key0 + colbase + g * 4);
                                float s0, s1, s2, s3;
                                f2_unpack(f2_fma(f2_pack_bits(v[g * 4], v[g * 4 + 1]), scale2, f2_pack(kb.x, kb.y)), s0,
                                          s1);
                                f2_unpack(f2_fma(f2_pack_bits(v[g * 4 + 2], v[g * 4 + 3]), scale2, f2_pack(kb.z, kb.w)),
                                          s2, s3);
                                cm = fmax3(cm, s0, s1);
                                cm = fmax3(cm, s2, s3);
                            }
                        } else {
#pragma unroll
                            for (int g = 0; g < 8; ++g)
                                cm = fmax3(cm, __uint_as_float(v[g * 2]), __uint_as_float(v[g * 2 + 1]));
                        }
                    };
                    tmem_ld16(s_addr, va);
                    tmem_ld_wait();
                    tmem_ld16(s_addr + 16, vb);
                    max16(va, 0);
                    tmem_ld_wait();
                    tmem_ld16(s_addr + 32, va);
                    max16(vb, 16);
                    tmem_ld_wait();
                    tmem_ld16(s_addr + 48, vb);
                    max16(va, 32);
                    tmem_ld_wait();
                    max16(vb, 48);
                }
                if (!has_bias) cm *= p.scale_log2;
                float* xch = xbase + (c & 1) * 256;
                xch[half * 128 + r] = cm;
                bar_sync_named(1 + t, GROUP);
                cm = fmaxf(cm, xch[(half ^ 1) * 128 + r]);
                const float m_new = fmaxf(m, cm);
                float m_use;
                if (m_new - m <= 8.f)
                    m_use = m;
                else
                    m_use = m_new == -INFINITY ? 0.f : m_new;
                const float alpha = exp2f(m - m_use);
                if (j > 0) {
                    if (!mbar_wait(&o_done[t], (c - 1) & 1, abort_flag)) ok = false;
                    tc_fence_after();
                    if (__any_sync(0xffffffffu, alpha != 1.f)) {
                        uint32_t v[32];
                        tmem_ld32(col_o + lane_addr + half * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        tmem_st32(col_o + lane_addr + half * 32, v);
                        tmem_st_wait();
                    }
                }
                uint64_t rs2 = f2_pack(0.f, 0.f);
                {
                    uint32_t va[16], vb[16];
                    const uint64_t negm2 = f2_pack(-m_use, -m_use);
                    auto prob16 = [&](const uint32_t(&v)[16], int colbase) {
#pragma unroll
                        for (int g = 0; g < 2; ++g) {
                            float pr[8];
#pragma unroll
                            for (int hq = 0; hq < 2; ++hq) {
                                const int key = key0 + colbase + g * 8 + hq * 4;
                                uint4 kh = make_uint4(0, 0, 0, 0);
                                if (p.thr32) kh = *reinterpret_cast<const uint4*>(s_kh + key);
                                const uint32_t khv[4] = {kh.x, kh.y, kh.z, kh.w};
                                const int e0 = g * 8 + hq * 4;
                                uint64_t x01, x23;
                                if (has_bias) {
                                    const float4 kb = *reinterpret_cast<const float4*>(kbt + key);
                                    x01 = f2_add(f2_fma(f2_pack_bits(v[e0], v[e0 + 1]), scale2, f2_pack(kb.x, kb.y)),
                                                 negm2);
                                    x23 = f2_add(f2_fma(f2_pack_bits(v[e0 + 2], v[e0 + 3]), scale2, f2_pack(kb.z, kb.w)),
                                                 negm2);
                                } else {
                                    x01 = f2_fma(f2_pack_bits(v[e0], v[e0 + 1]), scale2, negm2);
                                    x23 = f2_fma(f2_pack_bits(v[e0 + 2], v[e0 + 3]), scale2, negm2);
                                }
                                float x[4], e[4];
                                f2_unpack(x01, x[0], x[1]);
                                f2_unpack(x23, x[2], x[3]);
#pragma unroll
                                for (int i = 0; i < 4; ++i) e[i] = ex2_approx(x[i]);
                                rs2 = f2_add(rs2, f2_pack(e[0], e[1]));
                                rs2 = f2_add(rs2, f2_pack(e[2], e[3]));
#pragma unroll
                                for (int i = 0; i < 4; ++i)
                                    pr[hq * 4 + i] = (!p.thr32 || drop_keep(row_hash, khv[i], p.thr32)) ? e[i] : 0.f;
                            }
                            uint4 qv;
                            qv.x = pack2<T>(pr[0], pr[1]);
                            qv.y = pack2<T>(pr[2], pr[3]);
                            qv.z = pack2<T>(pr[4], pr[5]);
                            qv.w = pack2<T>(pr[6], pr[7]);
                            *reinterpret_cast<uint4*>(prow + ((static_cast<uint32_t>(colbase / 8 + g) ^ sw) << 4)) = qv;
                        }
                    };
                    tmem_ld16(s_addr, va);
                    tmem_ld_wait();
                    tmem_ld16(s_addr + 16, vb);
                    prob16(va, 0);
                    tmem_ld_wait();
                    tmem_ld16(s_addr + 32, va);
                    prob16(vb, 16);
                    tmem_ld_wait();
                    tmem_ld16(s_addr + 48, vb);
                    prob16(va, 32);
                    tmem_ld_wait();
                    tc_fence_before();
                    mbar_arrive(&s_free[t]);
                    prob16(vb, 48);
                }
                float rs_lo, rs_hi;
                f2_unpack(rs2, rs_lo, rs_hi);
                l = l * alpha + (rs_lo + rs_hi);
                m = m_new == -INFINITY ? -INFINITY : m_use;
                fence_proxy_async();
                tc_fence_before();
                mbar_arrive(&p_ready[t]);
            }
            // ---- the item's output: wait for its last product, take O out of tensor memory, release it
            const int c_last = k * nchunks + nchunks - 1;
            if (!mbar_wait(&o_done[t], c_last & 1, abort_flag)) ok = false;
            tc_fence_after();
            float* xch = xbase + 2 * 256;
            xch[half * 128 + r] = l;
            bar_sync_named(1 + t, GROUP);
            l += xch[(half ^ 1) * 128 + r];
            const float inv_l = l > 0.f ? p.inv_keep / l : 0.f;
            uint32_t v[32];
            tmem_ld32(col_o + lane_addr + half * 32, v);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(&o_free[t]);
            if (ok) {
                T* orow = reinterpret_cast<T*>(p.O) + b * p.o_sb + static_cast<long long>(q) * p.o_ss + h * p.o_sh +
                          half * 32;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint4 qv;
                    qv.x = pack2<T>(__uint_as_float(v[g * 8]) * inv_l, __uint_as_float(v[g * 8 + 1]) * inv_l);
                    qv.y = pack2<T>(__uint_as_float(v[g * 8 + 2]) * inv_l, __uint_as_float(v[g * 8 + 3]) * inv_l);
                    qv.z = pack2<T>(__uint_as_float(v[g * 8 + 4]) * inv_l, __uint_as_float(v[g * 8 + 5]) * inv_l);
                    qv.w = pack2<T>(__uint_as_float(v[g * 8 + 6]) * inv_l, __uint_as_float(v[g * 8 + 7]) * inv_l);
                    *reinterpret_cast<uint4*>(orow + g * 8) = qv;
                }
                if (half == 0)
                    p.lse[(static_cast<long long>(b) * p.H + h) * p.S + q] =
                        (m == -INFINITY ? 0.f : m) * 0.6931471805599453f + __logf(fmaxf(l, 1e-30f));
            }
            mbar_arrive(&item_done[buf]);
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
    if (warp == 16) {
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
    p.thr32 = drop_threshold(a.p_drop);
    p.inv_keep = a.p_drop > 0.f ? 1.f / (1.f - a.p_drop) : 1.f;
    p.seed = drop_seed(a.seed, a.offset);
    p.err = error_word_ptr();
    if (!p.err) return -3;
    // sequences of whole query-tile pairs that fit the per-key tables run on the persistent kernel
    static int persist_env = -1;
    if (persist_env < 0) {
        const char* e = getenv("RB_ATTN_PERSISTENT");
        persist_env = (e && e[0] == '0') ? 0 : 1;
    }
    if (persist_env && a.S % (2 * AQ) == 0 && a.S <= KB_MAX) {
        auto pk = attn_fwd_persist_kernel<T>;
        static bool pattr[64] = {};
        int pdev = 0;
        cudaGetDevice(&pdev);
        if (!pattr[pdev & 63]) {
            if (cudaFuncSetAttribute(pk, cudaFuncAttributeMaxDynamicSharedMemorySize, ATTP_SMEM) != cudaSuccess)
                return -4;
            pattr[pdev & 63] = true;
        }
        const long long nitems = static_cast<long long>(a.B) * a.H * (a.S / (2 * AQ));
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, pdev);
        if (sms <= 0) sms = 148;
        const int grid = nitems < sms ? static_cast<int>(nitems) : sms;
        pk<<<grid, ATT_THREADS, ATTP_SMEM, st>>>(tq, tk, tv, p, static_cast<int>(nitems));
        return cudaGetLastError() == cudaSuccess ? 0 : -1;
    }
    const bool fast = (a.S + AK - 1) / AK * AK <= KB_MAX;
    auto kern = fast ? attn_fwd_kernel<T, true> : attn_fwd_kernel<T, false>;
    static bool attr_set[64][2] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63][fast]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) != cudaSuccess)
            return -4;
        attr_set[dev & 63][fast] = true;
    }
    dim3 grid((a.S + 2 * AQ - 1) / (2 * AQ), a.H, a.B);
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
