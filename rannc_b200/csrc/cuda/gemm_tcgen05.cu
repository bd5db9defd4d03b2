// Dense GEMM on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), sm_100a.
//
//   D[b] = epilogue( alpha * op(A[b]) * op(B[b]) )      op(A): M x K, op(B): K x N
//
// A is "K-major" when stored [M, K] row-major and "MN-major" when stored
// [K, M] row-major; B is K-major when stored [N, K] (the nn.Linear weight
// layout) and MN-major when stored [K, N].  The three GEMMs of a linear layer
// map onto it without a transposed copy:
//   forward  Y  = X  W^T : A = X  (K-major),  B = W  (K-major)
//   dgrad    dX = dY W   : A = dY (K-major),  B = W  (MN-major)
//   wgrad    dW = dY^T X : A = dY (MN-major), B = X  (MN-major)
//
// Structure: persistent CTAs (one per SM), 128 x 256 output tile, K step 64,
// 4-stage TMA->smem ring, fp32 accumulators double-buffered in TMEM (2 x 256
// columns) so the epilogue of tile i overlaps the main loop of tile i+1.
// Warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..9 = epilogue (with K = 1024 a tile's main loop is
// only 16 k steps, and four warps could not drain a 128 x 256 accumulator in that time).
//
// PAIR variant (cta_group::2): two CTAs of a cluster -- the two SMs of a TPC -- share a 256 x 256 tile.
// Each CTA loads its own 128 rows of A and HALF of the B tile (so a k step moves 32 KiB per SM instead
// of 48 KiB: the single-CTA tile is limited by the L2 -> shared-memory path, not by the tensor core),
// one thread of the first CTA issues the MMAs for both, and each CTA keeps and drains the accumulator of
// its own 128 rows.  Completion of both CTAs' loads is counted on the first CTA's barrier; stage-free
// and accumulator-full signals go to both CTAs with one multicast commit.  No load is multicast.
//
// This kernel takes the place of the cuBLAS calls the reference reaches through
// aten::linear / aten::matmul in its TorchScript interpreter
// (src/torch/TorchDriver.cpp:566) and in src/distop/DistMatmul.cpp:97-214.
#include "gemm_tcgen05.h"

#include <cstdlib>
#include <mutex>

#include "tc_common.cuh"

namespace rb {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int EPI_WARPS = 8;                         // two per TMEM lane quarter: each drains 128 of the 256 columns
constexpr int EPI_THREADS = 32 * EPI_WARPS;
constexpr int GEMM_THREADS = 64 + EPI_THREADS;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 8;

template <bool PAIR>
struct Cfg {
    static constexpr int STAGES = PAIR ? 6 : 4;
    static constexpr int B_ROWS = PAIR ? BN / 2 : BN;       // extent of the B tile one CTA loads
    static constexpr int B_STAGE_BYTES = B_ROWS * BK * 2;   // 16 / 32 KiB
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
    static constexpr int TILE_M = PAIR ? 2 * BM : BM;       // rows of the output tile of a CTA (pair)
};

struct GemmKernelParams {
    int M, N, K, batch;
    int a_major, b_major;
    int num_m_blocks, num_n_blocks, num_tiles, num_kb;
    int base_tiles, split_k, kb_per_split;  // split-K: num_tiles = base_tiles * split_k
    int rs_nranks, rs_cols;                 // reduce-scatter epilogue: column block j -> rs_peer[j]
    void* rs_peer[8];
    // all-gather prologue: B is assembled in local memory from column shards held by the ranks of a group
    int ag_nranks, ag_my_idx, ag_rows, ag_cols;  // shard r = [ag_rows, ag_cols] at ag_src[r]
    const void* ag_src[8];
    void* ag_dst;                                // [ag_rows, ag_nranks * ag_cols] (the B operand)
    unsigned int* ag_flags;                      // [8] counters, zero at launch: CTAs done copying shard r
    void* D;
    const void* bias;
    const void* residual;
    const void* aux_in;
    void* aux_out;
    long long ldd, strideD;
    float alpha;
    int flags;
    int* err;
    // implicit-GEMM convolution: see RbGemmArgs
    int conv_kb_per_tap, conv_b_tap_cols, b_row_shift;
    int map_hp, map_wp, map_h, map_w, map_pad;
    int conv_shift[49];
};

__device__ __forceinline__ void tile_coords(const GemmKernelParams& p, int tile, int& mb, int& nb,
                                            int& b, int& kb_begin, int& kb_end) {
    const int ks = tile / p.base_tiles;
    tile -= ks * p.base_tiles;
    kb_begin = ks * p.kb_per_split;
    kb_end = min(p.num_kb, kb_begin + p.kb_per_split);
    const int per_batch = p.num_m_blocks * p.num_n_blocks;
    b = tile / per_batch;
    int t = tile - b * per_batch;
    const int group_sz = GROUP_M * p.num_n_blocks;
    const int g = t / group_sz;
    const int first_m = g * GROUP_M;
    const int gm = min(GROUP_M, p.num_m_blocks - first_m);
    t -= g * group_sz;
    mb = first_m + (t % gm);
    nb = t / gm;
}

template <typename T>
__device__ __forceinline__ void load32(const T* ptr, bool vec_ok, int valid, float (&v)[32]) {
    if (vec_ok) {
        if constexpr (sizeof(T) == 2) {
            const uint4* p4 = reinterpret_cast<const uint4*>(ptr);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 q = p4[i];
                const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i * 8 + j] = to_f32<T>(e[j]);
            }
        } else {
            const float4* p4 = reinterpret_cast<const float4*>(ptr);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float4 q = p4[i];
                v[i * 4 + 0] = q.x;
                v[i * 4 + 1] = q.y;
                v[i * 4 + 2] = q.z;
                v[i * 4 + 3] = q.w;
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (j < valid) ? to_f32<T>(ptr[j]) : 0.f;
    }
}

template <typename T>
__device__ __forceinline__ void store32(T* ptr, bool vec_ok, int valid, const float (&v)[32]) {
    if (vec_ok) {
        if constexpr (sizeof(T) == 2) {
            uint4* p4 = reinterpret_cast<uint4*>(ptr);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 q;
                T* e = reinterpret_cast<T*>(&q);
#pragma unroll
                for (int j = 0; j < 8; ++j) e[j] = from_f32<T>(v[i * 8 + j]);
                p4[i] = q;
            }
        } else {
            float4* p4 = reinterpret_cast<float4*>(ptr);
#pragma unroll
            for (int i = 0; i < 8; ++i)
                p4[i] = make_float4(v[i * 4], v[i * 4 + 1], v[i * 4 + 2], v[i * 4 + 3]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < valid) ptr[j] = from_f32<T>(v[j]);
    }
}

template <typename InT, typename OutT, bool PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                        const __grid_constant__ CUtensorMap tmB, const GemmKernelParams p) {
    constexpr int STAGES = Cfg<PAIR>::STAGES;
    constexpr int B_STAGE_BYTES = Cfg<PAIR>::B_STAGE_BYTES;
    constexpr int STAGE_BYTES = Cfg<PAIR>::STAGE_BYTES;
    constexpr int TILE_M = Cfg<PAIR>::TILE_M;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* full = bars;                  // [STAGES]
    uint64_t* empty = bars + STAGES;        // [STAGES]
    uint64_t* tfull = bars + 2 * STAGES;    // [2]
    uint64_t* tempty = bars + 2 * STAGES + 2;  // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // PAIR: rank of this CTA in its pair; the first CTA issues the MMAs and owns the `full` / `tempty` counts
    const uint32_t crank = PAIR ? cluster_ctarank() : 0u;
    const int tile0 = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int tile_step = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tfull[a], 1);
            mbar_init(&tempty[a], PAIR ? 2 * EPI_WARPS : EPI_THREADS);   // PAIR: one arrival per epilogue warp of both CTAs
        }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 2) {
        if (PAIR) {
            tmem_alloc_pair(tmem_slot, TMEM_COLS);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, TMEM_COLS);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();   // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer ----------------
            int stage = 0;
            uint32_t phase = 0;
            uint32_t ag_ready = 0;
            bool ok = true;
            for (int tile = tile0; tile < p.num_tiles && ok; tile += tile_step) {
                int mb, nb, b, kb_begin, kb_end;
                tile_coords(p, tile, mb, nb, b, kb_begin, kb_end);
                const int m0 = mb * TILE_M + static_cast<int>(crank) * BM;
                const int n0 = nb * BN + (PAIR ? static_cast<int>(crank) * (BN / 2) : 0);
                for (int kbi = kb_begin; kbi < kb_end; ++kbi) {
                    int kb = kbi;
                    if (p.ag_nranks > 1) {
                        // start with the k-range (or column block) this rank holds itself; wait until every
                        // CTA has copied the shard this step reads into the local B buffer
                        int shard;
                        if (p.b_major == 0) {
                            kb = kbi + p.ag_my_idx * (p.ag_cols / BK);
                            if (kb >= p.num_kb) kb -= p.num_kb;
                            shard = (kb * BK) / p.ag_cols;
                        } else {
                            shard = n0 / p.ag_cols;
                        }
                        if (!(ag_ready & (1u << shard))) {
                            bool got = false;
                            const uint64_t t0 = globaltimer_ns();
                            for (uint32_t it = 0; it < RB_MBAR_SPIN_LIMIT && !*abort_flag; ++it) {
                                unsigned int v;
                                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.ag_flags + shard) : "memory");
                                if (v >= gridDim.x) {
                                    got = true;
                                    break;
                                }
                                if ((it & 0xff) == 0xff && globaltimer_ns() - t0 > RB_WAIT_LIMIT_NS) break;
                                __nanosleep(64);
                            }
                            if (!got) {
                                *abort_flag = 1;
                                ok = false;
                                break;
                            }
                            asm volatile("fence.proxy.async.global;" ::: "memory");
                            ag_ready |= 1u << shard;
                        }
                    }
                    if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) {
                        ok = false;
                        break;
                    }
                    uint8_t* a_dst = sA + stage * A_STAGE_BYTES;
                    uint8_t* b_dst = sB + stage * B_STAGE_BYTES;
                    const int k0 = kb * BK;
                    // A (K-major) reads columns ax of rows ay..; B (MN-major) reads columns +bx of rows bk..
                    int ax = k0, ay = m0, bx = 0, bk = k0 + p.b_row_shift;
                    if (p.conv_kb_per_tap > 0) {
                        const int tap = kb / p.conv_kb_per_tap;
                        ax = (kb - tap * p.conv_kb_per_tap) * BK;
                        ay = m0 + p.conv_shift[tap];
                        if (p.b_major != 0) {
                            bx = tap * p.conv_b_tap_cols;
                            bk = ax;
                        }
                    }
                    if constexpr (PAIR) {
                        // both CTAs' bytes are counted on the first CTA's barrier
                        if (crank == 0) mbar_arrive_expect_tx(&full[stage], 2 * STAGE_BYTES);
                        const uint32_t fb = mapa_shared(smem_u32(&full[stage]), 0);
                        if (p.a_major == 0) {
                            tma_load_3d_pair(a_dst, &tmA, fb, ax, ay, b);
                        } else {
#pragma unroll
                            for (int c = 0; c < BM / 64; ++c)
                                tma_load_3d_pair(a_dst + c * (BK * 128), &tmA, fb, m0 + c * 64, k0, b);
                        }
                        if (p.b_major == 0) {
                            tma_load_3d_pair(b_dst, &tmB, fb, k0, n0, b);
                        } else {
#pragma unroll
                            for (int c = 0; c < Cfg<PAIR>::B_ROWS / 64; ++c)
                                tma_load_3d_pair(b_dst + c * (BK * 128), &tmB, fb, n0 + bx + c * 64, bk, b);
                        }
                    } else {
                        mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
                        if (p.a_major == 0) {
                            tma_load_3d(a_dst, &tmA, &full[stage], ax, ay, b);
                        } else {
#pragma unroll
                            for (int c = 0; c < BM / 64; ++c)
                                tma_load_3d(a_dst + c * (BK * 128), &tmA, &full[stage], m0 + c * 64,
                                            k0, b);
                        }
                        if (p.b_major == 0) {
                            tma_load_3d(b_dst, &tmB, &full[stage], k0, n0, b);
                        } else {
#pragma unroll
                            for (int c = 0; c < BN / 64; ++c)
                                tma_load_3d(b_dst + c * (BK * 128), &tmB, &full[stage], n0 + bx + c * 64,
                                            bk, b);
                        }
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && crank == 0) {
            // ---------------- MMA issuer (PAIR: the first CTA issues for both) ----------------
            constexpr int fmt = (sizeof(InT) == 2 && std::is_same<InT, __nv_bfloat16>::value) ? 1 : 0;
            const uint32_t idesc = make_idesc_f16(fmt, p.a_major, p.b_major, TILE_M, BN);
            // per-UMMA_K (16 elements) advance of the smem start address
            const uint32_t a_kstep = (p.a_major == 0) ? 32u : 2048u;
            const uint32_t b_kstep = (p.b_major == 0) ? 32u : 2048u;
            const uint32_t a_lbo = (p.a_major == 0) ? 16u : BK * 128u;
            const uint32_t b_lbo = (p.b_major == 0) ? 16u : BK * 128u;
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int it = 0;
            for (int tile = tile0; tile < p.num_tiles && ok; tile += tile_step, ++it) {
                const int acc = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!(PAIR ? mbar_wait_cluster(&tempty[acc], acc_phase ^ 1, abort_flag)
                           : mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag)))
                    break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                int mb_, nb_, b_, kb_begin, kb_end;
                tile_coords(p, tile, mb_, nb_, b_, kb_begin, kb_end);
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!(PAIR ? mbar_wait_cluster(&full[stage], phase, abort_flag)
                               : mbar_wait(&full[stage], phase, abort_flag))) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(sA + stage * A_STAGE_BYTES);
                    const uint32_t b_addr = smem_u32(sB + stage * B_STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t da = make_smem_desc_sw128(a_addr + k * a_kstep, a_lbo, 1024);
                        const uint64_t db = make_smem_desc_sw128(b_addr + k * b_kstep, b_lbo, 1024);
                        if constexpr (PAIR)
                            umma_f16_pair(d_tmem, da, db, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
                        else
                            umma_f16(d_tmem, da, db, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
                    }
                    if constexpr (PAIR)
                        umma_commit_pair(&empty[stage], 3);   // frees the stage in both CTAs
                    else
                        umma_commit(&empty[stage]);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok) {
                    if constexpr (PAIR)
                        umma_commit_pair(&tfull[acc], 3);
                    else
                        umma_commit(&tfull[acc]);
                }
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5) ----------------
        if (p.ag_nranks > 1) {
            // all-gather prologue: the epilogue threads of every CTA copy their share of each peer's
            // shard into the local B buffer (plain 16-byte peer loads), in the order the k loop consumes
            // them (own shard first); a counter per shard tells the TMA producers when it is whole
            const int t = threadIdx.x - 64;
            const int vec_per_row = p.ag_cols / 8;
            const long long total = static_cast<long long>(p.ag_rows) * vec_per_row;
            const long long dst_ld = static_cast<long long>(p.ag_nranks) * p.ag_cols;
            for (int rr = 0; rr < p.ag_nranks; ++rr) {
                const int r = (p.ag_my_idx + rr) % p.ag_nranks;   // the order in which the k loop needs them
                const uint4* src = reinterpret_cast<const uint4*>(p.ag_src[r]);
                InT* dst = reinterpret_cast<InT*>(p.ag_dst) + static_cast<long long>(r) * p.ag_cols;
                for (long long i = static_cast<long long>(blockIdx.x) * EPI_THREADS + t; i < total;
                     i += static_cast<long long>(gridDim.x) * EPI_THREADS * 4) {
                    uint4 v[4];
                    long long idx[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        idx[u] = i + static_cast<long long>(u) * gridDim.x * EPI_THREADS;
                        if (idx[u] < total) v[u] = src[idx[u]];
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (idx[u] < total) {
                            const long long row = idx[u] / vec_per_row, c = idx[u] - row * vec_per_row;
                            *reinterpret_cast<uint4*>(dst + row * dst_ld + c * 8) = v[u];
                        }
                    }
                }
                asm volatile("fence.proxy.async.global;" ::: "memory");
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
                if (t == 0) atomicAdd(p.ag_flags + r, 1u);
            }
        }
        const int q = warp & 3;  // TMEM lane quarter this warp may access
        const int chalf = (warp - 2) >> 2;   // which 128 of the tile's 256 columns this warp drains
        const int row_in_tile = q * 32 + lane;
        const bool has_bias = p.flags & RB_GEMM_BIAS;
        const bool has_res = p.flags & RB_GEMM_RESIDUAL;
        const bool act_gelu = p.flags & RB_GEMM_GELU;
        const bool act_dgelu = p.flags & RB_GEMM_DGELU;
        const bool aux_out = p.flags & RB_GEMM_AUX_OUT;
        const bool accum = p.flags & RB_GEMM_ACCUM;
        const bool in_al = (p.ldd % 8 == 0);
        const bool out_al = (sizeof(OutT) == 2) ? (p.ldd % 8 == 0) : (p.ldd % 4 == 0);
        int it = 0;
        for (int tile = tile0; tile < p.num_tiles; tile += tile_step, ++it) {
            int mb, nb, b, kb_begin, kb_end;
            tile_coords(p, tile, mb, nb, b, kb_begin, kb_end);
            const int acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            if (!mbar_wait(&tfull[acc], acc_phase, abort_flag)) break;
            tc_fence_after();
            int row = mb * TILE_M + static_cast<int>(crank) * BM + row_in_tile;
            bool row_ok = row < p.M;
            if (p.map_hp > 0 && row_ok) {
                // rows are positions of a zero-padded image grid: only the interior is stored
                const int per_img = p.map_hp * p.map_wp;
                const int img = row / per_img;
                const int rem = row - img * per_img;
                const int yy = rem / p.map_wp - p.map_pad;
                const int xx = rem - (rem / p.map_wp) * p.map_wp - p.map_pad;
                row_ok = yy >= 0 && yy < p.map_h && xx >= 0 && xx < p.map_w;
                row = (img * p.map_h + yy) * p.map_w + xx;
            }
            const long long row_off = static_cast<long long>(b) * p.strideD +
                                      static_cast<long long>(row_ok ? row : 0) * p.ldd;
#pragma unroll 1
            for (int c = chalf * (BN / 64); c < (chalf + 1) * (BN / 64); ++c) {
                const int col = nb * BN + c * 32;
                if (col >= p.N) break;
                uint32_t r[32];
                tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 32, r);
                tmem_ld_wait();
                if (!row_ok) continue;
                const int valid = min(32, p.N - col);
                const bool full_chunk = valid == 32;
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
                if constexpr (std::is_same<OutT, float>::value) {
                    if (p.split_k > 1 || p.rs_nranks > 1) {
                        // partial sums (a K slice, and/or one replica's share of a reduce-scatter):
                        // accumulate with vector reductions.  With rs_nranks > 1 the output columns
                        // are split in equal blocks and block j lives in rank j's buffer, so the
                        // reduction goes to that peer's memory over NVLink.
                        float* dptr = reinterpret_cast<float*>(p.D) + row_off + col;
                        if (p.rs_nranks > 1) {
                            const int owner = col / p.rs_cols;
                            dptr = reinterpret_cast<float*>(p.rs_peer[owner]) + row_off + (col - owner * p.rs_cols);
                        }
                        if (full_chunk && out_al) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dptr + j),
                                             "f"(v[j]), "f"(v[j + 1]), "f"(v[j + 2]), "f"(v[j + 3])
                                             : "memory");
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (j < valid) atomicAdd(dptr + j, v[j]);
                        }
                        continue;
                    }
                }
                if (has_bias) {
                    float t[32];
                    load32(reinterpret_cast<const InT*>(p.bias) + col, full_chunk, valid, t);
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] += t[j];
                }
                if (aux_out)
                    store32(reinterpret_cast<InT*>(p.aux_out) + row_off + col, full_chunk && in_al,
                            valid, v);
                if (act_gelu) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
                }
                if (act_dgelu) {
                    float t[32];
                    load32(reinterpret_cast<const InT*>(p.aux_in) + row_off + col,
                           full_chunk && in_al, valid, t);
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] *= gelu_erf_grad(t[j]);
                }
                if (has_res) {
                    float t[32];
                    load32(reinterpret_cast<const InT*>(p.residual) + row_off + col,
                           full_chunk && in_al, valid, t);
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] += t[j];
                }
                OutT* dptr = reinterpret_cast<OutT*>(p.D) + row_off + col;
                if (accum) {
                    float t[32];
                    load32(dptr, full_chunk && out_al, valid, t);
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] += t[j];
                }
                store32(dptr, full_chunk && out_al, valid, v);
            }
            tc_fence_before();
            if constexpr (PAIR) {
                // the accumulator may be overwritten once the epilogue warps of BOTH CTAs have drained it
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty[acc]), 0));
            } else {
                mbar_arrive(&tempty[acc]);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            atomicExch(p.err, ERR_MBAR_TIMEOUT);
            // let bulk copies that may still be in flight land before the CTA's
            // shared memory is released
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000) {
            }
        }
        __syncthreads();
    }
    // PAIR: neither CTA leaves (or frees tensor memory) while the other may still signal its barriers or
    // its MMAs may still write this CTA's accumulators
    if (PAIR) cluster_sync_all();
    if (warp == 2) {
        tc_fence_after();
        if (PAIR)
            tmem_dealloc_pair(tmem_base, TMEM_COLS);
        else
            tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault,
                                             &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

int make_tmap_3d(CUtensorMap* out, const void* base, int dtype_16bit_kind, uint64_t d0, uint64_t d1,
                 uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0,
                 uint32_t b1, int swizzle128) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return -100;
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
    cuuint32_t box[3] = {b0, b1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMapDataType dt =
        dtype_16bit_kind == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = CUDA_SUCCESS;
    for (int attempt = 0; attempt < 2; ++attempt) {
        r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE,
               swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_ERROR_INVALID_CONTEXT) break;
        // a thread that has made no runtime call yet (an autograd worker whose first operator is ours) has
        // no context bound for driver entry points: bind the device's primary context and try again
        cudaFree(nullptr);
    }
    return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 1000;
}

int make_tmap_4d(CUtensorMap* out, const void* base, int fmt, uint64_t d0, uint64_t d1, uint64_t d2,
                 uint64_t d3, uint64_t s1, uint64_t s2, uint64_t s3, uint32_t b0, uint32_t b1) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return -100;
    cuuint64_t dims[4] = {d0, d1, d2, d3};
    cuuint64_t strides[3] = {s1, s2, s3};
    cuuint32_t box[4] = {b0, b1, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUtensorMapDataType dt =
        fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = CUDA_SUCCESS;
    for (int attempt = 0; attempt < 2; ++attempt) {
        r = fn(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_ERROR_INVALID_CONTEXT) break;
        cudaFree(nullptr);
    }
    return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 1000;
}

// fp32 tensor, 4-D, 128-byte swizzle: box [b0 <= 32 elements, b1 rows, 1, 1]
int make_tmap_4d_f32(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3,
                     uint64_t s1, uint64_t s2, uint64_t s3, uint32_t b0, uint32_t b1) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return -100;
    cuuint64_t dims[4] = {d0, d1, d2, d3};
    cuuint64_t strides[3] = {s1, s2, s3};
    cuuint32_t box[4] = {b0, b1, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = CUDA_SUCCESS;
    for (int attempt = 0; attempt < 2; ++attempt) {
        r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_ERROR_INVALID_CONTEXT) break;
        cudaFree(nullptr);
    }
    return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 1000;
}

static __device__ int g_error_word = 0;

int* error_word_ptr() {
    // one address per device
    static int* ptrs[64] = {nullptr};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return nullptr;
    if (!ptrs[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_error_word) != cudaSuccess) return nullptr;
        ptrs[dev] = static_cast<int*>(p);
    }
    return ptrs[dev];
}

int num_sms() {
    static int n[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return 148;
    if (!n[dev]) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
    return n[dev];
}

template <typename InT, typename OutT, bool PAIR>
static int launch(const RbGemmArgs& a, const CUtensorMap& tmA, const CUtensorMap& tmB,
                  const GemmKernelParams& p, cudaStream_t stream) {
    auto kern = gemm_tcgen05_kernel<InT, OutT, PAIR>;
    constexpr int smem = Cfg<PAIR>::SMEM_BYTES;
    static bool attr_set[64] = {false};
    static int max_clusters[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return -static_cast<int>(e);
        attr_set[dev & 63] = true;
    }
    if (!PAIR) {
        int grid = p.num_tiles < num_sms() ? p.num_tiles : num_sms();
        if (a.max_ctas > 0 && grid > a.max_ctas) grid = a.max_ctas;
        kern<<<grid, GEMM_THREADS, smem, stream>>>(tmA, tmB, p);
        cudaError_t e = cudaGetLastError();
        return e == cudaSuccess ? 0 : -static_cast<int>(e);
    }
    // one cluster of two CTAs per TPC; persistent over the pair tiles
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (!max_clusters[dev & 63]) {
        cfg.gridDim = dim3(num_sms(), 1, 1);
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) n = num_sms() / 2;
        max_clusters[dev & 63] = n;
    }
    int clusters = p.num_tiles < max_clusters[dev & 63] ? p.num_tiles : max_clusters[dev & 63];
    if (a.max_ctas > 1 && clusters > a.max_ctas / 2) clusters = a.max_ctas / 2;
    cfg.gridDim = dim3(2 * clusters, 1, 1);
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, p);
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

// RB_GEMM_PAIR_GATHER=1 also puts the gather -> GEMM variant on the pair kernel (same prologue code).  Measured
// with four local slices it is no faster there (0.230 ms against 0.223 ms for M 8192, N = K = 4096: the
// prologue copy, not the main loop, is what the variant adds), so it stays on the single-CTA kernel; the
// scatter epilogue does gain from the pair kernel (0.224 ms against 0.248 ms) and uses it.
static bool pair_gather_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("RB_GEMM_PAIR_GATHER");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}

// RB_GEMM_PAIR=0 keeps every GEMM on the single-CTA kernel
static bool pair_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("RB_GEMM_PAIR");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

}  // namespace rb

extern "C" int rb_gemm(const RbGemmArgs* a, void* stream_) {
    using namespace rb;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (a->M <= 0 || a->N <= 0 || a->K <= 0 || a->batch <= 0) return 0;
    // TMA needs 16-byte aligned bases and row strides
    if ((reinterpret_cast<uintptr_t>(a->A) & 15) || (reinterpret_cast<uintptr_t>(a->B) & 15) ||
        (a->lda % 8) || (a->ldb % 8) || (a->batch > 1 && ((a->strideA % 8) || (a->strideB % 8))))
        return -2;
    GemmKernelParams p;
    p.M = static_cast<int>(a->M);
    p.N = static_cast<int>(a->N);
    p.K = static_cast<int>(a->K);
    p.batch = static_cast<int>(a->batch);
    p.a_major = a->a_major;
    p.b_major = a->b_major;
    // The pair kernel (256 x 256 tile over two SMs) serves every GEMM with enough work to fill the GPU:
    // enough tiles, or few tiles and a long K that is split (weight gradients); the gather prologue and the
    // scatter epilogue are the same code in both variants.  Small problems stay on the single-CTA kernel.
    const bool accum32 = a->out_dtype == 1 && a->flags == RB_GEMM_ACCUM;
    bool pair = pair_enabled() && (a->ag_nranks <= 1 || pair_gather_enabled());
    if (pair) {
        const long long pt = ((a->M + 2 * BM - 1) / (2 * BM)) * ((a->N + BN - 1) / BN) * a->batch;
        const long long kbs = (a->K + BK - 1) / BK;
        if (pt < num_sms() / 2 && !(accum32 && a->M > BM && pt * (kbs / 4) >= num_sms() / 2)) pair = false;
    }
    p.num_m_blocks = pair ? (p.M + 2 * BM - 1) / (2 * BM) : (p.M + BM - 1) / BM;
    p.num_n_blocks = (p.N + BN - 1) / BN;
    p.base_tiles = p.num_m_blocks * p.num_n_blocks * p.batch;
    p.num_kb = (p.K + BK - 1) / BK;
    p.ag_nranks = a->ag_nranks > 1 ? a->ag_nranks : 0;
    p.ag_my_idx = a->ag_my_idx;
    p.ag_rows = a->ag_rows;
    p.ag_cols = a->ag_cols;
    p.ag_dst = const_cast<void*>(a->B);
    p.ag_flags = static_cast<unsigned int*>(a->ag_flags);
    for (int r = 0; r < 8; ++r) p.ag_src[r] = a->ag_nranks > 1 ? a->ag_src[r] : nullptr;
    if (p.ag_nranks > 1) {
        // shards are column blocks of the stored B matrix: [rows, ag_cols] each, ag_cols a multiple of the tile
        const long long stored_cols = a->b_major == 0 ? a->K : a->N;
        if (a->ag_nranks > 8 || a->batch != 1 || !a->ag_flags || a->ag_cols % 256 ||
            static_cast<long long>(a->ag_cols) * a->ag_nranks != stored_cols || a->ldb != stored_cols)
            return -6;
        cudaMemsetAsync(a->ag_flags, 0, 8 * sizeof(unsigned int), stream);
    }
    p.split_k = 1;
    p.rs_nranks = a->rs_nranks > 1 ? a->rs_nranks : 0;
    p.rs_cols = a->rs_nranks > 1 ? static_cast<int>(a->N / a->rs_nranks) : 0;
    for (int r = 0; r < 8; ++r) p.rs_peer[r] = a->rs_nranks > 1 ? a->rs_peer[r] : nullptr;
    if (p.rs_nranks > 1 && (a->out_dtype != 1 || a->flags != RB_GEMM_ACCUM || a->N % a->rs_nranks || p.rs_cols % 32 ||
                            a->rs_nranks > 8 || a->batch != 1))
        return -5;
    // Few output tiles and a long K (weight gradients): split K over CTAs and accumulate with
    // reductions.  Only for fp32 outputs that accumulate and have no other epilogue work.
    const int units = pair ? num_sms() / 2 : num_sms();   // CTAs (or CTA pairs) that run at once
    if (accum32 && p.base_tiles < units && p.num_kb >= 8) {
        double best = 0.0;
        for (int s = 1; s <= 32 && s * 4 <= p.num_kb; ++s) {
            const int work = p.base_tiles * s;
            const int waves = (work + units - 1) / units;
            const double eff = static_cast<double>(work) / (waves * units) - 0.005 * s;
            if (eff > best + 1e-9) {
                best = eff;
                p.split_k = s;
            }
        }
    }
    p.kb_per_split = (p.num_kb + p.split_k - 1) / p.split_k;
    p.split_k = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;
    p.num_tiles = p.base_tiles * p.split_k;
    p.D = a->D;
    p.bias = a->bias;
    p.residual = a->residual;
    p.aux_in = a->aux_in;
    p.aux_out = a->aux_out;
    p.ldd = a->ldd;
    p.strideD = a->strideD;
    p.alpha = a->alpha;
    p.flags = a->flags;
    p.err = error_word_ptr();
    if (!p.err) return -3;
    p.conv_kb_per_tap = 0;
    p.conv_b_tap_cols = 0;
    p.b_row_shift = a->b_major != 0 ? a->b_row_shift : 0;
    p.map_hp = a->map_hp;
    p.map_wp = a->map_wp;
    p.map_h = a->map_h;
    p.map_w = a->map_w;
    p.map_pad = a->map_pad;
    for (int t = 0; t < 49; ++t) p.conv_shift[t] = 0;
    if (a->conv_taps > 0) {
        // A must be K-major with conv_c (a multiple of the k step) columns; no batch, gather or scatter
        if (a->conv_taps > 49 || a->a_major != 0 || a->conv_c % BK || a->lda != a->conv_c || a->batch != 1 ||
            a->K != static_cast<int64_t>(a->conv_taps) * a->conv_c || a->ag_nranks > 1 || a->rs_nranks > 1 ||
            (a->b_major != 0 && a->conv_b_tap_cols % 8))
            return -7;
        p.conv_kb_per_tap = a->conv_c / BK;
        p.conv_b_tap_cols = a->conv_b_tap_cols;
        for (int t = 0; t < a->conv_taps; ++t) p.conv_shift[t] = a->conv_shift[t];
    }
    if (a->map_hp > 0 && (a->batch != 1 || a->rs_nranks > 1 || a->map_wp <= 0)) return -7;

    CUtensorMap tmA, tmB;
    int rc;
    const uint64_t sA = a->batch > 1 ? a->strideA * 2 : (a->a_major == 0 ? a->M : a->K) * a->lda * 2;
    const uint64_t sB = a->batch > 1 ? a->strideB * 2 : (a->b_major == 0 ? a->N : a->K) * a->ldb * 2;
    if (a->conv_taps > 0)
        rc = make_tmap_3d(&tmA, a->A, a->in_dtype, a->conv_c, a->M, 1, a->lda * 2, a->M * a->lda * 2, BK, BM, 1);
    else if (a->a_major == 0)
        rc = make_tmap_3d(&tmA, a->A, a->in_dtype, a->K, a->M, a->batch, a->lda * 2, sA, BK, BM, 1);
    else
        rc = make_tmap_3d(&tmA, a->A, a->in_dtype, a->M, a->K, a->batch, a->lda * 2, sA, 64, BK, 1);
    if (rc) return rc;
    if (a->b_major == 0)
        rc = make_tmap_3d(&tmB, a->B, a->in_dtype, a->K, a->N, a->batch, a->ldb * 2, sB, BK, pair ? BN / 2 : BN, 1);
    else if (a->conv_taps > 0)
        // the stored matrix is [conv_c rows, conv_taps * conv_b_tap_cols columns]: tap t's [conv_c, N] block
        // starts at column t * conv_b_tap_cols
        rc = make_tmap_3d(&tmB, a->B, a->in_dtype, static_cast<uint64_t>(a->conv_taps) * a->conv_b_tap_cols,
                          a->conv_c, 1, a->ldb * 2, static_cast<uint64_t>(a->conv_c) * a->ldb * 2, 64, BK, 1);
    else
        rc = make_tmap_3d(&tmB, a->B, a->in_dtype, a->N, a->K, a->batch, a->ldb * 2, sB, 64, BK, 1);
    if (rc) return rc;

    if (a->in_dtype == 1) {
        if (a->out_dtype == 0)
            return pair ? launch<__nv_bfloat16, __nv_bfloat16, true>(*a, tmA, tmB, p, stream)
                        : launch<__nv_bfloat16, __nv_bfloat16, false>(*a, tmA, tmB, p, stream);
        return pair ? launch<__nv_bfloat16, float, true>(*a, tmA, tmB, p, stream)
                    : launch<__nv_bfloat16, float, false>(*a, tmA, tmB, p, stream);
    } else {
        if (a->out_dtype == 0)
            return pair ? launch<__half, __half, true>(*a, tmA, tmB, p, stream)
                        : launch<__half, __half, false>(*a, tmA, tmB, p, stream);
        return pair ? launch<__half, float, true>(*a, tmA, tmB, p, stream)
                    : launch<__half, float, false>(*a, tmA, tmB, p, stream);
    }
}

// Copies the device error word into `host_dst` (pinned host memory) on `stream` without waiting: the caller
// reads the value once work enqueued before the copy has finished (an event, or the next synchronisation).
extern "C" int rb_error_peek_async(int* host_dst, void* stream) {
    int* p = rb::error_word_ptr();
    if (!p || !host_dst) return -3;
    return cudaMemcpyAsync(host_dst, p, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)) ==
                   cudaSuccess
               ? 0
               : -4;
}

// Reads (and clears) the device error word.  Synchronises the device.
extern "C" int rb_read_error(int clear) {
    int* p = rb::error_word_ptr();
    if (!p) return -3;
    int v = 0;
    if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -4;
    if (clear && v) {
        int z = 0;
        cudaMemcpy(p, &z, sizeof(int), cudaMemcpyHostToDevice);
    }
    return v;
}
