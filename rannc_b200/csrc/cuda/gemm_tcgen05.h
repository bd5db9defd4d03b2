// C ABI of the tcgen05 GEMM (see gemm_tcgen05.cu).  Called from Python through
// ctypes with raw device pointers and the current CUDA stream.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum RbGemmFlags {
    RB_GEMM_BIAS = 1,       // v += bias[n]            (bias in the input dtype)
    RB_GEMM_GELU = 2,       // v = gelu(v)             (erf form)
    RB_GEMM_DGELU = 4,      // v *= gelu'(aux_in[m,n])
    RB_GEMM_RESIDUAL = 8,   // v += residual[m,n]
    RB_GEMM_ACCUM = 16,     // v += D[m,n]             (gradient accumulation)
    RB_GEMM_AUX_OUT = 32,   // aux_out[m,n] = v before the activation
};

typedef struct RbGemmArgs {
    const void* A;
    const void* B;
    void* D;
    const void* bias;
    const void* residual;
    const void* aux_in;
    void* aux_out;
    int64_t M, N, K, batch;
    int64_t lda, ldb, ldd;              // leading dimensions, elements
    int64_t strideA, strideB, strideD;  // batch strides, elements
    int32_t a_major;    // 0: A stored [M,K]; 1: A stored [K,M]
    int32_t b_major;    // 0: B stored [N,K]; 1: B stored [K,N]
    int32_t in_dtype;   // 0 fp16, 1 bf16
    int32_t out_dtype;  // 0 same as input, 1 fp32
    int32_t flags;
    int32_t max_ctas;   // 0 = one per SM
    float alpha;
    int32_t rs_nranks;  // > 1: reduce-scatter epilogue (fp32 output, RB_GEMM_ACCUM only): the N columns are split
                        // in rs_nranks equal blocks (multiples of 32); block j is ADDED into rs_peer[j], a
                        // [M, N / rs_nranks] fp32 buffer with leading dimension ldd in rank j's memory
    void* rs_peer[8];
    // all-gather prologue (ag_nranks > 1): B (stored [rows, ag_nranks * ag_cols], ldb = that width) is a local
    // buffer the kernel fills itself from the column shards ag_src[r] ([ag_rows, ag_cols] each, in rank r's
    // memory, own shard included) while the GEMM already consumes the shards that have arrived
    int32_t ag_nranks, ag_my_idx, ag_rows, ag_cols;
    void* ag_flags;        // 8 x uint32 of local device memory (cleared by the call)
    const void* ag_src[8];
    // implicit-GEMM convolution (conv_taps > 0).  A is the zero-padded channels-last activation seen as
    // [rows = N * Hp * Wp, conv_c] (lda = conv_c); the K dimension runs over conv_taps x conv_c: k-block kb reads
    // channels (kb mod conv_c/64) * 64 of the rows m + conv_shift[kb / (conv_c/64)] -- rows outside the matrix
    // read as zero.  With B stored [K, N] (b_major = 1) tap t's block starts conv_b_tap_cols * t columns further
    // right and its rows are the tap's own channel range.  No filter-sized copy of the activation exists.
    int32_t conv_taps, conv_c, conv_b_tap_cols;
    int32_t b_row_shift;   // b_major = 1: the rows of B that k-block kb reads start at kb * 64 + b_row_shift
    int32_t conv_shift[49];
    // output rows are positions of the padded grid: only the interior (map_pad <= y < map_pad + map_h, same for
    // x) is stored, at row (n * map_h + y - map_pad) * map_w + (x - map_pad) of D.  map_hp = 0: rows are rows.
    int32_t map_hp, map_wp, map_h, map_w, map_pad;
} RbGemmArgs;

// returns 0 on success, <0 on a host-side error (-2: operand not 16 B aligned)
int rb_gemm(const RbGemmArgs* args, void* stream);
// device error word: 0 ok, 1 mbarrier wait ran out, 2 peer wait ran out
int rb_read_error(int clear);
// asynchronous copy of the error word into pinned host memory (no synchronisation)
int rb_error_peek_async(int* host_dst, void* stream);

#ifdef __cplusplus
}
#include <cuda.h>
namespace rb {
int make_tmap_3d(CUtensorMap* out, const void* base, int dtype_16bit_kind, uint64_t d0, uint64_t d1,
                 uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0,
                 uint32_t b1, int swizzle128);
int* error_word_ptr();
int num_sms();
}  // namespace rb
#endif
