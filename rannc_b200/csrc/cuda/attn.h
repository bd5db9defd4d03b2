// C ABI of the fused attention kernels (attn_fwd.cu, attn_bwd.cu).
// Tensors are addressed as element (b, s, h, d) = base + b*sb + s*ss + h*sh + d
// (d contiguous), so Q/K/V may be slices of one fused QKV projection output.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct RbAttnArgs {
    const void* Q;
    const void* K;
    const void* V;
    void* O;
    float* lse;             // [B, H, S]
    const float* key_bias;  // [B, S] additive bias on the scores, or null
    // backward only
    const void* dO;
    void* dQ;
    void* dK;
    void* dV;
    float* delta;     // [B, H, S] scratch: rowsum(dO * O)
    float* dq_accum;  // [B, S, H, D] fp32 scratch, zeroed by the callee
    int64_t q_sb, q_ss, q_sh;
    int64_t k_sb, k_ss, k_sh;
    int64_t v_sb, v_ss, v_sh;
    int64_t o_sb, o_ss, o_sh;
    int64_t do_sb, do_ss, do_sh;
    int64_t dq_sb, dq_ss, dq_sh;
    int64_t dk_sb, dk_ss, dk_sh;
    int64_t dv_sb, dv_ss, dv_sh;
    int32_t B, H, S, D;
    int32_t dtype;  // 0 fp16, 1 bf16
    int32_t pad_;
    float scale;
    float p_drop;
    uint64_t seed, offset;
} RbAttnArgs;

int rb_attn_fwd(const RbAttnArgs* args, void* stream);
int rb_attn_bwd(const RbAttnArgs* args, void* stream);

#ifdef __cplusplus
}
#include <cuda.h>
#include <cuda_runtime.h>
namespace rb {
int make_tmap_4d(CUtensorMap* out, const void* base, int fmt, uint64_t d0, uint64_t d1, uint64_t d2,
                 uint64_t d3, uint64_t s1, uint64_t s2, uint64_t s3, uint32_t b0, uint32_t b1);
int make_tmap_4d_f32(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3,
                     uint64_t s1, uint64_t s2, uint64_t s3, uint32_t b0, uint32_t b1);
int* error_word_ptr();
}
#endif
