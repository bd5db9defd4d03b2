// C ABI of the fused reduce-scatter + Adam + all-gather kernel (rs_adam.cu).
#pragma once
#include <stdint.h>

#define RB_MAX_PEERS 8

#ifdef __cplusplus
extern "C" {
#endif

typedef struct RbRsAdamArgs {
    const void* peer_grad[RB_MAX_PEERS];   // fp32 flat gradient buffer of every rank of the owner set
    void* peer_param[RB_MAX_PEERS];        // 16-bit flat parameter buffer of every rank
    void* peer_flags[RB_MAX_PEERS];        // flag block of every rank: uint32 [2][RB_MAX_PEERS], zero-initialised
    const void* mc_grad;                   // multicast address of the gradient buffers, or null
    void* mc_param;                        // multicast address of the parameter buffers, or null
    float* master;                         // this rank's fp32 master shard
    float* m;
    float* v;
    void* done_counter;                    // one zero-initialised uint32 in local device memory
    int64_t lo, len;                       // shard [lo, lo + len) in elements; multiples of 8
    int32_t nranks, my_idx;
    uint32_t epoch;                        // strictly increasing per launch, same on every rank
    float grad_mul;                        // 1/world * 1/loss_scale
    float lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2;
    int32_t adamw;                         // 0 Adam, 1 AdamW, 2 SGD (beta1 = momentum, beta2 = dampening,
                                           // eps > 0.5 = Nesterov, bias_corr1 == 0 = first step; v unused)
    int32_t dtype16;                       // 0 fp16, 1 bf16
    int32_t num_ctas;                      // 0: 148
    int32_t mode;                          // 0: everything in one launch (= RB_RS_BEGIN | END | PULL | UPDATE);
                                           // otherwise a combination of the RB_RS_* bits below
    const float* ctrl;                     // optional [gradient multiplier, skip flag]
    uint64_t max_polls;                    // bound of every flag wait (0: 2^26 polls of >= 100 ns)
    float* sumsq;                          // optional: += sum of squares of the reduced, scaled gradients
} RbRsAdamArgs;

// mode bits: a launch may do the reduction alone (during backward, bucket by bucket, after a separate
// rb_peer_barrier) and leave the update to a later launch that reads the reduced gradients back.
#define RB_RS_BEGIN 1        // handshake before: every peer's gradients of this range are final
#define RB_RS_END 2          // handshake after: every peer has finished reading / writing this rank's buffers
#define RB_RS_PULL 4         // sum the range over all ranks (else: read this rank's own buffer only)
#define RB_RS_UPDATE 8       // optimizer update of the master shard + write of the 16-bit values to every rank
#define RB_RS_STORE_GRAD 16  // write the reduced, scaled gradient into this rank's own gradient buffer

// 0 on success.  A wait that runs out sets the device error word to 2 and the kernel returns.
int rb_rs_adam_ag(const RbRsAdamArgs* args, void* stream);
// polls `flag` until it reaches `expected` or `max_polls` ran out (error word 2); for tests of the bound
int rb_wait_flag_probe(const void* flag, unsigned int expected, unsigned long long max_polls, void* stream);

#ifdef __cplusplus
}
#endif
