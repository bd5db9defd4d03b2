// LayerNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for users of
// this library whose code runs where cudaMalloc is off limits: inside a
// real-time or latency-critical loop that may not touch the allocator, under a
// memory pool that owns every byte of the device and hands none out at run
// time, or in a host process that is only allowed to pass in buffers it was
// given.  The regular entry point (rb_ln_bwd, norm.cu) needs a scratch buffer
// from its caller for the per-CTA partial sums of dgamma / dbeta; this variant
// keeps that scratch inside the library instead, in a fixed
// `static __device__` array, so the caller passes inputs and outputs only.
//
// Limits and rules
//   * The scratch array holds RB_LN_NOALLOC_MAX_FLOATS floats (4.6 MiB).  Every
//     GPU that loads the library carries it until the process exits.
//   * A call needs rb_ln_bwd_grid(rows) * 2 * H floats of it; a call that needs
//     more is rejected with RB_LN_NOALLOC_TOO_LARGE and nothing is launched
//     (every row count fits for H <= 2048; H = 3072 fits up to 394 rows and
//     H = 4096 up to 296 rows; a width the kernel does not cover at all is
//     rejected with RB_LN_NOALLOC_BAD_WIDTH).
//   * The first call on a device looks up the device address of the array
//     (cudaGetSymbolAddress, with that device current) and remembers it.  Make
//     that first call before any stream capture begins.  The address that is
//     used is the CURRENT device's: make the device that owns `stream` current
//     before calling, as for any launch.  The lookup may run on several host
//     threads at once (the cached addresses are atomics).
//   * All calls on one device share the one array.  Nothing in it has to start
//     at zero -- every word a call reads was written by the same call -- but two
//     calls that overlap on the GPU (different streams, no ordering between
//     them) race on it.  Order them on one stream or with events.
//   * The function calls no cudaMalloc / cudaFree and no allocating library
//     routine.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RB_LN_NOALLOC_MAX_FLOATS (296 * 2 * 2048)

enum {
    RB_LN_NOALLOC_OK = 0,
    RB_LN_NOALLOC_LAUNCH_FAILED = -1,
    RB_LN_NOALLOC_BAD_WIDTH = -2,   // H is not one of 256, 512, 768, 1024, 1536, 2048, 3072, 4096
    RB_LN_NOALLOC_NO_SYMBOL = -6,   // cudaGetSymbolAddress failed on this device
    RB_LN_NOALLOC_TOO_LARGE = -7,   // rows x H needs more scratch than the library holds
};

// Same arguments and results as rb_ln_bwd, minus the scratch pointer:
//   dz [rows, H], dx [rows, H] (only written when p > 0), dgamma / dbeta fp32 [H]
//   (accumulate != 0 adds to them).  dtype: 0 fp16, 1 bf16.
int rb_ln_bwd_noalloc(const void* dy, const void* z, const void* gamma, const float* mean,
                      const float* rstd, void* dz, void* dx, float* dgamma, float* dbeta, int rows, int H,
                      float p, uint64_t seed, uint64_t offset, int accumulate, int dtype, void* stream);

// One-line description of a return code of rb_ln_bwd_noalloc.
const char* rb_ln_bwd_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
