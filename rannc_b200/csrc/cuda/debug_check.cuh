// Checked build of the kernel library (-DRB_DEBUG_BOUNDS, `python -m rannc_b200.build --debug`).
//
// compute-sanitizer is not available where this library is developed, so the memory-safety net is built in:
// in a checked build every entry point whose kernel indexes memory with DATA (token ids, class labels, row
// offsets supplied by the caller) first runs a small kernel that looks at those values and, for anything out of
// range, records ERR_BOUNDS in the device error word (rb_read_error) instead of letting the access happen or
// trapping.  The consuming kernels themselves skip out-of-range rows in every build; what the checked build
// adds is that the event is reported.  Host-side argument checks (alignment, strides, extents against the
// tensor-map rules) are promoted from "return -2" to a message on stderr that names the argument.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "tc_common.cuh"

namespace rb {

int* error_word_ptr();

#ifdef RB_DEBUG_BOUNDS
// values[i] must lie in [lo, hi) unless it equals `skip` (an ignore / padding marker)
static __global__ void debug_range_kernel(const long long* __restrict__ values, long long n, long long lo, long long hi,
                                   long long skip, int* __restrict__ err) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long v = values[i];
        if (v != skip && (v < lo || v >= hi)) atomicExch(err, ERR_BOUNDS);
    }
}

inline void debug_check_range(const long long* values, long long n, long long lo, long long hi, long long skip,
                              cudaStream_t st) {
    int* err = error_word_ptr();
    if (!err || n <= 0) return;
    long long g = (n + 255) / 256;
    if (g > 1024) g = 1024;
    debug_range_kernel<<<static_cast<unsigned>(g), 256, 0, st>>>(values, n, lo, hi, skip, err);
}
#define RB_DEBUG_RANGE(values, n, lo, hi, skip, st) ::rb::debug_check_range(values, n, lo, hi, skip, st)
#define RB_DEBUG_ARG(cond, what)                                                                  \
    do {                                                                                          \
        if (!(cond)) fprintf(stderr, "rannc_b200 kernels (checked build): %s:%d: %s\n", __FILE__, \
                             __LINE__, what);                                                     \
    } while (0)
#else
#define RB_DEBUG_RANGE(values, n, lo, hi, skip, st) ((void)0)
#define RB_DEBUG_ARG(cond, what) ((void)0)
#endif

}  // namespace rb
