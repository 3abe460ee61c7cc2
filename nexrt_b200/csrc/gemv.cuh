// Work partition shared by the CUDA-core GEMV kernels (gemv_cta.cuh): a balanced contiguous split of
// rows over the CTAs of a launch.
#pragma once

#include "common.cuh"

namespace nexrt {

// Rows [lo, hi) of `total` tasks owned by CTA `b` of `n` (balanced contiguous partition).
__device__ __forceinline__ void cta_range(int total, int b, int n, int* lo, int* hi) {
    const int base = total / n, rem = total % n;
    *lo = b * base + min(b, rem);
    *hi = *lo + base + (b < rem ? 1 : 0);
}

}  // namespace nexrt
