// Shared tail of every row-parallel projection: in-kernel all-reduce of the CTA's output rows
// over the LL channel, then the bf16 residual update.  The CTA that computed rows
// [row0, row0+nrows) is also the one that reduces them, so no grid-wide synchronisation exists.
#pragma once

#include "ll.cuh"

namespace nexrt {

// res: shared memory [M][nrows] fp32 partial sums of this rank.
// partial_out (library-baseline arm only): when non-null the CTA stores its fp32 partial sums there ([M][H]) and leaves
// both the exchange and the residual to the nodes that follow (a library all-reduce and a residual-add kernel).
__device__ __forceinline__ void allreduce_residual(const LLChannel& ch, unsigned int site, const float* res, int M, int row0, int nrows,
                                                   int H, __nv_bfloat16* __restrict__ x, bool add_residual = true, float* partial_out = nullptr) {
    if (partial_out != nullptr) {
        for (int idx = threadIdx.x; idx < M * nrows; idx += blockDim.x)
            partial_out[static_cast<size_t>(idx / nrows) * H + row0 + idx % nrows] = res[idx];
        return;
    }
    LLCall call{0u, 0u};
    if (ch.world > 1) call = ll_begin(ch, site);
    for (int idx = threadIdx.x; idx < M * nrows; idx += blockDim.x) {
        const int m = idx / nrows, r = idx % nrows;
        const size_t o = static_cast<size_t>(m) * H + row0 + r;
        const float sum = ll_allreduce_f32(ch, call, static_cast<unsigned int>(o), res[idx]);
        x[o] = __float2bfloat16_rn(add_residual ? __bfloat162float(x[o]) + sum : sum);
    }
}

}  // namespace nexrt
