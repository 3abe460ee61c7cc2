// Warp-level streaming GEMV building blocks: block-scaled FP8 (e4m3, 128x128 fp32 scales) and
// BF16 weight rows against up to four fp32 activation rows held in shared memory.
//
// The arithmetic is the reference's `acc += scale * dot128` (nex_n2_5_pro/kernels/full_attn/
// nex_n2_5_pro_qkv_proj_ctypes.cu:108-123); the layout is new: activations are staged
// "quad-major" - element k of a row of width K lives at ((k%16)/4 * K/16 + k/16) * 4 + k%4 -
// so that the four 16-byte shared-memory loads that pair with one 16-byte weight load are
// conflict-free for every K that is a multiple of 16, and one routine serves full-warp rows
// and the 128-byte rows of a tensor-parallel expert down-projection alike.
#pragma once

#include "common.cuh"

namespace nexrt {

// Staging position of element k for 16-element (fp8) and 8-element (bf16) lane chunks.
__device__ __forceinline__ int perm16(int k, int K) { return ((((k & 15) >> 2) * (K >> 4) + (k >> 4)) << 2) + (k & 3); }
__device__ __forceinline__ int perm8(int k, int K) { return ((((k & 7) >> 2) * (K >> 3) + (k >> 3)) << 2) + (k & 3); }

template <int EPL>
__device__ __forceinline__ int perm_pos(int k, int K) {
    return EPL == 16 ? perm16(k, K) : perm8(k, K);
}

// rmsnorm(x) * gamma for `rows` bf16 rows -> staged fp32.  `red` is 32 floats of shared memory.
template <int EPL>
__device__ __forceinline__ void stage_rmsnorm(float* xs, const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, int rows,
                                              int H, float eps, float* red) {
    for (int r = 0; r < rows; ++r) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = __bfloat162float(x[static_cast<size_t>(r) * H + i]);
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, red);
        const float inv = rsqrtf(ss / static_cast<float>(H) + eps);
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = __bfloat162float(x[static_cast<size_t>(r) * H + i]);
            xs[r * H + perm_pos<EPL>(i, H)] = v * inv * gamma[i];
        }
    }
    __syncthreads();
}

template <int LPR>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// NR fp8 weight rows x MB activation rows.  `w[n]` points at row n (K bytes), `s[n]` at that
// row's scale row (K/128 floats).  LPR lanes (index `sub`) cooperate on the rows; K must be a
// multiple of LPR*16.  On return acc[n][m] is the full dot product on every lane of the group.
template <int MB, int NR, int LPR>
__device__ __forceinline__ void gemv_fp8(const uint8_t* const (&w)[NR], const float* const (&s)[NR], int K, const float* __restrict__ xs,
                                         int sub, float (&acc)[NR][MB]) {
    const int q = K >> 4;
#pragma unroll
    for (int n = 0; n < NR; ++n)
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[n][m] = 0.f;
#pragma unroll 2
    for (int c = sub; c < q; c += LPR) {
        uint4 wv[NR];
#pragma unroll
        for (int n = 0; n < NR; ++n) wv[n] = ld_stream16(w[n] + c * 16);
        float sc[NR];
#pragma unroll
        for (int n = 0; n < NR; ++n) sc[n] = __ldg(s[n] + (c >> 3));
        float part[NR][MB];
#pragma unroll
        for (int n = 0; n < NR; ++n)
#pragma unroll
            for (int m = 0; m < MB; ++m) part[n][m] = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float wf[NR][4];
#pragma unroll
            for (int n = 0; n < NR; ++n) {
                const uint32_t word = j == 0 ? wv[n].x : j == 1 ? wv[n].y : j == 2 ? wv[n].z : wv[n].w;
                e4m3x4_to_float4(word, wf[n]);
            }
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                const float4 xv = *reinterpret_cast<const float4*>(xs + m * K + ((j * q + c) << 2));
#pragma unroll
                for (int n = 0; n < NR; ++n) {
                    part[n][m] = fmaf(wf[n][0], xv.x, part[n][m]);
                    part[n][m] = fmaf(wf[n][1], xv.y, part[n][m]);
                    part[n][m] = fmaf(wf[n][2], xv.z, part[n][m]);
                    part[n][m] = fmaf(wf[n][3], xv.w, part[n][m]);
                }
            }
        }
#pragma unroll
        for (int n = 0; n < NR; ++n)
#pragma unroll
            for (int m = 0; m < MB; ++m) acc[n][m] = fmaf(part[n][m], sc[n], acc[n][m]);
    }
#pragma unroll
    for (int n = 0; n < NR; ++n)
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[n][m] = group_sum<LPR>(acc[n][m]);
}

// NR bf16 weight rows x MB activation rows executed by a full warp (router, gate rows, LM
// head).  XEPL names the permutation the staging buffer was written with (8: bf16-only kernels,
// 16: kernels that also stream fp8 rows from the same buffer).  K must be a multiple of 256.
template <int MB, int NR, int XEPL>
__device__ __forceinline__ void gemv_bf16(const __nv_bfloat16* const (&w)[NR], int K, const float* __restrict__ xs, int lane,
                                          float (&acc)[NR][MB]) {
#pragma unroll
    for (int n = 0; n < NR; ++n)
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[n][m] = 0.f;
#pragma unroll 2
    for (int k0 = 0; k0 < K; k0 += 256) {
        uint4 wv[NR];
#pragma unroll
        for (int n = 0; n < NR; ++n) wv[n] = ld_stream16(w[n] + k0 + lane * 8);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float wf[NR][4];
#pragma unroll
            for (int n = 0; n < NR; ++n) {
                const uint32_t a = j == 0 ? wv[n].x : wv[n].z, b = j == 0 ? wv[n].y : wv[n].w;
                wf[n][0] = __uint_as_float(a << 16);
                wf[n][1] = __uint_as_float(a & 0xffff0000u);
                wf[n][2] = __uint_as_float(b << 16);
                wf[n][3] = __uint_as_float(b & 0xffff0000u);
            }
            const int pos = perm_pos<XEPL>(k0 + lane * 8 + j * 4, K);
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                const float4 xv = *reinterpret_cast<const float4*>(xs + m * K + pos);
#pragma unroll
                for (int n = 0; n < NR; ++n) {
                    acc[n][m] = fmaf(wf[n][0], xv.x, acc[n][m]);
                    acc[n][m] = fmaf(wf[n][1], xv.y, acc[n][m]);
                    acc[n][m] = fmaf(wf[n][2], xv.z, acc[n][m]);
                    acc[n][m] = fmaf(wf[n][3], xv.w, acc[n][m]);
                }
            }
        }
    }
#pragma unroll
    for (int n = 0; n < NR; ++n)
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[n][m] = warp_sum(acc[n][m]);
}

// Rows [lo, hi) of `total` tasks owned by CTA `b` of `n` (balanced contiguous partition).
__device__ __forceinline__ void cta_range(int total, int b, int n, int* lo, int* hi) {
    const int base = total / n, rem = total % n;
    *lo = b * base + min(b, rem);
    *hi = *lo + base + (b < rem ? 1 : 0);
}

}  // namespace nexrt
