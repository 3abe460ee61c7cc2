// Gated delta net (linear attention) layer, front half and recurrence, for 1..8 token rows.
//
//   gdn_front : input RMSNorm -> block-scaled FP8 GEMV of the q|k|v|z rows -> causal conv1d(4)
//               over a position-indexed history ring + SiLU; the bf16 b/a rows ->
//               beta = sigmoid(b), g = -exp(A_log) * softplus(a + dt_bias).
//   gdn_core  : gated delta rule, one token after another, over a position-indexed ring of
//               fp32 states so that a speculative step can be committed up to any row.
//
// Replaces the reference's LinearFrontSplitCtaSk4Kernel (nex_n2_5_pro/kernels/linear_attn/
// nex_n2_5_pro_linear_front_gemv_ctypes.cu:88-224), RecurrentCoreTransposedSharedNormKernel
// (…linear_recurrent_core_ctypes.cu:62-171) and their M=4 / M=8 ring variants
// (…m4_gdn_front_ring_ctypes.cu:112-394, …m8_gdn_core_ctypes.cu:88-239) with one pair of
// kernels whose row count and head counts are run-time arguments.  The history ring holds the
// pre-convolution value of every channel at position p in slot p % conv_ring, and the state
// before consuming position p lives in slot p % state_ring: nothing is shifted or overwritten
// in place, so rejected rows need no rollback.
#include "api.h"
#include "gemv.cuh"
#include "gemv_cta.cuh"

namespace nexrt {

struct GdnFrontArgs {
    const __nv_bfloat16* x;      // [M][H] residual stream
    const float* in_ln;          // [H] 1 + w
    const uint8_t* front_w;      // [R][H] fp8, rows q|k|v|z
    const float* front_s;        // [R/128][H/128]
    const __nv_bfloat16* ba_w;   // [2 nv][H]: b rows then a rows
    const float* conv_w;         // [C][4]
    const float* a_log;          // [nv]
    const float* dt_bias;        // [nv]
    const int* ctl;
    float* conv_ring;            // [conv_ring][C]
    float* qkv;                  // [M][C] after conv + SiLU
    float* z;                    // [M][R - C]
    float* beta;                 // [M][nv]
    float* g;                    // [M][nv]
    int H, R, C, nv, M, conv_ring_len;
    float eps;
};

template <int MB>
__global__ void __launch_bounds__(512, 1) gdn_front_kernel(GdnFrontArgs a) {
    constexpr int U = MB == 1 ? 8 : 4;
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[32];
    pdl_launch_dependents();
    int r0, r1, b0, b1;
    cta_range(a.R, blockIdx.x, gridDim.x, &r0, &r1);
    cta_range(2 * a.nv, blockIdx.x, gridDim.x, &b0, &b1);
    const int nrows = r1 - r0, nba = b1 - b0;
    if (nrows) prefetch_l2_range(a.front_w + static_cast<size_t>(r0) * a.H, static_cast<size_t>(nrows) * a.H);
    const GemvGeom gf = gemv_geom(a.H / 16, blockDim.x), gb = gemv_geom(a.H / 8, blockDim.x);
    float* xs = smem;                                                   // [MB][H]
    float* part = xs + static_cast<size_t>(MB) * a.H;                   // fp8 rows
    float* part_ba = part + gemv_part_floats((a.R + gridDim.x - 1) / gridDim.x, MB, gf);
    pdl_wait();
    const int C0 = a.ctl[kCtlCommittedLen];
    for (int m0 = 0; m0 < a.M; m0 += MB) {
        const int mb = min(MB, a.M - m0);
        if (m0) __syncthreads();
        stage_rmsnorm_plain(xs, a.x + static_cast<size_t>(m0) * a.H, a.in_ln, mb, a.H, a.eps, red);
        gemv_cta<MB, U>(PlainFp8{a.front_w, a.front_s, a.H}, r0, nrows, xs, a.H, part);
        if (nba) gemv_cta<MB, 2>(PlainBf16{a.ba_w, a.H}, b0, nba, xs, a.H, part_ba);
        __syncthreads();
        for (int rl = threadIdx.x; rl < nrows; rl += blockDim.x) {
            const int row = r0 + rl;
            float pre[MB];
#pragma unroll
            for (int m = 0; m < MB; ++m) pre[m] = gemv_result(part, rl, m, MB, gf.wpr);
            if (row < a.C) {
                const float4 cw = *reinterpret_cast<const float4*>(a.conv_w + static_cast<size_t>(row) * 4);
                const int ring = a.conv_ring_len;
                for (int m = 0; m < mb; ++m) {
                    const int p = C0 + m0 + m;
                    a.conv_ring[static_cast<size_t>(p % ring) * a.C + row] = pre[m];
                }
                for (int m = 0; m < mb; ++m) {
                    const int p = C0 + m0 + m;
                    // taps at positions p-3..p; slots of positions before the sequence start hold zero
                    float h[3];
#pragma unroll
                    for (int j = 0; j < 3; ++j) {
                        const int mm = m - 3 + j;
                        h[j] = (mm >= 0) ? pre[mm < 0 ? 0 : mm] : a.conv_ring[static_cast<size_t>((p - 3 + j + ring) % ring) * a.C + row];
                    }
                    const float v = fmaf(cw.x, h[0], fmaf(cw.y, h[1], fmaf(cw.z, h[2], cw.w * pre[m])));
                    a.qkv[static_cast<size_t>(m0 + m) * a.C + row] = silu_f(v);
                }
            } else {
                for (int m = 0; m < mb; ++m) a.z[static_cast<size_t>(m0 + m) * (a.R - a.C) + (row - a.C)] = pre[m];
            }
        }
        for (int rl = threadIdx.x; rl < nba; rl += blockDim.x) {
            const int row = b0 + rl;     // [0, nv): b rows, [nv, 2nv): a rows
            for (int m = 0; m < mb; ++m) {
                const float v = gemv_result(part_ba, rl, m, MB, gb.wpr);
                if (row < a.nv) a.beta[(m0 + m) * a.nv + row] = sigmoid_f(v);
                else {
                    const int h = row - a.nv;
                    a.g[(m0 + m) * a.nv + h] = -__expf(a.a_log[h]) * softplus_f(v + a.dt_bias[h]);
                }
            }
        }
    }
}

struct GdnCoreArgs {
    const float* qkv;     // [M][C]: q heads | k heads | v heads, 128 wide each
    const float* beta;    // [M][nv]
    const float* g;       // [M][nv]
    const int* ctl;
    float* state_ring;    // [state_ring][nv][128 v][128 k]
    float* out;           // [M][nv*128]
    int nqk, nv, M, state_ring_len, C;
};

// grid (nv, 128 / warps-per-CTA); one warp per value column, lane holds 4 key rows.
__global__ void __launch_bounds__(256) gdn_core_kernel(GdnCoreArgs a) {
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int head = blockIdx.x, col = blockIdx.y * nwarps + warp;
    const int qk_head = head / (a.nv / a.nqk);
    const size_t head_stride = static_cast<size_t>(128) * 128, slot_stride = head_stride * a.nv;
    const size_t elem = head * head_stride + static_cast<size_t>(col) * 128 + lane * 4;
    pdl_wait();
    const int C0 = a.ctl[kCtlCommittedLen];
    float4 S = *reinterpret_cast<const float4*>(a.state_ring + static_cast<size_t>(C0 % a.state_ring_len) * slot_stride + elem);
    for (int m = 0; m < a.M; ++m) {
        const float* row = a.qkv + static_cast<size_t>(m) * a.C;
        const float4 q4 = *reinterpret_cast<const float4*>(row + qk_head * 128 + lane * 4);
        const float4 k4 = *reinterpret_cast<const float4*>(row + (a.nqk + qk_head) * 128 + lane * 4);
        const float v = row[(2 * a.nqk + head) * 128 + col];
        const float qn = rsqrtf(warp_sum(q4.x * q4.x + q4.y * q4.y + q4.z * q4.z + q4.w * q4.w) + 1e-6f) * 0.08838834764831845f;
        const float kn = rsqrtf(warp_sum(k4.x * k4.x + k4.y * k4.y + k4.z * k4.z + k4.w * k4.w) + 1e-6f);
        const float decay = __expf(a.g[m * a.nv + head]), b = a.beta[m * a.nv + head];
        S.x *= decay; S.y *= decay; S.z *= decay; S.w *= decay;
        const float kx = k4.x * kn, ky = k4.y * kn, kz = k4.z * kn, kw = k4.w * kn;
        const float kv = warp_sum(kx * S.x + ky * S.y + kz * S.z + kw * S.w);
        const float delta = (v - kv) * b;
        S.x = fmaf(kx, delta, S.x); S.y = fmaf(ky, delta, S.y); S.z = fmaf(kz, delta, S.z); S.w = fmaf(kw, delta, S.w);
        const float o = warp_sum(q4.x * S.x + q4.y * S.y + q4.z * S.z + q4.w * S.w) * qn;
        *reinterpret_cast<float4*>(a.state_ring + static_cast<size_t>((C0 + m + 1) % a.state_ring_len) * slot_stride + elem) = S;
        if (lane == 0) a.out[static_cast<size_t>(m) * a.nv * 128 + head * 128 + col] = o;
    }
}

}  // namespace nexrt

using namespace nexrt;

extern "C" int nexrt_gdn_front(const void* x, const void* in_ln, const void* front_w, const void* front_s, const void* ba_w,
                               const void* conv_w, const void* a_log, const void* dt_bias, const void* ctl, void* conv_ring, void* qkv,
                               void* z, void* beta, void* g, int H, int R, int C, int nv, int M, int conv_ring_len, float eps, int n_cta,
                               void* stream) {
    if (M < 1 || M > kMaxRows || H % 256 || conv_ring_len < M + 3) return cudaErrorInvalidValue;
    GdnFrontArgs a{static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(in_ln), static_cast<const uint8_t*>(front_w),
                   static_cast<const float*>(front_s), static_cast<const __nv_bfloat16*>(ba_w), static_cast<const float*>(conv_w),
                   static_cast<const float*>(a_log), static_cast<const float*>(dt_bias), static_cast<const int*>(ctl),
                   static_cast<float*>(conv_ring), static_cast<float*>(qkv), static_cast<float*>(z), static_cast<float*>(beta),
                   static_cast<float*>(g), H, R, C, nv, M, conv_ring_len, eps};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int mb = M == 1 ? 1 : 4;
    const size_t smem = sizeof(float) * (static_cast<size_t>(mb) * H + gemv_part_floats((R + n_cta - 1) / n_cta, mb, gemv_geom(H / 16, 512)) +
                                         gemv_part_floats((2 * nv + n_cta - 1) / n_cta, mb, gemv_geom(H / 8, 512)));
    if (M == 1) return launch(gdn_front_kernel<1>, dim3(n_cta), dim3(512), smem, st, a);
    return launch(gdn_front_kernel<4>, dim3(n_cta), dim3(512), smem, st, a);
}

extern "C" int nexrt_gdn_core(const void* qkv, const void* beta, const void* g, const void* ctl, void* state_ring, void* out, int nqk, int nv,
                              int M, int state_ring_len, int C, void* stream) {
    if (M < 1 || M > kMaxRows || state_ring_len < M + 1 || nv % nqk) return cudaErrorInvalidValue;
    GdnCoreArgs a{static_cast<const float*>(qkv), static_cast<const float*>(beta), static_cast<const float*>(g),
                  static_cast<const int*>(ctl), static_cast<float*>(state_ring), static_cast<float*>(out), nqk, nv, M, state_ring_len, C};
    return launch(gdn_core_kernel, dim3(nv, 128 / 8), dim3(256), 0, static_cast<cudaStream_t>(stream), a);
}
