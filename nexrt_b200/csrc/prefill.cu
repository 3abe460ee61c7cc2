// Small kernels of the wide prefill path (chunks of 16..128 prompt tokens per pass).  The chunk's projections,
// router and experts are tcgen05 GEMMs over all rows (tc_gemm.cu), so every weight is streamed once per chunk;
// the sequential parts (conv ring, delta rule, causal attention) reuse the multi-row step kernels eight rows at
// a time, each sub-step reading its base position from its own copy of the control block.  What is left are the
// glue kernels here: embedding rows from an id list, the control-block table, the GDN output gate + quantisation,
// the expert activation of the dense expert product, and the residual add over K-split planes.
//
// The reference has no counterpart: its prefill runs inside SGLang (nex_n2_5_pro/sglang_prefill/bridge.py:310-398).
#include <cuda_fp8.h>

#include "api.h"
#include "common.cuh"

namespace nexrt {
namespace {

__global__ void __launch_bounds__(256) prefill_embed_kernel(const __nv_bfloat16* __restrict__ embed, const int* __restrict__ ids, __nv_bfloat16* __restrict__ x,
                                                            int* status, int H, int vocab) {
    const int m = blockIdx.x;
    int id = ids[m];
    if (id >= vocab || id < 0) {
        if (threadIdx.x == 0 && status) atomicCAS(status, 0, static_cast<int>(kStatusBadToken));
        id = 0;
    }
    const uint4* src = reinterpret_cast<const uint4*>(embed + static_cast<size_t>(id) * H);
    uint4* dst = reinterpret_cast<uint4*>(x + static_cast<size_t>(m) * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// table[j] = copy of the control block whose committed length is advanced by j * rows: sub-step j of a chunk reads
// its base position from table[j] exactly like a decode step reads it from the control block itself
__global__ void prefill_ctl_kernel(const int* __restrict__ ctl, int* __restrict__ table, int n_sub, int rows) {
    const int j = blockIdx.x, w = threadIdx.x;
    if (j >= n_sub || w >= kCtlWords) return;
    int v = ctl[w];
    if (w == kCtlCommittedLen) v += j * rows;
    table[j * kCtlWords + w] = v;
}

__global__ void prefill_advance_kernel(int* ctl, int rows) {
    if (threadIdx.x == 0) ctl[kCtlCommittedLen] += rows;
}

__device__ __forceinline__ void quant_block4(const float v[4], __nv_fp8_storage_t* dst, float* scale_out, int lane) {
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = warp_max(amax);
    const float scale = fmaxf(amax, 1e-12f) / 448.f;
    const float inv = 1.f / scale;
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) packed |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(v[i] * inv, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
    reinterpret_cast<uint32_t*>(dst)[lane] = packed;
    if (lane == 0) *scale_out = scale;
}

// GDN output gate: per 128-wide head rmsnorm(o) * gnorm_w * silu(z), then e4m3 with one scale per head (= per 128-wide
// K block of the out-projection).  One warp per (row, head).
__global__ void __launch_bounds__(256) gdn_gate_quant_kernel(const float* __restrict__ o, const float* __restrict__ z, const float* __restrict__ gnorm_w,
                                                             __nv_fp8_storage_t* __restrict__ xq, float* __restrict__ sx, int K, int T, float eps) {
    const int lane = threadIdx.x & 31;
    const int heads = K / 128;
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= T * heads) return;
    const int m = item / heads, h = item % heads;
    const size_t base = static_cast<size_t>(m) * K + h * 128 + lane * 4;
    const float4 ov = *reinterpret_cast<const float4*>(o + base);
    const float4 zz = *reinterpret_cast<const float4*>(z + base);
    const float4 gw = *reinterpret_cast<const float4*>(gnorm_w + lane * 4);
    const float inv = rsqrtf(warp_sum(ov.x * ov.x + ov.y * ov.y + ov.z * ov.z + ov.w * ov.w) / 128.f + eps);
    const float v[4] = {gw.x * ov.x * inv * silu_f(zz.x), gw.y * ov.y * inv * silu_f(zz.y), gw.z * ov.z * inv * silu_f(zz.z), gw.w * ov.w * inv * silu_f(zz.w)};
    quant_block4(v, xq + static_cast<size_t>(m) * K + h * 128, sx + static_cast<size_t>(m) * heads + h, lane);
}

// Expert activation of the dense expert product.  gu [T][n_total * 2I] holds gate|up of EVERY expert for every row (the
// gate/up GEMM runs over all experts: at these row counts almost every expert is routed to by some row, and the weights
// are what costs); only the S routed (row, expert) pairs are turned into h = silu(gate) * up * route weight, quantised
// per 128 columns into hq [T][n_total * I] with scales hs [T][n_total * I / 128].  Both were zeroed before: a zero scale
// removes an unrouted block from the down product.  One warp per (row, slot, 128-column block).
__global__ void __launch_bounds__(256) moe_dense_act_kernel(const float* __restrict__ gu, const int* __restrict__ ids, const float* __restrict__ wts,
                                                            __nv_fp8_storage_t* __restrict__ hq, float* __restrict__ hs, int I, int S, int T, int n_total) {
    const int lane = threadIdx.x & 31;
    const int nb = I / 128;
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= T * S * nb) return;
    const int b = item % nb, s = (item / nb) % S, m = item / (nb * S);
    const int e = min(max(ids[m * S + s], 0), n_total - 1);
    const float wt = wts[m * S + s];
    const float* g = gu + (static_cast<size_t>(m) * n_total + e) * 2 * I + b * 128 + lane * 4;
    const float4 gt = *reinterpret_cast<const float4*>(g), up = *reinterpret_cast<const float4*>(g + I);
    const float v[4] = {silu_f(gt.x) * up.x * wt, silu_f(gt.y) * up.y * wt, silu_f(gt.z) * up.z * wt, silu_f(gt.w) * up.w * wt};
    quant_block4(v, hq + (static_cast<size_t>(m) * n_total + e) * I + b * 128, hs + (static_cast<size_t>(m) * n_total + e) * nb + b, lane);
}

// out = sum of the K-split planes y[ks][n]; with x != null the sum is added to the bf16 residual rows instead
// (x = bf16(x + sum)), with sum_out != null it is kept in fp32 (input of a host-launched all-reduce).
__global__ void __launch_bounds__(256) planes_residual_kernel(__nv_bfloat16* x, const float* __restrict__ y, float* sum_out, size_t n, int ksplit) {
    const size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    float4 t = *reinterpret_cast<const float4*>(y + i);
    for (int ks = 1; ks < ksplit; ++ks) {
        const float4 v = *reinterpret_cast<const float4*>(y + static_cast<size_t>(ks) * n + i);
        t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
    }
    if (sum_out) *reinterpret_cast<float4*>(sum_out + i) = t;
    if (x) {
        __nv_bfloat162* xp = reinterpret_cast<__nv_bfloat162*>(x + i);
        const float2 a = __bfloat1622float2(xp[0]), b = __bfloat1622float2(xp[1]);
        xp[0] = __floats2bfloat162_rn(a.x + t.x, a.y + t.y);
        xp[1] = __floats2bfloat162_rn(b.x + t.z, b.y + t.w);
    }
}

// rmsnorm(x[t]) * gamma of every chunk row, written in the forms the chunk's GEMMs take (each output optional):
//   xq / sx : e4m3 with one scale per 128 columns (FP8 projections, expert gate/up),
//   xn      : fp32 (the bf16 b/a rows of the GDN front are projected from it),
//   planes  : bf16 hi + lo per token, [T][2][K] (the router: x = hi + lo to about 2^-17, two accumulating GEMMs).
__global__ void __launch_bounds__(256) norm_rows_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, __nv_fp8_storage_t* __restrict__ xq,
                                                        float* __restrict__ sx, float* __restrict__ xn, __nv_bfloat16* __restrict__ planes, int K, float eps) {
    __shared__ float red[32];
    __shared__ float rinv_s;
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const __nv_bfloat16* xr = x + static_cast<size_t>(t) * K;
    float ss = 0.f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        const float v = __bfloat162float(xr[k]);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) rinv_s = rsqrtf(v / K + eps);
    }
    __syncthreads();
    const float rinv = rinv_s;
    const int KB = K / 128;
    for (int kb = threadIdx.x >> 5; kb < KB; kb += blockDim.x >> 5) {     // one warp per 128-column block
        const int k0 = kb * 128 + lane * 4;
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = __bfloat162float(xr[k0 + i]) * rinv * gamma[k0 + i];
        if (xn) *reinterpret_cast<float4*>(xn + static_cast<size_t>(t) * K + k0) = make_float4(v[0], v[1], v[2], v[3]);
        if (planes) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __nv_bfloat16 hi = __float2bfloat16_rn(v[i]);
                planes[(static_cast<size_t>(t) * 2) * K + k0 + i] = hi;
                planes[(static_cast<size_t>(t) * 2 + 1) * K + k0 + i] = __float2bfloat16_rn(v[i] - __bfloat162float(hi));
            }
        }
        if (xq) quant_block4(v, xq + static_cast<size_t>(t) * K + kb * 128, sx + static_cast<size_t>(t) * KB + kb, lane);
    }
}

}  // namespace
}  // namespace nexrt

using namespace nexrt;

extern "C" {

int nexrt_prefill_embed(const void* embed, const void* ids, void* x, void* status, int H, int vocab, int T, void* stream) {
    if (T < 1 || H % 8) return cudaErrorInvalidValue;
    prefill_embed_kernel<<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(embed), static_cast<const int*>(ids),
                                                                             static_cast<__nv_bfloat16*>(x), static_cast<int*>(status), H, vocab);
    return cudaGetLastError();
}

int nexrt_prefill_ctl(const void* ctl, void* table, int n_sub, int rows, void* stream) {
    if (n_sub < 1 || rows < 1) return cudaErrorInvalidValue;
    prefill_ctl_kernel<<<n_sub, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const int*>(ctl), static_cast<int*>(table), n_sub, rows);
    return cudaGetLastError();
}

int nexrt_prefill_advance(void* ctl, int rows, void* stream) {
    prefill_advance_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<int*>(ctl), rows);
    return cudaGetLastError();
}

int nexrt_gdn_gate_quant(const void* o, const void* z, const void* gnorm_w, void* xq, void* sx, int K, int T, float eps, void* stream) {
    if (T < 1 || K % 128) return cudaErrorInvalidValue;
    const int items = T * (K / 128);
    gdn_gate_quant_kernel<<<(items + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float*>(o), static_cast<const float*>(z), static_cast<const float*>(gnorm_w), static_cast<__nv_fp8_storage_t*>(xq),
        static_cast<float*>(sx), K, T, eps);
    return cudaGetLastError();
}

int nexrt_moe_dense_act(const void* gu, const void* ids, const void* wts, void* hq, void* hs, int I, int S, int T, int n_total, void* stream) {
    if (T < 1 || I % 128 || S < 1) return cudaErrorInvalidValue;
    const int items = T * S * (I / 128);
    moe_dense_act_kernel<<<(items + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float*>(gu), static_cast<const int*>(ids), static_cast<const float*>(wts), static_cast<__nv_fp8_storage_t*>(hq),
        static_cast<float*>(hs), I, S, T, n_total);
    return cudaGetLastError();
}

int nexrt_planes_residual(void* x, const void* y, void* sum_out, int64_t n, int ksplit, void* stream) {
    if (n < 4 || n % 4 || ksplit < 1) return cudaErrorInvalidValue;
    const int64_t threads = n / 4;
    planes_residual_kernel<<<static_cast<unsigned int>((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(x), static_cast<const float*>(y), static_cast<float*>(sum_out), static_cast<size_t>(n), ksplit);
    return cudaGetLastError();
}

int nexrt_norm_rows(const void* x, const void* gamma, void* xq, void* sx, void* xn, void* planes, int K, int T, float eps, void* stream) {
    if (T < 1 || K < 128 || K % 128) return cudaErrorInvalidValue;
    norm_rows_kernel<<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(gamma),
                                                                         static_cast<__nv_fp8_storage_t*>(xq), static_cast<float*>(sx), static_cast<float*>(xn),
                                                                         static_cast<__nv_bfloat16*>(planes), K, eps);
    return cudaGetLastError();
}

}  // extern "C"
