// Dense BF16 projection for 1..8 token rows on the tensor cores (DFlash draft stack, MTP helpers).
//
//   y[m][r] = sum_k W[r][k] * f(in[m])[k]
//
// One CTA per 16 weight rows, the 8 warps split K; BF16 weights go from global memory to registers
// to mma.m16n8k16 against the activation split into bf16 hi + lo columns (2^-16 relative).
// Input transforms f: RMSNorm * gamma of bf16 rows, plain fp32 rows, or SwiGLU of fp32 [gate | up].
// Outputs: fp32 rows, or the in-kernel all-reduce over the LL channel followed by the residual
// add (or plain store) into bf16 rows.
//
// Replaces the reference's DFlash projection kernels DfM8FoldedQkvFt16Split2ProjKernel,
// DfM8FoldedContextKvFt16Split2ProjKernel (nex_n2_5_pro/kernels/dflash/
// nex_n2_5_pro_dflash_qkv_ckv_front_ctypes.cu:198-406), DfOProjTcGemmKernel + DfOProjTcReduceKernel
// (…dflash_oproj_tc_ctypes.cu:171-342), DfRmsNormKernel / DfMlpGateUpGemmKernel /
// DfMlpDownGemmKernel / DfMlpDownReduceKernel (…dflash_mlp_tc_ctypes.cu:96-507) and
// DfTargetHiddenProjGemmKernel + …ReduceKernel (…dflash_target_hidden_proj_ctypes.cu:81-266).
#include "api.h"
#include "epilogue.cuh"
#include "gemv_cta.cuh"
#include "ll.cuh"
#include "mma_gemv.cuh"

namespace nexrt {

struct DenseArgs {
    const void* in;            // in_mode 0: bf16 [M][K]; 1: fp32 [M][K]; 2: fp32 [M][2K] (gate | up)
    const float* gamma;        // in_mode 0: [K] norm multiplier (1 + w)
    const __nv_bfloat16* w;    // [R][K]
    float* out;                // out_mode 0: fp32 [M][R]
    __nv_bfloat16* x;          // out_mode 1/2: bf16 [M][R] rows, residual add / overwrite
    int R, K, M, in_mode, out_mode, ld_in;
    float eps;
    LLChannel ch;
    unsigned int site;
};

template <int MP>
__global__ void __launch_bounds__(256, 2) dense_bf16_kernel(DenseArgs a) {
    constexpr int NB = 8;
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[32];
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int row0 = blockIdx.x * kRowsPerGroup, nwin = a.K / 32;
    const int KS = min(nwarps, nwin);
    float* xs = smem;                                                           // [MP][K]
    float* tiles = xs + static_cast<size_t>(MP) * a.K;                          // [8][16][8]
    float* res = tiles + 8 * 128;                                               // [kMaxRows][16]
    __nv_bfloat16* xh = reinterpret_cast<__nv_bfloat16*>(res + kMaxRows * kRowsPerGroup);   // [MP*2][K]
    MmaWarpBf16<NB> mw(a.w, a.K, row0, warp, KS, warp < KS ? nwin : 0);
    mw.preload();
    RowNorm<4> norm;
    if (a.in_mode == 0) norm.preload_gamma(a.gamma, a.K);
    pdl_wait();
    for (int m0 = 0; m0 < a.M; m0 += MP) {
        const int mb = min(MP, a.M - m0);
        if (m0) { __syncthreads(); mw.next_pass(); }
        if (a.in_mode == 0) {
            norm.template run<3>(nullptr, xs, static_cast<const __nv_bfloat16*>(a.in) + static_cast<size_t>(m0) * a.K, mb, a.K, a.eps, red);
        } else if (a.in_mode == 3) {
            const size_t ld = a.ld_in ? a.ld_in : a.K;
            const __nv_bfloat16* in = static_cast<const __nv_bfloat16*>(a.in) + static_cast<size_t>(m0) * ld;
            for (int idx = threadIdx.x * 2; idx < mb * a.K; idx += blockDim.x * 2) {
                const int m = idx / a.K, k = idx % a.K;
                const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(in + static_cast<size_t>(m) * ld + k));
                *reinterpret_cast<float2*>(xs + idx) = v;
            }
            __syncthreads();
        } else if (a.in_mode == 1) {
            const float* in = static_cast<const float*>(a.in) + static_cast<size_t>(m0) * a.K;
            for (int idx = threadIdx.x * 4; idx < mb * a.K; idx += blockDim.x * 4)
                *reinterpret_cast<float4*>(xs + idx) = *reinterpret_cast<const float4*>(in + idx);
            __syncthreads();
        } else {
            const float* in = static_cast<const float*>(a.in) + static_cast<size_t>(m0) * 2 * a.K;
            for (int idx = threadIdx.x * 4; idx < mb * a.K; idx += blockDim.x * 4) {
                const int m = idx / a.K, k = idx % a.K;
                const float4 g = *reinterpret_cast<const float4*>(in + static_cast<size_t>(m) * 2 * a.K + k);
                const float4 u = *reinterpret_cast<const float4*>(in + static_cast<size_t>(m) * 2 * a.K + a.K + k);
                *reinterpret_cast<float4*>(xs + idx) = make_float4(silu_f(g.x) * u.x, silu_f(g.y) * u.y, silu_f(g.z) * u.z, silu_f(g.w) * u.w);
            }
            __syncthreads();
        }
        split_bf16_rows(xh, xs, mb, a.K);
        float d[4];
        mw.run(xh, mb * 2, d);
        if (warp < KS) mw.store(tiles + warp * 128, d);
        __syncthreads();
        if (threadIdx.x < kRowsPerGroup * mb) {
            const int rl = threadIdx.x % kRowsPerGroup, m = threadIdx.x / kRowsPerGroup;
            const float v = mma_bf16_result(tiles, KS, rl, m);
            if (a.out_mode == 0) a.out[static_cast<size_t>(m0 + m) * a.R + row0 + rl] = v;
            else res[(m0 + m) * kRowsPerGroup + rl] = v;
        }
    }
    if (a.out_mode != 0) {
        __syncthreads();
        allreduce_residual(a.ch, a.site, res, a.M, row0, kRowsPerGroup, a.R, a.x, a.out_mode == 1);
    }
}

// k rows -> per-head RMSNorm (1+w) + partial NeoX RoPE at positions base + m -> bf16 K cache; v rows
// -> bf16 V cache.  Used for the context rows of the DFlash draft (their K/V come from projected
// target features, reference DfQkvCkvPostRowsSplit2Kernel, …dflash_qkv_ckv_front_ctypes.cu:222-406).
// kv [M][ld] fp32 with k heads at k_off and v heads at v_off.  One warp per (row, head).
__global__ void __launch_bounds__(256) kv_publish_kernel(const float* __restrict__ kv, int ld, int k_off, int v_off, const float* __restrict__ kn,
                                                         const float2* __restrict__ rope_table, const int* __restrict__ ctl,
                                                         __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int hd,
                                                         int kvh, int M, int cache_len, int rotary, float eps, int ring) {
    __shared__ float rope_buf[8][256];
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int C0 = ctl[kCtlCommittedLen], half = rotary / 2, el = hd / 32;
    for (int v = blockIdx.x * nwarps + warp; v < M * kvh; v += gridDim.x * nwarps) {
        const int m = v / kvh, h = v % kvh, pos = C0 + m;
        if (pos < 0) continue;
        const int slot = ring > 0 ? pos % ring : pos;
        if (slot >= cache_len) continue;
        const float* ks = kv + static_cast<size_t>(m) * ld + k_off + h * hd;
        const float* vs = kv + static_cast<size_t>(m) * ld + v_off + h * hd;
        float e[8], ss = 0.f;
        for (int i = 0; i < el; ++i) { e[i] = ks[lane + 32 * i]; ss = fmaf(e[i], e[i], ss); }
        const float inv = rsqrtf(warp_sum(ss) / static_cast<float>(hd) + eps);
        for (int i = 0; i < el; ++i) e[i] *= inv * kn[lane + 32 * i];
        // RoPE partners live in other lanes: exchange through this warp's slice of shared memory
        float* buf = rope_buf[warp];
        for (int i = 0; i < el; ++i) buf[lane + 32 * i] = e[i];
        __syncwarp();
        float r[8];
        for (int i = 0; i < el; ++i) {
            const int dim = lane + 32 * i;
            r[i] = e[i];
            if (dim < rotary) {
                const int f = dim < half ? dim : dim - half;
                const float2 cs = rope_table[static_cast<size_t>(pos) * half + f];
                const float partner = dim < half ? -buf[dim + half] : buf[dim - half];
                r[i] = e[i] * cs.x + partner * cs.y;
            }
        }
        __syncwarp();
        __nv_bfloat16* kd = k_cache + (static_cast<size_t>(h) * cache_len + slot) * hd;
        __nv_bfloat16* vd = v_cache + (static_cast<size_t>(h) * cache_len + slot) * hd;
        for (int i = 0; i < el; ++i) {
            kd[lane + 32 * i] = __float2bfloat16_rn(r[i]);
            vd[lane + 32 * i] = __float2bfloat16_rn(vs[lane + 32 * i]);
        }
    }
}

}  // namespace nexrt

using namespace nexrt;

extern "C" int nexrt_dense_bf16(const void* in, const void* gamma, const void* w, void* out, void* x, int R, int K, int M, int in_mode,
                                int out_mode, int ld_in, float eps, const NexrtLLChannel* ch, unsigned int site, void* stream) {
    if (M < 1 || M > kMaxRows || R % 16 || K % 32 || in_mode < 0 || in_mode > 3 || out_mode < 0 || out_mode > 2) return cudaErrorInvalidValue;
    if (in_mode == 0 && K > 4096) return cudaErrorInvalidValue;
    if (out_mode != 0 && (ch == nullptr || (ch->world > 1 && ch->slots < static_cast<unsigned int>(kMaxRows) * R))) return cudaErrorInvalidValue;
    DenseArgs a{};
    a.in = in; a.gamma = static_cast<const float*>(gamma); a.w = static_cast<const __nv_bfloat16*>(w); a.out = static_cast<float*>(out);
    a.x = static_cast<__nv_bfloat16*>(x); a.R = R; a.K = K; a.M = M; a.in_mode = in_mode; a.out_mode = out_mode; a.ld_in = ld_in; a.eps = eps; a.site = site;
    if (ch) a.ch = *ch;
    const int mp = M == 1 ? 1 : (K <= 4096 ? 4 : (K <= 8192 ? 2 : 1));
    const size_t smem = sizeof(float) * (static_cast<size_t>(mp) * K + 8 * 128 + kMaxRows * 16) + sizeof(__nv_bfloat16) * static_cast<size_t>(mp) * 2 * K;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 g(R / 16), b(256);
    if (mp == 1) return launch(dense_bf16_kernel<1>, g, b, smem, st, a);
    if (mp == 2) return launch(dense_bf16_kernel<2>, g, b, smem, st, a);
    return launch(dense_bf16_kernel<4>, g, b, smem, st, a);
}

extern "C" int nexrt_kv_publish(const void* kv, int ld, int k_off, int v_off, const void* kn, const void* rope_table, const void* ctl,
                                void* k_cache, void* v_cache, int hd, int kvh, int M, int cache_len, int rotary, float eps, int ring,
                                void* stream) {
    if (M < 1 || M > 128 || hd % 32 || hd > 256 || rotary > hd || rotary % 2) return cudaErrorInvalidValue;
    const int ctas = M * kvh <= 8 ? 1 : (M * kvh + 7) / 8;     // eight vectors per CTA (a prefill chunk publishes up to 128 rows)
    return launch(kv_publish_kernel, dim3(ctas < 16 ? ctas : 16), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const float*>(kv), ld, k_off, v_off,
                  static_cast<const float*>(kn), static_cast<const float2*>(rope_table), static_cast<const int*>(ctl),
                  static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), hd, kvh, M, cache_len, rotary, eps, ring);
}
