// Mixer output projection fused with the tensor-parallel all-reduce and the residual add.
//
//   x[m] += all_reduce_sum_over_ranks( W_out[:, local] @ f(in[m]) )
//
// One kernel does: the input transform f (identity for attention, per-head gated RMSNorm *
// silu(z) for the gated delta net, or the context-parallel LSE merge * sigmoid(gate)), the
// block-scaled FP8 GEMV of this rank's column slice, the in-kernel all-reduce over NVSwitch
// (one 8-byte self-tagged packet per value, published with `multimem.st` or peer stores, summed
// in rank order), and the bf16 residual update.  Every rank ends with a bitwise identical
// residual stream, which is also the "all-gather" that feeds the next projection.
//
// Replaces the reference's LinearFinalOProjFusedPushKernel (nex_n2_5_pro/kernels/linear_attn/
// nex_n2_5_pro_linear_final_o_proj_ctypes.cu:51-259), OProjFusedPushKernel and
// WholeVectorReduceKernel (…full_attn/nex_n2_5_pro_o_proj_reduce_ctypes.cu:51-289), the CP tail
// (…cp_tail_ctypes.cu:117-211) and the M=4/M=8 o_proj kernels (…m4_attn_oproj_fused_ctypes.cu,
// …m8_attn_oproj_ctypes.cu, …m4_gdn_oproj_fused_ctypes.cu, …m8_gdn_oproj_ctypes.cu).
#include "api.h"
#include "epilogue.cuh"
#include "gemv.cuh"
#include "gemv_cta.cuh"
#include "mma_gemv.cuh"
#include "ll.cuh"

namespace nexrt {

struct OProjArgs {
    const float* in;        // [M][K]
    const float* z;         // mode 1: [M][K]; mode 2: gate [M][K]
    const float* gnorm_w;   // mode 1: [hd]
    const uint8_t* w;       // [H][K] fp8
    const float* s;         // [H/128][K/128]
    __nv_bfloat16* x;       // [M][H] residual stream (read-modify-write)
    int H, K, M, mode, hd;
    int overwrite;          // 1: x = reduced projection (no residual add)
    float eps;
    float* partial_out;     // library-baseline arm: fp32 partial sums go here, no exchange, no residual
    LLChannel ch;
    unsigned int site;
    LLChannel cp;           // mode 2: partial inbox of the context-parallel group
    unsigned int cp_site;
};

template <int MB>
__global__ void __launch_bounds__(512, 1) oproj_allreduce_kernel(OProjArgs a) {
    constexpr int U = MB == 1 ? 8 : 4;
    extern __shared__ __align__(16) float smem[];
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    int row0, row1;
    cta_range(a.H, blockIdx.x, gridDim.x, &row0, &row1);
    const int nrows = row1 - row0, max_rows = (a.H + gridDim.x - 1) / gridDim.x;
    if (nrows) prefetch_l2_range(a.w + static_cast<size_t>(row0) * a.K, static_cast<size_t>(nrows) * a.K);
    const GemvGeom gg = gemv_geom(a.K / 16, blockDim.x);
    float* xs = smem;                                        // [MB][K]
    float* part = xs + static_cast<size_t>(MB) * a.K;        // [max_rows][wpr][MB]
    float* res = part + gemv_part_floats(max_rows, MB, gg);  // [kMaxRows][nrows]
    GemvCta<MB, U, PlainFp8> gemv(PlainFp8{a.w, a.s, a.K}, row0, nrows, a.K);
    gemv.preload();
    pdl_wait();
    LLCall cpcall{0u, 0u};
    if (a.mode == 2) cpcall = ll_begin(a.cp, a.cp_site);
    for (int m0 = 0; m0 < a.M; m0 += MB) {
        const int mb = min(MB, a.M - m0);
        if (m0) __syncthreads();
        if (a.mode == 0) {
            for (int idx = threadIdx.x; idx < mb * a.K; idx += blockDim.x) xs[idx] = a.in[static_cast<size_t>(m0) * a.K + idx];
        } else if (a.mode == 1) {
            // gated RMSNorm per 128-wide head: gnorm_w * o * rsqrt(mean o^2 + eps) * silu(z)
            const int heads = a.K / 128;
            for (int v = warp; v < mb * heads; v += nwarps) {
                const int m = v / heads, h = v % heads;
                const size_t base = static_cast<size_t>(m0 + m) * a.K + h * 128 + lane * 4;
                const float4 o = *reinterpret_cast<const float4*>(a.in + base);
                const float4 zz = *reinterpret_cast<const float4*>(a.z + base);
                const float4 gw = *reinterpret_cast<const float4*>(a.gnorm_w + lane * 4);
                const float inv = rsqrtf(warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w) / 128.f + a.eps);
                float4 r;
                r.x = gw.x * o.x * inv * silu_f(zz.x);
                r.y = gw.y * o.y * inv * silu_f(zz.y);
                r.z = gw.z * o.z * inv * silu_f(zz.z);
                r.w = gw.w * o.w * inv * silu_f(zz.w);
                *reinterpret_cast<float4*>(xs + m * a.K + h * 128 + lane * 4) = r;
            }
        } else {
            // context-parallel merge: for every (row, local head, dim) combine the partial contexts
            // of the cp ranks with their log2-domain LSE weights, then gate.
            const int hd = a.hd, heads = a.K / hd;
            for (int idx = threadIdx.x; idx < mb * a.K; idx += blockDim.x) {
                const int m = idx / a.K, k = idx % a.K, lh = k / hd, d = k % hd;
                const unsigned int base = (static_cast<unsigned int>(m0 + m) * heads + lh) * (hd + 1);
                float lse[kMaxWorld], ctx[kMaxWorld], mx = -INFINITY;
                for (int sr = 0; sr < a.cp.world; ++sr) {
                    unsigned int pl, pc;
                    ll_wait(a.cp, cpcall, sr, base + hd, &pl, kStatusCpTimeout);
                    ll_wait(a.cp, cpcall, sr, base + d, &pc, kStatusCpTimeout);
                    lse[sr] = __uint_as_float(pl);
                    ctx[sr] = __uint_as_float(pc);
                    mx = fmaxf(mx, lse[sr]);
                }
                float num = 0.f, den = 0.f;
                for (int sr = 0; sr < a.cp.world; ++sr) {
                    const float wgt = lse[sr] == -INFINITY ? 0.f : exp2f(lse[sr] - mx);
                    num = fmaf(wgt, ctx[sr], num);
                    den += wgt;
                }
                const float gt = a.z[static_cast<size_t>(m0 + m) * a.K + k];
                xs[m * a.K + k] = (den > 0.f ? num / den : 0.f) * sigmoid_f(gt);
            }
        }
        __syncthreads();
        if (m0 == 0) gemv.run(xs, part);
        else gemv_cta<MB, U>(PlainFp8{a.w, a.s, a.K}, row0, nrows, xs, a.K, part);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nrows * mb; idx += blockDim.x) {
            const int rl = idx / mb, m = idx % mb;
            res[(m0 + m) * nrows + rl] = gemv_result(part, rl, m, MB, gg.wpr);
        }
    }
    __syncthreads();
    allreduce_residual(a.ch, a.site, res, a.M, row0, nrows, a.H, a.x, a.overwrite == 0, a.partial_out);
}

// Tensor-core form: one CTA per 16 output rows, the 8 warps split K (see mma_gemv.cuh); the CTA
// that computed the rows reduces them across the ranks and updates the residual.
template <int MP>
__global__ void __launch_bounds__(256, 2) oproj_allreduce_mma_kernel(OProjArgs a) {
    constexpr int TERMS = MmaShape<MP>::TERMS, NT = MmaShape<MP>::NT, TILE = MmaShape<MP>::TILE, NB = 8;
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[32];
    __shared__ float descale[MP];
    TraceCta tr;
    tr.begin(kTrOproj);
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int row0 = blockIdx.x * kRowsPerGroup, nwin = a.K / kWin;
    const int KS = min(nwarps, nwin);                                   // warps that share the K range
    float* xs = smem;                                                   // [MP][K]
    float* tiles = xs + static_cast<size_t>(MP) * a.K;                  // [KS][16][8]
    float* res = tiles + 8 * TILE;                                       // [kMaxRows][16]
    uint8_t* xq = reinterpret_cast<uint8_t*>(res + kMaxRows * kRowsPerGroup);   // [MP*TERMS][K]
    const MmaPlain src{a.w, a.s, a.K};
    MmaWarp<NB, MmaPlain> mw(row0, warp, KS, warp < KS ? nwin : 0);
    mw.preload(src);
    pdl_wait();
    tr.mark(1);
    LLCall cpcall{0u, 0u};
    if (a.mode == 2) cpcall = ll_begin(a.cp, a.cp_site);
    for (int m0 = 0; m0 < a.M; m0 += MP) {
        const int mb = min(MP, a.M - m0);
        if (m0) { __syncthreads(); mw.next_pass(); }
        if (a.mode == 0) {
            for (int idx = threadIdx.x * 4; idx < mb * a.K; idx += blockDim.x * 4)
                *reinterpret_cast<float4*>(xs + idx) = *reinterpret_cast<const float4*>(a.in + static_cast<size_t>(m0) * a.K + idx);
        } else if (a.mode == 1) {
            const int heads = a.K / 128;
            const float4 gw = *reinterpret_cast<const float4*>(a.gnorm_w + lane * 4);
            for (int v = warp; v < mb * heads; v += nwarps) {
                const int m = v / heads, h = v % heads;
                const size_t base = static_cast<size_t>(m0 + m) * a.K + h * 128 + lane * 4;
                const float4 o = *reinterpret_cast<const float4*>(a.in + base);
                const float4 zz = *reinterpret_cast<const float4*>(a.z + base);
                const float inv = rsqrtf(warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w) / 128.f + a.eps);
                float4 r;
                r.x = gw.x * o.x * inv * silu_f(zz.x);
                r.y = gw.y * o.y * inv * silu_f(zz.y);
                r.z = gw.z * o.z * inv * silu_f(zz.z);
                r.w = gw.w * o.w * inv * silu_f(zz.w);
                *reinterpret_cast<float4*>(xs + m * a.K + h * 128 + lane * 4) = r;
            }
        } else {
            const int hd = a.hd, heads = a.K / hd;
            for (int idx = threadIdx.x; idx < mb * a.K; idx += blockDim.x) {
                const int m = idx / a.K, k = idx % a.K, lh = k / hd, d = k % hd;
                const unsigned int base = (static_cast<unsigned int>(m0 + m) * heads + lh) * (hd + 1);
                float lse[kMaxWorld], ctx[kMaxWorld], mx = -INFINITY;
                for (int sr = 0; sr < a.cp.world; ++sr) {
                    unsigned int pl, pc;
                    ll_wait(a.cp, cpcall, sr, base + hd, &pl, kStatusCpTimeout);
                    ll_wait(a.cp, cpcall, sr, base + d, &pc, kStatusCpTimeout);
                    lse[sr] = __uint_as_float(pl);
                    ctx[sr] = __uint_as_float(pc);
                    mx = fmaxf(mx, lse[sr]);
                }
                float num = 0.f, den = 0.f;
                for (int sr = 0; sr < a.cp.world; ++sr) {
                    const float wgt = lse[sr] == -INFINITY ? 0.f : exp2f(lse[sr] - mx);
                    num = fmaf(wgt, ctx[sr], num);
                    den += wgt;
                }
                const float gt = a.z[static_cast<size_t>(m0 + m) * a.K + k];
                xs[m * a.K + k] = (den > 0.f ? num / den : 0.f) * sigmoid_f(gt);
            }
        }
        __syncthreads();
        act_split<TERMS>(xq, xs, mb, a.K, red, descale);
        float d[NT][4];
        mw.template run<NT>(src, xq, a.K, mb * TERMS, d);
        if (warp < KS) mw.template store<NT>(tiles + warp * TILE, d);
        __syncthreads();
        if (threadIdx.x < kRowsPerGroup * mb) {
            const int rl = threadIdx.x % kRowsPerGroup, m = threadIdx.x / kRowsPerGroup;
            res[(m0 + m) * kRowsPerGroup + rl] = mma_result<TERMS, NT>(tiles, KS, rl, m, descale[m]);
        }
    }
    __syncthreads();
    tr.mark(2);
    allreduce_residual(a.ch, a.site, res, a.M, row0, kRowsPerGroup, a.H, a.x, a.overwrite == 0, a.partial_out);
    tr.mark(3);
}

// Staging half of the wide out-projection (multi-row steps): one CTA per token row builds the projection's input
// (mode 0 plain copy, 1 GDN gated RMSNorm with z, 2 context-parallel merge of the group's partials) and writes it as
// three e4m3 planes [3M][K] plus a power-of-two scale per row - the B operand of the tcgen05 GEMM that follows
// (nexrt_tc_oproj_allreduce in tc_moe.cu), which also does the all-reduce and the residual.
__global__ void __launch_bounds__(256) oproj_stage_split_kernel(OProjArgs a, uint8_t* planes, float* descale_out) {
    extern __shared__ __align__(16) float xs[];          // [K]
    __shared__ float red[32];
    __shared__ float ds[1];
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int m = blockIdx.x;
    pdl_wait();
    if (a.mode == 0) {
        for (int idx = threadIdx.x * 4; idx < a.K; idx += blockDim.x * 4)
            *reinterpret_cast<float4*>(xs + idx) = *reinterpret_cast<const float4*>(a.in + static_cast<size_t>(m) * a.K + idx);
    } else if (a.mode == 1) {
        const int heads = a.K / 128;
        const float4 gw = *reinterpret_cast<const float4*>(a.gnorm_w + lane * 4);
        for (int h = warp; h < heads; h += nwarps) {
            const size_t base = static_cast<size_t>(m) * a.K + h * 128 + lane * 4;
            const float4 o = *reinterpret_cast<const float4*>(a.in + base);
            const float4 zz = *reinterpret_cast<const float4*>(a.z + base);
            const float inv = rsqrtf(warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w) / 128.f + a.eps);
            *reinterpret_cast<float4*>(xs + h * 128 + lane * 4) =
                make_float4(gw.x * o.x * inv * silu_f(zz.x), gw.y * o.y * inv * silu_f(zz.y), gw.z * o.z * inv * silu_f(zz.z), gw.w * o.w * inv * silu_f(zz.w));
        }
    } else {
        const LLCall cpcall = ll_begin(a.cp, a.cp_site);
        const int hd = a.hd, heads = a.K / hd;
        for (int k = threadIdx.x; k < a.K; k += blockDim.x) {
            const int lh = k / hd, d = k % hd;
            const unsigned int base = (static_cast<unsigned int>(m) * heads + lh) * (hd + 1);
            float lse[kMaxWorld], ctx[kMaxWorld], mx = -INFINITY;
            for (int sr = 0; sr < a.cp.world; ++sr) {
                unsigned int pl, pc;
                ll_wait(a.cp, cpcall, sr, base + hd, &pl, kStatusCpTimeout);
                ll_wait(a.cp, cpcall, sr, base + d, &pc, kStatusCpTimeout);
                lse[sr] = __uint_as_float(pl);
                ctx[sr] = __uint_as_float(pc);
                mx = fmaxf(mx, lse[sr]);
            }
            float num = 0.f, den = 0.f;
            for (int sr = 0; sr < a.cp.world; ++sr) {
                const float wgt = lse[sr] == -INFINITY ? 0.f : exp2f(lse[sr] - mx);
                num = fmaf(wgt, ctx[sr], num);
                den += wgt;
            }
            xs[k] = (den > 0.f ? num / den : 0.f) * sigmoid_f(a.z[static_cast<size_t>(m) * a.K + k]);
        }
    }
    __syncthreads();
    act_split<3>(planes + static_cast<size_t>(m) * 3 * a.K, xs, 1, a.K, red, ds);
    if (threadIdx.x == 0) descale_out[m] = ds[0];
}

}  // namespace nexrt

using namespace nexrt;

extern "C" int nexrt_oproj_stage_split(const void* in, const void* z, const void* gnorm_w, void* planes, void* descale, int K, int M, int mode, float eps,
                                       int hd, const NexrtLLChannel* cp, unsigned int cp_site, void* stream) {
    mode &= 3;
    if (M < 1 || M > kMaxRows || K % 128 || mode < 0 || mode > 2) return cudaErrorInvalidValue;
    if (mode == 2 && (cp == nullptr || hd <= 0 || K % hd)) return cudaErrorInvalidValue;
    OProjArgs a{};
    a.in = static_cast<const float*>(in); a.z = static_cast<const float*>(z); a.gnorm_w = static_cast<const float*>(gnorm_w);
    a.K = K; a.M = M; a.mode = mode; a.hd = hd; a.eps = eps;
    if (cp) { a.cp = *cp; a.cp_site = cp_site; }
    return launch(oproj_stage_split_kernel, dim3(M), dim3(256), sizeof(float) * K, static_cast<cudaStream_t>(stream), a, static_cast<uint8_t*>(planes),
                  static_cast<float*>(descale));
}

extern "C" int nexrt_oproj_allreduce(const void* in, const void* z, const void* gnorm_w, const void* w, const void* s, void* x, int H, int K,
                                     int M, int mode, float eps, int hd, const NexrtLLChannel* ch, unsigned int site,
                                     const NexrtLLChannel* cp, unsigned int cp_site, int n_cta, void* stream) {
    const int overwrite = (mode & 4) ? 1 : 0;
    mode &= 3;
    if (M < 1 || M > kMaxRows || K % 128 || H % 2 || ch == nullptr || mode < 0 || mode > 2) return cudaErrorInvalidValue;
    if (mode == 2 && (cp == nullptr || hd <= 0 || K % hd)) return cudaErrorInvalidValue;
    if (ch->world > 1 && ch->slots < static_cast<unsigned int>(kMaxRows) * H) return cudaErrorInvalidValue;
    OProjArgs a{};
    a.in = static_cast<const float*>(in); a.z = static_cast<const float*>(z); a.gnorm_w = static_cast<const float*>(gnorm_w);
    a.w = static_cast<const uint8_t*>(w); a.s = static_cast<const float*>(s); a.x = static_cast<__nv_bfloat16*>(x);
    a.H = H; a.K = K; a.M = M; a.mode = mode; a.hd = hd; a.overwrite = overwrite; a.eps = eps; a.ch = *ch; a.site = site;
    a.partial_out = partial_out_buffer();
    if (cp) { a.cp = *cp; a.cp_site = cp_site; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int mp = M == 1 ? 1 : (M == 2 ? 2 : 4), terms = 3;
    const size_t smem_mma = sizeof(float) * (static_cast<size_t>(mp) * K + 8 * 256 + kMaxRows * 16) + static_cast<size_t>(mp) * terms * K;
    // wide K with several rows (an unsharded out-projection at tensor-parallel 1) does not fit the tensor-core
    // kernel's staging buffers: those shapes take the CUDA-core kernel
    if ((gemv_mode() & 2) && H % 16 == 0 && K % 64 == 0 && smem_mma <= 200 * 1024) {
        dim3 g(H / 16), b(256);
        if (mp == 1) return launch(oproj_allreduce_mma_kernel<1>, g, b, smem_mma, st, a);
        if (mp == 2) return launch(oproj_allreduce_mma_kernel<2>, g, b, smem_mma, st, a);
        return launch(oproj_allreduce_mma_kernel<4>, g, b, smem_mma, st, a);
    }
    const int mb = M == 1 ? 1 : 4;
    const int max_rows = (H + n_cta - 1) / n_cta;
    const size_t smem = sizeof(float) * (static_cast<size_t>(mb) * K + gemv_part_floats(max_rows, mb, gemv_geom(K / 16, gemv_threads())) +
                                         static_cast<size_t>(kMaxRows) * max_rows);
    dim3 g(n_cta), b(gemv_threads());
    if (mb == 1) return launch(oproj_allreduce_kernel<1>, g, b, smem, st, a);
    return launch(oproj_allreduce_kernel<4>, g, b, smem, st, a);
}
