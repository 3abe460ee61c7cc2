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
#include "mma_gemv.cuh"

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
    int ba_rows_pad;             // rows of ba_w padded to a multiple of 16 (0: not padded)
    unsigned long long* events;  // optional in-kernel event ring: CTA 0 records %globaltimer at phase boundaries
};

// Per-row tail of the front: history-ring write, causal conv1d(4) + SiLU for the q|k|v rows, plain
// store for the z rows.  pre[m] is the projection of row `row` for token row m0 + m.
template <int MB>
__device__ __forceinline__ void gdn_front_row(const GdnFrontArgs& a, int row, const float (&pre)[MB], int m0, int mb, int C0, const float4& cw) {
    if (row < a.C) {
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

__device__ __forceinline__ void gdn_ba_row(const GdnFrontArgs& a, int row, float v, int mm) {
    if (row < a.nv) a.beta[mm * a.nv + row] = sigmoid_f(v);
    else {
        const int h = row - a.nv;
        a.g[mm * a.nv + h] = -__expf(a.a_log[h]) * softplus_f(v + a.dt_bias[h]);
    }
}

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
    float* gs = part_ba + gemv_part_floats((2 * a.nv + gridDim.x - 1) / gridDim.x, MB, gb);   // [H] norm multiplier
    GemvCta<MB, U, PlainFp8> gemv(PlainFp8{a.front_w, a.front_s, a.H}, r0, nrows, a.H);
    gemv.preload();
    for (int i = threadIdx.x; i < a.H; i += blockDim.x) gs[i] = a.in_ln[i];
    if (nrows) prefetch_l2_range(a.conv_w + static_cast<size_t>(r0) * 4, static_cast<size_t>(nrows) * 16);
    pdl_wait();
    const int C0 = a.ctl[kCtlCommittedLen];
    for (int m0 = 0; m0 < a.M; m0 += MB) {
        const int mb = min(MB, a.M - m0);
        if (m0) __syncthreads();
        stage_rmsnorm_plain(xs, a.x + static_cast<size_t>(m0) * a.H, gs, mb, a.H, a.eps, red);
        if (m0 == 0) gemv.run(xs, part);
        else gemv_cta<MB, U>(PlainFp8{a.front_w, a.front_s, a.H}, r0, nrows, xs, a.H, part);
        if (nba) gemv_cta<MB, 2>(PlainBf16{a.ba_w, a.H}, b0, nba, xs, a.H, part_ba);
        __syncthreads();
        for (int rl = threadIdx.x; rl < nrows; rl += blockDim.x) {
            float pre[MB];
#pragma unroll
            for (int m = 0; m < MB; ++m) pre[m] = gemv_result(part, rl, m, MB, gf.wpr);
            float4 cw = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r0 + rl < a.C) cw = *reinterpret_cast<const float4*>(a.conv_w + static_cast<size_t>(r0 + rl) * 4);
            gdn_front_row<MB>(a, r0 + rl, pre, m0, mb, C0, cw);
        }
        for (int rl = threadIdx.x; rl < nba; rl += blockDim.x)
            for (int m = 0; m < mb; ++m) gdn_ba_row(a, b0 + rl, gemv_result(part_ba, rl, m, MB, gb.wpr), m0 + m);
    }
}

// Tensor-core form of the front: one CTA per 16 weight rows, the 8 warps split K, FP8 weights go
// from global memory to registers to mma.m16n8k32 against the exact e4m3 split of the normalised
// activation.  MP token rows per pass (1, 2 or 4).  The first 2*nv CTAs also do one b/a row each.
#define NEXRT_EVENT(i) do { if (a.events != nullptr && blockIdx.x == 0 && threadIdx.x == 0) a.events[i] = globaltimer_ns(); } while (0)

// LOOP: the grid is smaller than the number of 16-row groups and a CTA walks several of them (one-row steps on wide shards);
// a separate instantiation, so that the one-group form the 8-way deployment runs keeps its register allocation.
template <int MP, bool LOOP = false>
__global__ void __launch_bounds__(256, 2) gdn_front_mma_kernel(GdnFrontArgs a) {
    constexpr int TERMS = MmaShape<MP>::TERMS, NT = MmaShape<MP>::NT, TILE = MmaShape<MP>::TILE, NB = 8, KS = 8;
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[32];
    NEXRT_EVENT(0);
    TraceCta tr;
    tr.begin(kTrGdnFront);
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5;
    const int row0 = blockIdx.x * kRowsPerGroup, nwin = a.H / kWin;
    // the first 2 * nv CTAs also project one bf16 b/a row each (CUDA cores, weights preloaded)
    const int ba_row = static_cast<int>(blockIdx.x) < 2 * a.nv ? static_cast<int>(blockIdx.x) : -1;
    const bool ba_cta = ba_row >= 0;
    float* xs = smem;                                                      // [MP][H]   (b/a CTAs only)
    float* tiles = xs + static_cast<size_t>(MP) * a.H;                     // [KS][TILE]
    float* part_ba = tiles + KS * TILE;                                    // [wpr][MP]
    uint8_t* xq = reinterpret_cast<uint8_t*>(part_ba + 64);                // [MP*TERMS][H]
    float* gpark = reinterpret_cast<float*>(xq + static_cast<size_t>(MP) * TERMS * a.H);   // [H] norm multiplier, parked until the norm
    __nv_bfloat16* bpark = reinterpret_cast<__nv_bfloat16*>(gpark + a.H);                  // [H] this CTA's b/a row (b/a CTAs only)
    float4* cpark = reinterpret_cast<float4*>(bpark + a.H);                                // [16] conv taps of the CTA's rows
    const MmaPlain src{a.front_w, a.front_s, a.H};
    MmaWarp<NB, MmaPlain> mw(row0, warp, KS, nwin);
    mw.preload(src);
    // b/a row of this CTA and the conv taps of its 16 rows: asynchronous copies into shared memory (no registers held across
    // the wait); thread t owns elements [16 t, 16 t + 16) of the bf16 row and reads back only what it copied itself
    const bool ba_thread = ba_cta && static_cast<int>(threadIdx.x) * 16 < a.H;
    if (ba_thread) {
        const __nv_bfloat16* p = a.ba_w + static_cast<size_t>(ba_row) * a.H + threadIdx.x * 16;
        const unsigned int dst = static_cast<unsigned int>(__cvta_generic_to_shared(bpark + threadIdx.x * 16));
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(p) : "memory");
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst + 16u), "l"(p + 8) : "memory");
    }
    const bool conv_thread = threadIdx.x < kRowsPerGroup && row0 + static_cast<int>(threadIdx.x) < a.C;
    if (conv_thread) {
        const unsigned int dst = static_cast<unsigned int>(__cvta_generic_to_shared(cpark + threadIdx.x));
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(a.conv_w + static_cast<size_t>(row0 + threadIdx.x) * 4) : "memory");
    }
    NEXRT_EVENT(1);
    RowNorm<4> norm;
    norm.preload_gamma_async(gpark, a.in_ln, a.H);
    NEXRT_EVENT(2);
    pdl_wait();
    tr.mark(1);
    NEXRT_EVENT(3);
    const int C0 = a.ctl[kCtlCommittedLen];
    for (int m0 = 0; m0 < a.M; m0 += MP) {
        const int mb = min(MP, a.M - m0);
        if (m0) { __syncthreads(); mw.next_pass(); }
        norm.template run<TERMS>(xq, ba_cta ? xs : nullptr, a.x + static_cast<size_t>(m0) * a.H, mb, a.H, a.eps, red, &tr);
        tr.mark(4);
        NEXRT_EVENT(4);
        float d[NT][4];
        mw.template run<NT>(src, xq, a.H, mb * TERMS, d, &tr);
        mw.template store<NT>(tiles + warp * TILE, d);
        tr.mark(2);
        NEXRT_EVENT(5);
        if (ba_cta) {
            // dot of the b/a row with the normalised fp32 rows (xs, written by the norm above): per-warp partials
            float wf[16];
            if (ba_thread) {
                const uint4* bp = reinterpret_cast<const uint4*>(bpark + threadIdx.x * 16);
                unpack8_bf16(bp[0], wf);
                unpack8_bf16(bp[1], wf + 8);
            }
            for (int m = 0; m < mb; ++m) {
                float acc = 0.f;
                if (ba_thread) {
                    const float* xr = xs + static_cast<size_t>(m) * a.H + threadIdx.x * 16;
#pragma unroll
                    for (int e = 0; e < 16; e += 4) {
                        const float4 xv = *reinterpret_cast<const float4*>(xr + e);
                        acc = fmaf(wf[e], xv.x, fmaf(wf[e + 1], xv.y, fmaf(wf[e + 2], xv.z, fmaf(wf[e + 3], xv.w, acc))));
                    }
                }
                acc = warp_sum(acc);
                if ((threadIdx.x & 31) == 0) part_ba[m * 8 + warp] = acc;
            }
        }
        __syncthreads();
        tr.mark(5);
        NEXRT_EVENT(7);
        if (threadIdx.x < kRowsPerGroup) {
            float pre[MP];
#pragma unroll
            for (int m = 0; m < MP; ++m) pre[m] = m < mb ? mma_result<TERMS, NT>(tiles, KS, threadIdx.x, m, kSplitDescale) : 0.f;
            const float4 cw = conv_thread ? cpark[threadIdx.x] : make_float4(0.f, 0.f, 0.f, 0.f);
            gdn_front_row<MP>(a, row0 + threadIdx.x, pre, m0, mb, C0, cw);
        } else if (ba_cta && threadIdx.x >= 32 && threadIdx.x < 32 + mb) {
            const int m = threadIdx.x - 32;
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) v += part_ba[m * 8 + w];      // fixed order over the 8 warps
            gdn_ba_row(a, ba_row, v, m0 + m);
        }
        NEXRT_EVENT(6);
    }
    if constexpr (MP == 1 && LOOP) {
        // One-row steps on wide shards (tensor-parallel 1 or 2: up to 1280 row groups): the grid is capped at the CTAs the
        // machine holds at once and a CTA walks its further groups here - the row is normalised and split once per CTA, not
        // once per group, and only the weight stream repeats.
        for (int rg = row0 + static_cast<int>(gridDim.x) * kRowsPerGroup; rg < a.R; rg += static_cast<int>(gridDim.x) * kRowsPerGroup) {
            __syncthreads();
            mw.row0 = rg;
            mw.preloaded = false;
            float d[NT][4];
            mw.template run<NT>(src, xq, a.H, TERMS, d);
            mw.template store<NT>(tiles + warp * TILE, d);
            __syncthreads();
            if (threadIdx.x < kRowsPerGroup) {
                const int row = rg + static_cast<int>(threadIdx.x);
                float pre[MP] = {mma_result<TERMS, NT>(tiles, KS, threadIdx.x, 0, kSplitDescale)};
                const float4 cw = row < a.C ? *reinterpret_cast<const float4*>(a.conv_w + static_cast<size_t>(row) * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                gdn_front_row<MP>(a, row, pre, 0, 1, C0, cw);
            }
        }
    }
    tr.mark(3);
}

// Tail of the wide front (multi-row steps): the q|k|v|z projections of all rows were produced by the tcgen05 rows
// GEMM into pre[M][R]; this kernel applies the per-channel conv ring + SiLU / the z store (one thread per weight
// row, all token rows in registers), and extra CTAs project the bf16 b/a rows from the fp32 normalised rows xn.
__global__ void __launch_bounds__(256) gdn_front_tail_kernel(GdnFrontArgs a, const float* __restrict__ pre, const float* __restrict__ xn, int row_ctas,
                                                             int ksplit) {
    TraceCta tr;
    tr.begin(kTrHelper);
    pdl_launch_dependents();
    pdl_wait();
    tr.mark(1);
    if (static_cast<int>(blockIdx.x) < row_ctas) {
        const int row = blockIdx.x * blockDim.x + threadIdx.x;
        if (row >= a.R) return;
        // Every load of the thread is requested before the first use: the three history taps (positions C0 - 3 .. C0 - 1
        // of the ring, independent of this step's projections), the conv weights, and up to 8 x 8 K-split partials.  In
        // program order (sum, store the ring, read the ring back) the same work is four dependent trips to L2.
        const bool conv = row < a.C;
        const int C0 = a.ctl[kCtlCommittedLen], ring = a.conv_ring_len;
        float hist[3] = {0.f, 0.f, 0.f};
        float4 cw = make_float4(0.f, 0.f, 0.f, 0.f);
        if (conv) {
#pragma unroll
            for (int j = 0; j < 3; ++j) hist[j] = __ldcg(a.conv_ring + static_cast<size_t>((C0 - 3 + j + ring) % ring) * a.C + row);
            cw = *reinterpret_cast<const float4*>(a.conv_w + static_cast<size_t>(row) * 4);
        }
        constexpr int kMaxSplit = 8;
        float part[kMaxRows][kMaxSplit];
#pragma unroll
        for (int m = 0; m < kMaxRows; ++m)
#pragma unroll
            for (int ks = 0; ks < kMaxSplit; ++ks)
                part[m][ks] = (m < a.M && ks < ksplit) ? __ldcg(pre + (static_cast<size_t>(ks) * a.M + m) * a.R + row) : 0.f;
        float p[kMaxRows];
#pragma unroll
        for (int m = 0; m < kMaxRows; ++m) {
            p[m] = 0.f;
#pragma unroll
            for (int ks = 0; ks < kMaxSplit; ++ks) p[m] += part[m][ks];      // K-split partials, fixed order (absent ones are zero)
        }
        if (!conv) {
#pragma unroll
            for (int m = 0; m < kMaxRows; ++m)
                if (m < a.M) a.z[static_cast<size_t>(m) * (a.R - a.C) + (row - a.C)] = p[m];
        } else {
            // window of the causal conv: positions C0 - 3 .. C0 + M - 1
#pragma unroll
            for (int m = 0; m < kMaxRows; ++m) {
                if (m < a.M) {
                    const float h0 = m >= 3 ? p[m - 3 < 0 ? 0 : m - 3] : hist[m], h1 = m >= 2 ? p[m - 2 < 0 ? 0 : m - 2] : hist[m + 1],
                                h2 = m >= 1 ? p[m - 1 < 0 ? 0 : m - 1] : hist[m + 2 > 2 ? 2 : m + 2];
                    const float v = fmaf(cw.x, h0, fmaf(cw.y, h1, fmaf(cw.z, h2, cw.w * p[m])));
                    a.conv_ring[static_cast<size_t>((C0 + m) % ring) * a.C + row] = p[m];
                    a.qkv[static_cast<size_t>(m) * a.C + row] = silu_f(v);
                }
            }
        }
        tr.mark(3);
        return;
    }
    // one warp per (b/a row, token row)
    const int lane = threadIdx.x & 31;
    const int item = (blockIdx.x - row_ctas) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= 2 * a.nv * a.M) return;
    const int row = item / a.M, m = item % a.M;
    const __nv_bfloat16* w = a.ba_w + static_cast<size_t>(row) * a.H;
    const float* xr = xn + static_cast<size_t>(m) * a.H;
    float acc = 0.f;
#pragma unroll 4
    for (int k = lane * 8; k < a.H; k += 256) {      // unrolled so that the loads of four steps are in flight together
        float wf[8];
        unpack8_bf16(*reinterpret_cast<const uint4*>(w + k), wf);
        const float4 x0 = *reinterpret_cast<const float4*>(xr + k), x1 = *reinterpret_cast<const float4*>(xr + k + 4);
        acc = fmaf(wf[0], x0.x, fmaf(wf[1], x0.y, fmaf(wf[2], x0.z, fmaf(wf[3], x0.w, acc))));
        acc = fmaf(wf[4], x1.x, fmaf(wf[5], x1.y, fmaf(wf[6], x1.z, fmaf(wf[7], x1.w, acc))));
    }
    acc = warp_sum(acc);
    if (lane == 0) gdn_ba_row(a, row, acc, m);
    tr.mark(3);
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

// One row of the delta rule for one value column: S is this lane's 4 key rows of the column's state.
// One reduction round per row: with S the decayed state, k^ = k / |k| and delta = (v - k^.S) b, the output is
// q.(S + k^ delta) = q.S + (q.k^) delta, so the five lane sums q.q, k.k, q.k, k.S and q.S are reduced side by side
// and neither the delta nor the output waits for a second, dependent reduction (the reference's core kernel
// reduces k.S and q.S_new one after the other, linear_attn/nex_n2_5_pro_linear_recurrent_core_ctypes.cu:117-146).
__device__ __forceinline__ float gdn_core_row(const float4& q, const float4& k, float v, float decay, float b, float4& S) {
    S.x *= decay; S.y *= decay; S.z *= decay; S.w *= decay;
    float qq = q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
    float kk = k.x * k.x + k.y * k.y + k.z * k.z + k.w * k.w;
    float qk = q.x * k.x + q.y * k.y + q.z * k.z + q.w * k.w;
    float ks = k.x * S.x + k.y * S.y + k.z * S.z + k.w * S.w;
    float qs = q.x * S.x + q.y * S.y + q.z * S.z + q.w * S.w;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        qq += __shfl_xor_sync(0xffffffffu, qq, off);
        kk += __shfl_xor_sync(0xffffffffu, kk, off);
        qk += __shfl_xor_sync(0xffffffffu, qk, off);
        ks += __shfl_xor_sync(0xffffffffu, ks, off);
        qs += __shfl_xor_sync(0xffffffffu, qs, off);
    }
    const float qn = rsqrtf(qq + 1e-6f) * 0.08838834764831845f, kn = rsqrtf(kk + 1e-6f);
    const float delta = (v - ks * kn) * b;
    const float kd = kn * delta;
    S.x = fmaf(k.x, kd, S.x); S.y = fmaf(k.y, kd, S.y); S.z = fmaf(k.z, kd, S.z); S.w = fmaf(k.w, kd, S.w);
    return (qs + qk * kd) * qn;
}

// grid (nv, 128 / warps-per-CTA); one warp per value column, lane holds 4 key rows.
// ROWS = true (multi-row steps): every row's operands are requested before the recurrence starts (they do not depend on the
// state): inside the loop a row's loads cannot move above the previous row's state store, and each row would pay its own
// trip to L2 (8.5 -> 6.9 us at 8 rows).  The one-row step keeps the plain form, which measured 0.7 us faster there.
template <bool ROWS>
__global__ void __launch_bounds__(256) gdn_core_kernel(GdnCoreArgs a) {
    TraceCta tr;
    tr.begin(kTrGdnCore);
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int head = blockIdx.x, col = blockIdx.y * nwarps + warp;
    const int qk_head = head / (a.nv / a.nqk);
    const size_t head_stride = static_cast<size_t>(128) * 128, slot_stride = head_stride * a.nv;
    const size_t elem = head * head_stride + static_cast<size_t>(col) * 128 + lane * 4;
    pdl_wait();
    tr.mark(1);
    const int C0 = a.ctl[kCtlCommittedLen];
    if constexpr (!ROWS) {
        float4 S = *reinterpret_cast<const float4*>(a.state_ring + static_cast<size_t>(C0 % a.state_ring_len) * slot_stride + elem);
        for (int m = 0; m < a.M; ++m) {
            const float* row = a.qkv + static_cast<size_t>(m) * a.C;
            const float4 q4 = *reinterpret_cast<const float4*>(row + qk_head * 128 + lane * 4);
            const float4 k4 = *reinterpret_cast<const float4*>(row + (a.nqk + qk_head) * 128 + lane * 4);
            const float v = row[(2 * a.nqk + head) * 128 + col];
            const float decay = __expf(a.g[m * a.nv + head]), b = a.beta[m * a.nv + head];
            const float o = gdn_core_row(q4, k4, v, decay, b, S);
            *reinterpret_cast<float4*>(a.state_ring + static_cast<size_t>((C0 + m + 1) % a.state_ring_len) * slot_stride + elem) = S;
            if (lane == 0) a.out[static_cast<size_t>(m) * a.nv * 128 + head * 128 + col] = o;
        }
    } else {
        float4 q4[kMaxRows], k4[kMaxRows];
        float vv[kMaxRows], gg[kMaxRows], bb[kMaxRows];
#pragma unroll
        for (int m = 0; m < kMaxRows; ++m) {
            if (m < a.M) {
                const float* row = a.qkv + static_cast<size_t>(m) * a.C;
                q4[m] = __ldcg(reinterpret_cast<const float4*>(row + qk_head * 128 + lane * 4));
                k4[m] = __ldcg(reinterpret_cast<const float4*>(row + (a.nqk + qk_head) * 128 + lane * 4));
                vv[m] = __ldcg(row + (2 * a.nqk + head) * 128 + col);
                gg[m] = __ldcg(a.g + m * a.nv + head);
                bb[m] = __ldcg(a.beta + m * a.nv + head);
            }
        }
        float4 S = *reinterpret_cast<const float4*>(a.state_ring + static_cast<size_t>(C0 % a.state_ring_len) * slot_stride + elem);
#pragma unroll
        for (int m = 0; m < kMaxRows; ++m) {
            if (m >= a.M) break;
            const float o = gdn_core_row(q4[m], k4[m], vv[m], __expf(gg[m]), bb[m], S);
            *reinterpret_cast<float4*>(a.state_ring + static_cast<size_t>((C0 + m + 1) % a.state_ring_len) * slot_stride + elem) = S;
            if (lane == 0) a.out[static_cast<size_t>(m) * a.nv * 128 + head * 128 + col] = o;
        }
    }
    tr.mark(3);
}

}  // namespace nexrt

using namespace nexrt;

static unsigned long long* g_events = nullptr;
// Optional event ring (8 x u64 device memory) filled by CTA 0 of the tensor-core front kernel.
extern "C" int nexrt_set_event_ring(void* ring) {
    g_events = static_cast<unsigned long long*>(ring);
    return 0;
}

extern "C" int nexrt_gdn_front(const void* x, const void* in_ln, const void* front_w, const void* front_s, const void* ba_w,
                               const void* conv_w, const void* a_log, const void* dt_bias, const void* ctl, void* conv_ring, void* qkv,
                               void* z, void* beta, void* g, int H, int R, int C, int nv, int M, int conv_ring_len, float eps, int ba_rows_pad,
                               int n_cta, void* stream) {
    if (M < 1 || M > kMaxRows || H % 256 || conv_ring_len < M + 3) return cudaErrorInvalidValue;
    GdnFrontArgs a{static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(in_ln), static_cast<const uint8_t*>(front_w),
                   static_cast<const float*>(front_s), static_cast<const __nv_bfloat16*>(ba_w), static_cast<const float*>(conv_w),
                   static_cast<const float*>(a_log), static_cast<const float*>(dt_bias), static_cast<const int*>(ctl),
                   static_cast<float*>(conv_ring), static_cast<float*>(qkv), static_cast<float*>(z), static_cast<float*>(beta),
                   static_cast<float*>(g), H, R, C, nv, M, conv_ring_len, eps, ba_rows_pad, g_events};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if ((gemv_mode() & 1) && R % 16 == 0 && H % 512 == 0 && H <= 4096 && R / 16 >= 2 * nv) {
        const int mp = M == 1 ? 1 : (M == 2 ? 2 : 4);
        const size_t smem = sizeof(float) * (static_cast<size_t>(mp) * H + 8 * 256 + 64) + static_cast<size_t>(mp) * 3 * H + sizeof(float) * H +
                            sizeof(__nv_bfloat16) * H + 16 * sizeof(float4);
        dim3 g(R / 16), b(256);
        // one row: no more CTAs than the machine holds at once (two per SM), but at least the 2 nv that carry a b/a row
        if (mp == 1 && R / 16 > max(2 * n_cta, 2 * nv)) return launch(gdn_front_mma_kernel<1, true>, dim3(max(2 * n_cta, 2 * nv)), b, smem, st, a);
        if (mp == 1) return launch(gdn_front_mma_kernel<1>, g, b, smem, st, a);
        if (mp == 2) return launch(gdn_front_mma_kernel<2>, g, b, smem, st, a);
        return launch(gdn_front_mma_kernel<4>, g, b, smem, st, a);
    }
    const int mb = M == 1 ? 1 : 4;
    const size_t smem = sizeof(float) * (static_cast<size_t>(mb + 1) * H + gemv_part_floats((R + n_cta - 1) / n_cta, mb, gemv_geom(H / 16, gemv_threads())) +
                                         gemv_part_floats((2 * nv + n_cta - 1) / n_cta, mb, gemv_geom(H / 8, gemv_threads())));
    if (M == 1) return launch(gdn_front_kernel<1>, dim3(n_cta), dim3(gemv_threads()), smem, st, a);
    return launch(gdn_front_kernel<4>, dim3(n_cta), dim3(gemv_threads()), smem, st, a);
}

// Tail of the wide front: pre [M][R] fp32 projections, xn [M][H] fp32 normalised rows (see gdn_front_tail_kernel).
extern "C" int nexrt_gdn_front_tail(const void* pre, const void* xn, const void* ba_w, const void* conv_w, const void* a_log, const void* dt_bias,
                                    const void* ctl, void* conv_ring, void* qkv, void* z, void* beta, void* g, int H, int R, int C, int nv, int M,
                                    int conv_ring_len, int ksplit, void* stream) {
    if (M < 1 || M > kMaxRows || H % 256 || conv_ring_len < M + 3) return cudaErrorInvalidValue;
    GdnFrontArgs a{nullptr, nullptr, nullptr, nullptr, static_cast<const __nv_bfloat16*>(ba_w), static_cast<const float*>(conv_w),
                   static_cast<const float*>(a_log), static_cast<const float*>(dt_bias), static_cast<const int*>(ctl),
                   static_cast<float*>(conv_ring), static_cast<float*>(qkv), static_cast<float*>(z), static_cast<float*>(beta),
                   static_cast<float*>(g), H, R, C, nv, M, conv_ring_len, 0.f, 0, nullptr};
    const int row_ctas = (R + 255) / 256, ba_ctas = (2 * nv * M + 7) / 8;
    return launch(gdn_front_tail_kernel, dim3(row_ctas + ba_ctas), dim3(256), 0, static_cast<cudaStream_t>(stream), a, static_cast<const float*>(pre),
                  static_cast<const float*>(xn), row_ctas, ksplit);
}

extern "C" int nexrt_gdn_core(const void* qkv, const void* beta, const void* g, const void* ctl, void* state_ring, void* out, int nqk, int nv,
                              int M, int state_ring_len, int C, void* stream) {
    if (M < 1 || M > kMaxRows || state_ring_len < M + 1 || nv % nqk) return cudaErrorInvalidValue;
    GdnCoreArgs a{static_cast<const float*>(qkv), static_cast<const float*>(beta), static_cast<const float*>(g),
                  static_cast<const int*>(ctl), static_cast<float*>(state_ring), static_cast<float*>(out), nqk, nv, M, state_ring_len, C};
    if (M == 1) return launch(gdn_core_kernel<false>, dim3(nv, 128 / 8), dim3(256), 0, static_cast<cudaStream_t>(stream), a);
    return launch(gdn_core_kernel<true>, dim3(nv, 128 / 8), dim3(256), 0, static_cast<cudaStream_t>(stream), a);
}
