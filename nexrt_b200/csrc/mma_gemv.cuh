// Tensor-core streaming GEMV for FP8 weights with exact-split FP8 activations.
//
// The batch-1 projections are bound by instruction issue, not by bytes: decoding e4m3 to fp32
// and multiplying on the CUDA cores costs about 40 instructions per 16 weight bytes.  Here the
// weight bytes go from global memory to registers and straight into the tensor cores, which do
// the decode and the multiply-accumulate in fp32.  FP8 x FP8 needs an FP8 activation, so the
// activation is split exactly into a sum of e4m3 terms,
//     x' = t1 + t2 / 16 + t3 / 256,   t1 = e4m3(x'), t2 = e4m3(16 (x' - t1)), t3 = e4m3(16 (16 (x' - t1) - t2)),
// (relative error 2^-12, better than bf16; the factor 16 keeps every term in e4m3's normal range), and the terms occupy separate columns of the N=8
// operand: D[16 rows][8] += W[16][32] * T[32][8].  The per-128x128-block weight scale multiplies
// the fp32 partial of each 64-byte k-window (`acc += scale * partial`, the arithmetic of the
// reference's CUDA-core kernels, e.g. nex_n2_5_pro/kernels/full_attn/
// nex_n2_5_pro_qkv_proj_ctypes.cu:108-123).
//
// Fragment mapping: lane (g = lane / 4, t = lane % 4) loads 16 contiguous bytes of weight row g and
// of row g + 8 at byte offset 16 t of a 64-byte k-window and feeds them to two
// mma.m16n8k32 instructions; because the reduction index may be permuted freely, the same byte
// positions of activation column g form the B fragment, so every operand is one aligned 16-byte
// load and nothing is shuffled or staged.
#pragma once

#include "common.cuh"

namespace nexrt {

constexpr int kWin = 64;          // bytes of K one warp-wide load pair covers
constexpr int kRowsPerGroup = 16; // rows of one MMA tile

__device__ __forceinline__ void mma_e4m3_16x8x32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.f), "f"(v));
    return static_cast<uint8_t>(r & 0xff);
}
__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
    return e4m3x2_to_float2(static_cast<uint16_t>(b)).x;
}

// Fixed power-of-two prescale of the split: normalised activations are bounded by sqrt(K) times
// the norm multiplier, so 2 keeps |x'| well under the e4m3 limit of 448 while leaving 2^-11 of
// absolute resolution; saturation of the first term is absorbed by the later terms.
constexpr float kSplitScale = 2.0f;
constexpr float kSplitDescale = 0.5f;
constexpr float kTermStep = 16.0f;        // scale between consecutive split terms
constexpr float kTermInv = 1.0f / 16.0f;

// e4m3 split of 4 values at once: TERMS packed words (byte i of word t = term t of value i).
template <int TERMS>
__device__ __forceinline__ void split4(float (&r)[4], uint32_t (&out)[TERMS]) {
#pragma unroll
    for (int term = 0; term < TERMS; ++term) {
        uint16_t lo, hi;
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(r[1]), "f"(r[0]));
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(r[3]), "f"(r[2]));
        out[term] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
        if (term + 1 < TERMS) {
            // the residual is re-scaled by 16 so that every term uses the normal range of e4m3
            // (min normal 2^-6) instead of dying in its subnormals: x' = t1 + t2 / 16 + t3 / 256
            const float2 a = e4m3x2_to_float2(lo), b = e4m3x2_to_float2(hi);
            r[0] = (r[0] - a.x) * kTermStep; r[1] = (r[1] - a.y) * kTermStep;
            r[2] = (r[2] - b.x) * kTermStep; r[3] = (r[3] - b.y) * kTermStep;
        }
    }
}

// Split `rows` fp32 activation rows xs[m][K] (shared memory, not normalised) into TERMS e4m3 byte
// planes xq[(m * TERMS + term)][K] after scaling each row by the power of two that brings its
// largest magnitude into [128, 256).  descale[m] (shared memory) receives the inverse factor.
// `red` is 32 floats.  K must be a multiple of 4.
template <int TERMS>
__device__ __forceinline__ void act_split(uint8_t* xq, const float* xs, int rows, int K, float* red, float* descale) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    for (int m = 0; m < rows; ++m) {
        float mx = 0.f;
        for (int k = threadIdx.x * 4; k < K; k += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(xs + m * K + k);
            mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
        }
        mx = warp_max(mx);
        __syncthreads();
        if (lane == 0) red[warp] = mx;
        __syncthreads();
        float t = 0.f;
        for (int w = 0; w < nw; ++w) t = fmaxf(t, red[w]);
        int e = 0;
        if (t > 0.f && t < 3.0e38f) frexpf(t, &e);          // t = f * 2^e, f in [0.5, 1)
        const float up = exp2f(static_cast<float>(8 - e));    // largest magnitude -> [128, 256)
        if (threadIdx.x == 0) descale[m] = exp2f(static_cast<float>(e - 8));
        for (int k = threadIdx.x * 4; k < K; k += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(xs + m * K + k);
            float r[4] = {v.x * up, v.y * up, v.z * up, v.w * up};
            uint32_t out[TERMS];
            split4<TERMS>(r, out);
#pragma unroll
            for (int term = 0; term < TERMS; ++term)
                *reinterpret_cast<uint32_t*>(xq + static_cast<size_t>(m * TERMS + term) * K + k) = out[term];
        }
    }
    __syncthreads();
}

// Fused prologue of the tensor-core kernels: rmsnorm(x[m]) * gamma for `rows` bf16 rows of width K
// straight into the e4m3 byte planes xq[(m * TERMS + term)][K] (one pass over registers, one
// block-wide reduction per row).  If `xs` is non-null the normalised fp32 row is also kept there.
// `red` is 32 floats of shared memory.  K must be a multiple of 4.
template <int TERMS>
__device__ __forceinline__ void norm_split_rows(uint8_t* xq, float* xs, const __nv_bfloat16* __restrict__ x, const float* gamma, int rows,
                                                int K, float eps, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    for (int m = 0; m < rows; ++m) {
        float ss = 0.f;
        for (int k = threadIdx.x * 4; k < K; k += blockDim.x * 4) {
            const uint2 u = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(m) * K + k);
            const float v0 = __uint_as_float(u.x << 16), v1 = __uint_as_float(u.x & 0xffff0000u);
            const float v2 = __uint_as_float(u.y << 16), v3 = __uint_as_float(u.y & 0xffff0000u);
            ss = fmaf(v0, v0, fmaf(v1, v1, fmaf(v2, v2, fmaf(v3, v3, ss))));
        }
        ss = warp_sum(ss);
        if (m) __syncthreads();
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < nw; ++w) tot += red[w];
        const float inv = rsqrtf(tot / static_cast<float>(K) + eps);
        for (int k = threadIdx.x * 4; k < K; k += blockDim.x * 4) {
            const uint2 u = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(m) * K + k);
            const float4 gm = *reinterpret_cast<const float4*>(gamma + k);
            float r[4] = {__uint_as_float(u.x << 16) * inv * gm.x, __uint_as_float(u.x & 0xffff0000u) * inv * gm.y,
                          __uint_as_float(u.y << 16) * inv * gm.z, __uint_as_float(u.y & 0xffff0000u) * inv * gm.w};
            if (xs) *reinterpret_cast<float4*>(xs + static_cast<size_t>(m) * K + k) = make_float4(r[0], r[1], r[2], r[3]);
#pragma unroll
            for (int i = 0; i < 4; ++i) r[i] *= kSplitScale;
            uint32_t out[TERMS];
            split4<TERMS>(r, out);
#pragma unroll
            for (int term = 0; term < TERMS; ++term)
                *reinterpret_cast<uint32_t*>(xq + static_cast<size_t>(m * TERMS + term) * K + k) = out[term];
        }
    }
    __syncthreads();
}

// Register-resident form of the same prologue.  Every global load a thread needs is issued
// before anything is consumed: the norm multiplier (a constant) before the programmatic-dependency
// wait, the activation right after it, so the prologue costs one memory round trip instead of one
// per loop iteration.  A thread owns up to NCH groups of 4 consecutive elements: K <= NCH * 4 *
// blockDim.x.
//
// The norm multiplier can be parked in shared memory instead of registers (preload_gamma_async): an asynchronous
// global-to-shared copy issued before the wait, read back by the thread that issued it.  The kernels that also hold a
// whole K range of weight bytes in registers are at the 128-register limit, and a spilled weight register is reloaded
// from local memory inside the tensor-core loop - an L2 round trip per K window when the line has left L1.
template <int NCH>
struct RowNorm {
    float4 gm[NCH];
    const float* park = nullptr;
    __device__ __forceinline__ void preload_gamma(const float* __restrict__ gamma, int K) {
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            const int k = (c * blockDim.x + threadIdx.x) * 4;
            gm[c] = k < K ? *reinterpret_cast<const float4*>(gamma + k) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    // park_smem: K floats of shared memory, 16-byte aligned
    __device__ __forceinline__ void preload_gamma_async(float* park_smem, const float* __restrict__ gamma, int K) {
        park = park_smem;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            const int k = (c * blockDim.x + threadIdx.x) * 4;
            if (k < K) {
                const unsigned int dst = static_cast<unsigned int>(__cvta_generic_to_shared(park_smem + k));
                asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gamma + k) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // xq: e4m3 byte planes [(m * TERMS + term)][K] or null; xs: fp32 rows [m][K] or null.
    // L2_LOADS: read x with ld.global.cg (used when the rows are read before this grid's dependency wait and
    // must not be served from a cache line an earlier grid left on this SM).
    template <int TERMS, bool L2_LOADS = false>
    __device__ __forceinline__ void run(uint8_t* xq, float* xs, const __nv_bfloat16* __restrict__ x, int rows, int K, float eps, float* red,
                                        TraceCta* tr = nullptr) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
        if (park != nullptr) asm volatile("cp.async.wait_group 0;" ::: "memory");   // this thread's own copies: no barrier needed
        for (int m = 0; m < rows; ++m) {
            uint2 u[NCH];
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const int k = (c * blockDim.x + threadIdx.x) * 4;
                const uint2* px = reinterpret_cast<const uint2*>(x + static_cast<size_t>(m) * K + k);
                u[c] = k < K ? (L2_LOADS ? __ldcg(px) : *px) : make_uint2(0u, 0u);
            }
            float v[NCH][4], ss = 0.f;
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                v[c][0] = __uint_as_float(u[c].x << 16); v[c][1] = __uint_as_float(u[c].x & 0xffff0000u);
                v[c][2] = __uint_as_float(u[c].y << 16); v[c][3] = __uint_as_float(u[c].y & 0xffff0000u);
#pragma unroll
                for (int i = 0; i < 4; ++i) ss = fmaf(v[c][i], v[c][i], ss);
            }
            ss = warp_sum(ss);
            if (m) __syncthreads();
            if (lane == 0) red[warp] = ss;
            __syncthreads();
            float tot = 0.f;
            for (int w = 0; w < nw; ++w) tot += red[w];
            const float inv = rsqrtf(tot / static_cast<float>(K) + eps);
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const int k = (c * blockDim.x + threadIdx.x) * 4;
                if (k < K) {
                    const float4 g4 = park != nullptr ? *reinterpret_cast<const float4*>(park + k) : gm[c];
                    float r[4] = {v[c][0] * inv * g4.x, v[c][1] * inv * g4.y, v[c][2] * inv * g4.z, v[c][3] * inv * g4.w};
                    if (xs) *reinterpret_cast<float4*>(xs + static_cast<size_t>(m) * K + k) = make_float4(r[0], r[1], r[2], r[3]);
                    if (xq) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) r[i] *= kSplitScale;
                        uint32_t out[TERMS];
                        split4<TERMS>(r, out);
#pragma unroll
                        for (int term = 0; term < TERMS; ++term)
                            *reinterpret_cast<uint32_t*>(xq + static_cast<size_t>(m * TERMS + term) * K + k) = out[term];
                    }
                }
            }
        }
        __syncthreads();
    }
};

// Same split for activations that are already fp32 in shared memory (no normalisation).
template <int TERMS>
__device__ __forceinline__ void split_rows(uint8_t* xq, const float* xs, int rows, int K, float prescale) {
    for (int idx = threadIdx.x * 4; idx < rows * K; idx += blockDim.x * 4) {
        const int m = idx / K, k = idx % K;
        const float4 v = *reinterpret_cast<const float4*>(xs + idx);
        float r[4] = {v.x * prescale, v.y * prescale, v.z * prescale, v.w * prescale};
        uint32_t out[TERMS];
        split4<TERMS>(r, out);
#pragma unroll
        for (int term = 0; term < TERMS; ++term)
            *reinterpret_cast<uint32_t*>(xq + static_cast<size_t>(m * TERMS + term) * K + k) = out[term];
    }
    __syncthreads();
}

// ---- row sources: address of the 16-byte piece of (row, window) and the scale of that window ----
struct MmaPlain {           // W [rows][K] fp8, S [rows/128][K/128]
    const uint8_t* w; const float* s; int K;
    __device__ __forceinline__ const uint8_t* ptr(int row, int win) const { return w + static_cast<size_t>(row) * K + win * kWin; }
    __device__ __forceinline__ float scale(int row, int win) const { return ld_const_f32(s + (row >> 7) * (K >> 7) + (win >> 1)); }
};

struct MmaExpertUp {        // virtual rows (slot, i) of the selected experts: W13 [E+1][2I][H]
    const uint8_t* w; const float* s; const int* ids; int H, I2;
    __device__ __forceinline__ const uint8_t* ptr(int v, int win) const {
        const int e = ids[v / I2], i = v % I2;
        return w + (static_cast<size_t>(e) * I2 + i) * H + win * kWin;
    }
    __device__ __forceinline__ float scale(int v, int win) const {
        const int e = ids[v / I2], i = v % I2;
        return ld_const_f32(s + (static_cast<size_t>(e) * (I2 >> 7) + (i >> 7)) * (H >> 7) + (win >> 1));
    }
};

struct MmaExpertDown {      // virtual K = [slot][I]: W2 [E+1][H][I]
    const uint8_t* w; const float* s; const int* ids; int H, I;
    __device__ __forceinline__ const uint8_t* ptr(int row, int win) const {
        const int wps = I / kWin, slot = win / wps, kw = win % wps;
        return w + (static_cast<size_t>(ids[slot]) * H + row) * I + kw * kWin;
    }
    __device__ __forceinline__ float scale(int row, int win) const {
        const int wps = I / kWin, slot = win / wps, kw = win % wps;
        return ld_const_f32(s + (static_cast<size_t>(ids[slot]) * (H >> 7) + (row >> 7)) * (I >> 7) + (kw >> 1));
    }
};

// One warp: 16 rows starting at row0, windows w0, w0 + wstride, ... (< nwin_total).  NB windows
// are in flight at a time.  On return d[4] holds this warp's share of D in the MMA accumulator
// layout: d0 (row g, col 2t), d1 (row g, col 2t+1), d2 (row g+8, col 2t), d3 (row g+8, col 2t+1).
template <int NB, typename Src>
struct MmaWarp {
    uint4 ra[NB], rb[NB];
    float sc[NB];           // one scale per window: rows g and g + 8 of a 16-row tile (row0 a multiple of 16) share their 128-row block
    int row0, w0, wstride, nwin, g, t;
    bool preloaded;

    __device__ __forceinline__ MmaWarp(int r0, int first, int stride, int total) : row0(r0), w0(first), wstride(stride), nwin(total) {
        const int lane = threadIdx.x & 31;
        g = lane >> 2; t = lane & 3;
        preloaded = false;
    }
    __device__ __forceinline__ void load(const Src& src, int wbase) {
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            const int win = wbase + i * wstride;
            if (win < nwin) {
                ra[i] = ld_stream16(src.ptr(row0 + g, win) + t * 16);
                rb[i] = ld_stream16(src.ptr(row0 + g + 8, win) + t * 16);
                sc[i] = src.scale(row0 + g, win);
            } else {
                ra[i] = make_uint4(0u, 0u, 0u, 0u);
                rb[i] = make_uint4(0u, 0u, 0u, 0u);
                sc[i] = 0.f;
            }
        }
    }
    // Only for sources that do not depend on data written by earlier kernels of the step.
    __device__ __forceinline__ void preload(const Src& src) { load(src, w0); preloaded = true; }
    // Before another pass over the SAME weights (the next block of token rows): when one load covers every window of this
    // warp, the registers still hold them and the pass starts without a trip to L2.  Sources whose rows change between
    // passes (expert ids per token row) clear `preloaded` themselves instead.
    __device__ __forceinline__ void next_pass() { preloaded = w0 + NB * wstride >= nwin; }

    // xq: shared memory [ncols][Kx] byte planes; columns >= ncols are zero.  NT n-tiles of 8 columns.
    template <int NT>
    __device__ __forceinline__ void run(const Src& src, const uint8_t* xq, int Kx, int ncols, float (&d)[NT][4], TraceCta* tr = nullptr) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) d[nt][0] = d[nt][1] = d[nt][2] = d[nt][3] = 0.f;
        for (int wbase = w0; wbase < nwin; wbase += NB * wstride) {
            if (!(preloaded && wbase == w0)) load(src, wbase);
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                const int win = wbase + i * wstride;
                if (win >= nwin) break;                 // uniform across the warp
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int col = nt * 8 + g;
                    uint4 xb = make_uint4(0u, 0u, 0u, 0u);
                    if (col < ncols) xb = *reinterpret_cast<const uint4*>(xq + static_cast<size_t>(col) * Kx + win * kWin + t * 16);
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_e4m3_16x8x32(c, ra[i].x, rb[i].x, ra[i].y, rb[i].y, xb.x, xb.y);
                    mma_e4m3_16x8x32(c, ra[i].z, rb[i].z, ra[i].w, rb[i].w, xb.z, xb.w);
                    d[nt][0] = fmaf(c[0], sc[i], d[nt][0]); d[nt][1] = fmaf(c[1], sc[i], d[nt][1]);
                    d[nt][2] = fmaf(c[2], sc[i], d[nt][2]); d[nt][3] = fmaf(c[3], sc[i], d[nt][3]);
                }
                if (tr && i == 0 && wbase == w0) tr->mark(6);   // timeline: the first window's weights were there and are consumed
            }
        }
        if (tr) tr->mark(7);                                    // timeline: every window consumed
    }
    // Write the accumulator tile to shared memory: tile[16 rows][8 * NT cols].
    template <int NT>
    __device__ __forceinline__ void store(float* tile, const float (&d)[NT][4]) const {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            tile[g * 8 * NT + nt * 8 + 2 * t] = d[nt][0]; tile[g * 8 * NT + nt * 8 + 2 * t + 1] = d[nt][1];
            tile[(g + 8) * 8 * NT + nt * 8 + 2 * t] = d[nt][2]; tile[(g + 8) * 8 * NT + nt * 8 + 2 * t + 1] = d[nt][3];
        }
    }
};

// Sum over the k-split warps and the split terms, in a fixed order.
// tiles: [ksplit][16][8 * NT]; returns y for (row in group, m).
template <int TERMS, int NT>
__device__ __forceinline__ float mma_result(const float* tiles, int ksplit, int row, int m, float descale) {
    float v = 0.f;
    for (int ks = 0; ks < ksplit; ++ks) {
        const float* tl = tiles + (static_cast<size_t>(ks) * 16 + row) * 8 * NT + m * TERMS;
        float w = 1.f;
#pragma unroll
        for (int term = 0; term < TERMS; ++term) { v = fmaf(tl[term], w, v); w *= kTermInv; }
    }
    return v * descale;
}

// ---- bf16 weights (router, gate rows): mma.m16n8k16 with the activation as bf16 hi + lo columns ----
__device__ __forceinline__ void mma_bf16_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// fp32 rows xs[m][K] (shared memory) -> bf16 planes xh[(m * 2 + term)][K]: hi = bf16(x), lo = bf16(x - hi).
__device__ __forceinline__ void split_bf16_rows(__nv_bfloat16* xh, const float* xs, int rows, int K) {
    for (int idx = threadIdx.x * 2; idx < rows * K; idx += blockDim.x * 2) {
        const int m = idx / K, k = idx % K;
        const float2 v = *reinterpret_cast<const float2*>(xs + idx);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(v.x, v.y);
        const float2 hf = __bfloat1622float2(hi);
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x - hf.x, v.y - hf.y);
        *reinterpret_cast<__nv_bfloat162*>(xh + static_cast<size_t>(m * 2) * K + k) = hi;
        *reinterpret_cast<__nv_bfloat162*>(xh + static_cast<size_t>(m * 2 + 1) * K + k) = lo;
    }
    __syncthreads();
}

// One warp: 16 bf16 weight rows starting at row0 of W [rows][K], 64-byte windows (32 elements)
// w0, w0 + wstride, ... < nwin.  Same lane mapping as the fp8 routine.
template <int NB>
struct MmaWarpBf16 {
    uint4 ra[NB], rb[NB];
    const __nv_bfloat16* w;
    int K, row0, w0, wstride, nwin, g, t;
    bool preloaded;
    __device__ __forceinline__ MmaWarpBf16(const __nv_bfloat16* wt, int k, int r0, int first, int stride, int total)
        : w(wt), K(k), row0(r0), w0(first), wstride(stride), nwin(total) {
        const int lane = threadIdx.x & 31;
        g = lane >> 2; t = lane & 3;
        preloaded = false;
    }
    __device__ __forceinline__ void load(int wbase) {
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            const int win = wbase + i * wstride;
            if (win < nwin) {
                ra[i] = ld_stream16(w + static_cast<size_t>(row0 + g) * K + win * 32 + t * 8);
                rb[i] = ld_stream16(w + static_cast<size_t>(row0 + g + 8) * K + win * 32 + t * 8);
            } else {
                ra[i] = make_uint4(0u, 0u, 0u, 0u);
                rb[i] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    }
    __device__ __forceinline__ void preload() { load(w0); preloaded = true; }
    __device__ __forceinline__ void next_pass() { preloaded = w0 + NB * wstride >= nwin; }   // see MmaWarp::next_pass
    // xh: shared memory bf16 planes [ncols][K]
    __device__ __forceinline__ void run(const __nv_bfloat16* xh, int ncols, float (&d)[4]) {
        d[0] = d[1] = d[2] = d[3] = 0.f;
        for (int wbase = w0; wbase < nwin; wbase += NB * wstride) {
            if (!(preloaded && wbase == w0)) load(wbase);
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                const int win = wbase + i * wstride;
                if (win >= nwin) break;
                uint4 xb = make_uint4(0u, 0u, 0u, 0u);
                if (g < ncols) xb = *reinterpret_cast<const uint4*>(xh + static_cast<size_t>(g) * K + win * 32 + t * 8);
                mma_bf16_16x8x16(d, ra[i].x, rb[i].x, ra[i].y, rb[i].y, xb.x, xb.y);
                mma_bf16_16x8x16(d, ra[i].z, rb[i].z, ra[i].w, rb[i].w, xb.z, xb.w);
            }
        }
    }
    __device__ __forceinline__ void store(float* tile, const float (&d)[4]) const {
        tile[g * 8 + 2 * t] = d[0]; tile[g * 8 + 2 * t + 1] = d[1];
        tile[(g + 8) * 8 + 2 * t] = d[2]; tile[(g + 8) * 8 + 2 * t + 1] = d[3];
    }
};

// tiles [ksplit][16][8]: value of (row, m) = sum over k-split warps of hi + lo columns.
__device__ __forceinline__ float mma_bf16_result(const float* tiles, int ksplit, int row, int m) {
    float v = 0.f;
    for (int ks = 0; ks < ksplit; ++ks) {
        const float* tl = tiles + (static_cast<size_t>(ks) * 16 + row) * 8 + m * 2;
        v += tl[0] + tl[1];
    }
    return v;
}

// Row passes of the tensor-core kernels: 3 split terms per token row, so one n-tile of 8 columns
// holds 2 rows and two n-tiles hold 4 (5 would fit; 4 keeps the passes even for 8 rows).
template <int MP> struct MmaShape { static constexpr int TERMS = 3, NT = MP <= 2 ? 1 : 2, TILE = 16 * 8 * NT; };

}  // namespace nexrt
