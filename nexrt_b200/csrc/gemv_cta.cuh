// CTA-cooperative, k-stationary streaming GEMV for the latency-bound batch-1 regime.
//
// Every thread of the CTA owns one 16-byte chunk position of the reduction dimension: it keeps the
// matching activation values (up to MB rows x 16) in registers for the whole kernel and walks
// down the CTA's weight rows, issuing U independent 16-byte streaming loads before it consumes
// any of them.  All 512 threads are busy whatever the number of rows a CTA owns (17 rows per CTA
// at tensor-parallel 8), the bytes of the CTA's whole weight slice are requested in one or two
// waves, and the activation is read from shared memory once per thread instead of once per
// weight chunk.  Row partials are reduced with warp shuffles, then across the warps of a row in a
// fixed order through shared memory (deterministic).
//
// The reference reaches the same goal with split-K across the warps of small CTAs
// (LinearFrontSplitCtaSk4Kernel, nex_n2_5_pro/kernels/linear_attn/
// nex_n2_5_pro_linear_front_gemv_ctypes.cu:88-224); here one routine serves all seven GEMV sites
// through a small "row source" functor.
#pragma once

#include "common.cuh"

namespace nexrt {

// Threads per CTA of every GEMV-type kernel.  256 threads at <= 128 registers let the CTAs of two
// consecutive kernels share an SM, which is what makes the early weight preload of the next
// kernel overlap the tail of the current one under programmatic dependent launch.
// (Kernels are compiled for up to 512 threads at <= 128 registers; the launch width is a run-time
// setting so both shapes can be measured.)
int& gemv_threads_ref();
inline int gemv_threads() { return gemv_threads_ref(); }
// Bit mask of the kernels that use the tensor-core GEMV where the shape allows (1: projection
// fronts, 2: out-projection, 4: expert gate/up, 8: expert down, 16: router and gate rows, 32: attention key loop; 64: the
// attention decode runs as thread-block clusters with a DSMEM combine); 0 selects the CUDA-core kernels.
int& gemv_mode_ref();
inline int gemv_mode() { return gemv_mode_ref(); }

// ---- row sources ------------------------------------------------------------------------------
// at(chunk) fixes the thread's chunk; ptr(r)/scale(r) then address row r of the CTA's range.

struct PlainFp8 {                       // W [rows][K] fp8, S [rows/128][K/128]
    const uint8_t* w; const float* s; int K;
    static constexpr int EPL = 16;
    size_t off; int kb, KB;
    __device__ __forceinline__ void at(int chunk) { off = static_cast<size_t>(chunk) * 16; kb = chunk >> 3; KB = K / kScaleBlock; }
    __device__ __forceinline__ const void* ptr(int r) const { return w + static_cast<size_t>(r) * K + off; }
    __device__ __forceinline__ float scale(int r) const { return __ldg(s + (r >> 7) * KB + kb); }
};

struct PlainBf16 {                      // W [rows][K] bf16
    const __nv_bfloat16* w; int K;
    static constexpr int EPL = 8;
    size_t off;
    __device__ __forceinline__ void at(int chunk) { off = static_cast<size_t>(chunk) * 8; }
    __device__ __forceinline__ const void* ptr(int r) const { return w + static_cast<size_t>(r) * K + off; }
    __device__ __forceinline__ float scale(int) const { return 1.f; }
};

struct ExpertUp {                       // virtual rows (slot, i): W13 [E+1][2I][H] fp8 of the selected experts
    const uint8_t* w; const float* s; const int* ids; int H, I2;   // I2 = 2 * I_local; ids: shared memory [S]
    static constexpr int EPL = 16;
    size_t off; int kb, KB;
    __device__ __forceinline__ void at(int chunk) { off = static_cast<size_t>(chunk) * 16; kb = chunk >> 3; KB = H / kScaleBlock; }
    __device__ __forceinline__ const void* ptr(int v) const {
        const int e = ids[v / I2], i = v % I2;
        return w + (static_cast<size_t>(e) * I2 + i) * H + off;
    }
    __device__ __forceinline__ float scale(int v) const {
        const int e = ids[v / I2], i = v % I2;
        return __ldg(s + (static_cast<size_t>(e) * (I2 / kScaleBlock) + (i >> 7)) * KB + kb);
    }
};

struct ExpertDown {                     // virtual K = S x I: W2 [E+1][H][I] fp8, chunk -> (slot, k)
    const uint8_t* w; const float* s; const int* ids; int H, I;     // ids: shared memory [S]
    static constexpr int EPL = 16;
    const uint8_t* base; const float* sbase; int SB;
    __device__ __forceinline__ void at(int chunk) {
        const int cps = I >> 4, slot = chunk / cps, kc = chunk % cps, e = ids[slot];
        SB = I / kScaleBlock;
        base = w + static_cast<size_t>(e) * H * I + kc * 16;
        sbase = s + static_cast<size_t>(e) * (H / kScaleBlock) * SB + (kc >> 3);
    }
    __device__ __forceinline__ const void* ptr(int r) const { return base + static_cast<size_t>(r) * I; }
    __device__ __forceinline__ float scale(int r) const { return __ldg(sbase + (r >> 7) * SB); }
};

// ---- geometry ---------------------------------------------------------------------------------
struct GemvGeom {
    int chunks;   // 16-byte chunks per (virtual) row
    int tpr;      // threads cooperating on one row
    int rpp;      // rows processed per pass
    int wpr;      // partials per row (warps per row, 1 for sub-warp groups)
    int kblocks;  // passes over the reduction dimension (chunks > threads)
};

__host__ __device__ inline GemvGeom gemv_geom(int chunks, int threads) {
    GemvGeom g;
    g.chunks = chunks;
    if (chunks >= 32) g.tpr = min(((chunks + 31) / 32) * 32, threads);
    else g.tpr = chunks <= 8 ? 8 : chunks <= 16 ? 16 : 32;
    g.rpp = threads / g.tpr;
    g.wpr = g.tpr >= 32 ? g.tpr / 32 : 1;
    g.kblocks = (chunks + g.tpr - 1) / g.tpr;
    return g;
}

// shared-memory floats needed for the partials of `nrows` rows
__host__ __device__ inline size_t gemv_part_floats(int nrows, int mb, const GemvGeom& g) { return static_cast<size_t>(nrows) * g.wpr * mb; }

template <int EPL>
__device__ __forceinline__ void unpack_chunk(const uint4& v, float* f) {
    if (EPL == 16) unpack16_fp8(v, f);
    else unpack8_bf16(v, f);
}

// The GEMV as an object so that its first batch of weight loads can be issued BEFORE the
// programmatic-dependency wait (weights are constants, so they may be fetched while the previous
// kernel of the stream is still running) and consumed after the activation has been staged.
//
//   GemvCta<MB, U, Src> g(src, row0, nrows, Kx);   g.preload();   pdl_wait();   ... stage xs ...
//   g.run(xs, part);   __syncthreads();   gemv_result(part, ...)
//
// xs: shared memory [MB][Kx] fp32 in natural order (Kx = chunks * EPL).  Rows [row0, row0+nrows).
// part: shared memory [nrows][wpr][MB].
template <int MB, int U, typename Src>
struct GemvCta {
    static constexpr int EPL = Src::EPL;
    Src src;
    GemvGeom g;
    int row0, nrows, Kx, rsub, kc, lane, wir, jn;
    bool row_thread, preloaded;
    uint4 wv[U];
    float sc[U];

    __device__ __forceinline__ GemvCta(const Src& s, int r0, int nr, int kx) : src(s), row0(r0), nrows(nr), Kx(kx) {
        g = gemv_geom(Kx / EPL, blockDim.x);
        const int tid = threadIdx.x;
        rsub = tid / g.tpr; kc = tid % g.tpr; lane = tid & 31;
        row_thread = rsub < g.rpp;
        wir = g.tpr >= 32 ? kc >> 5 : 0;
        jn = (nrows + g.rpp - 1) / g.rpp;
        preloaded = false;
    }

    __device__ __forceinline__ void load_batch(int j0, bool live) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int rl = (j0 + u) * g.rpp + rsub;
            const bool ok = live && rl < nrows;
            const int r = row0 + (ok ? rl : 0);
            wv[u] = ok ? ld_stream16(src.ptr(r)) : make_uint4(0u, 0u, 0u, 0u);
            sc[u] = ok ? src.scale(r) : 0.f;
        }
    }

    // Issue the loads of the first batch (k-block 0).  Only for row sources that do not depend on
    // data produced by earlier kernels of the step.
    __device__ __forceinline__ void preload() {
        const bool live = row_thread && kc < g.chunks;
        src.at(live ? kc : 0);
        load_batch(0, live);
        preloaded = true;
    }

    __device__ __forceinline__ void run(const float* __restrict__ xs, float* __restrict__ part) {
        for (int kb = 0; kb < g.kblocks; ++kb) {
            const int chunk = kb * g.tpr + kc;
            const bool live = row_thread && chunk < g.chunks;
            float xr[MB][EPL];
            if (!(preloaded && kb == 0)) src.at(live ? chunk : 0);
#pragma unroll
            for (int m = 0; m < MB; ++m)
#pragma unroll
                for (int e = 0; e < EPL; e += 4) {
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (live) v = *reinterpret_cast<const float4*>(xs + static_cast<size_t>(m) * Kx + chunk * EPL + e);
                    xr[m][e] = v.x; xr[m][e + 1] = v.y; xr[m][e + 2] = v.z; xr[m][e + 3] = v.w;
                }
            for (int j0 = 0; j0 < jn; j0 += U) {
                if (!(preloaded && kb == 0 && j0 == 0)) load_batch(j0, live);
                float acc[MB][U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    float wf[EPL];
                    unpack_chunk<EPL>(wv[u], wf);
#pragma unroll
                    for (int m = 0; m < MB; ++m) {
                        float a0 = 0.f, a1 = 0.f;
#pragma unroll
                        for (int e = 0; e < EPL; e += 2) {
                            a0 = fmaf(wf[e], xr[m][e], a0);
                            a1 = fmaf(wf[e + 1], xr[m][e + 1], a1);
                        }
                        acc[m][u] = (a0 + a1) * sc[u];
                    }
                }
                if (g.tpr >= 32) {
                    // transpose-reduce: U values per lane -> lane l ends with the warp total of value
                    // index sel(l); about 2U shuffles instead of 5U
#pragma unroll
                    for (int m = 0; m < MB; ++m) {
                        int sel = 0;
#pragma unroll
                        for (int w = U / 2, o = 16; w >= 1; w >>= 1, o >>= 1) {
                            const bool hi = (lane & o) != 0;
#pragma unroll
                            for (int i = 0; i < w; ++i) {
                                const float send = hi ? acc[m][i] : acc[m][i + w];
                                const float keep = hi ? acc[m][i + w] : acc[m][i];
                                acc[m][i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                            }
                            if (hi) sel += w;
                        }
#pragma unroll
                        for (int o = 16 / U; o >= 1; o >>= 1) acc[m][0] += __shfl_xor_sync(0xffffffffu, acc[m][0], o);
                        constexpr int kLow = 32 / U;   // lanes whose low bits are zero write: one writer per value
                        if ((lane & (kLow - 1)) == 0) {
                            const int rl = (j0 + sel) * g.rpp + rsub;
                            if (row_thread && rl < nrows) {
                                float* p = part + (static_cast<size_t>(rl) * g.wpr + wir) * MB + m;
                                *p = (kb == 0 ? 0.f : *p) + acc[m][0];
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int rl = (j0 + u) * g.rpp + rsub;
#pragma unroll
                        for (int m = 0; m < MB; ++m) {
                            float a = acc[m][u];
                            for (int o = g.tpr >> 1; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                            if (kc == 0 && row_thread && rl < nrows) {
                                float* p = part + (static_cast<size_t>(rl) * g.wpr + wir) * MB + m;
                                *p = (kb == 0 ? 0.f : *p) + a;
                            }
                        }
                    }
                }
            }
        }
    }
};

// One-shot form (no early preload).
template <int MB, int U, typename Src>
__device__ __forceinline__ void gemv_cta(Src src, int row0, int nrows, const float* __restrict__ xs, int Kx, float* __restrict__ part) {
    GemvCta<MB, U, Src> g(src, row0, nrows, Kx);
    g.run(xs, part);
}

// Fixed-order sum of the partials of (row_local, m).
__device__ __forceinline__ float gemv_result(const float* part, int row_local, int m, int mb, int wpr) {
    const float* p = part + static_cast<size_t>(row_local) * wpr * mb + m;
    float v = 0.f;
    for (int w = 0; w < wpr; ++w) v += p[w * mb];
    return v;
}

// Stage rmsnorm(x) * gamma of `rows` bf16 rows into shared memory in natural order (gamma may
// point at shared memory that was filled before the dependency wait).
__device__ __forceinline__ void stage_rmsnorm_plain(float* xs, const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, int rows,
                                                    int H, float eps, float* red) {
    for (int r = 0; r < rows; ++r) {
        float ss = 0.f;
        for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
            const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + static_cast<size_t>(r) * H + i));
            xs[r * H + i] = v.x;
            xs[r * H + i + 1] = v.y;
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, ss));
        }
        ss = block_sum(ss, red);
        const float inv = rsqrtf(ss / static_cast<float>(H) + eps);
        for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
            const float2 gm = *reinterpret_cast<const float2*>(gamma + i);
            xs[r * H + i] *= inv * gm.x;
            xs[r * H + i + 1] *= inv * gm.y;
        }
    }
    __syncthreads();
}

}  // namespace nexrt
