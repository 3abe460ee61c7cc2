// Expert projections of a multi-row step (4-row MTP verify, 8-row DFlash verify, prefill chunks) on the
// 5th-generation tensor cores, with the tensor-parallel all-reduce fused into the down-projection's epilogue.
//
//   rows_norm_split : rmsnorm(x[m]) * gamma -> three e4m3 planes per row (x' = t1 + t2/16 + t3/256, exact to
//                     2^-12), laid out as a [3M, H] matrix: the B operand of the gate/up product
//   tc_moe_l1       : one CTA per (distinct expert of the step, 128 gate/up rows).  The expert's FP8 rows are
//                     the A operand (TMA -> shared memory -> tcgen05.mma, M = 128), all 3M activation planes
//                     the B operand (N = 32), so an expert chosen by several rows is streamed once; the 128x128
//                     block scale multiplies each K block's TMEM result on its way into fp32 registers
//   rows_h_split    : h = silu(gate) * up * route weight -> three planes per row, [3M, S*I], power-of-two scale
//   tc_moe_l2       : one CTA per (row, 128 output rows): K runs over the row's S experts (each K block takes its
//                     A tile from another expert's down matrix), then the epilogue all-reduces its 128 values
//                     over the LL packet channel (multimem.st through the NVSwitch alias, or peer stores), adds
//                     the residual and writes bf16 x - compute tile and collective in one kernel.
//
// Same arithmetic as the mma.sync kernels of moe.cu (exact three-term activation split, fp32 accumulation,
// block scale per K block), so the verify rows agree with the one-row decode path.  Replaces the reference's
// WGMMA expert kernels of the 8-row family (kernels/moe/nex_n2_5_pro_m8_moe_l1_wgmma_ctypes.cu,
// nex_n2_5_pro_m8_moe_l2_ctypes.cu) and its route plan (…m8_route_plan…): the plan here is a scan of the 88
// expert ids by each CTA.
#include <cuda.h>
#include <cuda_runtime.h>

#include "api.h"
#include "common.cuh"
#include "ll.cuh"
#include "mma_gemv.cuh"
#include "tc_common.cuh"

namespace {
using namespace nexrt;
using namespace nexrt::tc;

constexpr int kBN = 32;                              // 3 planes x up to 8 rows, padded
constexpr int kA = kBM * kSpan;                      // 16 KB weight tile
constexpr int kB = kBN * kSpan;                      // 4 KB activation tile
constexpr int kStage = kA + kB;
constexpr int smem_bytes(bool) { return 1024 + 4 * kStage + 1024; }

struct TcMoeArgs {
    const float* w_s;       // block scales of the weight matrix, [rows / 128][K / 128] over the flattened experts
    const int* ids;         // [M][S]
    const float* descale;   // [M] (down projection only)
    float* gu;              // [M][S][2I] (gate/up only)
    __nv_bfloat16* x;       // [M][H] residual stream (down projection only)
    int H, I, S, M;
    int n_total;            // experts in the weight matrix (routed + shared); ids are clamped into [0, n_total)
    int overwrite;          // shared down projection: write the reduced sum instead of adding it to x
    int ksplit;             // gate/up and plain GEMM: CTAs per row tile along K (partial planes [ksplit][M][S][rows])
    LLChannel ch;
    unsigned int site;
    int* status;
    int trace_kind;         // timeline builds: which record list this launch writes (kTrTcMoeL1, ...)
};

// DOWN = false: gate/up of one distinct expert for every row that routes to it.
// DOWN = true : down projection of one row over its S experts + all-reduce + residual.
// BF16 = true (plain rows GEMM only): bf16 weights without block scales, two bf16 planes (hi, lo) per row.
// Four shared-memory stages and EIGHT tensor-memory accumulator buffers, two CTAs per SM: what bounds one CTA's K walk is
// the round trip commit -> epilogue wakes -> tcgen05.ld -> buffer released -> issuer wakes (about 2 us on B200), so the
// number of K blocks in flight is what sets the rate; 8 buffers x 32 columns x 2 CTAs use all 512 TMEM columns.
// SHARED = true (with DOWN): one weight matrix for all rows (out-projection): the epilogue all-reduces every row.
template <bool DOWN, bool BF16 = false, bool SHARED = false>
__global__ void __launch_bounds__(kThreads, 2) tc_moe_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcMoeArgs a) {
    constexpr int NS = 4;                // shared-memory stages
    constexpr int NAB = 8;               // accumulator buffers in tensor memory
    extern __shared__ uint8_t smem_raw[];
    __shared__ int s_user[kMaxRows];     // gate/up: slot of row m that uses this CTA's expert, or -1
    __shared__ float s_wscale[kMaxKBlocks + 16 * 8];   // block scale of every K block this CTA walks (no load in the loop)
    TraceCta tr;
    tr.begin(a.trace_kind);
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int I2 = 2 * a.I;
    int m, slot, mt, expert = 0;
    int ks = 0;                                          // index of this CTA's K range
    if (DOWN) { mt = blockIdx.x; m = blockIdx.y; slot = 0; }
    else {
        const int n_mt = static_cast<int>(gridDim.x) / a.ksplit;
        mt = blockIdx.x % n_mt; ks = blockIdx.x / n_mt; slot = blockIdx.y; m = blockIdx.z;
    }
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base);
    uint8_t* smem = base + 1024;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * NS + 2 * NAB);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NS + 2 * NAB + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (NS + s); };
    auto tfull = [&](int b) { return bar0 + 8u * (2 * NS + b); };
    auto tempty = [&](int b) { return bar0 + 8u * (2 * NS + NAB + b); };
    constexpr uint32_t kCols = NAB * kBN;

    constexpr int kElems = BF16 ? kSpan / 2 : kSpan;   // elements of K per 128-byte block
    constexpr int TERMS = BF16 ? 2 : 3;                // activation planes per row
    const int kpe = DOWN ? a.I / 128 : a.H / kElems;   // K blocks per expert
    // split K: each of the ksplit CTAs of a row tile walks a contiguous range of K blocks; partial sums go to separate
    // output planes that the consumer adds in a fixed order
    const int ksplit = DOWN ? 1 : a.ksplit;
    const int kb_per = (kpe + ksplit - 1) / ksplit;
    const int kb0 = ks * kb_per;
    const int KB = DOWN ? a.S * kpe : max(0, min(kb_per, kpe - kb0));
    // everything that does not depend on the predecessor's output happens before the dependency wait
    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
        for (int b = 0; b < NAB; ++b) { mbar_init(tfull(b), 1); mbar_init(tempty(b), 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), kCols);
    pdl_wait();
    tr.mark(1);
    bool active = true;
    if (!DOWN) {
        // route plan: the first row that names an expert computes it for every row that does
        expert = a.ids[m * a.S + slot];
        for (int m2 = 0; m2 < m; ++m2)
            for (int s2 = 0; s2 < a.S; ++s2)
                if (a.ids[m2 * a.S + s2] == expert) active = false;   // uniform for the CTA
        if (threadIdx.x < kMaxRows) {
            int u = -1;
            if (static_cast<int>(threadIdx.x) >= m && static_cast<int>(threadIdx.x) < a.M)
                for (int s2 = 0; s2 < a.S; ++s2)
                    if (a.ids[threadIdx.x * a.S + s2] == expert) u = s2;
            s_user[threadIdx.x] = u;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int n_kb = active ? KB : 0;

    // weight rows of K block kb start at this row of the flattened expert matrix
    auto expert_of = [&](int kb) { return min(max(DOWN ? a.ids[m * a.S + kb / kpe] : expert, 0), a.n_total - 1); };   // kb: index in this CTA's range
    const int rows_per_expert = DOWN ? a.H : I2;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < n_kb; ++kb) {
                const int s = kb % NS;
                if (!mbar_wait(empty(s), ((kb / NS) & 1) ^ 1, abort_flag)) break;
                mbar_expect_tx(full(s), kA + kB);
                const uint32_t dst = smem_u32(smem + s * kStage);
                const int e = expert_of(kb);
                tma_load_2d(dst, &map_w, ((kb0 + kb) % kpe) * kElems, e * rows_per_expert + mt * kBM, full(s));
                tma_load_2d(dst + kA, &map_x, (kb0 + kb) * kElems, 0, full(s));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc<!BF16>(kBN);
            for (int kb = 0; kb < n_kb; ++kb) {
                const int s = kb % NS, buf = kb % NAB;
                if (!mbar_wait(tempty(buf), ((kb / NAB) & 1) ^ 1, abort_flag)) break;
                if (!mbar_wait(full(s), (kb / NS) & 1, abort_flag)) break;
                tc_fence_after();
                const uint32_t a0 = smem_u32(smem + s * kStage);
                const uint64_t da = smem_desc(a0), db = smem_desc(a0 + kA);
#pragma unroll
                for (int k = 0; k < 4; ++k) tc_mma<!BF16>(tmem_base + buf * kBN, da + 2u * k, db + 2u * k, idesc, k != 0);
                tc_commit(empty(s));
                tc_commit(tfull(buf));
            }
        }
    } else {
        const int q = warp & 3;
        const int row = mt * kBM + 32 * q + lane;        // row inside the expert's matrix
        constexpr int NC = (DOWN && !SHARED) ? 4 : kBN;   // columns this thread accumulates
        float acc[NC];
#pragma unroll
        for (int n = 0; n < NC; ++n) acc[n] = 0.f;
        // the block scales of the whole K walk go to shared memory first: a global load per K block would sit in the
        // serial chain tmem-full -> load -> scale -> accumulate
        if (!BF16) {
            for (int kb = threadIdx.x - 64; kb < n_kb; kb += 128) {
                const int e = expert_of(kb);
                s_wscale[kb] = __ldg(a.w_s + (static_cast<size_t>(e) * (rows_per_expert / 128) + mt) * kpe + (kb0 + kb) % kpe);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        bool ok = true;
        for (int kb = 0; kb < n_kb && ok; ++kb) {
            const int buf = kb % NAB;
            ok = mbar_wait(tfull(buf), (kb / NAB) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(32 * q) << 16) + buf * kBN;
            const float w = BF16 ? 1.f : s_wscale[kb];
            if (DOWN && !SHARED) {
                float p[4];
                tmem_ld4(taddr + 3 * m, p);
                tmem_ld_wait();
#pragma unroll
                for (int n = 0; n < 3; ++n) acc[n] = fmaf(p[n], w, acc[n]);
            } else {
                float p[kBN];
                tmem_ld16(taddr, p);
                tmem_ld16(taddr + 16, p + 16);
                tmem_ld_wait();
#pragma unroll
                for (int n = 0; n < kBN; ++n) acc[n] = fmaf(p[n], w, acc[n]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty(buf));
        }
        if (ok && active) {
            if (DOWN && SHARED) {
                LLCall call{0u, 0u};
                if (a.ch.world > 1) call = ll_begin(a.ch, a.site);
#pragma unroll
                for (int m2 = 0; m2 < kMaxRows; ++m2) {
                    if (m2 < a.M) {
                        const float val = (acc[3 * m2] + acc[3 * m2 + 1] * (1.f / 16.f) + acc[3 * m2 + 2] * (1.f / 256.f)) * a.descale[m2];
                        const size_t o = static_cast<size_t>(m2) * a.H + row;
                        const float sum = ll_allreduce_f32(a.ch, call, static_cast<unsigned int>(o), val);
                        a.x[o] = __float2bfloat16_rn(a.overwrite ? sum : __bfloat162float(a.x[o]) + sum);
                    }
                }
            } else if (DOWN) {
                const float val = (acc[0] + acc[1] * (1.f / 16.f) + acc[2] * (1.f / 256.f)) * a.descale[m];
                LLCall call{0u, 0u};
                if (a.ch.world > 1) call = ll_begin(a.ch, a.site);
                const size_t o = static_cast<size_t>(m) * a.H + row;
                const float sum = ll_allreduce_f32(a.ch, call, static_cast<unsigned int>(o), val);
                a.x[o] = __float2bfloat16_rn(__bfloat162float(a.x[o]) + sum);
            } else {
#pragma unroll
                for (int m2 = 0; m2 < kMaxRows; ++m2) {
                    const int u = s_user[m2];
                    if (u >= 0 && row < I2) {
                        const float val = BF16 ? acc[TERMS * m2] + acc[TERMS * m2 + 1]
                                               : (acc[3 * m2] + acc[3 * m2 + 1] * (1.f / 16.f) + acc[3 * m2 + 2] * (1.f / 256.f)) * kSplitDescale;
                        a.gu[(static_cast<size_t>(ks) * a.M * a.S + static_cast<size_t>(m2) * a.S + u) * I2 + row] = val;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 50000) {
        }
        if (threadIdx.x == 0 && a.status) atomicCAS(a.status, 0, static_cast<int>(kStatusPipeTimeout));
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_free(tmem_base, kCols);
    }
    tr.mark(3);
}

// rmsnorm(x[m]) * gamma -> planes[(3m + term)][H]; xn (optional) keeps the normalised row in fp32
__global__ void __launch_bounds__(256) rows_norm_split_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, uint8_t* planes, float* xn,
                                                              int H, float eps) {
    __shared__ float red[32];
    TraceCta tr;
    tr.begin(kTrHelper);
    pdl_launch_dependents();
    RowNorm<4> norm;
    norm.preload_gamma(gamma, H);
    pdl_wait();
    tr.mark(1);
    const int m = blockIdx.x;
    norm.template run<3>(planes + static_cast<size_t>(m) * 3 * H, xn ? xn + static_cast<size_t>(m) * H : nullptr, x + static_cast<size_t>(m) * H, 1, H, eps, red);
    tr.mark(3);
}

// rmsnorm(x[m]) * gamma -> bf16 planes[(2m + {hi, lo})][H]: x' = hi + lo to ~2^-17
__global__ void __launch_bounds__(256) rows_norm_split_bf16_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, __nv_bfloat16* planes,
                                                                   uint8_t* planes_e4m3, int H, float eps) {
    __shared__ float red[32];
    extern __shared__ __align__(16) float xs[];
    TraceCta tr;
    tr.begin(kTrHelper);
    pdl_launch_dependents();
    RowNorm<4> norm;
    norm.preload_gamma(gamma, H);
    pdl_wait();
    tr.mark(1);
    const int m = blockIdx.x;
    norm.template run<3>(nullptr, xs, x + static_cast<size_t>(m) * H, 1, H, eps, red);
    split_bf16_rows(planes + static_cast<size_t>(m) * 2 * H, xs, 1, H);
    if (planes_e4m3 != nullptr) split_rows<3>(planes_e4m3 + static_cast<size_t>(m) * 3 * H, xs, 1, H, kSplitScale);   // same rows for the expert kernels
    tr.mark(3);
}

// h = silu(gate) * up * route weight -> planes[(3m + term)][S * I], descale[m]
__global__ void __launch_bounds__(256) rows_h_split_kernel(const float* __restrict__ gu, const float* __restrict__ wts, uint8_t* planes, float* descale,
                                                           int I, int S, int M, int ksplit) {
    extern __shared__ __align__(16) float hs[];
    __shared__ float red[32];
    __shared__ float ds[1];
    TraceCta tr;
    tr.begin(kTrHelper);
    pdl_launch_dependents();
    pdl_wait();
    tr.mark(1);
    const int m = blockIdx.x, VK = S * I;
    for (int k = threadIdx.x * 4; k < VK; k += blockDim.x * 4) {
        const int sl = k / I, i = k % I;
        const float* g = gu + (static_cast<size_t>(m) * S + sl) * 2 * I;
        float4 gt = *reinterpret_cast<const float4*>(g + i), up = *reinterpret_cast<const float4*>(g + I + i);
        for (int ks = 1; ks < ksplit; ++ks) {           // K-split partial planes of the gate/up product, fixed order
            const float* gk = g + static_cast<size_t>(ks) * M * S * 2 * I;
            const float4 g2 = *reinterpret_cast<const float4*>(gk + i), u2 = *reinterpret_cast<const float4*>(gk + I + i);
            gt.x += g2.x; gt.y += g2.y; gt.z += g2.z; gt.w += g2.w;
            up.x += u2.x; up.y += u2.y; up.z += u2.z; up.w += u2.w;
        }
        const float wt = wts[m * S + sl];
        *reinterpret_cast<float4*>(hs + k) = make_float4(silu_f(gt.x) * up.x * wt, silu_f(gt.y) * up.y * wt, silu_f(gt.z) * up.z * wt, silu_f(gt.w) * up.w * wt);
    }
    __syncthreads();
    act_split<3>(planes + static_cast<size_t>(m) * 3 * VK, hs, 1, VK, red, ds);
    if (threadIdx.x == 0) descale[m] = ds[0];
    tr.mark(3);
}

template <bool DOWN, bool BF16 = false, bool SHARED = false>
int launch_tc_moe(const CUtensorMap& mw, const CUtensorMap& mx, const TcMoeArgs& a, dim3 grid, cudaStream_t st) {
    static bool configured = false;
    auto kern = tc_moe_kernel<DOWN, BF16, SHARED>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(DOWN));
        if (e != cudaSuccess) return static_cast<int>(e);
        configured = true;
    }
    if (const cudaError_t e = pipe_budget_install()) return static_cast<int>(e);
    return launch(kern, grid, dim3(kThreads), static_cast<size_t>(smem_bytes(DOWN)), st, mw, mx, a);
}

}  // namespace

extern "C" {

// Gate/up projections of all rows' experts.  planes: e4m3 [3M][H] scratch, written here.
int nexrt_tc_moe_l1(const void* x, const void* post_ln, const void* w13, const void* w13_s, const void* ids, void* gu, void* planes, int H, int I, int S,
                    int M, int n_experts_total, int ksplit, float eps, int planes_ready, int* status, void* stream) {
    if (M < 1 || M > kMaxRows || H % 128 || H > 4096 || I % 64 || S < 1 || S > 16 || ksplit < 1 || ksplit > 4) return cudaErrorInvalidValue;
    auto st = static_cast<cudaStream_t>(stream);
    if (!planes_ready) {      // the router of this step did not leave the planes: make them here
        int e = launch(rows_norm_split_kernel, dim3(M), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(post_ln),
                       static_cast<uint8_t*>(planes), static_cast<float*>(nullptr), H, eps);
        if (e) return e;
    }
    CUtensorMap mw, mx;
    const uint64_t wrows = static_cast<uint64_t>(n_experts_total) * 2 * I;
    if (!tensor_map(&mw, w13, wrows, H, H, kBM, false) || !tensor_map(&mx, planes, 3 * M, H, H, kBN, false)) return cudaErrorInvalidValue;
    TcMoeArgs a{};
    a.w_s = static_cast<const float*>(w13_s); a.ids = static_cast<const int*>(ids); a.gu = static_cast<float*>(gu);
    a.H = H; a.I = I; a.S = S; a.M = M; a.n_total = n_experts_total; a.ksplit = ksplit; a.status = status;
    a.trace_kind = kTrTcMoeL1;
    return launch_tc_moe<false>(mw, mx, a, dim3(2 * I / kBM * ksplit, S, M), st);
}

// rmsnorm(x[m]) * gamma for M rows -> e4m3 planes [3M][H] (and, if xn != null, the fp32 rows [M][H]).
int nexrt_rows_norm_split(const void* x, const void* gamma, void* planes, void* xn, int H, int M, float eps, void* stream) {
    if (M < 1 || M > kMaxRows || H % 4 || H > 4096) return cudaErrorInvalidValue;
    return launch(rows_norm_split_kernel, dim3(M), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(x),
                  static_cast<const float*>(gamma), static_cast<uint8_t*>(planes), static_cast<float*>(xn), H, eps);
}

// out[m][r] = sum_k W[r][k] * xhat[m][k] for M rows at once: W [R][K] e4m3 with 128x128 block scales, xhat given as
// the planes of nexrt_rows_norm_split.  The weights are streamed once for all rows.  zero_ids: M zero int32 words.
// ksplit > 1 splits K over that many CTAs per row tile: out then holds ksplit partial planes [ksplit][M][R] for the
// consumer to add in order.
int nexrt_tc_rows_gemm(const void* w, const void* w_s, const void* planes, void* out, const void* zero_ids, int R, int K, int M, int ksplit, int* status,
                       void* stream) {
    if (M < 1 || M > kMaxRows || R % 128 || K % 128 || K > 8192 || ksplit < 1 || ksplit > 8) return cudaErrorInvalidValue;
    CUtensorMap mw, mx;
    if (!tensor_map(&mw, w, R, K, K, kBM, false) || !tensor_map(&mx, planes, 3 * M, K, K, kBN, false)) return cudaErrorInvalidValue;
    TcMoeArgs a{};
    a.w_s = static_cast<const float*>(w_s); a.ids = static_cast<const int*>(zero_ids); a.gu = static_cast<float*>(out);
    a.H = K; a.I = R / 2; a.S = 1; a.M = M; a.n_total = 1; a.ksplit = ksplit; a.status = status;     // one "expert" of R rows, named by every row
    a.trace_kind = kTrTcRows;
    return launch_tc_moe<false>(mw, mx, a, dim3(R / kBM * ksplit, 1, 1), static_cast<cudaStream_t>(stream));
}

// Router logits of M rows: partial[ks][m][r] = sum over the K range ks of W[r][k] * xhat[m][k], W bf16 [rows][K] (rows
// need not be a multiple of 128; rows_pad is the row stride of the output), xhat = rmsnorm(x) * gamma as bf16 hi + lo
// planes written into `planes` ([2M][K] bf16 scratch).
int nexrt_tc_router_logits(const void* x, const void* gamma, const void* w, void* planes, void* partial, const void* zero_ids, int rows, int rows_pad, int K,
                           int M, int ksplit, float eps, void* planes_e4m3, int* status, void* stream) {
    if (M < 1 || M > kMaxRows || K % 64 || K > 4096 || rows_pad % 2 || rows_pad < rows || ksplit < 1 || ksplit > 16) return cudaErrorInvalidValue;
    auto st = static_cast<cudaStream_t>(stream);
    int e = launch(rows_norm_split_bf16_kernel, dim3(M), dim3(256), sizeof(float) * K, st, static_cast<const __nv_bfloat16*>(x),
                   static_cast<const float*>(gamma), static_cast<__nv_bfloat16*>(planes), static_cast<uint8_t*>(planes_e4m3), K, eps);
    if (e) return e;
    CUtensorMap mw, mx;
    if (!tensor_map(&mw, w, rows, K, K, kBM, true) || !tensor_map(&mx, planes, 2 * M, K, K, kBN, true)) return cudaErrorInvalidValue;
    TcMoeArgs a{};
    a.ids = static_cast<const int*>(zero_ids); a.gu = static_cast<float*>(partial);
    a.H = K; a.I = rows_pad / 2; a.S = 1; a.M = M; a.n_total = 1; a.ksplit = ksplit; a.status = status;
    a.trace_kind = kTrTcRouter;
    return launch_tc_moe<false, true>(mw, mx, a, dim3((rows + kBM - 1) / kBM * ksplit, 1, 1), st);
}

// Down projections + all-reduce + residual.  planes: e4m3 [3M][S*I] scratch, descale: fp32 [M] scratch.
int nexrt_tc_moe_l2_allreduce(const void* gu, const void* ids, const void* wts, const void* w2, const void* w2_s, void* x, void* planes, void* descale,
                              int H, int I, int S, int M, int n_experts_total, int gu_ksplit, const NexrtLLChannel* ch, unsigned int site, int* status,
                              void* stream) {
    if (M < 1 || M > kMaxRows || H % 128 || I % 128 || S < 1 || S > 16 || ch == nullptr) return cudaErrorInvalidValue;
    if (ch->world > 1 && ch->slots < static_cast<unsigned int>(kMaxRows) * H) return cudaErrorInvalidValue;
    auto st = static_cast<cudaStream_t>(stream);
    const int VK = S * I;
    int e = launch(rows_h_split_kernel, dim3(M), dim3(256), sizeof(float) * VK, st, static_cast<const float*>(gu), static_cast<const float*>(wts),
                   static_cast<uint8_t*>(planes), static_cast<float*>(descale), I, S, M, gu_ksplit < 1 ? 1 : gu_ksplit);
    if (e) return e;
    CUtensorMap mw, mx;
    const uint64_t wrows = static_cast<uint64_t>(n_experts_total) * H;
    if (!tensor_map(&mw, w2, wrows, I, I, kBM, false) || !tensor_map(&mx, planes, 3 * M, VK, VK, kBN, false)) return cudaErrorInvalidValue;
    TcMoeArgs a{};
    a.w_s = static_cast<const float*>(w2_s); a.ids = static_cast<const int*>(ids); a.descale = static_cast<const float*>(descale);
    a.x = static_cast<__nv_bfloat16*>(x); a.H = H; a.I = I; a.S = S; a.M = M; a.n_total = n_experts_total; a.ksplit = 1; a.ch = *ch; a.site = site; a.status = status;
    a.trace_kind = kTrTcMoeL2;
    return launch_tc_moe<true>(mw, mx, a, dim3(H / kBM, M), st);
}

// Wide out-projection: x[m] (+)= all-reduce(W * in[m]) for M rows; planes / descale come from nexrt_oproj_stage_split.
// W [H][K] e4m3 with block scales w_s [H/128][K/128]; zero_ids: M zero int32 words.
int nexrt_tc_oproj_allreduce(const void* planes, const void* descale, const void* w, const void* w_s, void* x, const void* zero_ids, int H, int K, int M,
                             int overwrite, const NexrtLLChannel* ch, unsigned int site, int* status, void* stream) {
    if (M < 1 || M > kMaxRows || H % 128 || K % 128 || K > 8192 || ch == nullptr) return cudaErrorInvalidValue;
    if (ch->world > 1 && ch->slots < static_cast<unsigned int>(kMaxRows) * H) return cudaErrorInvalidValue;
    CUtensorMap mw, mx;
    if (!tensor_map(&mw, w, H, K, K, kBM, false) || !tensor_map(&mx, planes, 3 * M, K, K, kBN, false)) return cudaErrorInvalidValue;
    TcMoeArgs a{};
    a.w_s = static_cast<const float*>(w_s); a.ids = static_cast<const int*>(zero_ids); a.descale = static_cast<const float*>(descale);
    a.x = static_cast<__nv_bfloat16*>(x); a.H = H; a.I = K; a.S = 1; a.M = M; a.n_total = 1; a.ksplit = 1; a.overwrite = overwrite ? 1 : 0;
    a.ch = *ch; a.site = site; a.status = status;
    a.trace_kind = kTrTcRows;
    return launch_tc_moe<true, false, true>(mw, mx, a, dim3(H / kBM, 1), static_cast<cudaStream_t>(stream));
}

}  // extern "C"
