// Mixture-of-experts FFN for 1..8 token rows at any tensor-parallel width.
//
//   moe_router        : post-attention RMSNorm -> bf16 GEMV over E routed experts + the shared
//                       expert gate row -> (last CTA to finish) top-k by packed (value, lowest id)
//                       keys, softmax over the selected logits, sigmoid of the shared gate.
//   moe_l1            : for every (row, selected expert) the gate/up rows of this rank's slice
//                       of the intermediate dimension, silu(g) * u, route weight folded in.
//   moe_l2_allreduce  : down projection summed over the selected experts, in-kernel all-reduce
//                       over the LL channel, residual add.
//
// Replaces the reference's GateGemvRowRawAndRmsCta0Kernel + GateTopKSingleCta…Kernel
// (nex_n2_5_pro/kernels/moe/nex_n2_5_pro_gate_gemv_ctypes.cu:92-323), L1K2PairPacked64…Kernel
// (…l1_pair_ctypes.cu:101-254), FusedL2ReducePushKernel (…fused_l2_reduce_ctypes.cu:100-280) and
// the M=4 / M=8 families (…m4_gate_gemm, m4_gate_topk, m4_l1_foldw, m4_moe_l2, m8_gate_gemm,
// m8_gate_topk, m8_moe_wm16, m8_moe_l2tc).  Softmax over all experts followed by top-k and
// renormalisation (reference moe.py:76-84) equals a softmax over the selected logits, which is
// what the router computes.
#include "api.h"
#include "no_alloc.h"
#include "epilogue.cuh"
#include "gemv.cuh"
#include "gemv_cta.cuh"
#include "mma_gemv.cuh"
#include "ll.cuh"

#include <atomic>

namespace nexrt {

// ---------------------------------------------------------------------------------------------
struct RouterArgs {
    const __nv_bfloat16* x;
    const float* post_ln;
    const __nv_bfloat16* w;   // [E+1][H]; row E is the shared-expert gate
    float* logits;            // [M][E+1]
    int* ids;                 // [M][topk+1]; last entry is E (the shared expert)
    float* wts;               // [M][topk+1]; last entry is sigmoid(shared gate)
    int* ticket;
    int H, E, topk, M;
    float eps;
    float* partial;           // tensor-core form: [4 k-quarters][M][rows_pad]
    int rows_pad;             // rows of w padded to a multiple of 16 (0: not padded)
    uint8_t* planes;          // optional [3M][H] e4m3: the normalised rows split for the tcgen05 expert kernels (CTA m writes row m)
    int no_tail;              // 1: stop after the partial logits; the expert gate/up kernel sums them and selects (moe_l1_mma_kernel)
};

constexpr int kRouterPartialSplit = 2;   // K halves of the partial-logit router (layout [2][M][rows_pad])

// Order-preserving image of an fp32 in u32 (never 0 for a finite value or an infinity), so that an integer max picks the
// largest logit.
__device__ __forceinline__ unsigned int router_key(float f) {
    const unsigned int b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float router_unkey(unsigned int o) { return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o); }

// Top-k of one token row by one warp from logits in shared memory.  Same selection (ties go to the lowest expert id) and the
// same softmax over the selected logits as router_topk below, but built from rank counts over values in shared memory
// instead of rounds of cross-lane reductions: on this GPU a `redux.sync` or a shuffle chain costs on the order of a
// hundred cycles, and ten to thirty of them in a row made the selection the longest phase of the gate/up kernel.
//   A  every lane finds the maximum of its 16 experts (a 4-level tree) and publishes it;
//   B  every lane counts the published maxima above its own (ties ordered by lane): the lane with exactly topk - 1 above
//      it holds T, a lower bound of the topk-th largest logit;
//   C  the experts with logit >= T - a few more than topk - are compacted into shared memory with 16 ballots as 64-bit
//      (key, ~id) words;
//   D  every lane counts, for its one or two candidates, the candidates above them: that count is the final position,
//      and ties resolve to the lowest id because ~id is part of the word;
//   E  the softmax over the selected logits is summed in rank order.
// More than 64 candidates (many equal logits) fall back to rounds over all 16 values per lane.
// ids / wts: [topk + 1] (shared or global); the last entry is the shared expert E with sigmoid(gate logit).  topk <= 31.
struct alignas(16) TopkScratch {      // 16-byte aligned and sized: gmax is read with 128-bit loads from every element of an array
    unsigned long long cand[64];
    unsigned int gmax[32];
    float val[32];
    unsigned int T;
};

__device__ __forceinline__ void router_topk_warp(const float* lg, int E, int topk, int* ids, float* wts, TopkScratch& sc) {
    const int lane = threadIdx.x & 31;
    const unsigned int lt_mask = (1u << lane) - 1u;
    unsigned int key[16];                       // 0 marks an empty entry
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int e = lane + 32 * i;
        key[i] = e < E ? router_key(lg[e]) : 0u;
    }
    unsigned int t8[8], t4[4];
#pragma unroll
    for (int i = 0; i < 8; ++i) t8[i] = max(key[2 * i], key[2 * i + 1]);
#pragma unroll
    for (int i = 0; i < 4; ++i) t4[i] = max(t8[2 * i], t8[2 * i + 1]);
    const unsigned int my = max(max(t4[0], t4[1]), max(t4[2], t4[3]));
    sc.gmax[lane] = my;
    __syncwarp();
    {
        int above = 0;
        const uint4* g4 = reinterpret_cast<const uint4*>(sc.gmax);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint4 v = g4[j];
            above += (v.x > my || (v.x == my && 4 * j < lane)) + (v.y > my || (v.y == my && 4 * j + 1 < lane)) +
                     (v.z > my || (v.z == my && 4 * j + 2 < lane)) + (v.w > my || (v.w == my && 4 * j + 3 < lane));
        }
        if (above == topk - 1) sc.T = my;
    }
    __syncwarp();
    const unsigned int T = sc.T;
    int n = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const bool in = key[i] != 0u && key[i] >= T;
        const unsigned int b = __ballot_sync(0xffffffffu, in);
        const int pos = n + __popc(b & lt_mask);
        if (in && pos < 64) sc.cand[pos] = (static_cast<unsigned long long>(key[i]) << 32) | static_cast<unsigned int>(~(lane + 32 * i));
        n += __popc(b);
    }
    __syncwarp();
    if (n <= 64) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int c = lane + 32 * h;
            if (c < n) {
                const unsigned long long mine = sc.cand[c];
                int above = 0;
                for (int j = 0; j < n; ++j) above += sc.cand[j] > mine ? 1 : 0;
                if (above < topk) {
                    ids[above] = static_cast<int>(~static_cast<unsigned int>(mine));
                    sc.val[above] = router_unkey(static_cast<unsigned int>(mine >> 32));
                }
            }
        }
    } else {
        for (int k = 0; k < topk; ++k) {
            unsigned int lm = 0u;
            int li = 0;
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (key[i] > lm) { lm = key[i]; li = i; }
            const unsigned int gm = redux_max_u32(lm);
            const unsigned int gi = redux_min_u32(lm == gm ? static_cast<unsigned int>(lane + 32 * li) : 0xffffffffu);
#pragma unroll
            for (int i = 0; i < 16; ++i) key[i] = gi == static_cast<unsigned int>(lane + 32 * i) ? 0u : key[i];
            if (lane == 0) { ids[k] = static_cast<int>(gi); sc.val[k] = router_unkey(gm); }
        }
    }
    __syncwarp();
    if (lane < topk) {
        const float top0 = sc.val[0];
        float denom = 0.f;
        for (int j = 0; j < topk; ++j) denom += __expf(sc.val[j] - top0);
        wts[lane] = __expf(sc.val[lane] - top0) / denom;
    } else if (lane == topk) {
        ids[lane] = E;
        wts[lane] = sigmoid_f(lg[E]);
    }
    __syncwarp();
}

// Top-k of every token row by the calling CTA: warp m owns row m, lane holds logits lane,
// lane + 32, ...; ties go to the lowest expert id; weights are a softmax over the selected logits.
// `src` holds the summed logits [M][E+1]: the global array (read through L2) or a shared-memory copy.
template <bool FROM_SMEM = false>
__device__ __forceinline__ void router_topk(const RouterArgs& a, const float* src) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int rows = a.E + 1;
    for (int m = warp; m < a.M; m += nwarps) {
        const float* lg = src + static_cast<size_t>(m) * rows;
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int e = lane + 32 * i;
            v[i] = e < a.E ? (FROM_SMEM ? lg[e] : __ldcg(lg + e)) : -INFINITY;
        }
        float top0 = 0.f, denom = 0.f, mine = 0.f;
        int mine_id = -1;
        for (int k = 0; k < a.topk; ++k) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (v[i] > bv) { bv = v[i]; bi = lane + 32 * i; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (k == 0) top0 = bv;
            const float ex = __expf(bv - top0);
            denom += ex;
            if (lane == k) { mine = ex; mine_id = bi; }
            if ((bi & 31) == lane) {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if (i == (bi >> 5)) v[i] = -INFINITY;
            }
        }
        const int S = a.topk + 1;
        if (lane < a.topk) {
            a.ids[m * S + lane] = mine_id;
            a.wts[m * S + lane] = mine / denom;
        } else if (lane == a.topk) {
            a.ids[m * S + lane] = a.E;
            a.wts[m * S + lane] = sigmoid_f(FROM_SMEM ? lg[a.E] : __ldcg(lg + a.E));
        }
    }
}

template <int MB>
__global__ void __launch_bounds__(512, 1) moe_router_kernel(RouterArgs a) {
    constexpr int U = MB == 1 ? 4 : 2;
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[32];
    __shared__ int s_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int rows = a.E + 1;
    int r0, r1;
    cta_range(rows, blockIdx.x, gridDim.x, &r0, &r1);
    const int nrows = r1 - r0;
    if (nrows) prefetch_l2_range(a.w + static_cast<size_t>(r0) * a.H, static_cast<size_t>(nrows) * a.H * 2);
    const GemvGeom gg = gemv_geom(a.H / 8, blockDim.x);
    float* xs = smem;
    float* part = xs + static_cast<size_t>(MB) * a.H;
    float* gs = part + gemv_part_floats((rows + gridDim.x - 1) / gridDim.x, MB, gg);   // [H] norm multiplier
    GemvCta<MB, U, PlainBf16> gemv(PlainBf16{a.w, a.H}, r0, nrows, a.H);
    gemv.preload();
    for (int i = threadIdx.x; i < a.H; i += blockDim.x) gs[i] = a.post_ln[i];
    pdl_wait();
    pdl_launch_dependents();   // after the wait: see the tensor-core router
    for (int m0 = 0; m0 < a.M; m0 += MB) {
        const int mb = min(MB, a.M - m0);
        if (m0) __syncthreads();
        stage_rmsnorm_plain(xs, a.x + static_cast<size_t>(m0) * a.H, gs, mb, a.H, a.eps, red);
        if (m0 == 0) gemv.run(xs, part);
        else gemv_cta<MB, U>(PlainBf16{a.w, a.H}, r0, nrows, xs, a.H, part);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nrows * mb; idx += blockDim.x) {
            const int rl = idx / mb, m = idx % mb;
            a.logits[static_cast<size_t>(m0 + m) * rows + r0 + rl] = gemv_result(part, rl, m, MB, gg.wpr);
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(a.ticket, 1) == static_cast<int>(gridDim.x) - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    router_topk(a, a.logits);
    if (threadIdx.x == 0) *a.ticket = 0;
}

// ---------------------------------------------------------------------------------------------
struct MoeL1Args {
    const __nv_bfloat16* x;
    const float* post_ln;
    const uint8_t* w13;     // [E+1][2I][H]: gate rows then up rows
    const float* w13_s;     // [E+1][2I/128][H/128]
    const int* ids;         // [M][S]
    float* gu;              // [M][S][2I] raw gate | up projections
    int H, I, S, M;
    float eps;
    int shared_expert;      // index whose weights may be prefetched before the dependency wait
    // routed form (tensor-core kernel only): the router left K-quarter partial logits and this kernel selects the experts
    const float* partial;   // [4][M][rows_pad] or null (ids come from memory)
    int rows_pad, E, topk;
    int* ids_out;           // [M][S]   written by CTA 0 for the down projection
    float* wts_out;         // [M][S]
    float* logits_out;      // [M][E+1] summed logits (inspection, tests)
    const uint8_t* w2;      // [E+1][H][I]: the selected experts' down weights are pulled towards L2 once the ids are known
    const void* pf;         // a later kernel's constant weights to pull towards L2 before the dependency wait (or null)
    unsigned long long pf_bytes;
};

__global__ void __launch_bounds__(512, 1) moe_l1_kernel(MoeL1Args a) {
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[32];
    __shared__ int s_ids[16];
    pdl_launch_dependents();
    const int I2 = 2 * a.I, vrows = a.S * I2;
    int v0, v1;
    cta_range(vrows, blockIdx.x, gridDim.x, &v0, &v1);
    const int nrows = v1 - v0;
    const size_t expert_bytes = static_cast<size_t>(I2) * a.H;
    {   // the shared expert (last slot) is known before routing: pull this CTA's rows of it towards L2
        const int s0 = max(v0, (a.S - 1) * I2), s1 = v1;
        if (s1 > s0) prefetch_l2_range(a.w13 + a.shared_expert * expert_bytes + static_cast<size_t>(s0 - (a.S - 1) * I2) * a.H,
                                       static_cast<size_t>(s1 - s0) * a.H);
    }
    const GemvGeom gg = gemv_geom(a.H / 16, blockDim.x);
    float* xs = smem;                 // [H]
    float* part = xs + a.H;
    float* gs = part + gemv_part_floats((vrows + gridDim.x - 1) / gridDim.x, 1, gg);   // [H] norm multiplier
    for (int i = threadIdx.x; i < a.H; i += blockDim.x) gs[i] = a.post_ln[i];
    pdl_wait();
    for (int m = 0; m < a.M; ++m) {
        if (m) __syncthreads();
        if (threadIdx.x < a.S) s_ids[threadIdx.x] = a.ids[m * a.S + threadIdx.x];
        stage_rmsnorm_plain(xs, a.x + static_cast<size_t>(m) * a.H, gs, 1, a.H, a.eps, red);
        gemv_cta<1, 8>(ExpertUp{a.w13, a.w13_s, s_ids, a.H, I2}, v0, nrows, xs, a.H, part);
        __syncthreads();
        for (int rl = threadIdx.x; rl < nrows; rl += blockDim.x)
            a.gu[static_cast<size_t>(m) * vrows + v0 + rl] = gemv_result(part, rl, 0, 1, gg.wpr);
    }
}

// ---------------------------------------------------------------------------------------------
struct MoeL2Args {
    const float* gu;        // [M][S][2I] raw gate | up projections
    const int* ids;         // [M][S]
    const float* wts;       // [M][S] route weights (shared-expert gate last)
    const uint8_t* w2;      // [E+1][H][I]
    const float* w2_s;      // [E+1][H/128][I/128]
    __nv_bfloat16* x;
    int H, I, S, M;
    LLChannel ch;
    unsigned int site;
    float* partial_out;     // library-baseline arm: fp32 partial sums go here, no exchange, no residual
};

__global__ void __launch_bounds__(512, 1) moe_l2_allreduce_kernel(MoeL2Args a) {
    extern __shared__ __align__(16) float smem[];
    __shared__ int s_ids[16];
    pdl_launch_dependents();
    int row0, row1;
    cta_range(a.H, blockIdx.x, gridDim.x, &row0, &row1);
    const int nrows = row1 - row0, max_rows = (a.H + gridDim.x - 1) / gridDim.x;
    const int VK = a.S * a.I;
    const GemvGeom gg = gemv_geom(VK / 16, blockDim.x);
    float* hs = smem;                                        // [VK]
    float* part = hs + VK;
    float* res = part + gemv_part_floats(max_rows, 1, gg);   // [kMaxRows][nrows]
    pdl_wait();
    for (int m = 0; m < a.M; ++m) {
        if (m) __syncthreads();
        // h = silu(gate) * up * route weight
        for (int k = threadIdx.x; k < VK; k += blockDim.x) {
            const int sl = k / a.I, i = k % a.I;
            const float* g = a.gu + (static_cast<size_t>(m) * a.S + sl) * 2 * a.I;
            hs[k] = silu_f(g[i]) * g[a.I + i] * a.wts[m * a.S + sl];
        }
        if (threadIdx.x < a.S) s_ids[threadIdx.x] = a.ids[m * a.S + threadIdx.x];
        __syncthreads();
        gemv_cta<1, 8>(ExpertDown{a.w2, a.w2_s, s_ids, a.H, a.I}, row0, nrows, hs, VK, part);
        __syncthreads();
        for (int rl = threadIdx.x; rl < nrows; rl += blockDim.x) res[m * nrows + rl] = gemv_result(part, rl, 0, 1, gg.wpr);
    }
    __syncthreads();
    allreduce_residual(a.ch, a.site, res, a.M, row0, nrows, a.H, a.x, true, a.partial_out);
}

// Router on the tensor cores: bf16 weights [rows_pad][H], one CTA per (16 rows, quarter of K), the
// 8 warps split the quarter; the CTA that takes the last ticket adds the four quarters in a
// fixed order and selects the experts.
// KQ: CTAs that share the reduction dimension of one 16-row group (4: 132 CTAs of 4 windows per warp; 2: 66 CTAs of 8
// windows per warp, the form of the routed one-row step, whose small grid leaves SM slots for the gate/up kernel that
// follows to become resident - and preload - while this one runs).
template <int MP, int KQ = 4>
__global__ void __launch_bounds__(256, 2) moe_router_mma_kernel(RouterArgs a) {
    constexpr int NB = 16 / KQ, KS = 8;
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[32];
    __shared__ int s_last;
    TraceCta tr;
    tr.begin(kTrRouter);
    const int warp = threadIdx.x >> 5;
    const int rg = blockIdx.x / KQ, kq = blockIdx.x % KQ, rows = a.E + 1;
    const int nq = a.H / 32 / KQ;                                       // 64-byte windows per quarter
    float* xs = smem;                                                   // [MP][H]
    float* tiles = xs + static_cast<size_t>(MP) * a.H;                  // [KS][16][8]
    __nv_bfloat16* xh = reinterpret_cast<__nv_bfloat16*>(tiles + KS * 128);   // [MP*2][H]
    MmaWarpBf16<NB> mw(a.w, a.H, rg * kRowsPerGroup, kq * nq + warp, KS, (kq + 1) * nq);
    mw.preload();
    RowNorm<4> norm;
    norm.preload_gamma(a.post_ln, a.H);
    pdl_wait();
    tr.mark(1);
    // Released only now: the expert gate/up kernel that follows normalises x (complete since the wait above)
    // before ITS dependency wait, which is safe only if it cannot start before x is final.
    pdl_launch_dependents();
    for (int m0 = 0; m0 < a.M; m0 += MP) {
        const int mb = min(MP, a.M - m0);
        if (m0) { __syncthreads(); mw.next_pass(); }
        norm.template run<3>(nullptr, xs, a.x + static_cast<size_t>(m0) * a.H, mb, a.H, a.eps, red);
        // the expert kernels of a multi-row step take the same normalised rows as three e4m3 planes: the CTA whose index
        // is the row's (modulo the grid: a router of few experts has fewer CTAs than the step has rows) writes them,
        // which saves them a kernel of their own
        if (a.planes != nullptr) {
            for (int m = 0; m < mb; ++m)
                if ((m0 + m) % static_cast<int>(gridDim.x) == static_cast<int>(blockIdx.x))
                    split_rows<3>(a.planes + static_cast<size_t>(m0 + m) * 3 * a.H, xs + static_cast<size_t>(m) * a.H, 1, a.H, kSplitScale);
        }
        split_bf16_rows(xh, xs, mb, a.H);
        float d[4];
        mw.run(xh, mb * 2, d);
        mw.store(tiles + warp * 128, d);
        __syncthreads();
        if (threadIdx.x < kRowsPerGroup * mb) {
            const int rl = threadIdx.x % kRowsPerGroup, m = threadIdx.x / kRowsPerGroup;
            a.partial[(static_cast<size_t>(kq) * a.M + m0 + m) * a.rows_pad + rg * kRowsPerGroup + rl] = mma_bf16_result(tiles, KS, rl, m);
        }
    }
    tr.mark(2);
    if (a.no_tail) { tr.mark(3); return; }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(a.ticket, 1) == static_cast<int>(gridDim.x) - 1);
    __syncthreads();
    if (!s_last) { tr.mark(3); return; }
    __threadfence();
    // sum the K quarters in a fixed order into shared memory (the scratch of the GEMV phase is free now);
    // three logits per thread are in flight together, so M = 1 needs one round trip to L2
    float* lg_s = smem;
    for (int idx0 = threadIdx.x; idx0 < a.M * rows; idx0 += 3 * blockDim.x) {
        float v[3][KQ];
#pragma unroll
        for (int u = 0; u < 3; ++u) {
            const int idx = idx0 + u * blockDim.x;
            const int m = idx / rows, e = idx % rows;
#pragma unroll
            for (int q = 0; q < KQ; ++q)
                v[u][q] = idx < a.M * rows ? __ldcg(a.partial + (static_cast<size_t>(q) * a.M + m) * a.rows_pad + e) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 3; ++u) {
            const int idx = idx0 + u * blockDim.x;
            if (idx < a.M * rows) {
                const float t = ((v[u][0] + v[u][1]) + v[u][2]) + v[u][3];
                lg_s[idx] = t;
                a.logits[idx] = t;
            }
        }
    }
    __syncthreads();
    router_topk<true>(a, lg_s);
    if (threadIdx.x == 0) *a.ticket = 0;
    tr.mark(3);
}

// Top-k stage of the wide router (multi-row steps): the logits arrive as K-split partial planes
// partial[ks][m][rows_pad] from the tcgen05 rows GEMM; they are added in a fixed order into shared memory, kept
// in a.logits for inspection, and selected exactly like the fused router does.
__global__ void __launch_bounds__(256) moe_topk_rows_kernel(RouterArgs a, int ksplit, int rpc) {
    extern __shared__ __align__(16) float lg_s[];
    __shared__ TopkScratch s_topk[8];
    TraceCta tr;
    tr.begin(kTrHelper);
    pdl_launch_dependents();
    pdl_wait();
    tr.mark(1);
    const int rows = a.E + 1;
    // one CTA per block of rpc token rows (one row per CTA in a decode step; a prefill chunk packs a few rows per CTA)
    const int m0 = blockIdx.x * rpc, mb = min(rpc, a.M - m0);
    // four consecutive experts per thread, every K-split plane of them requested before the first add (16-byte
    // loads, all in flight): the sum is one or two round trips to L2
    const int quads = a.rows_pad / 4;
    for (int q = threadIdx.x; q < mb * quads; q += blockDim.x) {
        const int m = q / quads, e0 = (q % quads) * 4;
        float4 v[16];
#pragma unroll
        for (int ks = 0; ks < 16; ++ks)
            v[ks] = ks < ksplit ? __ldcg(reinterpret_cast<const float4*>(a.partial + (static_cast<size_t>(ks) * a.M + m0 + m) * a.rows_pad + e0))
                                : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 t = v[0];
#pragma unroll
        for (int ks = 1; ks < 16; ++ks)
            if (ks < ksplit) { t.x += v[ks].x; t.y += v[ks].y; t.z += v[ks].z; t.w += v[ks].w; }
        const float tv[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (e0 + i < rows) {
                lg_s[m * rows + e0 + i] = tv[i];
                a.logits[(m0 + m) * rows + e0 + i] = tv[i];
            }
    }
    __syncthreads();
    const int S = a.topk + 1;
    for (int m = threadIdx.x >> 5; m < mb; m += blockDim.x >> 5)
        router_topk_warp(lg_s + static_cast<size_t>(m) * rows, a.E, a.topk, a.ids + static_cast<size_t>(m0 + m) * S, a.wts + static_cast<size_t>(m0 + m) * S,
                         s_topk[threadIdx.x >> 5]);
    __syncthreads();
    tr.mark(3);
}

// ---- tensor-core forms (see mma_gemv.cuh) ------------------------------------------------------
// Expert gate/up: one CTA per 16 virtual rows (slot, i), the 8 warps split K = H.
template <bool LOOP>      // LOOP: the grid is capped and a CTA walks several groups of 16 virtual rows (see gdn_front_mma_kernel)
__global__ void __launch_bounds__(256, 2) moe_l1_mma_kernel(MoeL1Args a) {
    constexpr int TERMS = 3, NB = 8, KS = 8, KQ = kRouterPartialSplit;
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[32];
    __shared__ int s_ids[16];
    __shared__ int s_ids_all[kMaxRows][16];
    __shared__ float s_wts_all[kMaxRows][16];
    __shared__ TopkScratch s_topk[KS];
    TraceCta tr;
    tr.begin(kTrMoeL1);
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5;
    const int I2 = 2 * a.I, vrows = a.S * I2;
    const int v0 = blockIdx.x * kRowsPerGroup, nwin = a.H / kWin;
    float* tiles = smem;                                             // [KS][16][8]
    uint8_t* xq = reinterpret_cast<uint8_t*>(tiles + KS * 128);      // [TERMS][H]
    float* lg_s = reinterpret_cast<float*>(xq + static_cast<size_t>(TERMS) * a.H);   // routed form: [M][E + 1]
    const bool shared_rows = v0 >= (a.S - 1) * I2;                   // the shared expert is known before routing
    if (threadIdx.x == 0) s_ids[a.S - 1] = a.shared_expert;
    __syncthreads();
    const MmaExpertUp src{a.w13, a.w13_s, s_ids, a.H, I2};
    MmaWarp<NB, MmaExpertUp> mw(v0, warp, KS, nwin);
    if (shared_rows) mw.preload(src);
    RowNorm<4> norm;
    norm.preload_gamma(a.post_ln, a.H);
    // idle until the router is done: warm L2 with the constant weights of a kernel further down the step
    prefetch_l2_slice(a.pf, a.pf_bytes, blockIdx.x, gridDim.x);
    tr.mark(4);
    // x was finished two kernels back (out-projection + all-reduce); the router, this grid's direct predecessor,
    // releases its dependents only after its own dependency wait, so x is complete and in L2 by now: row 0 is
    // normalised and split while the router is still working, only the expert ids need the wait.
    norm.template run<TERMS, true>(xq, nullptr, a.x, 1, a.H, a.eps, red);
    tr.mark(2);
    pdl_wait();
    tr.mark(1);
    if (a.partial != nullptr) {
        // the router stopped at its K-quarter partials: add them in a fixed order (every load of a thread in flight
        // together) and select the experts here, in every CTA alike; CTA 0 leaves ids / weights / logits for the rest
        const int rows = a.E + 1, total = a.M * rows;
        for (int idx0 = threadIdx.x; idx0 < total; idx0 += 3 * blockDim.x) {
            float v[3][KQ];
#pragma unroll
            for (int u = 0; u < 3; ++u) {
                const int idx = idx0 + u * blockDim.x, m = idx / rows, e = idx % rows;
#pragma unroll
                for (int q = 0; q < KQ; ++q)
                    v[u][q] = idx < total ? __ldcg(a.partial + (static_cast<size_t>(q) * a.M + m) * a.rows_pad + e) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 3; ++u) {
                const int idx = idx0 + u * blockDim.x;
                if (idx < total) {
                    float t = v[u][0];
#pragma unroll
                    for (int q = 1; q < KQ; ++q) t += v[u][q];
                    lg_s[idx] = t;
                    if (blockIdx.x == 0 && a.logits_out != nullptr) a.logits_out[idx] = t;
                }
            }
        }
        __syncthreads();
        tr.mark(5);
        for (int m = warp; m < a.M; m += KS) router_topk_warp(lg_s + static_cast<size_t>(m) * rows, a.E, a.topk, s_ids_all[m], s_wts_all[m], s_topk[warp]);
        __syncthreads();
        tr.mark(6);
        if (blockIdx.x == 0 && threadIdx.x < a.M * a.S) {
            const int m = threadIdx.x / a.S, sl = threadIdx.x % a.S;
            a.ids_out[threadIdx.x] = s_ids_all[m][sl];
            a.wts_out[threadIdx.x] = s_wts_all[m][sl];
        }
    }
    for (int m = 0; m < a.M; ++m) {
        if (m) { __syncthreads(); mw.preloaded = false; }
        if (threadIdx.x < a.S) s_ids[threadIdx.x] = a.partial != nullptr ? s_ids_all[m][threadIdx.x] : a.ids[m * a.S + threadIdx.x];
        if (m) norm.template run<TERMS>(xq, nullptr, a.x + static_cast<size_t>(m) * a.H, 1, a.H, a.eps, red);
        else __syncthreads();
        if (m == 0 && !shared_rows) mw.preload(src);                 // own gate/up rows first ...
        if (m == 0 && a.w2 != nullptr && a.M == 1) {
            // ... then the down weights of the selected experts towards L2 for the kernel that follows: one line per
            // thread of the S x H x I bytes
            const size_t per_expert = static_cast<size_t>(a.H) * a.I >> 7, lines = per_expert * a.S;
            const size_t per = (lines + gridDim.x - 1) / gridDim.x, lo = blockIdx.x * per, hi = lo + per < lines ? lo + per : lines;
            for (size_t l = lo + threadIdx.x; l < hi; l += blockDim.x) {
                const size_t sl = l / per_expert, off = l % per_expert;
                prefetch_l2(a.w2 + (static_cast<size_t>(s_ids[sl]) * per_expert + off) * 128);
            }
        }
        float d[1][4];
        mw.template run<1>(src, xq, a.H, TERMS, d);
        mw.template store<1>(tiles + warp * 128, d);
        __syncthreads();
        tr.mark(7);
        if (threadIdx.x < kRowsPerGroup)
            a.gu[static_cast<size_t>(m) * vrows + v0 + threadIdx.x] = mma_result<TERMS, 1>(tiles, KS, threadIdx.x, 0, kSplitDescale);
    }
    // One-row steps on wide shards: the grid is capped at the CTAs the machine holds at once; a CTA walks its further
    // groups of 16 virtual rows here.  The row was normalised and the experts selected once per CTA; only the weight
    // stream repeats.
    if (LOOP && a.M == 1) {
        for (int vg = v0 + static_cast<int>(gridDim.x) * kRowsPerGroup; vg < vrows; vg += static_cast<int>(gridDim.x) * kRowsPerGroup) {
            __syncthreads();
            mw.row0 = vg;
            mw.preloaded = false;
            float d[1][4];
            mw.template run<1>(src, xq, a.H, TERMS, d);
            mw.template store<1>(tiles + warp * 128, d);
            __syncthreads();
            if (threadIdx.x < kRowsPerGroup) a.gu[vg + threadIdx.x] = mma_result<TERMS, 1>(tiles, KS, threadIdx.x, 0, kSplitDescale);
        }
    }
    tr.mark(3);
}

// Expert down + all-reduce + residual: one CTA per 16 output rows, warps split the virtual K = S x I.
__global__ void __launch_bounds__(256, 2) moe_l2_allreduce_mma_kernel(MoeL2Args a) {
    constexpr int TERMS = 3, NB = 4;
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[32];
    __shared__ float descale[1];
    __shared__ int s_ids[16];
    TraceCta tr;
    tr.begin(kTrMoeL2);
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int row0 = blockIdx.x * kRowsPerGroup;
    const int VK = a.S * a.I, nwin = VK / kWin;
    const int KS = min(nwarps, nwin);
    float* hs = smem;                                                // [VK]
    float* tiles = hs + VK;                                          // [8][16][8]
    float* res = tiles + 8 * 128;                                    // [kMaxRows][16]
    uint8_t* xq = reinterpret_cast<uint8_t*>(res + kMaxRows * kRowsPerGroup);   // [TERMS][VK]
    const MmaExpertDown src{a.w2, a.w2_s, s_ids, a.H, a.I};
    pdl_wait();
    tr.mark(1);
    for (int m = 0; m < a.M; ++m) {
        if (m) __syncthreads();
        if (threadIdx.x < a.S) s_ids[threadIdx.x] = a.ids[m * a.S + threadIdx.x];
        __syncthreads();
        MmaWarp<NB, MmaExpertDown> mw(row0, warp, KS, warp < KS ? nwin : 0);
        mw.preload(src);                                             // weights stream while h is being built
        // h = silu(gate) * up * route weight
#pragma unroll 2
        for (int k = threadIdx.x * 4; k < VK; k += blockDim.x * 4) {
            const int sl = k / a.I, i = k % a.I;
            const float* g = a.gu + (static_cast<size_t>(m) * a.S + sl) * 2 * a.I;
            const float4 gt = *reinterpret_cast<const float4*>(g + i), up = *reinterpret_cast<const float4*>(g + a.I + i);
            const float wt = a.wts[m * a.S + sl];
            *reinterpret_cast<float4*>(hs + k) =
                make_float4(silu_f(gt.x) * up.x * wt, silu_f(gt.y) * up.y * wt, silu_f(gt.z) * up.z * wt, silu_f(gt.w) * up.w * wt);
        }
        __syncthreads();
        tr.mark(4);
        act_split<TERMS>(xq, hs, 1, VK, red, descale);
        tr.mark(5);
        float d[1][4];
        mw.template run<1>(src, xq, VK, TERMS, d);
        tr.mark(6);
        if (warp < KS) mw.template store<1>(tiles + warp * 128, d);
        __syncthreads();
        if (threadIdx.x < kRowsPerGroup) res[m * kRowsPerGroup + threadIdx.x] = mma_result<TERMS, 1>(tiles, KS, threadIdx.x, 0, descale[0]);
    }
    __syncthreads();
    tr.mark(2);
    allreduce_residual(a.ch, a.site, res, a.M, row0, kRowsPerGroup, a.H, a.x, true, a.partial_out);
    tr.mark(3);
}

}  // namespace nexrt

using namespace nexrt;

extern "C" int nexrt_moe_router(const void* x, const void* post_ln, const void* w, void* logits, void* ids, void* wts, void* ticket,
                                void* partial, int rows_pad, int H, int E, int topk, int M, float eps, int n_cta, void* planes, void* stream) {
    if (M < 1 || M > kMaxRows || H % 256 || E > 512 || topk < 1 || topk > 31 || topk > E) return cudaErrorInvalidValue;
    RouterArgs a{static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(post_ln), static_cast<const __nv_bfloat16*>(w),
                 static_cast<float*>(logits), static_cast<int*>(ids), static_cast<float*>(wts), static_cast<int*>(ticket), H, E, topk, M, eps,
                 static_cast<float*>(partial), rows_pad, static_cast<uint8_t*>(planes)};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if ((gemv_mode() & 16) && partial != nullptr && rows_pad >= E + 1 && rows_pad % 16 == 0 && H % 1024 == 0 && H <= 4096) {
        const int mp = M == 1 ? 1 : (M == 2 ? 2 : 4);
        const size_t smem_mma = sizeof(float) * (static_cast<size_t>(mp) * H + 8 * 128) + sizeof(__nv_bfloat16) * static_cast<size_t>(mp) * 2 * H;
        dim3 g(rows_pad / 16 * 4), b(256);
        if (mp == 1) return launch(moe_router_mma_kernel<1>, g, b, smem_mma, st, a);
        if (mp == 2) return launch(moe_router_mma_kernel<2>, g, b, smem_mma, st, a);
        return launch(moe_router_mma_kernel<4>, g, b, smem_mma, st, a);
    }
    if (planes != nullptr) return cudaErrorInvalidValue;   // only the tensor-core router writes the planes
    const int mb = M == 1 ? 1 : 4;
    const size_t smem = sizeof(float) * (static_cast<size_t>(mb + 1) * H + gemv_part_floats((E + 1 + n_cta - 1) / n_cta, mb, gemv_geom(H / 8, gemv_threads())));
    if (M == 1) return launch(moe_router_kernel<1>, dim3(n_cta), dim3(gemv_threads()), smem, st, a);
    return launch(moe_router_kernel<4>, dim3(n_cta), dim3(gemv_threads()), smem, st, a);
}

extern "C" int nexrt_moe_router_topk(const void* partial, int ksplit, int rows_pad, void* logits, void* ids, void* wts, int E, int topk, int M, void* stream) {
    if (M < 1 || M > 1024 || E > 512 || topk < 1 || topk > 31 || topk > E || ksplit < 1 || ksplit > 16 || rows_pad % 4) return cudaErrorInvalidValue;
    RouterArgs a{nullptr, nullptr, nullptr, static_cast<float*>(logits), static_cast<int*>(ids), static_cast<float*>(wts), nullptr, 0, E, topk, M, 0.f,
                 const_cast<float*>(static_cast<const float*>(partial)), rows_pad, nullptr};
    const int rpc = M <= kMaxRows ? 1 : 2;   // a decode step: one CTA per token row (the rows' partial sums and selections run side by side); prefill chunks: two rows per CTA
    return launch(moe_topk_rows_kernel, dim3((M + rpc - 1) / rpc), dim3(256), sizeof(float) * rpc * (E + 1), static_cast<cudaStream_t>(stream), a, ksplit, rpc);
}

extern "C" int nexrt_moe_l1(const void* x, const void* post_ln, const void* w13, const void* w13_s, const void* ids, void* gu, int H, int I,
                            int S, int M, float eps, int shared_expert, int n_cta, void* stream) {
    if (M < 1 || M > kMaxRows || H % 256 || I % 128 || S > 16) return cudaErrorInvalidValue;
    MoeL1Args a{};
    a.x = static_cast<const __nv_bfloat16*>(x); a.post_ln = static_cast<const float*>(post_ln); a.w13 = static_cast<const uint8_t*>(w13);
    a.w13_s = static_cast<const float*>(w13_s); a.ids = static_cast<const int*>(ids); a.gu = static_cast<float*>(gu);
    a.H = H; a.I = I; a.S = S; a.M = M; a.eps = eps; a.shared_expert = shared_expert;
    const int vrows = S * 2 * I;
    if ((gemv_mode() & 4) && H % 512 == 0 && H <= 4096) {
        const size_t smem_mma = sizeof(float) * 8 * 128 + static_cast<size_t>(3) * H;
        return (M == 1 && vrows / 16 > 2 * sm_count()) ? launch(moe_l1_mma_kernel<true>, dim3(2 * sm_count()), dim3(256), smem_mma, static_cast<cudaStream_t>(stream), a)
                                                 : launch(moe_l1_mma_kernel<false>, dim3(vrows / 16), dim3(256), smem_mma, static_cast<cudaStream_t>(stream), a);
    }
    const size_t smem = sizeof(float) * (static_cast<size_t>(2) * H + gemv_part_floats((vrows + n_cta - 1) / n_cta, 1, gemv_geom(H / 16, gemv_threads())));
    return launch(moe_l1_kernel, dim3(n_cta), dim3(gemv_threads()), smem, static_cast<cudaStream_t>(stream), a);
}

extern "C" int nexrt_moe_router_partial_split(void) { return nexrt::kRouterPartialSplit; }

// Routed pair of the one-row step: the router stops at its K-quarter partial logits (no ticket, no tail by one CTA) and
// the gate/up kernel - every CTA alike - adds them, selects the experts on the warp-reduce unit and goes straight on to
// its weight rows; its CTA 0 leaves ids / wts / logits in memory for the down projection.  While it waits for the
// router it pulls [pf, pf + pf_bytes) towards L2 (constant weights of a later kernel), and once the ids are known the
// selected experts' down weights (w2, may be null).
extern "C" int nexrt_moe_router_partial(const void* x, const void* post_ln, const void* w, void* partial, int rows_pad, int H, int E, int topk, int M,
                                        float eps, void* planes, void* stream) {
    if (M < 1 || M > kMaxRows || E > 512 || topk < 1 || topk > 31 || topk > E || partial == nullptr || rows_pad < E + 1 || rows_pad % 16 ||
        H % 1024 || H > 4096)
        return cudaErrorInvalidValue;
    RouterArgs a{};
    a.x = static_cast<const __nv_bfloat16*>(x); a.post_ln = static_cast<const float*>(post_ln); a.w = static_cast<const __nv_bfloat16*>(w);
    a.H = H; a.E = E; a.topk = topk; a.M = M; a.eps = eps; a.partial = static_cast<float*>(partial); a.rows_pad = rows_pad; a.no_tail = 1;
    a.planes = static_cast<uint8_t*>(planes);   // optional: the rows' e4m3 planes for the tcgen05 expert kernels (CTA m writes row m)
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int mp = M == 1 ? 1 : (M == 2 ? 2 : 4);
    const size_t smem_mma = sizeof(float) * (static_cast<size_t>(mp) * H + 8 * 128) + sizeof(__nv_bfloat16) * static_cast<size_t>(mp) * 2 * H;
    dim3 g(rows_pad / 16 * kRouterPartialSplit), b(256);
    if (mp == 1) return launch(moe_router_mma_kernel<1, kRouterPartialSplit>, g, b, smem_mma, st, a);
    if (mp == 2) return launch(moe_router_mma_kernel<2, kRouterPartialSplit>, g, b, smem_mma, st, a);
    return launch(moe_router_mma_kernel<4, kRouterPartialSplit>, g, b, smem_mma, st, a);
}

extern "C" int nexrt_moe_l1_routed(const void* x, const void* post_ln, const void* w13, const void* w13_s, const void* partial, int rows_pad, void* ids_out,
                                   void* wts_out, void* logits_out, void* gu, const void* w2, const void* pf, unsigned long long pf_bytes, int H, int I,
                                   int E, int topk, int M, float eps, void* stream) {
    const int S = topk + 1;
    if (M < 1 || M > kMaxRows || H % 512 || H > 4096 || I % 128 || S > 16 || E > 512 || topk < 1 || topk > E || partial == nullptr ||
        rows_pad < E + 1 || ids_out == nullptr || wts_out == nullptr)
        return cudaErrorInvalidValue;
    MoeL1Args a{};
    a.x = static_cast<const __nv_bfloat16*>(x); a.post_ln = static_cast<const float*>(post_ln); a.w13 = static_cast<const uint8_t*>(w13);
    a.w13_s = static_cast<const float*>(w13_s); a.gu = static_cast<float*>(gu);
    a.H = H; a.I = I; a.S = S; a.M = M; a.eps = eps; a.shared_expert = E;
    a.partial = static_cast<const float*>(partial); a.rows_pad = rows_pad; a.E = E; a.topk = topk;
    a.ids_out = static_cast<int*>(ids_out); a.wts_out = static_cast<float*>(wts_out); a.logits_out = static_cast<float*>(logits_out);
    a.w2 = static_cast<const uint8_t*>(w2); a.pf = pf; a.pf_bytes = pf_bytes;
    const int vrows = S * 2 * I;
    const size_t smem_mma = sizeof(float) * 8 * 128 + static_cast<size_t>(3) * H + sizeof(float) * static_cast<size_t>(M) * (E + 1);
    return (M == 1 && vrows / 16 > 2 * sm_count()) ? launch(moe_l1_mma_kernel<true>, dim3(2 * sm_count()), dim3(256), smem_mma, static_cast<cudaStream_t>(stream), a)
                                                 : launch(moe_l1_mma_kernel<false>, dim3(vrows / 16), dim3(256), smem_mma, static_cast<cudaStream_t>(stream), a);
}

extern "C" int nexrt_moe_l2_allreduce(const void* gu, const void* ids, const void* wts, const void* w2, const void* w2_s, void* x, int H, int I,
                                      int S, int M, const NexrtLLChannel* ch, unsigned int site, int n_cta, void* stream) {
    if (M < 1 || M > kMaxRows || I % 128 || S > 16 || ch == nullptr) return cudaErrorInvalidValue;
    if (ch->world > 1 && ch->slots < static_cast<unsigned int>(kMaxRows) * H) return cudaErrorInvalidValue;
    MoeL2Args a{};
    a.gu = static_cast<const float*>(gu); a.ids = static_cast<const int*>(ids); a.wts = static_cast<const float*>(wts);
    a.w2 = static_cast<const uint8_t*>(w2); a.w2_s = static_cast<const float*>(w2_s); a.x = static_cast<__nv_bfloat16*>(x);
    a.H = H; a.I = I; a.S = S; a.M = M; a.ch = *ch; a.site = site;
    a.partial_out = partial_out_buffer();
    if ((gemv_mode() & 8) && H % 16 == 0) {
        const size_t VK = static_cast<size_t>(S) * I;
        const size_t smem_mma = sizeof(float) * (VK + 8 * 128 + kMaxRows * 16) + 3 * VK;
        return launch(moe_l2_allreduce_mma_kernel, dim3(H / 16), dim3(256), smem_mma, static_cast<cudaStream_t>(stream), a);
    }
    const int max_rows = (H + n_cta - 1) / n_cta;
    const size_t smem = sizeof(float) * (static_cast<size_t>(S) * I + gemv_part_floats(max_rows, 1, gemv_geom(S * I / 16, gemv_threads())) +
                                         static_cast<size_t>(kMaxRows) * max_rows);
    return launch(moe_l2_allreduce_kernel, dim3(n_cta), dim3(gemv_threads()), smem, static_cast<cudaStream_t>(stream), a);
}

// ---- allocation-free router entry point (see no_alloc.h) ------------------------------------------
namespace {
constexpr size_t kNoAllocPartial = 4ull * NEXRT_ROUTER_NOALLOC_MAX_ROWS * NEXRT_ROUTER_NOALLOC_MAX_EXPERT_ROWS;   // floats
constexpr size_t kNoAllocLogits = static_cast<size_t>(NEXRT_ROUTER_NOALLOC_MAX_ROWS) * NEXRT_ROUTER_NOALLOC_MAX_EXPERT_ROWS;
constexpr size_t kNoAllocFloats = kNoAllocPartial + kNoAllocLogits + 64;   // + the ticket word (own 256-byte line)
}  // namespace

// Scratch of the allocation-free router: partial logits | logits | ticket.  In host code this name
// is only a stand-in for the symbol; the device address is obtained with cudaGetSymbolAddress.
static __device__ __align__(256) float g_router_noalloc_scratch[kNoAllocFloats];

extern "C" int nexrt_moe_router_noalloc(const void* x, const void* post_ln, const void* w, void* ids, void* wts, int rows_pad, int H, int E,
                                        int topk, int M, float eps, void* stream) {
    if (M < 1 || M > NEXRT_ROUTER_NOALLOC_MAX_ROWS || rows_pad > NEXRT_ROUTER_NOALLOC_MAX_EXPERT_ROWS || rows_pad % 16 || rows_pad < E + 1 ||
        H % 1024 || H > 4096 || E > 512 || topk < 1 || topk > 31 || topk > E)
        return cudaErrorInvalidValue;
    // one address per device, looked up on the first call made with that device current
    static std::atomic<float*> scratch_of_device[64];   // zero-initialised; every writer of a slot stores the same address
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    float* base = scratch_of_device[dev].load(std::memory_order_acquire);
    if (base == nullptr) {
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&base), g_router_noalloc_scratch);
        if (e != cudaSuccess) return static_cast<int>(e);
        scratch_of_device[dev].store(base, std::memory_order_release);
    }
    float* partial = base;
    float* logits = base + kNoAllocPartial;
    int* ticket = reinterpret_cast<int*>(base + kNoAllocPartial + kNoAllocLogits);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    e = cudaMemsetAsync(ticket, 0, sizeof(int), st);      // the ticket must start at zero whatever the last call left
    if (e != cudaSuccess) return static_cast<int>(e);
    RouterArgs a{static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(post_ln), static_cast<const __nv_bfloat16*>(w), logits,
                 static_cast<int*>(ids), static_cast<float*>(wts), ticket, H, E, topk, M, eps, partial, rows_pad, nullptr};
    const int mp = M == 1 ? 1 : (M == 2 ? 2 : 4);
    const size_t smem_mma = sizeof(float) * (static_cast<size_t>(mp) * H + 8 * 128) + sizeof(__nv_bfloat16) * static_cast<size_t>(mp) * 2 * H;
    dim3 g(rows_pad / 16 * 4), b(256);
    if (mp == 1) return launch(moe_router_mma_kernel<1>, g, b, smem_mma, st, a);
    if (mp == 2) return launch(moe_router_mma_kernel<2>, g, b, smem_mma, st, a);
    return launch(moe_router_mma_kernel<4>, g, b, smem_mma, st, a);
}
