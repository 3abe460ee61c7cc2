// Gated full attention for 1..8 token rows: projection front and split-KV decode.
//
//   attn_front  : input RMSNorm -> block-scaled FP8 GEMV of the (query|gate) per head, k and v
//                 rows; v is appended to the bf16 cache at positions C..C+M-1.
//   attn_decode : per-head q/k RMSNorm (1+w) + partial NeoX RoPE in the prologue, append of the
//                 new k rows, split-KV online-softmax decode with a staircase causal mask over the
//                 M rows, and an in-kernel combine by the last CTA to finish (ticket), which
//                 also applies ctx * sigmoid(gate).
//
// One pair of kernels replaces the reference's QkvGroupSplitKKernel + NormRopeFusedKernel +
// wgmma_fd4_mega (nex_n2_5_pro/kernels/full_attn/nex_n2_5_pro_qkv_proj_ctypes.cu:71-152,
// …norm_rope_ctypes.cu:83-173, …attn_fd4_wgmma_ctypes.cu:120-401) and their M=4 / M=8 and
// context-parallel variants.  There is no software grid barrier: the combine is done by
// whichever CTA takes the last ticket, so no CTA ever waits on another.
//
// Context parallel mode: the committed prefix [0, C) is cut into cp_size equal windows, the
// last rank of the group also takes the M new rows, every rank attends with the q heads of
// the whole group, and instead of the final context the kernel emits per-row partials
// (locally normalised context + log2-domain LSE) which it sends to the rank that owns each head.
#include "api.h"
#include "gemv.cuh"
#include "gemv_cta.cuh"
#include "mma_gemv.cuh"
#include "attn_mma.cuh"
#include "ll.cuh"

#include <cooperative_groups.h>

namespace nexrt {

struct AttnFrontArgs {
    const __nv_bfloat16* x;
    const float* in_ln;
    const uint8_t* w;        // [R][H]
    const float* s;          // [R/128][H/128]
    const int* ctl;
    float* q_raw;            // [M][nq][hd]
    float* gate;             // [M][ngate][hd]
    float* k_raw;            // [M][kvh][hd]
    __nv_bfloat16* v_cache;  // [kvh][cache_len][hd]
    int H, hd, nq, ngate, kvh, M, cache_len;
    float eps;
};

// Scatter one projected value: query / gate rows to scratch, k rows to scratch, v rows to the cache.
__device__ __forceinline__ void attn_front_row(const AttnFrontArgs& a, int row, int mm, float v, int C0, bool interleaved) {
    const int head = row / a.hd, d = row % a.hd;
    if (head < a.nq + a.ngate) {
        int qh, is_gate;
        if (interleaved) { qh = head >> 1; is_gate = head & 1; }
        else { is_gate = head >= a.nq; qh = is_gate ? head - a.nq : head; }
        if (is_gate) a.gate[(static_cast<size_t>(mm) * a.ngate + qh) * a.hd + d] = v;
        else a.q_raw[(static_cast<size_t>(mm) * a.nq + qh) * a.hd + d] = v;
    } else if (head < a.nq + a.ngate + a.kvh) {
        a.k_raw[(static_cast<size_t>(mm) * a.kvh + (head - a.nq - a.ngate)) * a.hd + d] = v;
    } else {
        const int kv = head - a.nq - a.ngate - a.kvh;
        if (C0 + mm < a.cache_len)      // a step past the end of the cache must not write outside it
            a.v_cache[(static_cast<size_t>(kv) * a.cache_len + C0 + mm) * a.hd + d] = __float2bfloat16_rn(v);
    }
}

// Row order of the weight: nq "query" heads; when ngate == nq each query head is followed by its
// gate head (checkpoint order query|gate per head), otherwise (context-parallel front) all nq
// query heads come first and the ngate gate heads after them; then k heads, then v heads.
template <int MB>
__global__ void __launch_bounds__(512, 1) attn_front_kernel(AttnFrontArgs a) {
    constexpr int U = MB == 1 ? 8 : 4;
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[32];
    pdl_launch_dependents();
    const int R = (a.nq + a.ngate + 2 * a.kvh) * a.hd;
    int r0, r1;
    cta_range(R, blockIdx.x, gridDim.x, &r0, &r1);
    const int nrows = r1 - r0;
    if (nrows) prefetch_l2_range(a.w + static_cast<size_t>(r0) * a.H, static_cast<size_t>(nrows) * a.H);
    const GemvGeom gf = gemv_geom(a.H / 16, blockDim.x);
    float* xs = smem;
    float* part = xs + static_cast<size_t>(MB) * a.H;
    float* gs = part + gemv_part_floats((R + gridDim.x - 1) / gridDim.x, MB, gf);   // [H] norm multiplier
    GemvCta<MB, U, PlainFp8> gemv(PlainFp8{a.w, a.s, a.H}, r0, nrows, a.H);
    gemv.preload();
    for (int i = threadIdx.x; i < a.H; i += blockDim.x) gs[i] = a.in_ln[i];
    pdl_wait();
    const int C0 = a.ctl[kCtlCommittedLen];
    const bool interleaved = a.ngate == a.nq;
    for (int m0 = 0; m0 < a.M; m0 += MB) {
        const int mb = min(MB, a.M - m0);
        if (m0) __syncthreads();
        stage_rmsnorm_plain(xs, a.x + static_cast<size_t>(m0) * a.H, gs, mb, a.H, a.eps, red);
        if (m0 == 0) gemv.run(xs, part);
        else gemv_cta<MB, U>(PlainFp8{a.w, a.s, a.H}, r0, nrows, xs, a.H, part);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nrows * mb; idx += blockDim.x) {
            const int rl = idx / mb, m = idx % mb;
            attn_front_row(a, r0 + rl, m0 + m, gemv_result(part, rl, m, MB, gf.wpr), C0, interleaved);
        }
    }
}

// Tensor-core form: one CTA per 16 weight rows, 8 warps split K (see mma_gemv.cuh).
template <int MP, bool LOOP = false>      // LOOP: see gdn_front_mma_kernel
__global__ void __launch_bounds__(256, 2) attn_front_mma_kernel(AttnFrontArgs a) {
    constexpr int TERMS = MmaShape<MP>::TERMS, NT = MmaShape<MP>::NT, TILE = MmaShape<MP>::TILE, NB = 8, KS = 8;
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[32];
    TraceCta tr;
    tr.begin(kTrAttnFront);
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5;
    const int row0 = blockIdx.x * kRowsPerGroup, nwin = a.H / kWin;
    float* tiles = smem;                                              // [KS][16][8]
    uint8_t* xq = reinterpret_cast<uint8_t*>(tiles + KS * TILE);       // [MP*TERMS][H]
    float* gpark = reinterpret_cast<float*>(xq + static_cast<size_t>(MP) * TERMS * a.H);   // [H] norm multiplier, parked until the norm
    const MmaPlain src{a.w, a.s, a.H};
    MmaWarp<NB, MmaPlain> mw(row0, warp, KS, nwin);
    mw.preload(src);
    RowNorm<4> norm;
    norm.preload_gamma_async(gpark, a.in_ln, a.H);
    pdl_wait();
    tr.mark(1);
    const int C0 = a.ctl[kCtlCommittedLen];
    const bool interleaved = a.ngate == a.nq;
    for (int m0 = 0; m0 < a.M; m0 += MP) {
        const int mb = min(MP, a.M - m0);
        if (m0) { __syncthreads(); mw.next_pass(); }
        norm.template run<TERMS>(xq, nullptr, a.x + static_cast<size_t>(m0) * a.H, mb, a.H, a.eps, red);
        float d[NT][4];
        mw.template run<NT>(src, xq, a.H, mb * TERMS, d);
        mw.template store<NT>(tiles + warp * TILE, d);
        __syncthreads();
        if (threadIdx.x < kRowsPerGroup * mb) {
            const int rl = threadIdx.x % kRowsPerGroup, m = threadIdx.x / kRowsPerGroup;
            attn_front_row(a, row0 + rl, m0 + m, mma_result<TERMS, NT>(tiles, KS, rl, m, kSplitDescale), C0, interleaved);
        }
    }
    if constexpr (MP == 1 && LOOP) {
        // further row groups of this CTA when the grid was capped (wide shards, one row): see gdn_front_mma_kernel
        const int R = (a.nq + a.ngate + 2 * a.kvh) * a.hd;
        for (int rg = row0 + static_cast<int>(gridDim.x) * kRowsPerGroup; rg < R; rg += static_cast<int>(gridDim.x) * kRowsPerGroup) {
            __syncthreads();
            mw.row0 = rg;
            mw.preloaded = false;
            float d[NT][4];
            mw.template run<NT>(src, xq, a.H, TERMS, d);
            mw.template store<NT>(tiles + warp * TILE, d);
            __syncthreads();
            if (threadIdx.x < kRowsPerGroup) attn_front_row(a, rg + threadIdx.x, 0, mma_result<TERMS, NT>(tiles, KS, threadIdx.x, 0, kSplitDescale), C0, interleaved);
        }
    }
    tr.mark(3);
}

struct AttnDecodeArgs {
    const float* q_raw;       // [M][nq][hd]
    const float* gate;        // [M][ngate][hd]
    const float* k_raw;       // [M][kvh][hd]
    const float* qn;          // [hd] 1 + w
    const float* kn;          // [hd]
    const float* inv_freq;    // [rotary/2]
    const float2* rope_table; // optional [cache_len][rotary/2] (cos, sin); null: computed with sincosf
    const int* ctl;
    __nv_bfloat16* k_cache;   // [kvh][cache_len][hd]
    const __nv_bfloat16* v_cache;
    float* ws_acc;            // [kvh][n_splits][rows][hd]
    float* ws_ml;             // [kvh][n_splits][rows][2]
    int* ticket;              // [kvh]
    float* out;               // [M][ngate*hd]   ctx * sigmoid(gate)      (cp_size == 1)
    int nq, ngate, kvh, M, cache_len, rotary, n_splits;
    float eps;
    // context parallel
    int ldq, ldk;             // row strides of q_raw / k_raw in floats (0: packed)
    int flags;                // 1: rows of the step see each other (non-causal block); 2: no output gate; 4: the new k rows are in the cache already; 8: control block readable before the dependency wait
    int window;               // > 0: sliding window, only the last `window` positions are attended
    int cp_size, cp_rank;     // window of the prefix this rank attends
    LLChannel ch;             // partial exchange inside the cp group (world == cp_size)
    unsigned int site;
    unsigned long long* events;   // optional timing ring: split 0 records phases 0..5, the combining CTA 6..9
};

// Tail of the wide front (multi-row steps): the projections of all rows come from the tcgen05 rows GEMM as K-split
// partial planes pre[ks][M][R]; one thread per weight row adds them in order and scatters the row's M values.
__global__ void __launch_bounds__(256) attn_front_tail_kernel(AttnFrontArgs a, const float* __restrict__ pre, int R, int ksplit) {
    TraceCta tr;
    tr.begin(kTrHelper);
    pdl_launch_dependents();
    pdl_wait();
    tr.mark(1);
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= R) return;
    const int C0 = a.ctl[kCtlCommittedLen];
    const bool interleaved = a.ngate == a.nq;
    // blockIdx.y names a block of eight token rows (one block in a decode step, several in a prefill chunk); the loads of
    // the block are all requested before the first scatter
    const int m0 = blockIdx.y * kMaxRows;
    float v[kMaxRows];
#pragma unroll
    for (int i = 0; i < kMaxRows; ++i) {
        v[i] = 0.f;
        if (m0 + i < a.M)
            for (int ks = 0; ks < ksplit; ++ks) v[i] += pre[(static_cast<size_t>(ks) * a.M + m0 + i) * R + row];
    }
#pragma unroll
    for (int i = 0; i < kMaxRows; ++i)
        if (m0 + i < a.M) attn_front_row(a, row, m0 + i, v[i], C0, interleaved);
    tr.mark(3);
}

constexpr int kRowsPerPass = 4;
constexpr int kMinKeysPerSplit = 128;   // short contexts stay on few CTAs: the combine's cost grows with the split count

constexpr int kRowsPerPassMma = 8;

// MMA: the key loop runs on the tensor cores (attn_mma.cuh), eight query rows per pass.
template <int HD, bool MMA>
__global__ void __launch_bounds__(256) attn_decode_kernel(AttnDecodeArgs a) {
    constexpr int RP = MMA ? kRowsPerPassMma : kRowsPerPass;
#define NEXRT_AEVENT(i, cond) do { if (a.events != nullptr && (cond) && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) a.events[i] = globaltimer_ns(); } while (0)
    NEXRT_AEVENT(0, blockIdx.x == 0);
    constexpr int EL = HD / 32;  // elements per lane
    extern __shared__ __align__(16) float smem[];
    __shared__ int s_last;
    TraceCta tr;
    tr.begin(kTrAttnDecode);
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int NW = 8;
    const int kv = blockIdx.y, split = blockIdx.x;
    const int G = a.nq / a.kvh;             // q heads attending one kv head
    const int rows = a.M * G;               // row index = m * G + head_in_group
    pdl_wait();
    tr.mark(1);
    NEXRT_AEVENT(1, blockIdx.x == 0);
    const int C0 = a.ctl[kCtlCommittedLen];
    // key window of this rank: [win_lo, win_hi) of positions, new rows included on the last cp rank
    int win_lo = 0, win_hi = min(C0 + a.M, a.cache_len);   // never read past the end of the cache
    if (a.window > 0) win_lo = max(0, win_hi - a.window);
    if (a.cp_size > 1) {
        const int share = C0 / a.cp_size;
        win_lo = a.cp_rank * share;
        win_hi = (a.cp_rank == a.cp_size - 1) ? min(C0 + a.M, a.cache_len) : (a.cp_rank + 1) * share;
    }
    const int n_keys = win_hi - win_lo;
    // At most one 16-key tile per warp (128 keys per CTA) while the context is short.  For longer contexts the
    // split count balances the two serial costs measured on B200: about 3 us per extra tile a warp walks against
    // about 1.1 us per 16 partials the combining CTA reads, which puts the optimum near 0.6 * sqrt(keys).
    int n_active = (n_keys + kMinKeysPerSplit - 1) / kMinKeysPerSplit;
    n_active = min(n_active, max(8, static_cast<int>(0.6f * sqrtf(static_cast<float>(n_keys)))));
    n_active = max(1, min(a.n_splits, n_active));
    if (split >= n_active) { tr.mark(3); return; }
    const int per = (n_keys + n_active - 1) / n_active;
    const int lo = win_lo + split * per, hi = min(win_hi, lo + per);

    float* q_s = smem;                                   // [rows][HD]  normalised, roped, pre-scaled
    float* k_s = q_s + static_cast<size_t>(rows) * HD;   // [M][HD]     normalised, roped, bf16 rounded
    float* part = k_s + static_cast<size_t>(a.M) * HD;   // [NW][RP][HD + 2]
    const float qscale = rsqrtf(static_cast<float>(HD)) * 1.4426950408889634f;
    const int half = a.rotary / 2;
    // ---- prologue: q and new-k normalisation + RoPE, one warp per vector
    for (int v = warp; v < rows + a.M; v += NW) {
        const bool is_q = v < rows;
        const int m = is_q ? v / G : v - rows;
        const size_t ldq = a.ldq ? a.ldq : static_cast<size_t>(a.nq) * HD, ldk = a.ldk ? a.ldk : static_cast<size_t>(a.kvh) * HD;
        const float* src = is_q ? a.q_raw + static_cast<size_t>(m) * ldq + static_cast<size_t>(kv * G + (v % G)) * HD
                                : a.k_raw + static_cast<size_t>(m) * ldk + static_cast<size_t>(kv) * HD;
        float* dst = is_q ? q_s + static_cast<size_t>(v) * HD : k_s + static_cast<size_t>(m) * HD;
        const float* gam = is_q ? a.qn : a.kn;
        float e[EL], ss = 0.f;
#pragma unroll
        for (int i = 0; i < EL; ++i) { e[i] = src[lane + 32 * i]; ss = fmaf(e[i], e[i], ss); }
        const float inv = rsqrtf(warp_sum(ss) / static_cast<float>(HD) + a.eps);
#pragma unroll
        for (int i = 0; i < EL; ++i) dst[lane + 32 * i] = e[i] * inv * gam[lane + 32 * i];
        __syncwarp();
        const float pos = static_cast<float>(C0 + m);
        float rot[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};   // rotary <= 256: up to 8 rotated dims per lane
        int ri[8] = {-1, -1, -1, -1, -1, -1, -1, -1};
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int i = lane + 32 * c;
            if (i >= a.rotary) break;
            const int f = i < half ? i : i - half;
            float sn, cs;
            if (a.rope_table != nullptr && C0 + m < a.cache_len) {   // the table has one row per cache position
                const float2 cssn = a.rope_table[static_cast<size_t>(C0 + m) * half + f];
                cs = cssn.x; sn = cssn.y;
            } else {
                sincosf(pos * a.inv_freq[f], &sn, &cs);
            }
            const float self = dst[i], other = i < half ? -dst[i + half] : dst[i - half];
            rot[c] = self * cs + other * sn;
            ri[c] = i;
        }
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 8; ++c)
            if (ri[c] >= 0) dst[ri[c]] = rot[c];
        __syncwarp();
#pragma unroll
        for (int i = 0; i < EL; ++i) {
            const float val = dst[lane + 32 * i];
            dst[lane + 32 * i] = is_q ? val * qscale : bf16_round(val);
        }
        if (!is_q && split == 0 && C0 + m < a.cache_len && !(a.flags & 4)) {
            // every rank keeps the full cache: the new k rows are appended by split 0
#pragma unroll
            for (int i = 0; i < EL; ++i)
                a.k_cache[(static_cast<size_t>(kv) * a.cache_len + C0 + m) * HD + lane + 32 * i] = __float2bfloat16_rn(dst[lane + 32 * i]);
        }
    }
    __syncthreads();
    NEXRT_AEVENT(2, split == 0);

    const __nv_bfloat16* kc = a.k_cache + static_cast<size_t>(kv) * a.cache_len * HD;
    const __nv_bfloat16* vc = a.v_cache + static_cast<size_t>(kv) * a.cache_len * HD;
    float* wsa = a.ws_acc + (static_cast<size_t>(kv) * a.n_splits + split) * rows * HD;
    float* wsm = a.ws_ml + (static_cast<size_t>(kv) * a.n_splits + split) * rows * 2;

    // cross-warp merge of the per-warp partials in `part` ([NW][RP][HD + 2]) into this split's workspace rows
    auto merge_warps = [&](int r0, int nr) {
        for (int idx = threadIdx.x; idx < nr * HD; idx += blockDim.x) {
            const int r = idx / HD, d = idx % HD;
            float M_ = -INFINITY;
            for (int w = 0; w < NW; ++w) M_ = fmaxf(M_, part[(static_cast<size_t>(w) * RP + r) * (HD + 2) + HD]);
            float L_ = 0.f, A_ = 0.f;
            for (int w = 0; w < NW; ++w) {
                const float* pr = part + (static_cast<size_t>(w) * RP + r) * (HD + 2);
                const float sc = pr[HD] == -INFINITY ? 0.f : exp2f(pr[HD] - M_);
                L_ = fmaf(pr[HD + 1], sc, L_);
                A_ = fmaf(pr[d], sc, A_);
            }
            wsa[static_cast<size_t>(r0 + r) * HD + d] = A_;
            if (d == 0) { wsm[(r0 + r) * 2] = M_; wsm[(r0 + r) * 2 + 1] = L_; }
        }
    };
    if constexpr (MMA) {
        // eight query rows per pass; wider steps (a verify step's rows x the heads of the kv group) walk the keys
        // once per pass - the K/V tiles of the later passes come from L2
        const AttnMmaKeys keys{kc, vc, k_s, C0, lo, hi};
        uint4* qf = reinterpret_cast<uint4*>(part + static_cast<size_t>(NW) * RP * (HD + 2));   // behind the per-warp partials
        // blockIdx.z names the pass: the passes of a wide step run side by side on different CTAs instead of one after
        // the other (their K/V tiles meet in L2); the ticket below counts splits x passes
        {
            const int r0 = static_cast<int>(blockIdx.z) * RP;
            const int nr = min(RP, rows - r0);
            const int gr = lane >> 2;
            const int my_limit = gr < nr ? ((a.flags & 1) ? C0 + a.M - 1 : C0 + (r0 + gr) / G) : -1;
            attn_mma_stage_q<HD>(qf, q_s + static_cast<size_t>(r0) * HD, nr);
            __syncthreads();
            attn_mma_pass<HD>(keys, qf, my_limit, warp, NW, lane, part + static_cast<size_t>(warp) * RP * (HD + 2));
            __syncthreads();
            NEXRT_AEVENT(3, split == 0);
            merge_warps(r0, nr);
            __syncthreads();
        }
        NEXRT_AEVENT(4, split == 0);
    } else {
    for (int r0 = 0; r0 < rows; r0 += kRowsPerPass) {
        const int nr = min(kRowsPerPass, rows - r0);
        float q[kRowsPerPass][EL], acc[kRowsPerPass][EL], mx[kRowsPerPass], l[kRowsPerPass];
        int limit[kRowsPerPass];
#pragma unroll
        for (int r = 0; r < kRowsPerPass; ++r) {
            const int rr = min(r0 + r, rows - 1);
#pragma unroll
            for (int i = 0; i < EL; ++i) { q[r][i] = q_s[static_cast<size_t>(rr) * HD + lane * EL + i]; acc[r][i] = 0.f; }
            mx[r] = -INFINITY; l[r] = 0.f;
            limit[r] = (r < nr) ? ((a.flags & 1) ? C0 + a.M - 1 : C0 + rr / G) : -1;   // last visible position of the row
        }
        constexpr int KBATCH = 8;   // keys whose K and V rows are in flight together per warp
        for (int pb = lo + warp; pb < hi; pb += NW * KBATCH) {
            uint4 kraw[KBATCH], vraw[KBATCH];
#pragma unroll
            for (int b = 0; b < KBATCH; ++b) {
                const int p = pb + b * NW;
                kraw[b] = make_uint4(0u, 0u, 0u, 0u);
                vraw[b] = make_uint4(0u, 0u, 0u, 0u);
                if (p < hi) {
                    if (EL == 8) {
                        if (p < C0) kraw[b] = *reinterpret_cast<const uint4*>(kc + static_cast<size_t>(p) * HD + lane * 8);
                        vraw[b] = *reinterpret_cast<const uint4*>(vc + static_cast<size_t>(p) * HD + lane * 8);
                    } else {
                        if (p < C0) {
                            const uint2 u = *reinterpret_cast<const uint2*>(kc + static_cast<size_t>(p) * HD + lane * 4);
                            kraw[b].x = u.x; kraw[b].y = u.y;
                        }
                        const uint2 u = *reinterpret_cast<const uint2*>(vc + static_cast<size_t>(p) * HD + lane * 4);
                        vraw[b].x = u.x; vraw[b].y = u.y;
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < KBATCH; ++b) {
                const int p = pb + b * NW;
                if (p >= hi) break;     // uniform across the warp
                float kf[EL], vf[EL];
                if (p < C0) {
                    if (EL == 8) unpack8_bf16(kraw[b], kf);
                    else {
                        kf[0] = __uint_as_float(kraw[b].x << 16); kf[1] = __uint_as_float(kraw[b].x & 0xffff0000u);
                        kf[2] = __uint_as_float(kraw[b].y << 16); kf[3] = __uint_as_float(kraw[b].y & 0xffff0000u);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < EL; ++i) kf[i] = k_s[static_cast<size_t>(p - C0) * HD + lane * EL + i];
                }
                if (EL == 8) unpack8_bf16(vraw[b], vf);
                else {
                    vf[0] = __uint_as_float(vraw[b].x << 16); vf[1] = __uint_as_float(vraw[b].x & 0xffff0000u);
                    vf[2] = __uint_as_float(vraw[b].y << 16); vf[3] = __uint_as_float(vraw[b].y & 0xffff0000u);
                }
#pragma unroll
                for (int r = 0; r < kRowsPerPass; ++r) {
                    float sdot = 0.f;
#pragma unroll
                    for (int i = 0; i < EL; ++i) sdot = fmaf(q[r][i], kf[i], sdot);
                    sdot = warp_sum(sdot);
                    if (p <= limit[r]) {
                        const float nm = fmaxf(mx[r], sdot);
                        const float corr = exp2f(mx[r] - nm), pw = exp2f(sdot - nm);
                        l[r] = l[r] * corr + pw;
#pragma unroll
                        for (int i = 0; i < EL; ++i) acc[r][i] = fmaf(pw, vf[i], acc[r][i] * corr);
                        mx[r] = nm;
                    }
                }
            }
        }
        // ---- merge the 8 warps of the CTA
        __syncthreads();
#pragma unroll
        for (int r = 0; r < kRowsPerPass; ++r) {
            float* pr = part + (static_cast<size_t>(warp) * kRowsPerPass + r) * (HD + 2);
#pragma unroll
            for (int i = 0; i < EL; ++i) pr[lane * EL + i] = acc[r][i];
            if (lane == 0) { pr[HD] = mx[r]; pr[HD + 1] = l[r]; }
        }
        __syncthreads();
        merge_warps(r0, nr);
        __syncthreads();
    }
    }

    // ---- ticket: the last CTA of this kv head to arrive combines all splits
    tr.mark(2);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(a.ticket + kv, 1) == n_active * static_cast<int>(gridDim.z) - 1);
    __syncthreads();
    NEXRT_AEVENT(5, split == 0);
    if (!s_last) { tr.mark(3); return; }
    __threadfence();
    NEXRT_AEVENT(6, true);
    const float* base_acc = a.ws_acc + static_cast<size_t>(kv) * a.n_splits * rows * HD;
    const float* base_ml = a.ws_ml + static_cast<size_t>(kv) * a.n_splits * rows * 2;
    LLCall call{0u, 0u};
    if (a.cp_size > 1) call = ll_begin(a.ch, a.site);
    // stage the (max, sum) pairs, turn them into per-(row, split) scales, then stream the partials
    float* sc = smem;                                        // [rows][n_active] scale of each split
    float* sl = sc + static_cast<size_t>(rows) * n_active;   // [rows][n_active] l, then [rows] totals
    __syncthreads();
    for (int idx = threadIdx.x; idx < rows * n_active; idx += blockDim.x) {
        const int r = idx / n_active, sp = idx % n_active;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(base_ml + (static_cast<size_t>(sp) * rows + r) * 2));
        sc[idx] = ml.x;
        sl[idx] = ml.y;
    }
    __syncthreads();
    float* rowM = sl + static_cast<size_t>(rows) * n_active;  // [rows] max
    float* rowL = rowM + rows;                                // [rows] total sum
    for (int r = warp; r < rows; r += NW) {
        float mxv = -INFINITY;
        for (int sp = lane; sp < n_active; sp += 32) mxv = fmaxf(mxv, sc[r * n_active + sp]);
        mxv = warp_max(mxv);
        float lsum = 0.f;
        for (int sp = lane; sp < n_active; sp += 32) {
            const float m_ = sc[r * n_active + sp];
            const float w_ = m_ == -INFINITY ? 0.f : exp2f(m_ - mxv);
            sc[r * n_active + sp] = w_;
            lsum = fmaf(sl[r * n_active + sp], w_, lsum);
        }
        lsum = warp_sum(lsum);
        if (lane == 0) { rowM[r] = mxv; rowL[r] = lsum; }
    }
    __syncthreads();
    NEXRT_AEVENT(7, true);
    // four consecutive dims of row r: normalise, gate and store (or send the partial to its owner in the cp group)
    auto finish4 = [&](int r, int d, const float4& A_, const float4& gt) {
        const float L_ = rowL[r], M_ = rowM[r];
        const int m = r / G, hg = r % G;   // head inside the kv group
        const float invl = L_ > 0.f ? 1.f / L_ : 0.f;
        float4 ctx = make_float4(A_.x * invl, A_.y * invl, A_.z * invl, A_.w * invl);
        if (a.cp_size == 1) {
            const int head = kv * G + hg;
            if (!(a.flags & 2)) {
                ctx.x *= sigmoid_f(gt.x); ctx.y *= sigmoid_f(gt.y); ctx.z *= sigmoid_f(gt.z); ctx.w *= sigmoid_f(gt.w);
            }
            *reinterpret_cast<float4*>(a.out + (static_cast<size_t>(m) * a.ngate + head) * HD + d) = ctx;
        } else {
            // head hg of the group belongs to cp rank hg / ngate; slot layout at the owner:
            // [m][local head][HD + 1] with the LSE in the last slot
            const int owner = hg / a.ngate, lh = hg % a.ngate;
            const unsigned int slot = (static_cast<unsigned int>(m) * a.ngate + lh) * (HD + 1) + d;
            const float lse = L_ > 0.f ? M_ + log2f(L_) : -INFINITY;
            ll_send(a.ch, call, owner, slot, __float_as_uint(ctx.x));
            ll_send(a.ch, call, owner, slot + 1, __float_as_uint(ctx.y));
            ll_send(a.ch, call, owner, slot + 2, __float_as_uint(ctx.z));
            ll_send(a.ch, call, owner, slot + 3, __float_as_uint(ctx.w));
            if (d == 0) ll_send(a.ch, call, owner, slot + HD, __float_as_uint(lse));
        }
    };
    const size_t stride = static_cast<size_t>(rows) * HD;
    // One thread per four consecutive output dims, 16 splits of them in flight as 16-byte loads: a decode row's
    // combine (up to 16 splits) is a single round trip to L2; the output gates are requested first.
    constexpr int WAY = 16;
    for (int q4 = threadIdx.x; q4 < rows * HD / 4; q4 += blockDim.x) {
        const int idx = q4 * 4, r = idx / HD, d = idx % HD;
        float4 gt = make_float4(0.f, 0.f, 0.f, 0.f);
        if (a.cp_size == 1 && !(a.flags & 2))
            gt = __ldcg(reinterpret_cast<const float4*>(a.gate + (static_cast<size_t>(r / G) * a.ngate + kv * G + r % G) * HD + d));
        float4 A_ = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4* pa = reinterpret_cast<const float4*>(base_acc + idx);
        for (int sp0 = 0; sp0 < n_active; sp0 += WAY) {
            float4 v[WAY];
#pragma unroll
            for (int i = 0; i < WAY; ++i)
                v[i] = (sp0 + i < n_active) ? __ldcg(pa + (sp0 + i) * (stride / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float* w_ = sc + r * n_active + sp0;
#pragma unroll
            for (int i = 0; i < WAY; ++i) {
                if (sp0 + i < n_active) {
                    const float w = w_[i];
                    A_.x = fmaf(v[i].x, w, A_.x); A_.y = fmaf(v[i].y, w, A_.y); A_.z = fmaf(v[i].z, w, A_.z); A_.w = fmaf(v[i].w, w, A_.w);
                }
            }
        }
        NEXRT_AEVENT(9, true);
        finish4(r, d, A_, gt);
        NEXRT_AEVENT(10, true);
    }
    __syncthreads();
    NEXRT_AEVENT(8, true);
    if (threadIdx.x == 0) a.ticket[kv] = 0;
    tr.mark(3);
#undef NEXRT_AEVENT
}


// ---- cluster form of the tensor-core decode (cp_size == 1) -------------------------------------------------------------
// The key window is cut over clusters of 8 CTAs.  Inside a cluster the 8 per-CTA partials (un-normalised context, max,
// sum) are combined through distributed shared memory: after one cluster barrier CTA c reads dims [c HD/8, (c+1) HD/8) of
// every row from all 8 CTAs, so the split-KV combine of a short context (one cluster = 1024 keys, one 16-key tile per
// warp) is one DSMEM round trip instead of fence + ticket + a last CTA re-reading everything from L2.  Longer contexts
// use up to n_splits / 8 clusters, whose partials (at most 18 per kv head) meet in a small ticketed tail.
//
// With `flags & 8` the committed length is read BEFORE the dependency wait (the step's first kernel releases its
// dependents only after its own wait and the head is the only writer of the control block, so the value is final), and
// the cache rows of this warp's first tile - positions below the committed length, written by earlier steps - are pulled
// into L1 while the projection front is still running.
//
// Replaces wgmma_fd4_mega's software grid barrier + combine (nex_n2_5_pro/kernels/full_attn/
// nex_n2_5_pro_attn_fd4_wgmma_ctypes.cu:98-118,389-401) with hardware cluster barriers; nothing here spins.
namespace cg = cooperative_groups;
constexpr int kClusterCtas = 8;       // portable cluster size
constexpr int kClusterCtasWide = 16;  // the largest (non-portable) size: twice the warps, so one 16-key tile per warp up to 2048 keys

template <int HD, int CL>
__global__ void __launch_bounds__(256) attn_decode_cluster_kernel(AttnDecodeArgs a) {
    constexpr int RP = kRowsPerPassMma, NW = 8, EL = HD / 32, SL = HD / CL;
    constexpr int kKeysPerCluster = CL * 8 * 16;   // one 16-key tile per warp
    extern __shared__ __align__(16) float smem[];
    __shared__ int s_last;
    TraceCta tr;
    tr.begin(kTrAttnDecode);
    cg::cluster_group cluster = cg::this_cluster();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kv = blockIdx.y, crank = static_cast<int>(cluster.block_rank()), cidx = blockIdx.x / CL;
    const int G = a.nq / a.kvh, rows = a.M * G;
    const bool early = (a.flags & 8) != 0;

    float* q_s = smem;                                   // [rows][HD]
    float* k_s = q_s + static_cast<size_t>(rows) * HD;   // [M][HD]
    float* part = k_s + static_cast<size_t>(a.M) * HD;   // [NW][RP][HD + 2]
    uint4* qf = reinterpret_cast<uint4*>(part + static_cast<size_t>(NW) * RP * (HD + 2));   // [HD / 16][32]
    float* cpart = reinterpret_cast<float*>(qf + (HD / 16) * 32);                            // [RP][HD] this CTA's partial
    float* cml = cpart + RP * HD;                                                            // [RP][2]  (max, sum)

    int C0 = 0, win_lo = 0, win_hi = 0, n_act = 1, lo = 0, hi = 0;
    auto ranges = [&]() {
        win_lo = 0;
        win_hi = min(C0 + a.M, a.cache_len);
        if (a.window > 0) win_lo = max(0, win_hi - a.window);
        if (a.cp_size > 1) {
            // context parallel: the committed prefix is cut into cp_size equal windows, the last rank of the group also
            // takes the rows of this step
            const int share = C0 / a.cp_size;
            win_lo = a.cp_rank * share;
            win_hi = (a.cp_rank == a.cp_size - 1) ? min(C0 + a.M, a.cache_len) : (a.cp_rank + 1) * share;
        }
        const int n_keys = win_hi - win_lo;
        n_act = max(1, min(static_cast<int>(gridDim.x) / CL, (n_keys + kKeysPerCluster / 2) / kKeysPerCluster));
        const int n_ctas = n_act * CL, idx = cidx * CL + crank;
        const int per = (n_keys + n_ctas - 1) / n_ctas;
        lo = min(win_hi, win_lo + idx * per);
        hi = min(win_hi, lo + per);
    };
    const __nv_bfloat16* kc = a.k_cache + static_cast<size_t>(kv) * a.cache_len * HD;
    const __nv_bfloat16* vc = a.v_cache + static_cast<size_t>(kv) * a.cache_len * HD;
    if (early) {
        C0 = *reinterpret_cast<const volatile int*>(a.ctl + kCtlCommittedLen);
        ranges();
        if (cidx < n_act) {
            // rows of this warp's first tile that earlier steps wrote: one lane per 128-byte line
            constexpr int LINES = HD * 2 / 128;
            const int t0 = lo + 16 * warp, t1 = min(min(t0 + 16, hi), C0);
            for (int i = lane; i < 16 * LINES; i += 32) {
                const int p = t0 + i / LINES;
                if (p < t1) {
                    prefetch_l1(kc + static_cast<size_t>(p) * HD + (i % LINES) * 64);
                    prefetch_l1(vc + static_cast<size_t>(p) * HD + (i % LINES) * 64);
                }
            }
        }
    }
    pdl_wait();
    tr.mark(1);
    if (!early) {
        C0 = a.ctl[kCtlCommittedLen];
        ranges();
    }
    if (cidx >= n_act) { tr.mark(3); return; }          // whole clusters leave: no barrier is left half attended

    const int r0 = static_cast<int>(blockIdx.z) * RP, nr = min(RP, rows - r0);
    // one cluster and no context parallelism: the cluster's combine is the final result; otherwise the clusters' partials
    // (and, context parallel, the other ranks') meet in the ticketed tail below
    const bool direct = n_act == 1 && a.cp_size == 1;
    // the output gates of this CTA's slice are needed only at the very end: request them now
    float gate_v = 0.f;
    const int fr = static_cast<int>(threadIdx.x) / SL, fd = crank * SL + static_cast<int>(threadIdx.x) % SL;   // (row, dim) of the final combine
    if (fr < nr && !(a.flags & 2) && direct)
        gate_v = __ldcg(a.gate + (static_cast<size_t>((r0 + fr) / G) * a.ngate + kv * G + (r0 + fr) % G) * HD + fd);

    const float qscale = rsqrtf(static_cast<float>(HD)) * 1.4426950408889634f;
    const int half = a.rotary / 2;
    // ---- q and new-k normalisation + RoPE, one warp per vector (same arithmetic as attn_decode_kernel)
    for (int v = warp; v < rows + a.M; v += NW) {
        const bool is_q = v < rows;
        const int m = is_q ? v / G : v - rows;
        const size_t ldq = a.ldq ? a.ldq : static_cast<size_t>(a.nq) * HD, ldk = a.ldk ? a.ldk : static_cast<size_t>(a.kvh) * HD;
        const float* src = is_q ? a.q_raw + static_cast<size_t>(m) * ldq + static_cast<size_t>(kv * G + (v % G)) * HD
                                : a.k_raw + static_cast<size_t>(m) * ldk + static_cast<size_t>(kv) * HD;
        float* dst = is_q ? q_s + static_cast<size_t>(v) * HD : k_s + static_cast<size_t>(m) * HD;
        const float* gam = is_q ? a.qn : a.kn;
        float e[EL], ss = 0.f;
#pragma unroll
        for (int i = 0; i < EL; ++i) { e[i] = src[lane + 32 * i]; ss = fmaf(e[i], e[i], ss); }
        const float inv = rsqrtf(warp_sum(ss) / static_cast<float>(HD) + a.eps);
#pragma unroll
        for (int i = 0; i < EL; ++i) dst[lane + 32 * i] = e[i] * inv * gam[lane + 32 * i];
        __syncwarp();
        const float pos = static_cast<float>(C0 + m);
        float rot[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        int ri[8] = {-1, -1, -1, -1, -1, -1, -1, -1};
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int i = lane + 32 * c;
            if (i >= a.rotary) break;
            const int f = i < half ? i : i - half;
            float sn, cs;
            if (a.rope_table != nullptr && C0 + m < a.cache_len) {
                const float2 cssn = a.rope_table[static_cast<size_t>(C0 + m) * half + f];
                cs = cssn.x; sn = cssn.y;
            } else {
                sincosf(pos * a.inv_freq[f], &sn, &cs);
            }
            const float self = dst[i], other = i < half ? -dst[i + half] : dst[i - half];
            rot[c] = self * cs + other * sn;
            ri[c] = i;
        }
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 8; ++c)
            if (ri[c] >= 0) dst[ri[c]] = rot[c];
        __syncwarp();
#pragma unroll
        for (int i = 0; i < EL; ++i) {
            const float val = dst[lane + 32 * i];
            dst[lane + 32 * i] = is_q ? val * qscale : bf16_round(val);
        }
        if (!is_q && cidx == 0 && crank == 0 && C0 + m < a.cache_len && !(a.flags & 4)) {
#pragma unroll
            for (int i = 0; i < EL; ++i)
                a.k_cache[(static_cast<size_t>(kv) * a.cache_len + C0 + m) * HD + lane + 32 * i] = __float2bfloat16_rn(dst[lane + 32 * i]);
        }
    }
    __syncthreads();
    tr.mark(4);

    // ---- this CTA's keys on the tensor cores, eight query rows
    {
        const AttnMmaKeys keys{kc, vc, k_s, C0, lo, hi};
        const int gr = lane >> 2;
        const int my_limit = gr < nr ? ((a.flags & 1) ? C0 + a.M - 1 : C0 + (r0 + gr) / G) : -1;
        attn_mma_stage_q<HD>(qf, q_s + static_cast<size_t>(r0) * HD, nr);
        __syncthreads();
        attn_mma_pass<HD>(keys, qf, my_limit, warp, NW, lane, part + static_cast<size_t>(warp) * RP * (HD + 2));
        __syncthreads();
    }
    tr.mark(5);
    // ---- the 8 warps of the CTA into one partial in shared memory
    for (int idx = threadIdx.x; idx < nr * HD; idx += blockDim.x) {
        const int r = idx / HD, d = idx % HD;
        float M_ = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M_ = fmaxf(M_, part[(static_cast<size_t>(w) * RP + r) * (HD + 2) + HD]);
        float L_ = 0.f, A_ = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float* pr = part + (static_cast<size_t>(w) * RP + r) * (HD + 2);
            const float sc = pr[HD] == -INFINITY ? 0.f : exp2f(pr[HD] - M_);
            L_ = fmaf(pr[HD + 1], sc, L_);
            A_ = fmaf(pr[d], sc, A_);
        }
        cpart[idx] = A_;
        if (d == 0) { cml[r * 2] = M_; cml[r * 2 + 1] = L_; }
    }
    tr.mark(2);
    cluster.sync();
    tr.mark(6);
    // ---- CTA c combines dims [c SL, (c + 1) SL) of every row over the cluster
    if (fr < nr) {
        float Av[CL], Mv[CL], Lv[CL], Mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < CL; ++c) {
            const float* rp = cluster.map_shared_rank(cpart, c);
            const float* rm = cluster.map_shared_rank(cml, c);
            Av[c] = rp[fr * HD + fd];
            Mv[c] = rm[fr * 2];
            Lv[c] = rm[fr * 2 + 1];
        }
#pragma unroll
        for (int c = 0; c < CL; ++c) Mx = fmaxf(Mx, Mv[c]);
        float A_ = 0.f, L_ = 0.f;
#pragma unroll
        for (int c = 0; c < CL; ++c) {
            const float w = Mv[c] == -INFINITY ? 0.f : exp2f(Mv[c] - Mx);
            A_ = fmaf(Av[c], w, A_);
            L_ = fmaf(Lv[c], w, L_);
        }
        const int row = r0 + fr;
        if (direct) {
            float ctx = L_ > 0.f ? A_ / L_ : 0.f;
            if (!(a.flags & 2)) ctx *= sigmoid_f(gate_v);
            a.out[(static_cast<size_t>(row / G) * a.ngate + kv * G + row % G) * HD + fd] = ctx;
        } else {
            a.ws_acc[((static_cast<size_t>(kv) * a.n_splits + cidx) * rows + row) * HD + fd] = A_;
            if (fd == 0) {
                float* ml = a.ws_ml + ((static_cast<size_t>(kv) * a.n_splits + cidx) * rows + row) * 2;
                ml[0] = Mx; ml[1] = L_;
            }
        }
    }
    if (!direct) __threadfence();
    cluster.sync();                                      // nobody leaves while a peer may still read its shared memory
    if (direct) { tr.mark(3); return; }

    // ---- several clusters (or a context-parallel group): the last cluster to arrive (per kv head, over all passes) merges
    // the clusters' partials, and ALL its CTAs share that work.  CTA 0 takes the ticket and stores the verdict into every
    // CTA's shared memory; the second cluster barrier makes it visible.  (With the tail in one CTA it was the longest
    // phase of the kernel: 13 us for 8 query rows, 33 us for the 16 rows of a context-parallel group.)
    if (crank == 0 && threadIdx.x == 0) {
        const int last = atomicAdd(a.ticket + kv, 1) == n_act * static_cast<int>(gridDim.z) - 1;
        if (last) a.ticket[kv] = 0;                      // every other cluster of this launch has taken its ticket already
#pragma unroll
        for (int c = 0; c < CL; ++c) *cluster.map_shared_rank(&s_last, c) = last;
    }
    cluster.sync();
    if (!s_last) { tr.mark(3); return; }
    tr.mark(7);
    __threadfence();
    const float* base_acc = a.ws_acc + static_cast<size_t>(kv) * a.n_splits * rows * HD;
    const float* base_ml = a.ws_ml + static_cast<size_t>(kv) * a.n_splits * rows * 2;
    constexpr int MAXC = 20;                             // clusters per kv head: n_splits (<= 160) / 8
    LLCall cpcall{0u, 0u};
    if (a.cp_size > 1) cpcall = ll_begin(a.ch, a.site);
    // Context parallel: two passes over the items - first everything that belongs to another rank is sent, then this
    // rank's own heads are merged - so that no rank sits in a wait while it still owes a peer its packets.
    for (int pass = 0; pass < (a.cp_size > 1 ? 2 : 1); ++pass)
    for (int q4 = crank * static_cast<int>(blockDim.x) + static_cast<int>(threadIdx.x); q4 < rows * HD / 4; q4 += CL * static_cast<int>(blockDim.x)) {
        const int idx = q4 * 4, r = idx / HD, d = idx % HD;
        const int m = r / G, hg = r % G;                 // token row, head inside the kv group
        // context parallel: head hg of the group belongs to cp rank hg / ngate; only the owner needs the gate
        const int owner = a.cp_size > 1 ? hg / a.ngate : 0, lh = a.cp_size > 1 ? hg % a.ngate : kv * G + hg;
        const bool mine = a.cp_size == 1 || owner == a.cp_rank;
        if (a.cp_size > 1 && mine != (pass == 1)) continue;
        float4 gt = make_float4(0.f, 0.f, 0.f, 0.f);
        if (!(a.flags & 2) && mine) gt = __ldcg(reinterpret_cast<const float4*>(a.gate + (static_cast<size_t>(m) * a.ngate + lh) * HD + d));
        float2 ml[MAXC];
        float4 v[MAXC];
#pragma unroll
        for (int c = 0; c < MAXC; ++c) {
            ml[c] = make_float2(-INFINITY, 0.f);
            v[c] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < n_act) {
                ml[c] = __ldcg(reinterpret_cast<const float2*>(base_ml + (static_cast<size_t>(c) * rows + r) * 2));
                v[c] = __ldcg(reinterpret_cast<const float4*>(base_acc + (static_cast<size_t>(c) * rows + r) * HD + d));
            }
        }
        float Mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < MAXC; ++c) Mx = fmaxf(Mx, ml[c].x);
        float4 A_ = make_float4(0.f, 0.f, 0.f, 0.f);
        float L_ = 0.f;
#pragma unroll
        for (int c = 0; c < MAXC; ++c) {
            const float w = ml[c].x == -INFINITY ? 0.f : exp2f(ml[c].x - Mx);
            L_ = fmaf(ml[c].y, w, L_);
            A_.x = fmaf(v[c].x, w, A_.x); A_.y = fmaf(v[c].y, w, A_.y); A_.z = fmaf(v[c].z, w, A_.z); A_.w = fmaf(v[c].w, w, A_.w);
        }
        const float invl = L_ > 0.f ? 1.f / L_ : 0.f;
        float4 ctx = make_float4(A_.x * invl, A_.y * invl, A_.z * invl, A_.w * invl);
        if (a.cp_size > 1) {
            // This rank's partial of (row m, head hg): locally normalised context and log2-domain LSE.  Partials of other
            // ranks' heads go to their owner as packets (every thread of the CTA sends its own four values); for this
            // rank's own heads the same thread then waits for the other ranks' packets and merges the cp_size partials
            // in rank order - once, here, instead of in every CTA of the out-projection that follows.
            const float lse = L_ > 0.f ? Mx + log2f(L_) : -INFINITY;
            const unsigned int slot = (static_cast<unsigned int>(m) * a.ngate + lh) * (HD + 1) + d;
            if (!mine) {
                ll_send(a.ch, cpcall, owner, slot, __float_as_uint(ctx.x));
                ll_send(a.ch, cpcall, owner, slot + 1, __float_as_uint(ctx.y));
                ll_send(a.ch, cpcall, owner, slot + 2, __float_as_uint(ctx.z));
                ll_send(a.ch, cpcall, owner, slot + 3, __float_as_uint(ctx.w));
                if (d == 0) ll_send(a.ch, cpcall, owner, (static_cast<unsigned int>(m) * a.ngate + lh) * (HD + 1) + HD, __float_as_uint(lse));
                continue;
            }
            float lses[kMaxWorld];
            float4 parts[kMaxWorld];
            float mx = -INFINITY;
            for (int sr = 0; sr < a.cp_size; ++sr) {
                if (sr == a.cp_rank) {
                    lses[sr] = lse;
                    parts[sr] = ctx;
                } else {
                    unsigned int pl, p0, p1, p2, p3;
                    ll_wait(a.ch, cpcall, sr, (static_cast<unsigned int>(m) * a.ngate + lh) * (HD + 1) + HD, &pl, kStatusCpTimeout);
                    ll_wait(a.ch, cpcall, sr, slot, &p0, kStatusCpTimeout);
                    ll_wait(a.ch, cpcall, sr, slot + 1, &p1, kStatusCpTimeout);
                    ll_wait(a.ch, cpcall, sr, slot + 2, &p2, kStatusCpTimeout);
                    ll_wait(a.ch, cpcall, sr, slot + 3, &p3, kStatusCpTimeout);
                    lses[sr] = __uint_as_float(pl);
                    parts[sr] = make_float4(__uint_as_float(p0), __uint_as_float(p1), __uint_as_float(p2), __uint_as_float(p3));
                }
                mx = fmaxf(mx, lses[sr]);
            }
            float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
            float den = 0.f;
            for (int sr = 0; sr < a.cp_size; ++sr) {
                const float wgt = lses[sr] == -INFINITY ? 0.f : exp2f(lses[sr] - mx);
                num.x = fmaf(wgt, parts[sr].x, num.x); num.y = fmaf(wgt, parts[sr].y, num.y);
                num.z = fmaf(wgt, parts[sr].z, num.z); num.w = fmaf(wgt, parts[sr].w, num.w);
                den += wgt;
            }
            const float invd = den > 0.f ? 1.f / den : 0.f;
            ctx = make_float4(num.x * invd, num.y * invd, num.z * invd, num.w * invd);
        }
        if (!(a.flags & 2)) {
            ctx.x *= sigmoid_f(gt.x); ctx.y *= sigmoid_f(gt.y); ctx.z *= sigmoid_f(gt.z); ctx.w *= sigmoid_f(gt.w);
        }
        *reinterpret_cast<float4*>(a.out + (static_cast<size_t>(m) * a.ngate + lh) * HD + d) = ctx;
    }
    tr.mark(3);
}

}  // namespace nexrt

using namespace nexrt;

// How many clusters of CL CTAs of this kernel the device runs at once (0: it cannot place one).  A cluster lives inside
// one GPC, so 144 CTAs in clusters of 16 are NOT one wave on 148 SMs: eight GPCs hold eight such clusters and the ninth
// runs after them - at long contexts, where every cluster has work, that doubled the kernel.  The launcher therefore never
// asks for more clusters than fit.  Asked once per kernel instantiation; also switches the non-portable cluster size on.
// Host-side queries only: safe while a stream is being captured.
template <int HD, int CL>
static int cluster_capacity(size_t smem) {
    static int cached = -1;                   // one answer per kernel instantiation
    auto kernel = attn_decode_cluster_kernel<HD, CL>;
    if (cached >= 0) return cached;
    cached = 0;
    if (CL > 8 && cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(CL, 1, 1);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    cached = n > 0 ? n : 0;
    return cached;
}

extern "C" int nexrt_attn_front_tail(const void* pre, const void* ctl, void* q_raw, void* gate, void* k_raw, void* v_cache, int hd, int nq, int ngate, int kvh,
                                     int M, int cache_len, int ksplit, void* stream) {
    if (M < 1 || M > 128 || ksplit < 1) return cudaErrorInvalidValue;   // no per-row state in the kernel: a prefill chunk goes through in one launch
    AttnFrontArgs a{nullptr, nullptr, nullptr, nullptr, static_cast<const int*>(ctl), static_cast<float*>(q_raw), static_cast<float*>(gate),
                    static_cast<float*>(k_raw), static_cast<__nv_bfloat16*>(v_cache), 0, hd, nq, ngate, kvh, M, cache_len, 0.f};
    const int R = (nq + ngate + 2 * kvh) * hd;
    return launch(attn_front_tail_kernel, dim3((R + 255) / 256, (M + kMaxRows - 1) / kMaxRows), dim3(256), 0, static_cast<cudaStream_t>(stream), a,
                  static_cast<const float*>(pre), R, ksplit);
}

extern "C" int nexrt_attn_front(const void* x, const void* in_ln, const void* w, const void* s, const void* ctl, void* q_raw, void* gate,
                                void* k_raw, void* v_cache, int H, int hd, int nq, int ngate, int kvh, int M, int cache_len, float eps,
                                int n_cta, void* stream) {
    if (M < 1 || M > kMaxRows || H % 256 || (hd != 128 && hd != 256)) return cudaErrorInvalidValue;
    AttnFrontArgs a{static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(in_ln), static_cast<const uint8_t*>(w),
                    static_cast<const float*>(s), static_cast<const int*>(ctl), static_cast<float*>(q_raw), static_cast<float*>(gate),
                    static_cast<float*>(k_raw), static_cast<__nv_bfloat16*>(v_cache), H, hd, nq, ngate, kvh, M, cache_len, eps};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int R = (nq + ngate + 2 * kvh) * hd;
    if ((gemv_mode() & 1) && H % 512 == 0 && H <= 4096) {
        const int mp = M == 1 ? 1 : (M == 2 ? 2 : 4), terms = 3;
        const size_t smem_mma = sizeof(float) * 8 * 256 + static_cast<size_t>(mp) * terms * H + sizeof(float) * H;
        dim3 g(R / 16), b(256);
        if (mp == 1 && R / 16 > 2 * n_cta) return launch(attn_front_mma_kernel<1, true>, dim3(2 * n_cta), b, smem_mma, st, a);   // capped: the kernel walks the rest
        if (mp == 1) return launch(attn_front_mma_kernel<1>, g, b, smem_mma, st, a);
        if (mp == 2) return launch(attn_front_mma_kernel<2>, g, b, smem_mma, st, a);
        return launch(attn_front_mma_kernel<4>, g, b, smem_mma, st, a);
    }
    const int mb = M == 1 ? 1 : 4;
    const size_t smem = sizeof(float) * (static_cast<size_t>(mb + 1) * H + gemv_part_floats((R + n_cta - 1) / n_cta, mb, gemv_geom(H / 16, gemv_threads())));
    if (M == 1) return launch(attn_front_kernel<1>, dim3(n_cta), dim3(gemv_threads()), smem, st, a);
    return launch(attn_front_kernel<4>, dim3(n_cta), dim3(gemv_threads()), smem, st, a);
}

// Optional timing ring (16 x u64 device memory) filled by the decode kernel of kv head 0; null switches it off.
static unsigned long long* g_attn_events = nullptr;
extern "C" int nexrt_set_attn_event_ring(void* ring) {
    g_attn_events = static_cast<unsigned long long*>(ring);
    return 0;
}

// 1 when nexrt_attn_decode with these settings runs the cluster kernel, which in context-parallel mode also merges the
// group's partials (its `out` is then the final gated context and the out-projection takes it as a plain input); 0 when
// the ticket kernel runs, which only sends the partials and leaves the merge to the out-projection (mode 2).
extern "C" int nexrt_attn_decode_merges_cp(int n_splits) {
    return ((gemv_mode() & 32) != 0 && (gemv_mode() & 64) != 0 && n_splits >= kClusterCtas) ? 1 : 0;
}

extern "C" size_t nexrt_attn_decode_smem(int hd, int nq, int kvh, int M) {
    const size_t rows = static_cast<size_t>(M) * (nq / kvh);
    const size_t main_floats = rows * hd + static_cast<size_t>(M) * hd + 8 * kRowsPerPassMma * (hd + 2) + static_cast<size_t>(hd / 16) * 32 * 4;
    const size_t n_sm = 160;  // upper bound of splits per kv head
    const size_t combine_floats = rows * n_sm * 2 + 2 * rows;
    return sizeof(float) * (main_floats > combine_floats ? main_floats : combine_floats);
}

extern "C" int nexrt_attn_decode(const void* q_raw, const void* gate, const void* k_raw, const void* qn, const void* kn, const void* inv_freq,
                                 const void* rope_table, const void* ctl, void* k_cache, const void* v_cache, void* ws_acc, void* ws_ml, void* ticket, void* out,
                                 int hd, int nq, int ngate, int kvh, int M, int cache_len, int rotary, int n_splits, float eps, int flags,
                                 int window, int ldq, int ldk, int cp_size, int cp_rank, const NexrtLLChannel* ch, unsigned int site, void* stream) {
    if (M < 1 || M > kMaxRows || nq % kvh || rotary > hd || rotary % 2) return cudaErrorInvalidValue;
    if (cp_size > 1 && ch == nullptr) return cudaErrorInvalidValue;
    if (n_splits > 160) return cudaErrorInvalidValue;
    AttnDecodeArgs a{};
    a.q_raw = static_cast<const float*>(q_raw); a.gate = static_cast<const float*>(gate); a.k_raw = static_cast<const float*>(k_raw);
    a.qn = static_cast<const float*>(qn); a.kn = static_cast<const float*>(kn); a.inv_freq = static_cast<const float*>(inv_freq);
    a.rope_table = static_cast<const float2*>(rope_table);
    a.ctl = static_cast<const int*>(ctl); a.k_cache = static_cast<__nv_bfloat16*>(k_cache);
    a.v_cache = static_cast<const __nv_bfloat16*>(v_cache); a.ws_acc = static_cast<float*>(ws_acc); a.ws_ml = static_cast<float*>(ws_ml);
    a.ticket = static_cast<int*>(ticket); a.out = static_cast<float*>(out);
    a.nq = nq; a.ngate = ngate; a.kvh = kvh; a.M = M; a.cache_len = cache_len; a.rotary = rotary; a.n_splits = n_splits; a.eps = eps;
    a.flags = flags; a.window = window; a.ldq = ldq; a.ldk = ldk;
    a.cp_size = cp_size; a.cp_rank = cp_rank; a.site = site;
    if (ch) a.ch = *ch;
    a.events = g_attn_events;
    const size_t smem = nexrt_attn_decode_smem(hd, nq, kvh, M);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool mma = (gemv_mode() & 32) != 0;
    if (mma && (gemv_mode() & 64) && n_splits >= kClusterCtas) {
        // cluster form: whole clusters along x; its shared memory adds this CTA's partial for the DSMEM combine
        const int passes_c = (M * (nq / kvh) + kRowsPerPassMma - 1) / kRowsPerPassMma;
        const size_t rows = static_cast<size_t>(M) * (nq / kvh);
        const size_t smem_c = sizeof(float) * (rows * hd + static_cast<size_t>(M) * hd + 8 * kRowsPerPassMma * (hd + 2) + static_cast<size_t>(hd / 16) * 32 * 4 +
                                               kRowsPerPassMma * hd + kRowsPerPassMma * 2);
        const size_t smem_max = sizeof(float) * (static_cast<size_t>(kMaxRows) * (nq / kvh) * hd + static_cast<size_t>(kMaxRows) * hd +
                                                 8 * kRowsPerPassMma * (hd + 2) + static_cast<size_t>(hd / 16) * 32 * 4 + kRowsPerPassMma * hd + kRowsPerPassMma * 2);
        // clusters of 16 (non-portable size) when asked for and when the device can place one: twice the warps per cluster, so a
        // context of up to 2048 keys is one 16-key tile per warp and still needs no cross-cluster tail
        const int groups = kvh * passes_c;                      // cluster rows of the grid (y x z)
        if ((gemv_mode() & 128) && n_splits >= kClusterCtasWide) {
            const int cap = hd == 256 ? cluster_capacity<256, kClusterCtasWide>(smem_max) : (hd == 128 ? cluster_capacity<128, kClusterCtasWide>(smem_max) : 0);
            if (cap > 0) {
                const int n_clusters = max(1, min(n_splits / kClusterCtasWide, cap / groups));
                const dim3 gw(n_clusters * kClusterCtasWide, kvh, passes_c);
                if (hd == 256) return launch_cluster(attn_decode_cluster_kernel<256, kClusterCtasWide>, gw, dim3(256), smem_c, st, kClusterCtasWide, a);
                return launch_cluster(attn_decode_cluster_kernel<128, kClusterCtasWide>, gw, dim3(256), smem_c, st, kClusterCtasWide, a);
            }
        }
        const int cap8 = hd == 256 ? cluster_capacity<256, kClusterCtas>(smem_max) : (hd == 128 ? cluster_capacity<128, kClusterCtas>(smem_max) : 0);
        const int n_clusters = max(1, min(n_splits / kClusterCtas, cap8 > 0 ? cap8 / groups : n_splits / kClusterCtas));
        const dim3 g(n_clusters * kClusterCtas, kvh, passes_c);
        if (hd == 256) return launch_cluster(attn_decode_cluster_kernel<256, kClusterCtas>, g, dim3(256), smem_c, st, kClusterCtas, a);
        if (hd == 128) return launch_cluster(attn_decode_cluster_kernel<128, kClusterCtas>, g, dim3(256), smem_c, st, kClusterCtas, a);
        return cudaErrorInvalidValue;
    }
    a.flags &= ~8;   // only the cluster kernel reads the control block before its dependency wait
    const int passes = (M * (nq / kvh) + kRowsPerPassMma - 1) / kRowsPerPassMma;     // tensor-core path: eight query rows per CTA
    if (hd == 256) return mma ? launch(attn_decode_kernel<256, true>, dim3(n_splits, kvh, passes), dim3(256), smem, st, a)
                              : launch(attn_decode_kernel<256, false>, dim3(n_splits, kvh), dim3(256), smem, st, a);
    if (hd == 128) return mma ? launch(attn_decode_kernel<128, true>, dim3(n_splits, kvh, passes), dim3(256), smem, st, a)
                              : launch(attn_decode_kernel<128, false>, dim3(n_splits, kvh), dim3(256), smem, st, a);
    return cudaErrorInvalidValue;
}
