// Tensor-core key loop of the decode attention for up to 8 query rows (the q heads that share one kv
// head, times the rows of the step): one warp walks 16-key tiles with mma.sync.m16n8k16 (bf16 inputs,
// fp32 accumulation).
//
//   S[rows x 16 keys]  = Q K^T   rows on the MMA M side (8 of 16 used), K read straight from the bf16 cache
//   O^T[dims x rows]  += V^T P^T rows on the MMA N side (all 8 used), V read straight from the cache
//
// Nothing is staged in shared memory and no matrix is transposed through it.  Each lane loads whole 16-byte
// pieces of a K or V row and the contraction / output dimensions are numbered so that those pieces ARE the
// fragments: a dot product does not care in which order its terms are added, so within every 64-dim block
// the four K steps take dims {16t + 4s .. 16t + 4s + 3} (t = lane % 4), and an output tile j of a 128-dim
// block holds dims {8g + j, 64 + 8g + j} (g = lane / 4).  V fragments pair two keys per register, built with
// one byte-permute per register.  The C fragment of S is already the B fragment of P^T.
//
// Q and P enter as bf16 hi + lo pairs (x = hi + lo to ~2^-17 relative), so the result matches an fp32
// evaluation on the bf16-rounded K/V the cache holds.  The reference's decode kernel does the same products with Hopper's
// wgmma m64n8k16 fed by TMA tiles (wgmma_fd4_mega, nex_n2_5_pro/kernels/full_attn/nex_n2_5_pro_attn_fd4_wgmma_ctypes.cu:120-401,
// keys on the M side, the 4 q heads padded to N = 8); wgmma does not exist on sm_100a, and with at most 8 query rows per kv
// head a warp-level mma.sync fed straight from the cache is the shape that fits.
#pragma once

#include "common.cuh"
#include "mma_gemv.cuh"

namespace nexrt {

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// hi/lo split of a pair: x = bf16(x) + bf16(x - bf16(x)) + O(2^-17 x)
__device__ __forceinline__ void split_pair(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    const float2 hf = __bfloat1622float2(h);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = pack_bf16(x - hf.x, y - hf.y);
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

struct AttnMmaKeys {
    const __nv_bfloat16* kc;   // [cache_len][HD] K cache of this kv head (positions < C0 are valid)
    const __nv_bfloat16* vc;   // [cache_len][HD] V cache (positions < C0 + M are valid)
    const float* k_new;        // shared memory [M][HD]: K rows of this step (bf16-rounded values in fp32)
    int C0;                    // committed length: positions >= C0 take K from k_new
    int lo, hi;                // key window of this CTA
};

// Query fragments in shared memory, built once per CTA: qf[(ks * 32 + lane) * 4 + {0,1,2,3}] = {hi(dims 0,1), hi(dims 2,3),
// lo(dims 0,1), lo(dims 2,3)} of row g at dims (ks / 4) * 64 + t * 16 + 4 * (ks % 4): one conflict-free 16-byte load per
// K step gives a lane its whole A fragment (hi and lo).  Needs HD / 16 * 32 * 16 bytes.
template <int HD>
__device__ __forceinline__ void attn_mma_stage_q(uint4* qf, const float* q_s, int rows) {
    constexpr int KS = HD / 16;
    for (int idx = threadIdx.x; idx < KS * 32; idx += blockDim.x) {
        const int ks = idx >> 5, lane = idx & 31, g = lane >> 2, t = lane & 3;
        const int d = (ks >> 2) * 64 + t * 16 + 4 * (ks & 3);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (g < rows) v = *reinterpret_cast<const float4*>(q_s + static_cast<size_t>(g) * HD + d);
        uint4 f;
        split_pair(v.x, v.y, f.x, f.z);
        split_pair(v.z, v.w, f.y, f.w);
        qf[idx] = f;
    }
}

__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }

// Runs one warp over the tiles {lo + 16 * (warp + nwarps * i)}.  qf: staged query fragments (attn_mma_stage_q).
// limit_row: last position row g may see.  Result: part[r][0..HD) un-normalised output, part[r][HD] running max,
// part[r][HD + 1] running sum, for r < 8 (rows beyond the step's rows come out as max = -inf, sum = 0).
//
// Per tile all K pieces are requested at once, the V rows of the tile and the K rows of the next tile are
// prefetched into L1 at the same moment, so the dependent phases (scores -> softmax -> values) meet warm lines.
// EXACT = false drops the lo terms of Q and P (bf16 operands, as flash-attention kernels use them: about 1e-3 relative
// on the output) and with them half of the tensor-core instructions.  Measured at 256K context it buys 6 us of a 69 us
// layer - the pass waits for one DRAM round trip per tile, not for the tensor pipes - and as a run-time branch in the
// decode kernel it cost the one-row step 1.9 us per attention layer, so no kernel instantiates it.
template <int HD, bool EXACT = true>
__device__ __forceinline__ void attn_mma_pass(const AttnMmaKeys& k, const uint4* qf, int limit_row, int warp, int nwarps, int lane, float* part) {
    constexpr int KS = HD / 16;    // K steps of the score product == output tiles of the value product
    constexpr int NB = HD / 64;
    const int g = lane >> 2, t = lane & 3;
    float o[KS][4];
#pragma unroll
    for (int j = 0; j < KS; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float mx = -INFINITY, l = 0.f;

    // 16 dims [d, d + 16) of key p as 8 packed bf16 pairs
    auto load_k = [&](int p, int d, uint32_t (&r)[8]) {
        if (p < k.C0) {
            const uint4* src = reinterpret_cast<const uint4*>(k.kc + static_cast<size_t>(p) * HD + d);
            const uint4 a = src[0], b = src[1];
            r[0] = a.x; r[1] = a.y; r[2] = a.z; r[3] = a.w; r[4] = b.x; r[5] = b.y; r[6] = b.z; r[7] = b.w;
        } else if (p < k.hi) {
            const float* src = k.k_new + static_cast<size_t>(p - k.C0) * HD + d;
#pragma unroll
            for (int i = 0; i < 8; ++i) r[i] = pack_bf16(src[2 * i], src[2 * i + 1]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) r[i] = 0u;
        }
    };
    // one lane per 128-byte line: rows [p0, p0 + 16) of a [.][HD] bf16 matrix
    auto prefetch_rows = [&](const __nv_bfloat16* base, int p0, int p_end) {
        constexpr int LINES = HD * 2 / 128;                  // lines per row
#pragma unroll
        for (int i = lane; i < 16 * LINES; i += 32) {
            const int p = p0 + i / LINES;
            if (p < p_end) prefetch_l1(base + static_cast<size_t>(p) * HD + (i % LINES) * 64);
        }
    };

    for (int tile = k.lo + 16 * warp; tile < k.hi; tile += 16 * nwarps) {
        // ---- request every K piece of the tile, then warm the lines the later phases will want
        uint32_t ka[NB][8], kb[NB][8];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            load_k(tile + g, b * 64 + t * 16, ka[b]);
            load_k(tile + 8 + g, b * 64 + t * 16, kb[b]);
        }
        prefetch_rows(k.vc, tile, k.hi);
        prefetch_rows(k.kc, tile + 16 * nwarps, min(k.hi, k.C0));
        // ---- scores of 16 keys: tile + g (s0) and tile + 8 + g (s1) on the N side
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const uint4 q = qf[ks * 32 + lane];
            const int b = ks >> 2, s = ks & 3;
            mma_bf16_16x8x16(s0, q.x, 0u, q.y, 0u, ka[b][2 * s], ka[b][2 * s + 1]);
            if (EXACT) mma_bf16_16x8x16(s0, q.z, 0u, q.w, 0u, ka[b][2 * s], ka[b][2 * s + 1]);
            mma_bf16_16x8x16(s1, q.x, 0u, q.y, 0u, kb[b][2 * s], kb[b][2 * s + 1]);
            if (EXACT) mma_bf16_16x8x16(s1, q.z, 0u, q.w, 0u, kb[b][2 * s], kb[b][2 * s + 1]);
        }
        // ---- mask and online softmax of row g (its 16 scores sit in the 4 lanes that share g)
        float sv[4] = {s0[0], s0[1], s1[0], s1[1]};
        const int kp[4] = {tile + 2 * t, tile + 2 * t + 1, tile + 8 + 2 * t, tile + 9 + 2 * t};
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (kp[i] > limit_row || kp[i] >= k.hi) sv[i] = -INFINITY;
        float tm = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
        tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
        tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
        const float mn = fmaxf(mx, tm);
        const float mu = mn == -INFINITY ? 0.f : mn;
        const float corr = mx == mn ? 1.f : exp2f(mx - mu);   // unchanged maximum (or a row that does not exist): no rescale
        float p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = exp2f(sv[i] - mu);
        l = fmaf(l, corr, (p[0] + p[1]) + (p[2] + p[3]));
        mx = mn;
        uint32_t ph0, pl0, ph1, pl1;
        split_pair(p[0], p[1], ph0, pl0);
        split_pair(p[2], p[3], ph1, pl1);
        // the accumulators of this lane belong to rows 2t and 2t + 1, whose state lives in lanes 8t and 8t + 4
        const float c0 = __shfl_sync(0xffffffffu, corr, 8 * t), c1 = __shfl_sync(0xffffffffu, corr, 8 * t + 4);
        if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
            for (int j = 0; j < KS; ++j) { o[j][0] *= c0; o[j][1] *= c1; o[j][2] *= c0; o[j][3] *= c1; }
        }
        // ---- O^T += V^T P^T
#pragma unroll
        for (int blk = 0; blk < HD / 128; ++blk) {
            uint4 v[4][2];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int p_ = kp[i];
                if (p_ < k.hi) {
                    const __nv_bfloat16* src = k.vc + static_cast<size_t>(p_) * HD + blk * 128 + g * 8;
                    v[i][0] = *reinterpret_cast<const uint4*>(src);
                    v[i][1] = *reinterpret_cast<const uint4*>(src + 64);
                } else {
                    v[i][0] = v[i][1] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
                auto word = [&](const uint4& q4) { return (j >> 1) == 0 ? q4.x : ((j >> 1) == 1 ? q4.y : ((j >> 1) == 2 ? q4.z : q4.w)); };
                const uint32_t a0 = prmt(word(v[0][0]), word(v[1][0]), sel), a1 = prmt(word(v[0][1]), word(v[1][1]), sel);
                const uint32_t a2 = prmt(word(v[2][0]), word(v[3][0]), sel), a3 = prmt(word(v[2][1]), word(v[3][1]), sel);
                mma_bf16_16x8x16(o[blk * 8 + j], a0, a1, a2, a3, ph0, ph1);
                if (EXACT) mma_bf16_16x8x16(o[blk * 8 + j], a0, a1, a2, a3, pl0, pl1);
            }
        }
    }
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    float* r0 = part + static_cast<size_t>(2 * t) * (HD + 2);
    float* r1 = r0 + (HD + 2);
#pragma unroll
    for (int j = 0; j < KS; ++j) {
        const int da = (j >> 3) * 128 + g * 8 + (j & 7), db = da + 64;
        r0[da] = o[j][0]; r1[da] = o[j][1];
        r0[db] = o[j][2]; r1[db] = o[j][3];
    }
    if (t == 0) {
        float* rg = part + static_cast<size_t>(g) * (HD + 2);
        rg[HD] = mx;
        rg[HD + 1] = l;
    }
}

}  // namespace nexrt
