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
#include "epilogue.cuh"
#include "gemv.cuh"
#include "ll.cuh"

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
};

template <int MB>
__global__ void __launch_bounds__(512, 1) moe_router_kernel(RouterArgs a) {
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[32];
    __shared__ int s_last;
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int rows = a.E + 1, pairs = (rows + 1) / 2;
    int t0, t1;
    cta_range(pairs, blockIdx.x, gridDim.x, &t0, &t1);
    if (t1 > t0) prefetch_l2_range(a.w + static_cast<size_t>(t0) * 2 * a.H, static_cast<size_t>(min(t1 * 2, rows) - t0 * 2) * a.H * 2);
    pdl_wait();
    for (int m0 = 0; m0 < a.M; m0 += MB) {
        const int mb = min(MB, a.M - m0);
        if (m0) __syncthreads();
        stage_rmsnorm<8>(smem, a.x + static_cast<size_t>(m0) * a.H, a.post_ln, mb, a.H, a.eps, red);
        for (int t = t0 + warp; t < t1; t += nwarps) {
            const int ra = t * 2, rb = min(t * 2 + 1, rows - 1);
            const __nv_bfloat16* w[2] = {a.w + static_cast<size_t>(ra) * a.H, a.w + static_cast<size_t>(rb) * a.H};
            float acc[2][MB];
            gemv_bf16<MB, 2, 8>(w, a.H, smem, lane, acc);
            if (lane == 0)
                for (int m = 0; m < mb; ++m) {
                    a.logits[static_cast<size_t>(m0 + m) * rows + ra] = acc[0][m];
                    if (rb != ra) a.logits[static_cast<size_t>(m0 + m) * rows + rb] = acc[1][m];
                }
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(a.ticket, 1) == static_cast<int>(gridDim.x) - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // ---- top-k: warp m owns row m; lane holds logits lane, lane+32, ...
    for (int m = warp; m < a.M; m += nwarps) {
        const float* lg = a.logits + static_cast<size_t>(m) * rows;
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int e = lane + 32 * i;
            v[i] = e < a.E ? __ldcg(lg + e) : -INFINITY;
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
            a.wts[m * S + lane] = sigmoid_f(__ldcg(lg + a.E));
        }
    }
    if (threadIdx.x == 0) *a.ticket = 0;
}

// ---------------------------------------------------------------------------------------------
struct MoeL1Args {
    const __nv_bfloat16* x;
    const float* post_ln;
    const uint8_t* w13;     // [E+1][2I][H]: gate rows then up rows
    const float* w13_s;     // [E+1][2I/128][H/128]
    const int* ids;         // [M][S]
    const float* wts;       // [M][S]
    float* h;               // [M][S][I]
    int H, I, S, M;
    float eps;
    int shared_expert;      // index whose weights may be prefetched before the dependency wait
};

__global__ void __launch_bounds__(512, 1) moe_l1_kernel(MoeL1Args a) {
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[32];
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int per_row = a.S * a.I, total = a.M * per_row;
    int t0, t1;
    cta_range(total, blockIdx.x, gridDim.x, &t0, &t1);
    const size_t expert_bytes = static_cast<size_t>(2) * a.I * a.H;
    {   // the shared expert is known before routing: pull this CTA's share of it towards L2
        const size_t share = expert_bytes / gridDim.x;
        prefetch_l2_range(a.w13 + a.shared_expert * expert_bytes + blockIdx.x * share, share);
    }
    pdl_wait();
    stage_rmsnorm<16>(smem, a.x, a.post_ln, a.M, a.H, a.eps, red);
    const int KB = a.H / kScaleBlock;
    for (int t = t0 + warp; t < t1; t += nwarps) {
        const int m = t / per_row, s_ = (t % per_row) / a.I, i = t % a.I;
        const int e = a.ids[m * a.S + s_];
        const uint8_t* base = a.w13 + e * expert_bytes;
        const uint8_t* w[2] = {base + static_cast<size_t>(i) * a.H, base + static_cast<size_t>(a.I + i) * a.H};
        const float* sb = a.w13_s + static_cast<size_t>(e) * (2 * a.I / kScaleBlock) * KB;
        const float* s[2] = {sb + (i / kScaleBlock) * KB, sb + ((a.I + i) / kScaleBlock) * KB};
        float acc[2][1];
        gemv_fp8<1, 2, 32>(w, s, a.H, smem + static_cast<size_t>(m) * a.H, lane, acc);
        if (lane == 0) a.h[t] = silu_f(acc[0][0]) * acc[1][0] * a.wts[m * a.S + s_];
    }
}

// ---------------------------------------------------------------------------------------------
struct MoeL2Args {
    const float* h;         // [M][S][I] (route weight already folded in)
    const int* ids;         // [M][S]
    const uint8_t* w2;      // [E+1][H][I]
    const float* w2_s;      // [E+1][H/128][I/128]
    __nv_bfloat16* x;
    int H, I, S, M;
    LLChannel ch;
    unsigned int site;
};

__global__ void __launch_bounds__(512, 1) moe_l2_allreduce_kernel(MoeL2Args a) {
    extern __shared__ __align__(16) float smem[];
    __shared__ int s_ids[16];
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    int r0, r1;
    cta_range(a.H / 2, blockIdx.x, gridDim.x, &r0, &r1);
    const int nrows = (r1 - r0) * 2, row0 = r0 * 2;
    const int VK = a.S * a.I, q = VK >> 4, cps = a.I >> 4;   // virtual row, its 16-byte chunks, chunks per slot
    float* hs = smem;               // [VK] quad-major
    float* res = smem + VK;         // [kMaxRows][nrows]
    const size_t expert_elems = static_cast<size_t>(a.H) * a.I;
    const int SB = a.I / kScaleBlock;
    pdl_wait();
    for (int m = 0; m < a.M; ++m) {
        if (m) __syncthreads();
        for (int k = threadIdx.x; k < VK; k += blockDim.x) hs[perm16(k, VK)] = a.h[static_cast<size_t>(m) * VK + k];
        if (threadIdx.x < a.S) s_ids[threadIdx.x] = a.ids[m * a.S + threadIdx.x];
        __syncthreads();
        for (int t = r0 + warp; t < r1; t += nwarps) {
            const int r = t * 2;
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll 2
            for (int c = lane; c < q; c += 32) {
                const int slot = c / cps, kc = c % cps;
                const int e = s_ids[slot];
                const uint8_t* wp = a.w2 + e * expert_elems + static_cast<size_t>(r) * a.I + kc * 16;
                const uint4 w0 = ld_stream16(wp), w1 = ld_stream16(wp + a.I);
                const float* sp = a.w2_s + (static_cast<size_t>(e) * (a.H / kScaleBlock) + r / kScaleBlock) * SB + (kc >> 3);
                const float sc0 = __ldg(sp), sc1 = __ldg(sp + (((r + 1) / kScaleBlock) - (r / kScaleBlock)) * SB);
                float p0 = 0.f, p1 = 0.f, f0[4], f1[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 xv = *reinterpret_cast<const float4*>(hs + ((j * q + c) << 2));
                    e4m3x4_to_float4(j == 0 ? w0.x : j == 1 ? w0.y : j == 2 ? w0.z : w0.w, f0);
                    e4m3x4_to_float4(j == 0 ? w1.x : j == 1 ? w1.y : j == 2 ? w1.z : w1.w, f1);
                    p0 = fmaf(f0[0], xv.x, p0); p0 = fmaf(f0[1], xv.y, p0); p0 = fmaf(f0[2], xv.z, p0); p0 = fmaf(f0[3], xv.w, p0);
                    p1 = fmaf(f1[0], xv.x, p1); p1 = fmaf(f1[1], xv.y, p1); p1 = fmaf(f1[2], xv.z, p1); p1 = fmaf(f1[3], xv.w, p1);
                }
                acc0 = fmaf(p0, sc0, acc0);
                acc1 = fmaf(p1, sc1, acc1);
            }
            acc0 = warp_sum(acc0);
            acc1 = warp_sum(acc1);
            if (lane == 0) {
                res[m * nrows + (r - row0)] = acc0;
                res[m * nrows + (r - row0) + 1] = acc1;
            }
        }
    }
    __syncthreads();
    allreduce_residual(a.ch, a.site, res, a.M, row0, nrows, a.H, a.x);
}

}  // namespace nexrt

using namespace nexrt;

extern "C" int nexrt_moe_router(const void* x, const void* post_ln, const void* w, void* logits, void* ids, void* wts, void* ticket, int H,
                                int E, int topk, int M, float eps, int n_cta, void* stream) {
    if (M < 1 || M > kMaxRows || H % 256 || E > 512 || topk < 1 || topk > 31 || topk > E) return cudaErrorInvalidValue;
    RouterArgs a{static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(post_ln), static_cast<const __nv_bfloat16*>(w),
                 static_cast<float*>(logits), static_cast<int*>(ids), static_cast<float*>(wts), static_cast<int*>(ticket), H, E, topk, M, eps};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (M == 1) return launch(moe_router_kernel<1>, dim3(n_cta), dim3(512), sizeof(float) * H, st, a);
    return launch(moe_router_kernel<4>, dim3(n_cta), dim3(512), sizeof(float) * 4 * H, st, a);
}

extern "C" int nexrt_moe_l1(const void* x, const void* post_ln, const void* w13, const void* w13_s, const void* ids, const void* wts, void* h,
                            int H, int I, int S, int M, float eps, int shared_expert, int n_cta, void* stream) {
    if (M < 1 || M > kMaxRows || H % 512 || I % 128 || S > 16) return cudaErrorInvalidValue;
    MoeL1Args a{static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(post_ln), static_cast<const uint8_t*>(w13),
                static_cast<const float*>(w13_s), static_cast<const int*>(ids), static_cast<const float*>(wts), static_cast<float*>(h),
                H, I, S, M, eps, shared_expert};
    return launch(moe_l1_kernel, dim3(n_cta), dim3(512), sizeof(float) * M * H, static_cast<cudaStream_t>(stream), a);
}

extern "C" int nexrt_moe_l2_allreduce(const void* h, const void* ids, const void* w2, const void* w2_s, void* x, int H, int I, int S, int M,
                                      const NexrtLLChannel* ch, unsigned int site, int n_cta, void* stream) {
    if (M < 1 || M > kMaxRows || I % 128 || S > 16 || H % 2 || ch == nullptr) return cudaErrorInvalidValue;
    if (ch->world > 1 && ch->slots < static_cast<unsigned int>(kMaxRows) * H) return cudaErrorInvalidValue;
    MoeL2Args a{};
    a.h = static_cast<const float*>(h); a.ids = static_cast<const int*>(ids); a.w2 = static_cast<const uint8_t*>(w2);
    a.w2_s = static_cast<const float*>(w2_s); a.x = static_cast<__nv_bfloat16*>(x); a.H = H; a.I = I; a.S = S; a.M = M; a.ch = *ch; a.site = site;
    const int max_rows = ((H / 2 + n_cta - 1) / n_cta) * 2;
    const size_t smem = sizeof(float) * (static_cast<size_t>(S) * I + static_cast<size_t>(kMaxRows) * max_rows);
    return launch(moe_l2_allreduce_kernel, dim3(n_cta), dim3(512), smem, static_cast<cudaStream_t>(stream), a);
}
