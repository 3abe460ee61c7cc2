// Kernels of the wide prefill path (chunks of 16..128 prompt tokens per pass) that are not GEMMs.  The chunk's
// projections, router and experts are tcgen05 GEMMs over all rows (tc_gemm.cu), so every weight is streamed once per
// chunk.  Here: embedding rows from an id list, the control-block table that gives each 8-row attention sub-step its
// base position, rmsnorm + quantisation of the chunk rows, the GDN layer's conv / gates / delta rule over the whole
// chunk, the GDN output gate + quantisation, the expert activation of the dense expert product, the skip list of
// unused experts, and the residual add over K-split planes with or without the tensor-parallel all-reduce.
//
// The reference has no counterpart: its prefill runs inside SGLang (nex_n2_5_pro/sglang_prefill/bridge.py:310-398).
#include <cuda_fp8.h>

#include "api.h"
#include "common.cuh"
#include "ll.cuh"
#include "mma_gemv.cuh"

namespace nexrt {
namespace {

__global__ void __launch_bounds__(256) prefill_embed_kernel(const __nv_bfloat16* __restrict__ embed, const int* __restrict__ ids, __nv_bfloat16* __restrict__ x,
                                                            int* status, int H, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x;
    int id = ids[m];
    if (id >= vocab || id < 0) {
        if (threadIdx.x == 0 && status) atomicCAS(status, 0, static_cast<int>(kStatusBadToken));
        id = 0;
    }
    const uint4* src = reinterpret_cast<const uint4*>(embed + static_cast<size_t>(id) * H);
    uint4* dst = reinterpret_cast<uint4*>(x + static_cast<size_t>(m) * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// table[j] = copy of the control block whose committed length is advanced by j * rows: sub-step j of a chunk reads
// its base position from table[j] exactly like a decode step reads it from the control block itself
__global__ void prefill_ctl_kernel(const int* __restrict__ ctl, int* __restrict__ table, int n_sub, int rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int j = blockIdx.x, w = threadIdx.x;
    if (j >= n_sub || w >= kCtlWords) return;
    int v = ctl[w];
    if (w == kCtlCommittedLen) v += j * rows;
    table[j * kCtlWords + w] = v;
}

// last node of a chunk: the committed length moves on, and so does the LL sequence base by the number of channel users
// of the chunk (what step_end does for a decode step)
__global__ void prefill_advance_kernel(int* ctl, int rows, unsigned int* seq, unsigned int n_sites) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        ctl[kCtlCommittedLen] += rows;
        if (seq != nullptr) *seq += n_sites;
    }
}

// One 128-column block (4 values per lane) to P e4m3 planes: plane 0 = e4m3(v / scale) with scale = amax / 448, plane p the
// residual of the planes before it at 16 times finer a scale (the step kernels' exact split, mma_gemv.cuh: split4), so that
// v = sum_p scale / 16^p * plane_p to 2^-4, 2^-8, 2^-12 of each value for P = 1, 2, 3.  Plane p of the values lies
// q_stride bytes and of the scales s_stride floats behind plane p - 1: the planes are extra token rows of the GEMM that
// follows, and its consumer adds their products like K-split partial sums.
template <int P>
__device__ __forceinline__ void quant_block4(const float v[4], __nv_fp8_storage_t* dst, float* scale_out, int lane, size_t q_stride, size_t s_stride) {
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = warp_max(amax);
    float scale = fmaxf(amax, 1e-12f) / 448.f;
    const float inv = 1.f / scale;
    float r[4] = {v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv};
    uint32_t out[P];
    split4<P>(r, out);
#pragma unroll
    for (int p = 0; p < P; ++p) {
        reinterpret_cast<uint32_t*>(dst + p * q_stride)[lane] = out[p];
        if (lane == 0) scale_out[p * s_stride] = scale;
        scale *= kTermInv;
    }
}

// GDN output gate: per 128-wide head rmsnorm(o) * gnorm_w * silu(z), then e4m3 with one scale per head (= per 128-wide
// K block of the out-projection).  One warp per (row, head).
template <int P>
__global__ void __launch_bounds__(256) gdn_gate_quant_kernel(const float* __restrict__ o, const float* __restrict__ z, const float* __restrict__ gnorm_w,
                                                             __nv_fp8_storage_t* __restrict__ xq, float* __restrict__ sx, int K, int T, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int heads = K / 128;
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= T * heads) return;
    const int m = item / heads, h = item % heads;
    const size_t base = static_cast<size_t>(m) * K + h * 128 + lane * 4;
    const float4 ov = *reinterpret_cast<const float4*>(o + base);
    const float4 zz = *reinterpret_cast<const float4*>(z + base);
    const float4 gw = *reinterpret_cast<const float4*>(gnorm_w + lane * 4);
    const float inv = rsqrtf(warp_sum(ov.x * ov.x + ov.y * ov.y + ov.z * ov.z + ov.w * ov.w) / 128.f + eps);
    const float v[4] = {gw.x * ov.x * inv * silu_f(zz.x), gw.y * ov.y * inv * silu_f(zz.y), gw.z * ov.z * inv * silu_f(zz.z), gw.w * ov.w * inv * silu_f(zz.w)};
    quant_block4<P>(v, xq + static_cast<size_t>(m) * K + h * 128, sx + static_cast<size_t>(m) * heads + h, lane, static_cast<size_t>(T) * K,
                    static_cast<size_t>(T) * heads);
}

// Expert activation of the dense expert product.  gu [T][n_total * 2I] holds gate|up of EVERY expert for every row (the
// gate/up GEMM runs over all experts: at these row counts almost every expert is routed to by some row, and the weights
// are what costs); only the S routed (row, expert) pairs are turned into h = silu(gate) * up * route weight, quantised
// per 128 columns into hq [T][n_total * I] with scales hs [T][n_total * I / 128].  Both were zeroed before: a zero scale
// removes an unrouted block from the down product.  One warp per (row, slot, 128-column block).
template <int P>
__global__ void __launch_bounds__(256) moe_dense_act_kernel(const float* __restrict__ gu, const int* __restrict__ ids, const float* __restrict__ wts,
                                                            __nv_fp8_storage_t* __restrict__ hq, float* __restrict__ hs, int I, int S, int T, int n_total,
                                                            int ksplit) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int nb = I / 128;
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= T * S * nb) return;
    const int b = item % nb, s = (item / nb) % S, m = item / (nb * S);
    const int e = min(max(ids[m * S + s], 0), n_total - 1);
    const float wt = wts[m * S + s];
    const float* g = gu + (static_cast<size_t>(m) * n_total + e) * 2 * I + b * 128 + lane * 4;
    float4 gt = *reinterpret_cast<const float4*>(g), up = *reinterpret_cast<const float4*>(g + I);
    for (int ks = 1; ks < ksplit; ++ks) {        // K-split partial planes of the gate/up product, added in plane order
        const float* gk = g + static_cast<size_t>(ks) * T * n_total * 2 * I;
        const float4 g2 = *reinterpret_cast<const float4*>(gk), u2 = *reinterpret_cast<const float4*>(gk + I);
        gt.x += g2.x; gt.y += g2.y; gt.z += g2.z; gt.w += g2.w;
        up.x += u2.x; up.y += u2.y; up.z += u2.z; up.w += u2.w;
    }
    const float v[4] = {silu_f(gt.x) * up.x * wt, silu_f(gt.y) * up.y * wt, silu_f(gt.z) * up.z * wt, silu_f(gt.w) * up.w * wt};
    quant_block4<P>(v, hq + (static_cast<size_t>(m) * n_total + e) * I + b * 128, hs + (static_cast<size_t>(m) * n_total + e) * nb + b, lane,
                    static_cast<size_t>(T) * n_total * I, static_cast<size_t>(T) * n_total * nb);
}

__global__ void moe_mark_used_kernel(const int* __restrict__ ids, int* __restrict__ used, int n_ids, int n_total) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_ids) used[min(max(ids[i], 0), n_total - 1)] = 1;
}

// out = sum of the K-split planes y[ks][n]; with x != null the sum is added to the bf16 residual rows instead
// (x = bf16(x + sum)), with sum_out != null it is kept in fp32 (input of a host-launched all-reduce).
__global__ void __launch_bounds__(256) planes_residual_kernel(__nv_bfloat16* x, const float* __restrict__ y, float* sum_out, size_t n, int ksplit) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    float4 t = *reinterpret_cast<const float4*>(y + i);
    for (int ks = 1; ks < ksplit; ++ks) {
        const float4 v = *reinterpret_cast<const float4*>(y + static_cast<size_t>(ks) * n + i);
        t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
    }
    if (sum_out) *reinterpret_cast<float4*>(sum_out + i) = t;
    if (x) {
        __nv_bfloat162* xp = reinterpret_cast<__nv_bfloat162*>(x + i);
        const float2 a = __bfloat1622float2(xp[0]), b = __bfloat1622float2(xp[1]);
        xp[0] = __floats2bfloat162_rn(a.x + t.x, a.y + t.y);
        xp[1] = __floats2bfloat162_rn(b.x + t.z, b.y + t.w);
    }
}

// Tensor-parallel form of the residual add: the sum of this rank's K-split planes is all-reduced inside the kernel, then
// x = bf16(x + sum).  A chunk moves megabytes per reduce, so the 8-byte tagged packets of the decode steps (half of every
// packet is the tag, one NVLink transaction per value) give way to a block protocol over the same symmetric inbox: the 256
// threads of a CTA store their 1024 values as plain 16-byte vectors into every rank's copy of region [half][this rank]
// (one multimem.st through the NVSwitch alias, or one store per peer), make them visible (fence.sys + barrier), and one
// thread publishes the call's tag in the CTA's flag word; the same CTA of every other rank does the same, so the CTA polls
// its flag word of each peer region (bounded like every LL wait, status latched on expiry), then adds the world's
// vectors in rank order: every rank gets the same bits.  Region layout: n floats of data, then one u32 flag per CTA.
// Halves alternate with the global call sequence as in ll.cuh: a peer can publish call k + 2 into a half only after this
// rank has left the kernel of call k.  CTA b waits for CTA b of every peer, so progress needs the CTAs of a call to be
// resident together or dispatched in the same order on every rank: the grid is n / 1024 <= 1024 CTAs, dispatched in
// index order (parallel/ll_model.py: BlockModel states the protocol on CPU threads, tests/test_ll_protocol_model.py).
__device__ __forceinline__ void st_sys_v4(float* p, const float4& v) {
    asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void mc_st_v4(float* p, const float4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ float4 ld_sys_v4(const float* p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_sys_u32(unsigned int* p, unsigned int v) { asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void mc_st_u32(unsigned int* p, unsigned int v) {
    asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(256) planes_allreduce_residual_kernel(__nv_bfloat16* x, const float* __restrict__ y, size_t n, int ksplit, LLChannel ch,
                                                                        unsigned int site) {
    __shared__ int s_ok[kMaxWorld];
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;     // n is a multiple of 1024: every thread has work
    float4 t = *reinterpret_cast<const float4*>(y + i);
    for (int ks = 1; ks < ksplit; ++ks) {
        const float4 v = *reinterpret_cast<const float4*>(y + static_cast<size_t>(ks) * n + i);
        t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
    }
    const LLCall call = ll_begin(ch, site);
    // byte offset of region [half][src] inside every rank's inbox, and of this CTA's flag word inside a region
    auto region = [&](int src) { return (static_cast<size_t>(call.half) * ch.world + src) * ch.slots * 8; };
    const size_t flag_off = n * 4 + static_cast<size_t>(blockIdx.x) * 4;
    const size_t mine = region(ch.rank);
    if (ch.mc != nullptr) {
        mc_st_v4(reinterpret_cast<float*>(reinterpret_cast<char*>(ch.mc) + mine) + i, t);
    } else {
        for (int p = 0; p < ch.world; ++p)
            if (p != ch.rank) st_sys_v4(reinterpret_cast<float*>(reinterpret_cast<char*>(ch.peer[p]) + mine) + i, t);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        // release pattern of the publishing thread itself: the barrier ordered the other threads' (already fenced) data
        // stores before this point, and this fence orders them, cumulatively, before the flag store that follows
        __threadfence_system();
        if (ch.mc != nullptr) {
            mc_st_u32(reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(ch.mc) + mine + flag_off), call.tag);
        } else {
            for (int p = 0; p < ch.world; ++p)
                if (p != ch.rank) st_sys_u32(reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(ch.peer[p]) + mine + flag_off), call.tag);
        }
    }
    // thread s waits for the flag of rank s
    if (static_cast<int>(threadIdx.x) < ch.world) {
        const int src = threadIdx.x;
        int ok = 1;
        if (src != ch.rank) {
            const unsigned int* f = reinterpret_cast<const unsigned int*>(reinterpret_cast<const char*>(ch.local) + region(src) + flag_off);
            if (ld_acquire_sys_u32(f) != call.tag) {
                const bool failed = *reinterpret_cast<volatile int*>(ch.status) != 0;     // a latched failure makes every later wait give up at once
                const unsigned long long t0 = globaltimer_ns();
                unsigned int spins = 0;
                while (ld_acquire_sys_u32(f) != call.tag) {
                    if (failed || ((++spins & 63u) == 0 && globaltimer_ns() - t0 > ch.budget_ns)) {
                        atomicCAS(ch.status, 0, static_cast<int>(kStatusReduceTimeout));
                        ok = 0;
                        break;
                    }
                }
            }
        }
        s_ok[src] = ok;
    }
    __syncthreads();
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int src = 0; src < ch.world; ++src) {
        float4 v = t;
        if (src != ch.rank)
            v = s_ok[src] ? ld_sys_v4(reinterpret_cast<const float*>(reinterpret_cast<const char*>(ch.local) + region(src)) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
    }
    __nv_bfloat162* xp = reinterpret_cast<__nv_bfloat162*>(x + i);
    const float2 a = __bfloat1622float2(xp[0]), b = __bfloat1622float2(xp[1]);
    xp[0] = __floats2bfloat162_rn(a.x + sum.x, a.y + sum.y);
    xp[1] = __floats2bfloat162_rn(b.x + sum.z, b.y + sum.w);
}

// rmsnorm(x[t]) * gamma of every chunk row, written in the forms the chunk's GEMMs take (each output optional):
//   xq / sx : e4m3 with one scale per 128 columns (FP8 projections, expert gate/up),
//   xn      : fp32 (the bf16 b/a rows of the GDN front are projected from it),
//   planes  : bf16 hi + lo per token, [T][2][K] (the router: x = hi + lo to about 2^-17, two accumulating GEMMs).
template <int P>
__global__ void __launch_bounds__(256) norm_rows_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, __nv_fp8_storage_t* __restrict__ xq,
                                                        float* __restrict__ sx, float* __restrict__ xn, __nv_bfloat16* __restrict__ planes, int K, float eps) {
    // thread t owns columns [8t, 8t + 8) of every 2048-column slab (K <= 8192): one 16-byte load per slab, the row stays in
    // registers between the two passes, and a 128-column quantisation block is 16 neighbouring lanes
    constexpr int NS = 4;
    __shared__ float red[32];
    pdl_launch_dependents();
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const int slabs = (K + 2047) / 2048;
    float g[NS][8];
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int k0 = i * 2048 + threadIdx.x * 8;
        if (i < slabs && k0 < K) {
            const float4 g0 = *reinterpret_cast<const float4*>(gamma + k0), g1 = *reinterpret_cast<const float4*>(gamma + k0 + 4);
            g[i][0] = g0.x; g[i][1] = g0.y; g[i][2] = g0.z; g[i][3] = g0.w; g[i][4] = g1.x; g[i][5] = g1.y; g[i][6] = g1.z; g[i][7] = g1.w;
        }
    }
    pdl_wait();
    const __nv_bfloat16* xr = x + static_cast<size_t>(t) * K;
    float v[NS][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int k0 = i * 2048 + threadIdx.x * 8;
        if (i < slabs && k0 < K) {
            unpack8_bf16(*reinterpret_cast<const uint4*>(xr + k0), v[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = fmaf(v[i][j], v[i][j], ss);
        }
    }
    const float rinv = rsqrtf(block_sum(ss, red) / K + eps);
    const int KB = K / 128;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int k0 = i * 2048 + threadIdx.x * 8;
        if (!(i < slabs && k0 < K)) continue;       // uniform per 16-lane group: K is a multiple of 128
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[i][j] = v[i][j] * rinv * g[i][j];
            amax = fmaxf(amax, fabsf(v[i][j]));
        }
        if (xn) {
            float* d = xn + static_cast<size_t>(t) * K + k0;
            *reinterpret_cast<float4*>(d) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
            *reinterpret_cast<float4*>(d + 4) = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
        }
        if (planes) {
            __align__(16) __nv_bfloat16 hi[8], lo[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                hi[j] = __float2bfloat16_rn(v[i][j]);
                lo[j] = __float2bfloat16_rn(v[i][j] - __bfloat162float(hi[j]));
            }
            *reinterpret_cast<uint4*>(planes + (static_cast<size_t>(t) * 2) * K + k0) = *reinterpret_cast<const uint4*>(hi);
            *reinterpret_cast<uint4*>(planes + (static_cast<size_t>(t) * 2 + 1) * K + k0) = *reinterpret_cast<const uint4*>(lo);
        }
        if (xq) {
            // the 16 lanes of a 128-column block share one scale (all 32 lanes take part in the shuffles)
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            float scale = fmaxf(amax, 1e-12f) / 448.f;
            const float inv = 1.f / scale;
            float r0[4] = {v[i][0] * inv, v[i][1] * inv, v[i][2] * inv, v[i][3] * inv}, r1[4] = {v[i][4] * inv, v[i][5] * inv, v[i][6] * inv, v[i][7] * inv};
            uint32_t w0[P], w1[P];
            split4<P>(r0, w0);
            split4<P>(r1, w1);
            // plane p = rows [p * T, (p + 1) * T) of xq / sx (T = gridDim.x): extra token rows of the GEMM that follows
#pragma unroll
            for (int p = 0; p < P; ++p) {
                const size_t row = static_cast<size_t>(p) * gridDim.x + t;
                *reinterpret_cast<uint2*>(xq + row * K + k0) = make_uint2(w0[p], w1[p]);
                if ((lane & 15) == 0) sx[row * KB + k0 / 128] = scale;
                scale *= kTermInv;
            }
        }
    }
}

// ---- GDN layer over a whole chunk -------------------------------------------------------------------------------
struct GdnChunkArgs {
    const float* pre;            // [T][R] projections of the chunk: q|k|v rows (C of them), then z rows
    const float* xn;             // [T][H] fp32 normalised rows (b/a projections)
    const __nv_bfloat16* ba_w;   // [2 nv][H]
    const float* conv_w;         // [C][4]
    const float* a_log;          // [nv]
    const float* dt_bias;        // [nv]
    const int* ctl;
    float* conv_ring;            // [ring][C], position-indexed
    float* qkv;                  // [T][C] after conv + SiLU
    float* z;                    // [T][R - C]
    float* beta;                 // [T][nv]
    float* g;                    // [T][nv]
    float* state_ring;           // [state_ring][nv][128 v][128 k]
    float* out;                  // [T][nv * 128]
    int H, R, C, nv, nqk, T, ring, state_ring_len;
};

// Conv ring + SiLU of the q|k|v rows, z store, b/a projections for all T rows in one launch: the same arithmetic as the
// step kernels (gdn.cu: gdn_front_row, gdn_ba_row), with the three-tap history carried in registers along the chunk.
__global__ void __launch_bounds__(256) gdn_front_chunk_kernel(GdnChunkArgs a, int row_ctas, int m_blocks, int ksplit) {
    pdl_launch_dependents();
    pdl_wait();
    if (static_cast<int>(blockIdx.x) < row_ctas * m_blocks) {
        // one thread per (weight row, block of eight token rows): the three taps before the block come from the chunk's own
        // projections (or, for the first block, from the ring), so the blocks do not depend on each other
        const int row = (blockIdx.x % row_ctas) * blockDim.x + threadIdx.x;
        const int m0 = (blockIdx.x / row_ctas) * 8;
        if (row >= a.R) return;
        const int C0 = a.ctl[kCtlCommittedLen];
        // the projection arrives as K-split partial planes pre[ks][T][R], added in plane order
        auto pre_sum = [&](int m) {
            float t = a.pre[static_cast<size_t>(m) * a.R + row];
            for (int ks = 1; ks < ksplit; ++ks) t += a.pre[(static_cast<size_t>(ks) * a.T + m) * a.R + row];
            return t;
        };
        float p[11];                       // rows m0 - 3 .. m0 + 7
#pragma unroll
        for (int i = 0; i < 8; ++i) p[3 + i] = m0 + i < a.T ? pre_sum(m0 + i) : 0.f;
        if (row >= a.C) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (m0 + i < a.T) a.z[static_cast<size_t>(m0 + i) * (a.R - a.C) + (row - a.C)] = p[3 + i];
            return;
        }
        const int ring = a.ring;
#pragma unroll
        for (int j = 0; j < 3; ++j)
            p[j] = m0 > 0 ? pre_sum(m0 - 3 + j) : a.conv_ring[static_cast<size_t>((C0 - 3 + j + ring) % ring) * a.C + row];
        const float4 cw = *reinterpret_cast<const float4*>(a.conv_w + static_cast<size_t>(row) * 4);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int m = m0 + i;
            if (m >= a.T) break;
            const float v = fmaf(cw.x, p[i], fmaf(cw.y, p[i + 1], fmaf(cw.z, p[i + 2], cw.w * p[i + 3])));
            a.qkv[static_cast<size_t>(m) * a.C + row] = silu_f(v);
            if (m >= a.T - 3) a.conv_ring[static_cast<size_t>((C0 + m) % ring) * a.C + row] = p[i + 3];   // later steps read the last three
        }
        return;
    }
    row_ctas *= m_blocks;
    // one warp per (b/a row, token row)
    const int lane = threadIdx.x & 31;
    const int item = (blockIdx.x - row_ctas) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= 2 * a.nv * a.T) return;
    const int row = item / a.T, m = item % a.T;
    const __nv_bfloat16* w = a.ba_w + static_cast<size_t>(row) * a.H;
    const float* xr = a.xn + static_cast<size_t>(m) * a.H;
    float acc = 0.f;
#pragma unroll 4
    for (int k = lane * 8; k < a.H; k += 256) {      // H % 256 == 0; unrolled so that the loads of four steps are in flight together
        float wf[8];
        unpack8_bf16(*reinterpret_cast<const uint4*>(w + k), wf);
        const float4 x0 = *reinterpret_cast<const float4*>(xr + k), x1 = *reinterpret_cast<const float4*>(xr + k + 4);
        acc = fmaf(wf[0], x0.x, fmaf(wf[1], x0.y, fmaf(wf[2], x0.z, fmaf(wf[3], x0.w, acc))));
        acc = fmaf(wf[4], x1.x, fmaf(wf[5], x1.y, fmaf(wf[6], x1.z, fmaf(wf[7], x1.w, acc))));
    }
    acc = warp_sum(acc);
    if (lane == 0) {
        if (row < a.nv) a.beta[m * a.nv + row] = sigmoid_f(acc);
        else {
            const int h = row - a.nv;
            a.g[m * a.nv + h] = -__expf(a.a_log[h]) * softplus_f(acc + a.dt_bias[h]);
        }
    }
}

// Delta rule over the T rows of a chunk: grid (nv, 128 / warps per CTA), one warp per value column, lane holds 4 key rows
// of the state column (the mapping and the arithmetic of gdn.cu: gdn_core_kernel, so the state is the one the step kernels
// would leave).  The state stays in registers along the chunk and only the state after the last row goes back to the ring.
// The inputs are staged 32 rows at a time in shared memory (coalesced loads, all in flight together) with k already
// normalised and the q scale per row, so the serial chain per row is one warp reduction and a few multiply-adds.
constexpr int kCoreRows = 32;
__global__ void __launch_bounds__(256) gdn_core_chunk_kernel(GdnChunkArgs a) {
    __shared__ __align__(16) float qs[kCoreRows][128];
    __shared__ __align__(16) float ks[kCoreRows][128];
    __shared__ float vs[kCoreRows][8], qn_s[kCoreRows], dec_s[kCoreRows], b_s[kCoreRows];
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;   // nwarps == 8
    const int head = blockIdx.x, col0 = blockIdx.y * nwarps, col = col0 + warp;
    const int qk_head = head / (a.nv / a.nqk);
    const size_t head_stride = static_cast<size_t>(128) * 128, slot_stride = head_stride * a.nv;
    const size_t elem = head * head_stride + static_cast<size_t>(col) * 128 + lane * 4;
    pdl_wait();
    const int C0 = a.ctl[kCtlCommittedLen];
    float4 S = *reinterpret_cast<const float4*>(a.state_ring + static_cast<size_t>(C0 % a.state_ring_len) * slot_stride + elem);
    for (int mb = 0; mb < a.T; mb += kCoreRows) {
        const int nr = min(kCoreRows, a.T - mb);
        __syncthreads();
        // warp w stages rows w, w + 8, ...: q (raw) with its scale, k normalised, the 8 v values of this CTA, decay, beta
        for (int r = warp; r < nr; r += nwarps) {
            const float* row = a.qkv + static_cast<size_t>(mb + r) * a.C;
            const float4 q4 = *reinterpret_cast<const float4*>(row + qk_head * 128 + lane * 4);
            const float4 k4 = *reinterpret_cast<const float4*>(row + (a.nqk + qk_head) * 128 + lane * 4);
            const float qn = rsqrtf(warp_sum(q4.x * q4.x + q4.y * q4.y + q4.z * q4.z + q4.w * q4.w) + 1e-6f) * 0.08838834764831845f;
            const float kn = rsqrtf(warp_sum(k4.x * k4.x + k4.y * k4.y + k4.z * k4.z + k4.w * k4.w) + 1e-6f);
            *reinterpret_cast<float4*>(&qs[r][lane * 4]) = q4;
            *reinterpret_cast<float4*>(&ks[r][lane * 4]) = make_float4(k4.x * kn, k4.y * kn, k4.z * kn, k4.w * kn);
            if (lane < 8) vs[r][lane] = row[(2 * a.nqk + head) * 128 + col0 + lane];
            if (lane == 8) qn_s[r] = qn;
            if (lane == 9) dec_s[r] = __expf(a.g[(mb + r) * a.nv + head]);
            if (lane == 10) b_s[r] = a.beta[(mb + r) * a.nv + head];
        }
        __syncthreads();
        // The output reduction of row r - 1 rides along with the k.S reduction of row r (two independent values per shuffle
        // step): a warp issues in order, so two back-to-back butterflies would cost twice the latency of one.
        float po = 0.f;       // this lane's part of q.S of the previous row
        for (int r = 0; r < nr; ++r) {
            const float4 k4 = *reinterpret_cast<const float4*>(&ks[r][lane * 4]);   // already k * kn
            const float decay = dec_s[r], b = b_s[r], v = vs[r][warp];
            S.x *= decay; S.y *= decay; S.z *= decay; S.w *= decay;
            float pk = k4.x * S.x + k4.y * S.y + k4.z * S.z + k4.w * S.w;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                pk += __shfl_xor_sync(0xffffffffu, pk, o);
                po += __shfl_xor_sync(0xffffffffu, po, o);
            }
            if (r > 0 && lane == 0) a.out[static_cast<size_t>(mb + r - 1) * a.nv * 128 + head * 128 + col] = po * qn_s[r - 1];
            const float delta = (v - pk) * b;
            S.x = fmaf(k4.x, delta, S.x); S.y = fmaf(k4.y, delta, S.y); S.z = fmaf(k4.z, delta, S.z); S.w = fmaf(k4.w, delta, S.w);
            const float4 q4 = *reinterpret_cast<const float4*>(&qs[r][lane * 4]);
            po = q4.x * S.x + q4.y * S.y + q4.z * S.z + q4.w * S.w;
        }
        po = warp_sum(po);
        if (lane == 0) a.out[static_cast<size_t>(mb + nr - 1) * a.nv * 128 + head * 128 + col] = po * qn_s[nr - 1];
    }
    *reinterpret_cast<float4*>(a.state_ring + static_cast<size_t>((C0 + a.T) % a.state_ring_len) * slot_stride + elem) = S;
}

}  // namespace
}  // namespace nexrt

using namespace nexrt;

extern "C" {

// Every kernel of this file starts with griddepcontrol.launch_dependents + griddepcontrol.wait and is launched with the
// programmatic-serialisation attribute (common.cuh: launch), so inside the captured chunk a kernel's launch latency
// overlaps the tail of its predecessor.

int nexrt_prefill_embed(const void* embed, const void* ids, void* x, void* status, int H, int vocab, int T, void* stream) {
    if (T < 1 || H % 8) return cudaErrorInvalidValue;
    return launch(prefill_embed_kernel, dim3(T), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(embed),
                  static_cast<const int*>(ids), static_cast<__nv_bfloat16*>(x), static_cast<int*>(status), H, vocab);
}

int nexrt_prefill_ctl(const void* ctl, void* table, int n_sub, int rows, void* stream) {
    if (n_sub < 1 || rows < 1) return cudaErrorInvalidValue;
    return launch(prefill_ctl_kernel, dim3(n_sub), dim3(32), 0, static_cast<cudaStream_t>(stream), static_cast<const int*>(ctl), static_cast<int*>(table), n_sub, rows);
}

int nexrt_prefill_advance(void* ctl, int rows, void* seq, unsigned int n_sites, void* stream) {
    return launch(prefill_advance_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), static_cast<int*>(ctl), rows, static_cast<unsigned int*>(seq),
                  n_sites);
}

int nexrt_planes_allreduce_residual(void* x, const void* y, int64_t n, int ksplit, const NexrtLLChannel* ch, unsigned int site, void* stream) {
    if (n < 1024 || n % 1024 || ksplit < 1 || ch == nullptr || ch->world < 2 || ch->slots < static_cast<unsigned int>(n)) return cudaErrorInvalidValue;
    const int64_t threads = n / 4;
    return launch(planes_allreduce_residual_kernel, dim3(static_cast<unsigned int>((threads + 255) / 256)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                  static_cast<__nv_bfloat16*>(x), static_cast<const float*>(y), static_cast<size_t>(n), ksplit, *ch, site);
}

// `terms` (1..3) = number of e4m3 planes the quantisers write: plane p occupies rows [p * T, (p + 1) * T) of xq / sx.
int nexrt_gdn_gate_quant(const void* o, const void* z, const void* gnorm_w, void* xq, void* sx, int K, int T, float eps, int terms, void* stream) {
    if (T < 1 || K % 128 || terms < 1 || terms > 3) return cudaErrorInvalidValue;
    const int items = T * (K / 128);
    auto go = [&](auto kern) {
        return launch(kern, dim3((items + 7) / 8), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const float*>(o), static_cast<const float*>(z),
                      static_cast<const float*>(gnorm_w), static_cast<__nv_fp8_storage_t*>(xq), static_cast<float*>(sx), K, T, eps);
    };
    return terms == 1 ? go(gdn_gate_quant_kernel<1>) : terms == 2 ? go(gdn_gate_quant_kernel<2>) : go(gdn_gate_quant_kernel<3>);
}

int nexrt_moe_dense_act(const void* gu, const void* ids, const void* wts, void* hq, void* hs, int I, int S, int T, int n_total, int ksplit, int terms,
                        void* stream) {
    if (T < 1 || I % 128 || S < 1 || ksplit < 1 || terms < 1 || terms > 3) return cudaErrorInvalidValue;
    const int items = T * S * (I / 128);
    auto go = [&](auto kern) {
        return launch(kern, dim3((items + 7) / 8), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const float*>(gu), static_cast<const int*>(ids),
                      static_cast<const float*>(wts), static_cast<__nv_fp8_storage_t*>(hq), static_cast<float*>(hs), I, S, T, n_total, ksplit);
    };
    return terms == 1 ? go(moe_dense_act_kernel<1>) : terms == 2 ? go(moe_dense_act_kernel<2>) : go(moe_dense_act_kernel<3>);
}


int nexrt_moe_mark_used(const void* ids, void* used, int n_ids, int n_total, void* stream) {
    if (n_ids < 1 || n_total < 1) return cudaErrorInvalidValue;
    auto s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(used, 0, sizeof(int) * n_total, s);
    if (e != cudaSuccess) return e;
    return launch(moe_mark_used_kernel, dim3((n_ids + 255) / 256), dim3(256), 0, s, static_cast<const int*>(ids), static_cast<int*>(used), n_ids, n_total);
}

int nexrt_planes_residual(void* x, const void* y, void* sum_out, int64_t n, int ksplit, void* stream) {
    if (n < 4 || n % 4 || ksplit < 1) return cudaErrorInvalidValue;
    const int64_t threads = n / 4;
    return launch(planes_residual_kernel, dim3(static_cast<unsigned int>((threads + 255) / 256)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                  static_cast<__nv_bfloat16*>(x), static_cast<const float*>(y), static_cast<float*>(sum_out), static_cast<size_t>(n), ksplit);
}

int nexrt_norm_rows(const void* x, const void* gamma, void* xq, void* sx, void* xn, void* planes, int K, int T, float eps, int terms, void* stream) {
    if (T < 1 || K < 256 || K % 256 || K > 8192 || terms < 1 || terms > 3) return cudaErrorInvalidValue;
    auto go = [&](auto kern) {
        return launch(kern, dim3(T), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(gamma),
                      static_cast<__nv_fp8_storage_t*>(xq), static_cast<float*>(sx), static_cast<float*>(xn), static_cast<__nv_bfloat16*>(planes), K, eps);
    };
    return terms == 1 ? go(norm_rows_kernel<1>) : terms == 2 ? go(norm_rows_kernel<2>) : go(norm_rows_kernel<3>);
}

// GDN layer of a chunk after its q|k|v|z projection (pre: ksplit partial planes [ksplit][T][R]): conv + gates (front) and
// the delta rule (core), T rows per launch.
int nexrt_gdn_chunk(const void* pre, const void* xn, const void* ba_w, const void* conv_w, const void* a_log, const void* dt_bias, const void* ctl,
                    void* conv_ring, void* qkv, void* z, void* beta, void* g, void* state_ring, void* out, int H, int R, int C, int nv, int nqk, int T,
                    int conv_ring_len, int state_ring_len, int ksplit, void* stream) {
    if (T < 1 || H % 256 || conv_ring_len < 3 || state_ring_len < 1 || nqk < 1 || nv % nqk || C != (2 * nqk + nv) * 128 || ksplit < 1) return cudaErrorInvalidValue;
    GdnChunkArgs a{static_cast<const float*>(pre), static_cast<const float*>(xn), static_cast<const __nv_bfloat16*>(ba_w), static_cast<const float*>(conv_w),
                   static_cast<const float*>(a_log), static_cast<const float*>(dt_bias), static_cast<const int*>(ctl), static_cast<float*>(conv_ring),
                   static_cast<float*>(qkv), static_cast<float*>(z), static_cast<float*>(beta), static_cast<float*>(g), static_cast<float*>(state_ring),
                   static_cast<float*>(out), H, R, C, nv, nqk, T, conv_ring_len, state_ring_len};
    auto s = static_cast<cudaStream_t>(stream);
    const int row_ctas = (R + 255) / 256, m_blocks = (T + 7) / 8, ba_ctas = (2 * nv * T + 7) / 8;
    int e = launch(gdn_front_chunk_kernel, dim3(row_ctas * m_blocks + ba_ctas), dim3(256), 0, s, a, row_ctas, m_blocks, ksplit);
    if (e != 0) return e;
    return launch(gdn_core_chunk_kernel, dim3(nv, 128 / 8), dim3(256), 0, s, a);
}

}  // extern "C"
