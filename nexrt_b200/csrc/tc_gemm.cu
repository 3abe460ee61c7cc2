// Tensor-core GEMM for many-row work (prefill chunks, wide verify): Y[T, R] = X[T, K] * W[R, K]^T on the
// 5th-generation tensor cores.
//
//   * operands are staged by TMA (cp.async.bulk.tensor.2d, 128-byte swizzle, no cluster qualifiers: every
//     CTA fetches its own tiles, which is also the only form allowed to read a peer GPU's memory),
//   * tcgen05.mma is issued by one thread; the weight tile is the A operand (M = 128 rows), the token tile
//     is the B operand (N = 16..64 tokens), accumulators live in tensor memory,
//   * FP8 variant: weights e4m3 with one fp32 scale per 128x128 block, activations e4m3 with one fp32 scale
//     per token and 128-wide K block.  Each K block is accumulated on its own in one of two TMEM buffers
//     and folded into fp32 registers with its scale product while the next block is being multiplied,
//   * BF16 variant: plain kind::f16 accumulation over the whole K extent, one read-back at the end.
//
// Warp roles: warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..5 = epilogue (each owns
// the 32 TMEM lanes its warp id selects).  Every wait is bounded by %globaltimer: on expiry the CTA raises
// an abort flag, all roles leave their loops, outstanding copies are given time to land, TMEM is freed
// and kStatusPipeTimeout is OR-ed into the caller's status word.
//
// The reference has no counterpart (its many-row GEMMs run inside SGLang during prefill); the block-scale
// handling follows the checkpoint format read by nex_n2_5_pro/weights.py:27-31.
#include <cuda.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <mutex>
#include <unordered_map>

#include "api.h"
#include "common.cuh"
#include "mma_gemv.cuh"
#include "tc_common.cuh"

namespace {
using namespace nexrt;
using namespace nexrt::tc;

template <int BN>
struct Layout {
    static constexpr int kA = kBM * kSpan;                 // 16 KB
    static constexpr int kB = BN * kSpan;
    static constexpr int kStage = kA + ((kB + 1023) / 1024) * 1024;
    static constexpr int kBars = 1024;
    // barriers first, then the stages, then the activation scales of this token tile ([kb][n], FP8 only)
    static int total(int kblocks, bool fp8) { return kBars + kStages * kStage + (fp8 ? kblocks * BN * 4 : 0) + 1024; }
};

struct Args {
    const float* sw;      // [ceil(R/128), KB] weight block scales (fp8 only)
    const float* sx;      // [T, KB] activation scales (fp8 only)
    void* y;              // [T, ldy]
    int T, R, KB, ldy;    // KB: K blocks of the whole product
    int out_mode;         // 0 fp32 store, 1 bf16 store, 2 fp32 accumulate (y += result)
    int* status;
    // split K: blockIdx.z walks K blocks [z * kb_per, (z + 1) * kb_per) and writes its partial sums to plane z of
    // y (planes are T * ldy elements apart); the consumer adds the planes in a fixed order
    int kb_per;
    // grouped K (expert down projections stored as [group][rows][group_kb * 128]): K block kb of the product is
    // block kb % group_kb of group kb / group_kb, whose rows start at (kb / group_kb) * group_rows; 0 = plain matrix
    int group_kb, group_rows;
    // optional skip list (dense expert products): used[g] == 0 means nothing is routed to group g.  Plain matrix: a row tile
    // whose group (m0 / used_rows) is unused does nothing; grouped K: the K blocks of unused groups are left out of the walk
    const int* used;
    int used_rows;
};

template <bool FP8, int BN>
__global__ void __launch_bounds__(kThreads, 2) tc_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, Args a) {
    using L = Layout<BN>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ float sws[kMaxKBlocks];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base);
    uint8_t* smem = base + L::kBars;
    float* sxs = reinterpret_cast<float*>(smem + kStages * L::kStage);
    // bars: [0, S) full, [S, 2S) empty, then kAccBufs tmem_full and kAccBufs tmem_empty
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * kStages + 2 * kAccBufs);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 2 * kAccBufs + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
    auto tfull = [&](int b) { return bar0 + 8u * (2 * kStages + b); };
    auto tempty = [&](int b) { return bar0 + 8u * (2 * kStages + kAccBufs + b); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * kBM, n0 = blockIdx.x * BN;     // token tiles of one weight tile are neighbours: they share it in L2
    // launched with programmatic serialisation: the grid may become resident while its predecessor drains; nothing of the
    // predecessor's output (skip list, activations, scales) is touched before the wait
    pdl_launch_dependents();
    pdl_wait();
    if (a.used != nullptr && a.group_kb == 0 && a.used[m0 / a.used_rows] == 0) return;   // the whole CTA: nothing allocated yet
    __shared__ unsigned short s_kb[kMaxKBlocks];               // K blocks this CTA walks (offsets from kb0), in order
    __shared__ int s_nact;
    const int kb0 = static_cast<int>(blockIdx.z) * a.kb_per;     // first K block of this CTA's range
    const int KBrange = max(0, min(a.kb_per, a.KB - kb0));
    constexpr uint32_t kCols = kAccBufs * BN;
    if (threadIdx.x < 32) {
        // compact the range to the blocks of used groups (all of them without a skip list)
        const int l = threadIdx.x;
        bool f[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int kb = l + 32 * h;
            f[h] = kb < KBrange && (a.used == nullptr || a.group_kb == 0 || a.used[(kb0 + kb) / a.group_kb] != 0);
        }
        const unsigned b0 = __ballot_sync(0xffffffffu, f[0]), b1 = __ballot_sync(0xffffffffu, f[1]);
        const unsigned lt = (1u << l) - 1u;
        if (f[0]) s_kb[__popc(b0 & lt)] = static_cast<unsigned short>(l);
        if (f[1]) s_kb[__popc(b0) + __popc(b1 & lt)] = static_cast<unsigned short>(l + 32);
        if (l == 0) s_nact = __popc(b0) + __popc(b1);
    }                 // power of two, 64..256 columns

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
        }
        for (int b = 0; b < kAccBufs; ++b) {
            mbar_init(tfull(b), 1);
            mbar_init(tempty(b), 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), kCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int KB = s_nact;

    if (warp == 0) {
        // ---- TMA producer -----------------------------------------------------------------------------
        if (lane == 0) {
            for (int kb = 0; kb < KB; ++kb) {
                const int s = kb % kStages;
                if (!mbar_wait(empty(s), ((kb / kStages) & 1) ^ 1, abort_flag)) break;
                mbar_expect_tx(full(s), L::kA + L::kB);
                const uint32_t dst = smem_u32(smem + s * L::kStage);
                constexpr int kElems = FP8 ? kSpan : kSpan / 2;          // elements of K per block
                const int kg = kb0 + s_kb[kb];
                if (a.group_kb > 0) tma_load_2d(dst, &map_w, (kg % a.group_kb) * kElems, (kg / a.group_kb) * a.group_rows + m0, full(s));
                else tma_load_2d(dst, &map_w, kg * kElems, m0, full(s));
                tma_load_2d(dst + L::kA, &map_x, kg * kElems, n0, full(s));
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer -------------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc<FP8>(BN);
            for (int kb = 0; kb < KB; ++kb) {
                const int s = kb % kStages;
                const int buf = FP8 ? (kb % kAccBufs) : 0;
                if (FP8 && !mbar_wait(tempty(buf), ((kb / kAccBufs) & 1) ^ 1, abort_flag)) break;
                if (!mbar_wait(full(s), (kb / kStages) & 1, abort_flag)) break;
                tc_fence_after();
                const uint32_t a0 = smem_u32(smem + s * L::kStage);
                const uint64_t da = smem_desc(a0), db = smem_desc(a0 + L::kA);
#pragma unroll
                for (int k = 0; k < 4; ++k)     // 4 x 32 bytes of K per stage; +2 in the 16-byte address field
                    tc_mma<FP8>(tmem_base + buf * BN, da + 2u * k, db + 2u * k, idesc, (FP8 ? k : (kb | k)) != 0);
                tc_commit(empty(s));            // smem stage reusable once these MMAs have read it
                if (FP8 || kb == KB - 1) tc_commit(tfull(buf));
            }
        }
    } else {
        // ---- epilogue: 4 warps, warp q owns TMEM lanes [32q, 32q+32) ----------------------------------
        const int q = warp & 3;
        const int row = m0 + 32 * q + lane;
        const int et = threadIdx.x - 64;        // 0..127
        if (FP8) {
            // activation scales of this token tile, read along K (neighbouring threads, neighbouring addresses)
            for (int i = et; i < KB * BN; i += 128) {
                const int n = i / KB, kb = i % KB;
                sxs[kb * BN + n] = (n0 + n < a.T) ? a.sx[static_cast<size_t>(n0 + n) * a.KB + kb0 + s_kb[kb]] : 0.f;
            }
            for (int i = et; i < KB; i += 128) {     // weight block scales of this row tile
                const int kg = kb0 + s_kb[i];
                sws[i] = a.group_kb > 0 ? __ldg(a.sw + (static_cast<size_t>(kg / a.group_kb) * (a.group_rows / kBM) + blockIdx.y) * a.group_kb + kg % a.group_kb)
                                        : __ldg(a.sw + static_cast<size_t>(blockIdx.y) * a.KB + kg);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        float acc[BN];
#pragma unroll
        for (int n = 0; n < BN; ++n) acc[n] = 0.f;
        bool ok = true;
        const int rounds = FP8 ? KB : 1;
        for (int r = 0; r < rounds && ok; ++r) {
            const int buf = FP8 ? (r % kAccBufs) : 0;
            ok = mbar_wait(tfull(buf), FP8 ? ((r / kAccBufs) & 1) : 0, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(32 * q) << 16) + buf * BN;
            if (FP8) {
                const float w = sws[r];
                const float4* sx4 = reinterpret_cast<const float4*>(sxs + r * BN);
                // all columns of the block are requested before the one wait (a tensor-memory round trip per 16 columns
                // was what bounded a CTA's K walk), and the buffer goes back to the issuer before the arithmetic
                float p[BN];
#pragma unroll
                for (int c = 0; c < BN; c += 16) tmem_ld16(taddr + c, p + c);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty(buf));
#pragma unroll
                for (int n = 0; n < BN; n += 4) {
                    const float4 sc = sx4[n >> 2];
                    acc[n] = fmaf(p[n], w * sc.x, acc[n]);
                    acc[n + 1] = fmaf(p[n + 1], w * sc.y, acc[n + 1]);
                    acc[n + 2] = fmaf(p[n + 2], w * sc.z, acc[n + 2]);
                    acc[n + 3] = fmaf(p[n + 3], w * sc.w, acc[n + 3]);
                }
            } else {
#pragma unroll
                for (int c = 0; c < BN; c += 16) tmem_ld16(taddr + c, acc + c);
                tmem_ld_wait();
            }
        }
        if (ok && row < a.R) {
            const size_t plane = static_cast<size_t>(blockIdx.z) * a.T * a.ldy;
#pragma unroll
            for (int n = 0; n < BN; ++n) {
                if (n0 + n >= a.T) break;
                const size_t o = plane + static_cast<size_t>(n0 + n) * a.ldy + row;
                if (a.out_mode == 0) {
                    static_cast<float*>(a.y)[o] = acc[n];
                } else if (a.out_mode == 1) {
                    static_cast<__nv_bfloat16*>(a.y)[o] = __float2bfloat16(acc[n]);
                } else {
                    static_cast<float*>(a.y)[o] += acc[n];
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // give copies and MMAs that were already issued time to land before the memory they target is released
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
}

// ---- row-wise activation quantisation: optional RMSNorm, then e4m3 with one scale per 128 columns ---------
// x [T, ldx] bf16 (or fp32 when x_fp32), gamma [K] fp32 or null, xq [P * T, K] e4m3, sx [P * T, K/128] fp32: P planes of T
// rows each, plane p the residual of the planes before it at a 16 times finer scale (the step kernels' exact split), so
// that a GEMM over all P * T rows followed by a sum of its row blocks multiplies by x to 2^-4, 2^-8 or 2^-12 of each value.
template <int P>
__global__ void act_quant_kernel(const void* __restrict__ x, int x_fp32, int ldx, const float* __restrict__ gamma, float eps,
                                 __nv_fp8_storage_t* __restrict__ xq, float* __restrict__ sx, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int KB = K / 128;
    __shared__ float red[32];
    __shared__ float rinv_s;
    auto load = [&](int k) -> float {
        return x_fp32 ? static_cast<const float*>(x)[static_cast<size_t>(t) * ldx + k]
                      : __bfloat162float(static_cast<const __nv_bfloat16*>(x)[static_cast<size_t>(t) * ldx + k]);
    };
    float rinv = 1.f;
    if (gamma) {
        float ss = 0.f;
        for (int k = threadIdx.x; k < K; k += blockDim.x) {
            const float v = load(k);
            ss += v * v;
        }
        ss = warp_sum(ss);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x < 32) {
            float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
            v = warp_sum(v);
            if (threadIdx.x == 0) rinv_s = rsqrtf(v / K + eps);
        }
        __syncthreads();
        rinv = rinv_s;
    }
    // one warp per 128-column block
    for (int kb = threadIdx.x >> 5; kb < KB; kb += blockDim.x >> 5) {
        float v[4];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = kb * 128 + (threadIdx.x & 31) * 4 + i;
            v[i] = load(k) * rinv * (gamma ? gamma[k] : 1.f);
            amax = fmaxf(amax, fabsf(v[i]));
        }
        amax = warp_max(amax);
        float scale = fmaxf(amax, 1e-12f) / 448.f;
        const float inv = 1.f / scale;
        float r[4] = {v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv};
        uint32_t out[P];
        split4<P>(r, out);
#pragma unroll
        for (int p = 0; p < P; ++p) {
            const size_t row = static_cast<size_t>(p) * gridDim.x + t;
            reinterpret_cast<uint32_t*>(xq + row * K + kb * 128)[threadIdx.x & 31] = out[p];
            if ((threadIdx.x & 31) == 0) sx[row * KB + kb] = scale;
            scale *= kTermInv;
        }
    }
}

template <bool FP8, int BN>
cudaError_t launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const Args& a, cudaStream_t stream) {
    using L = Layout<BN>;
    static bool configured = false;
    auto kern = tc_gemm_kernel<FP8, BN>;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total(kMaxKBlocks, FP8));
        if (e != cudaSuccess) return e;
        configured = true;
    }
    if (const cudaError_t e = pipe_budget_install()) return e;
    dim3 grid((a.T + BN - 1) / BN, (a.R + kBM - 1) / kBM, (a.KB + a.kb_per - 1) / a.kb_per);
    return static_cast<cudaError_t>(launch(kern, grid, dim3(kThreads), L::total(a.kb_per, FP8), stream, mw, mx, a));
}

}  // namespace

namespace {
// ---- host side: tensor maps ----------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

struct MapKey {
    const void* ptr;
    uint64_t rows, cols, ld;
    uint32_t box_rows, bf16;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows && bf16 == o.bf16; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        for (uint64_t v : {k.rows, k.cols, k.ld, static_cast<uint64_t>(k.box_rows), static_cast<uint64_t>(k.bf16)}) h = h * 1000003u ^ std::hash<uint64_t>()(v);
        return h;
    }
};

}  // namespace

// Row-major [rows, cols] matrix with leading dimension `ld` elements; box = box_rows x one 128-byte span.
bool nexrt::tc::tensor_map(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows, bool bf16) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{ptr, rows, cols, ld, box_rows, bf16 ? 1u : 0u};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const uint32_t esz = bf16 ? 2 : 1;
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * esz) & 15)) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * esz};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(kSpan / esz), box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    const CUresult r = fn(&m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}


extern "C" {

// Y[T, R] = dequant(Xq, sx) * dequant(Wq, sw)^T.  Wq [R, K] e4m3 (row stride ldw), sw [ceil(R/128), K/128],
// Xq [T, K] e4m3 (dense), sx [T, K/128].  K must be a multiple of 128 and at most 8192.
int nexrt_tc_gemm_fp8(const void* wq, const float* sw, int64_t ldw, const void* xq, const float* sx, void* y, int T, int R, int K, int ldy, int out_mode,
                      int* status, void* stream) {
    if (T <= 0 || R <= 0 || K <= 0 || K % 128 || K / 128 > kMaxKBlocks || out_mode < 0 || out_mode > 2) return cudaErrorInvalidValue;
    const int bn = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
    CUtensorMap mw, mx;
    if (!tensor_map(&mw, wq, R, K, ldw, kBM, false) || !tensor_map(&mx, xq, T, K, K, bn, false)) return cudaErrorInvalidValue;
    Args a{sw, sx, y, T, R, K / 128, ldy, out_mode, status, K / 128, 0, 0};
    auto s = static_cast<cudaStream_t>(stream);
    if (bn == 16) return launch_tc<true, 16>(mw, mx, a, s);
    if (bn == 32) return launch_tc<true, 32>(mw, mx, a, s);
    return launch_tc<true, 64>(mw, mx, a, s);
}

// The same product with K split over `ksplit` CTAs per tile (partial sums to ksplit fp32 planes of T * ldy elements each,
// which the consumer adds in plane order) and, when group_rows > 0, with W stored as `groups` matrices of
// [group_rows, group_k] one after the other (expert down projections): K = groups * group_k, R = group_rows, block
// scales sw [groups][group_rows / 128][group_k / 128].  Any K whose per-CTA share is at most 64 blocks.
int nexrt_tc_gemm_fp8_ex(const void* wq, const float* sw, int64_t ldw, const void* xq, const float* sx, void* y, int T, int R, int K, int ldy,
                         int ksplit, int group_k, int group_rows, const int* used, int used_rows, int* status, void* stream) {
    if (T <= 0 || R <= 0 || K <= 0 || K % 128 || ksplit < 1) return cudaErrorInvalidValue;
    const int KB = K / 128, kb_per = (KB + ksplit - 1) / ksplit;
    if (kb_per > kMaxKBlocks) return cudaErrorInvalidValue;
    if (group_rows > 0 && (group_k <= 0 || group_k % 128 || K % group_k || group_rows % kBM || R != group_rows)) return cudaErrorInvalidValue;
    const int bn = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
    CUtensorMap mw, mx;
    const bool okw = group_rows > 0 ? tensor_map(&mw, wq, static_cast<uint64_t>(K / group_k) * group_rows, group_k, ldw, kBM, false)
                                    : tensor_map(&mw, wq, R, K, ldw, kBM, false);
    if (!okw || !tensor_map(&mx, xq, T, K, K, bn, false)) return cudaErrorInvalidValue;
    if (used != nullptr && group_rows == 0 && (used_rows <= 0 || used_rows % kBM)) return cudaErrorInvalidValue;
    Args a{sw, sx, y, T, R, KB, ldy, 0, status, kb_per, group_rows > 0 ? group_k / 128 : 0, group_rows, used, used_rows};
    auto s = static_cast<cudaStream_t>(stream);
    if (bn == 16) return launch_tc<true, 16>(mw, mx, a, s);
    if (bn == 32) return launch_tc<true, 32>(mw, mx, a, s);
    return launch_tc<true, 64>(mw, mx, a, s);
}

// Y[T, R] = X[T, K] * W[R, K]^T, both bf16, fp32 accumulation.  K must be a multiple of 64, at most 4096.
int nexrt_tc_gemm_bf16(const void* w, int64_t ldw, const void* x, int64_t ldx, void* y, int T, int R, int K, int ldy, int out_mode, int* status,
                       void* stream) {
    if (T <= 0 || R <= 0 || K <= 0 || K % 64 || K / 64 > kMaxKBlocks || out_mode < 0 || out_mode > 2) return cudaErrorInvalidValue;
    const int bn = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
    CUtensorMap mw, mx;
    if (!tensor_map(&mw, w, R, K, ldw, kBM, true) || !tensor_map(&mx, x, T, K, ldx, bn, true)) return cudaErrorInvalidValue;
    Args a{nullptr, nullptr, y, T, R, K / 64, ldy, out_mode, status, K / 64, 0, 0};
    auto s = static_cast<cudaStream_t>(stream);
    if (bn == 16) return launch_tc<false, 16>(mw, mx, a, s);
    if (bn == 32) return launch_tc<false, 32>(mw, mx, a, s);
    return launch_tc<false, 64>(mw, mx, a, s);
}

// The bf16 product with K split over ksplit CTAs per tile: fp32 partial planes of T * ldy elements each.
int nexrt_tc_gemm_bf16_ex(const void* w, int64_t ldw, const void* x, int64_t ldx, void* y, int T, int R, int K, int ldy, int ksplit, int* status,
                          void* stream) {
    if (T <= 0 || R <= 0 || K <= 0 || K % 64 || ksplit < 1) return cudaErrorInvalidValue;
    const int KB = K / 64, kb_per = (KB + ksplit - 1) / ksplit;
    if (kb_per > kMaxKBlocks || (KB + kb_per - 1) / kb_per != ksplit) return cudaErrorInvalidValue;   // every plane needs a non-empty K range
    const int bn = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
    CUtensorMap mw, mx;
    if (!tensor_map(&mw, w, R, K, ldw, kBM, true) || !tensor_map(&mx, x, T, K, ldx, bn, true)) return cudaErrorInvalidValue;
    Args a{nullptr, nullptr, y, T, R, KB, ldy, 0, status, kb_per, 0, 0};
    auto s = static_cast<cudaStream_t>(stream);
    if (bn == 16) return launch_tc<false, 16>(mw, mx, a, s);
    if (bn == 32) return launch_tc<false, 32>(mw, mx, a, s);
    return launch_tc<false, 64>(mw, mx, a, s);
}

// Optional RMSNorm (gamma != null) followed by per-row, per-128-column e4m3 quantisation into `terms` (1..3) planes.
int nexrt_act_quant(const void* x, int x_fp32, int ldx, const float* gamma, float eps, void* xq, float* sx, int T, int K, int terms, void* stream) {
    if (T <= 0 || K <= 0 || K % 128 || terms < 1 || terms > 3) return cudaErrorInvalidValue;
    auto go = [&](auto kern) {
        return launch(kern, dim3(T), dim3(256), 0, static_cast<cudaStream_t>(stream), x, x_fp32, ldx, gamma, eps, static_cast<__nv_fp8_storage_t*>(xq), sx, K);
    };
    return terms == 1 ? go(act_quant_kernel<1>) : terms == 2 ? go(act_quant_kernel<2>) : go(act_quant_kernel<3>);
}

}  // extern "C"
