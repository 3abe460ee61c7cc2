// Shared device helpers for the sm_100a decode kernels: FP8 decode, warp reductions, bounded
// waits on %globaltimer, programmatic dependent launch (PDL) and the launch wrapper.
//
// Counterpart of the reference's nex_n2_5_pro/kernels/common/{pdl.cuh,oproj_common.cuh}; the
// geometry here is a run-time argument, not constexpr, so one binary serves every
// tensor-parallel width and the shrunk test geometry.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace nexrt {

constexpr int kScaleBlock = 128;   // edge of one FP8 scale block
constexpr int kMaxRows = 8;        // most token rows one step carries (M=1 decode, 4 MTP, 8 DFlash)
constexpr int kMaxWorld = 8;

// Sticky status codes written into a status word by any kernel that gives up.
enum Status : int {
    kStatusOk = 0,
    kStatusReduceTimeout = 1,   // a peer's packet did not arrive inside the wait budget
    kStatusNonFinite = 2,       // sampler saw a non-finite winning logit
    kStatusBadConfig = 3,       // sampler configuration out of range
    kStatusCpTimeout = 4,       // context-parallel partial did not arrive
    kStatusBadToken = 5,        // token id outside the vocabulary
    kStatusPipeTimeout = 6,     // an mbarrier / TMA / tensor-core completion did not arrive
};

// Control block shared by all three decode modes (int32[32]).  Python mirror: runtime/control.py.
enum Ctl : int {
    kCtlCommittedLen = 0,   // tokens whose state is committed == position of row 0
    kCtlStatus = 1,         // sticky OR of failure bits, 0 == healthy
    kCtlCommitCount = 2,    // tokens committed by the last step
    kCtlPending = 3,        // next row-0 token (sampled by the last step)
    kCtlIds = 4,            // [8] ids of the rows of the next step; ids[0] == pending
    kCtlEmitted = 12,       // [8] tokens emitted by the last step
    kCtlRows = 20,          // live rows of the step (1, 4 or 8)
    kCtlForcedCommit = 21,  // >0: commit exactly this many tokens (fixed-acceptance benchmarking)
    kCtlStepEpoch = 22,     // steps executed
    kCtlAccepted = 23,      // drafts accepted by the last step
    kCtlEos = 24,           // end-of-sequence id or -1
    kCtlStopPos = 25,       // index in emitted[] of the first EOS, or -1
    kCtlFlags = 26,
    kCtlForcedSeed = 27,    // seed of the forced-commit schedule (0: constant forced_commit)
    kCtlForcedMean10 = 28,  // mean accepted length x10 of the seeded schedule
    kCtlWords = 32,
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- FP8 e4m3 -> fp32 ---------------------------------------------------------------------
__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t v) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(v));
    __half2 h = *reinterpret_cast<__half2*>(&h2);
    return __half22float2(h);
}

__device__ __forceinline__ void e4m3x4_to_float4(uint32_t w, float* f) {
    float2 a = e4m3x2_to_float2(static_cast<uint16_t>(w & 0xffffu));
    float2 b = e4m3x2_to_float2(static_cast<uint16_t>(w >> 16));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// 16 fp8 weights (one uint4) dotted with 16 fp32 activations.
__device__ __forceinline__ float dot16_fp8(const uint4& w, const float* __restrict__ x) {
    float f[4], acc = 0.f;
    e4m3x4_to_float4(w.x, f); acc = fmaf(f[0], x[0], acc); acc = fmaf(f[1], x[1], acc); acc = fmaf(f[2], x[2], acc); acc = fmaf(f[3], x[3], acc);
    e4m3x4_to_float4(w.y, f); acc = fmaf(f[0], x[4], acc); acc = fmaf(f[1], x[5], acc); acc = fmaf(f[2], x[6], acc); acc = fmaf(f[3], x[7], acc);
    e4m3x4_to_float4(w.z, f); acc = fmaf(f[0], x[8], acc); acc = fmaf(f[1], x[9], acc); acc = fmaf(f[2], x[10], acc); acc = fmaf(f[3], x[11], acc);
    e4m3x4_to_float4(w.w, f); acc = fmaf(f[0], x[12], acc); acc = fmaf(f[1], x[13], acc); acc = fmaf(f[2], x[14], acc); acc = fmaf(f[3], x[15], acc);
    return acc;
}

__device__ __forceinline__ void unpack16_fp8(const uint4& w, float* f) {
    e4m3x4_to_float4(w.x, f);
    e4m3x4_to_float4(w.y, f + 4);
    e4m3x4_to_float4(w.z, f + 8);
    e4m3x4_to_float4(w.w, f + 12);
}

__device__ __forceinline__ void unpack8_bf16(const uint4& w, float* f) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(u[i] << 16);
        f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}

// Streaming 16-byte weight load: read-only path, do not keep in L1.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// One constant fp32 (a block scale) through the read-only path, as a volatile asm so that the load is ISSUED where it is
// written: a plain __ldg may be sunk by the compiler to its first use, which for a scale preloaded before the dependency
// wait means a full L2 round trip inside every iteration of the tensor-core loop that consumes it.
__device__ __forceinline__ float ld_const_f32(const float* p) {
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// Pull a byte range towards L2 with the whole CTA (used in the window before the dependency
// wait, where a kernel may touch only constant weights).
// CTA `b` of `n` pulls its share of [base, base + bytes) towards L2, one 128-byte line per prefetch: the way a kernel
// that is idle before its dependency wait warms the cache for a LATER kernel whose CTAs will not be resident in time to
// preload their weights themselves.
__device__ __forceinline__ void prefetch_l2_slice(const void* base, size_t bytes, int b, int n) {
    if (base == nullptr || bytes == 0) return;
    const size_t lines = (bytes + 127) >> 7, per = (lines + n - 1) / n;
    const size_t lo = static_cast<size_t>(b) * per, hi = lo + per < lines ? lo + per : lines;
    const char* p = static_cast<const char*>(base);
    for (size_t l = lo + threadIdx.x; l < hi; l += blockDim.x) prefetch_l2(p + (l << 7));
}

__device__ __forceinline__ unsigned int redux_max_u32(unsigned int v) {
    unsigned int r;
    asm volatile("redux.sync.max.u32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(v));
    return r;
}
__device__ __forceinline__ unsigned int redux_min_u32(unsigned int v) {
    unsigned int r;
    asm volatile("redux.sync.min.u32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(v));
    return r;
}

__device__ __forceinline__ void prefetch_l2_range(const void* base, size_t bytes) {
    const char* p = static_cast<const char*>(base);
    for (size_t off = static_cast<size_t>(threadIdx.x) * 128; off < bytes; off += static_cast<size_t>(blockDim.x) * 128)
        prefetch_l2(p + off);
}

// ---- programmatic dependent launch ----------------------------------------------------------
// Everything a kernel does before pdl_wait() may overlap the tail of the previous kernel in
// the stream and must therefore touch only data that no kernel of the step writes (weights).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Block-wide sum for blockDim.x <= 1024; `red` is 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    return t;
}


// ---- kernel timeline (trace build only: -DNEXRT_TRACE) ------------------------------------------
// Thread 0 of every CTA records %globaltimer at four points of its life - 0 entry, 1 dependency
// wait over, 2 a kernel-specific midpoint (own product finished, before the ticket / all-reduce),
// 3 exit - into a per-kind record list.  The slot comes from one atomicAdd issued at entry, whose
// latency hides behind the weight preload; the four stores are fire-and-forget.  The regular
// build compiles all of this to nothing, so the product kernels carry no extra registers.
enum TraceKind : int {
    kTrEmbed = 0, kTrGdnFront, kTrGdnCore, kTrOproj, kTrRouter, kTrMoeL1, kTrMoeL2, kTrAttnFront, kTrAttnDecode, kTrHead, kTrStepEnd,
    kTrTcMoeL1, kTrTcMoeL2, kTrTcRows, kTrTcRouter, kTrHelper, kTraceKinds = 16
};
constexpr int kTraceSlots = 20480;        // records per kind
constexpr int kTraceWords = 9;            // cta | grid << 32, t0, t1, t2, t3, then four kernel-specific extras t4..t7
#ifdef NEXRT_TRACE
static __constant__ unsigned long long* c_trace;   // [kTraceKinds cursors][kinds][slots][words]; one copy per translation unit
struct TraceCta {
    unsigned long long* rec;
    unsigned long long t0;
    __device__ __forceinline__ void begin(int kind) {
        rec = nullptr;
        if (threadIdx.x != 0 || c_trace == nullptr) return;
        t0 = globaltimer_ns();
        const unsigned long long slot = atomicAdd(c_trace + kind, 1ull);
        if (slot >= static_cast<unsigned long long>(kTraceSlots)) return;
        rec = c_trace + kTraceKinds + (static_cast<size_t>(kind) * kTraceSlots + slot) * kTraceWords;
        const unsigned long long cta = blockIdx.x + gridDim.x * (blockIdx.y + static_cast<unsigned long long>(gridDim.y) * blockIdx.z);
        rec[0] = cta | (static_cast<unsigned long long>(gridDim.x * gridDim.y * gridDim.z) << 32);
        rec[1] = t0;
    }
    __device__ __forceinline__ void mark(int phase) {
        if (threadIdx.x == 0 && rec != nullptr) rec[1 + phase] = globaltimer_ns();
    }
};
#else
struct TraceCta {
    __device__ __forceinline__ void begin(int) {}
    __device__ __forceinline__ void mark(int) {}
};
#endif

}  // namespace nexrt

// ---- host side --------------------------------------------------------------------------------
namespace nexrt {

// SMs of the current device (asked once per process).
static inline int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    }
    return n;
}

// Process-wide switch: launch with the programmatic-stream-serialisation attribute.
int& pdl_enabled();
// Kernels launched through launch() since the library was loaded (a capture counts its nodes with it).
unsigned long long& launch_counter();
// Library-baseline arm: when set, the projection kernels that end in an all-reduce store their fp32 partial sums here
// instead of exchanging them (see epilogue.cuh); null in normal operation.
float*& partial_out_buffer();

#ifdef NEXRT_TRACE
unsigned long long*& trace_buffer();   // device address of the trace buffer (step.cu), null: off
// Copies the buffer address into this translation unit's constant; called by every launch, so it must have
// run once (an eager step) before a stream capture begins.
static inline int trace_install() {
    static unsigned long long* installed = nullptr;
    unsigned long long* want = trace_buffer();
    if (want == installed) return 0;
    const cudaError_t e = cudaMemcpyToSymbol(c_trace, &want, sizeof(want));
    if (e == cudaSuccess) installed = want;
    return static_cast<int>(e);
}
#endif

template <typename... KArgs, typename... Args>
static inline int launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                  Args... args) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return static_cast<int>(e);
    }
#ifdef NEXRT_TRACE
    if (const int te = trace_install()) return te;
#endif
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    ++launch_counter();
    return static_cast<int>(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}


// Same launch with thread-block clusters of `cluster_x` CTAs along x (grid.x must be a multiple of it).
template <typename... KArgs, typename... Args>
static inline int launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_x, Args... args) {
    if (cluster_x < 1 || grid.x % cluster_x) return static_cast<int>(cudaErrorInvalidValue);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return static_cast<int>(e);
    }
#ifdef NEXRT_TRACE
    if (const int te = trace_install()) return te;
#endif
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    ++launch_counter();
    return static_cast<int>(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}

}  // namespace nexrt
