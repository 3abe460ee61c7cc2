// Device-side building blocks of the tcgen05 kernels (tc_gemm.cu, tc_moe.cu): mbarrier waits bounded on
// %globaltimer, TMA tile loads (no cluster qualifiers), tensor-memory allocation, tcgen05.mma / commit / ld
// wrappers, shared-memory and instruction descriptors - and the host-side tensor-map cache.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace nexrt {
namespace tc {


constexpr int kBM = 128;            // weight rows per CTA tile == MMA M
constexpr int kSpan = 128;          // bytes of K per stage == one swizzle span
constexpr int kStages = 4;           // 4 x (16 KB + token tile): two CTAs fit one SM and overlap each other's prologue and epilogue
constexpr int kAccBufs = 4;         // TMEM accumulator buffers of the FP8 variant (the MMA issuer runs this many K blocks ahead)
constexpr int kThreads = 192;
constexpr int kMaxKBlocks = 64;     // K <= 8192 (fp8) / 4096 (bf16)
// Budget of every mbarrier / TMA / tensor-core completion wait.  It follows NEXRT_WAIT_BUDGET_MS like the waits of the
// packet channel do (one knob bounds every device-side wait of the engine); unset, it is 200 ms.  The value sits in a
// per-translation-unit constant that the launch wrappers install once (pipe_budget_install) before their first launch.
static __constant__ uint64_t c_pipe_budget_ns = 200ull * 1000 * 1000;

static inline cudaError_t pipe_budget_install() {
    static bool done = false;
    if (done) return cudaSuccess;
    done = true;
    const char* env = getenv("NEXRT_WAIT_BUDGET_MS");
    if (env == nullptr || *env == 0) return cudaSuccess;
    const double ms = atof(env);
    if (!(ms > 0.0)) return cudaSuccess;
    const uint64_t ns = static_cast<uint64_t>(ms * 1e6);
    return cudaMemcpyToSymbol(c_pipe_budget_ns, &ns, sizeof(ns));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises the CTA's abort flag) when the budget runs out or when another
// role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t it = 0;; ++it) {
        if (mbar_try(bar, parity)) return true;
        if ((it & 63u) == 63u) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > c_pipe_budget_ns) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]^T; `accumulate` == 0 overwrites D.
template <bool FP8>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (FP8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// 16 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// 4 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, float* v) {
    uint32_t r[4];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are one 128-byte swizzle span: rows 128 B
// apart, groups of 8 rows 1024 B apart (stride byte offset), descriptor version 1, layout SWIZZLE_128B.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor: fp32 accumulator, both operands K-major, N in units of 8, M in units of 16.
template <bool FP8>
__host__ __device__ constexpr uint32_t instr_desc(int bn) {
    const uint32_t fmt = FP8 ? 0u /* e4m3 */ : 1u /* bf16 */;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(bn >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
}


// Row-major [rows, cols] matrix with leading dimension `ld` elements; box = box_rows x one 128-byte span.
// Encoded maps are cached per (pointer, shape); returns false when the driver entry point is missing or the
// operand breaks TMA's alignment rules.
bool tensor_map(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows, bool bf16);

}  // namespace tc
}  // namespace nexrt
