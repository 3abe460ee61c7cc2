// Step plumbing: embedding gather from the control block, the step-end node (sequence advance +
// host-visible mirror of the control block) and small utilities.
//
// Counterparts in the reference: EmbedGatherKernel / M4EmbedGatherKernel / M8EmbedGatherKernel
// (nex_n2_5_pro/kernels/embed/nex_n2_5_pro_embed_gather_ctypes.cu:37-55, …m4_embed_gather:47-81,
// …m8_embed_gather:60-100), CtlMirrorKernel (…util/nex_n2_5_pro_ctl_mirror_ctypes.cu:28-71) and
// ResidualAddKernel (…util/nex_n2_5_pro_residual_add_ctypes.cu:30-43).
#include "api.h"
#include "common.cuh"
#include "gemv_cta.cuh"

namespace nexrt {

int& gemv_threads_ref() {
    static int threads = 512;
    return threads;
}

int& gemv_mode_ref() {
    static int mode = 255;
    return mode;
}

int& pdl_enabled() {
    static int enabled = 1;
    return enabled;
}

unsigned long long& launch_counter() {
    static unsigned long long n = 0;
    return n;
}

float*& partial_out_buffer() {
    static float* buf = nullptr;
    return buf;
}

#ifdef NEXRT_TRACE
unsigned long long*& trace_buffer() {
    static unsigned long long* buf = nullptr;
    return buf;
}
#endif

// x[m] = embed[ids[m]] for the M rows named by the control block.  A negative id (the host
// learns of a failed step one replay late) is clamped to 0 so the speculative replay stays in
// bounds; an id beyond the vocabulary latches a status.
__global__ void __launch_bounds__(256) embed_gather_kernel(const __nv_bfloat16* __restrict__ embed, const int* __restrict__ ctl,
                                                           __nv_bfloat16* __restrict__ x, int* status, int H, int vocab, int M) {
    TraceCta tr;
    tr.begin(kTrEmbed);
    // The first kernel of a step releases its dependents only AFTER its own dependency wait: a later kernel of the step
    // can then only have started once everything before the step (the previous step's commit included) is complete, which
    // is what lets the attention decode read the committed length ahead of its own wait.
    pdl_wait();
    pdl_launch_dependents();
    tr.mark(1);
    const int m = blockIdx.x;
    int id = ctl[kCtlIds + m];
    if (id >= vocab) {
        if (threadIdx.x == 0) atomicCAS(status, 0, kStatusBadToken);
        id = 0;
    }
    if (id < 0) id = 0;
    const uint4* src = reinterpret_cast<const uint4*>(embed + static_cast<size_t>(id) * H);
    uint4* dst = reinterpret_cast<uint4*>(x + static_cast<size_t>(m) * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
    tr.mark(3);
}

// Last node of a step: advance the LL sequence base by the number of channel users of this
// graph, copy the control block into host-mapped memory, then publish the generation flag.
__global__ void __launch_bounds__(32) step_end_kernel(int* ctl, unsigned int* seq, unsigned int n_sites, int* mirror_host,
                                                      unsigned int* mirror_gen, int words) {
    TraceCta tr;
    tr.begin(kTrStepEnd);
    pdl_launch_dependents();
    pdl_wait();
    tr.mark(1);
    if (threadIdx.x == 0 && seq != nullptr) *seq += n_sites;
    if (mirror_host != nullptr) {
        const unsigned int gen = *mirror_gen + 1;
        int* dst = mirror_host + (gen & 1u) * (words + 1);
        if (static_cast<int>(threadIdx.x) < words) dst[threadIdx.x] = ctl[threadIdx.x];
        __syncwarp();
        __threadfence_system();
        if (threadIdx.x == 0) {
            *reinterpret_cast<volatile int*>(dst + words) = static_cast<int>(gen);
            *mirror_gen = gen;
        }
    }
    tr.mark(3);
}

// Empty node for the launch-floor fit: waits for its predecessor, optionally spins `body_ns` on %globaltimer, leaves.
__global__ void null_kernel(unsigned long long body_ns, int early_release, unsigned long long* clock_out) {
    if (early_release) pdl_launch_dependents();
    pdl_wait();
    const long long c0 = clock64();
    const unsigned long long t0 = globaltimer_ns();
    if (body_ns) {
        while (globaltimer_ns() - t0 < body_ns) {}
    }
    if (clock_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        // SM cycles against wall-clock nanoseconds over the spin: the SM clock this node actually ran at
        clock_out[0] = static_cast<unsigned long long>(clock64() - c0);
        clock_out[1] = globaltimer_ns() - t0;
    }
    if (!early_release) pdl_launch_dependents();
}

__global__ void residual_add_kernel(__nv_bfloat16* x, const float* y, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = __float2bfloat16_rn(__bfloat162float(x[i]) + y[i]);
}

}  // namespace nexrt

using namespace nexrt;

extern "C" int nexrt_set_pdl(int enabled) {
    pdl_enabled() = enabled ? 1 : 0;
    return 0;
}
extern "C" int nexrt_version(void) { return 101; }
extern "C" unsigned long long nexrt_launch_count(void) { return launch_counter(); }
// Library-baseline arm (fp32 [8][H] buffer or null): see partial_out_buffer() in common.cuh.
extern "C" int nexrt_set_partial_out(void* buffer) {
    partial_out_buffer() = static_cast<float*>(buffer);
    return 0;
}
// Trace build only: device buffer of kTraceKinds cursors followed by kTraceKinds * kTraceSlots records of kTraceWords
// 64-bit words (see common.cuh); null switches the timeline off.  Run one eager step after changing it and before
// capturing a graph, because every translation unit picks the address up at its next launch.
extern "C" int nexrt_set_trace(void* buffer) {
#ifdef NEXRT_TRACE
    trace_buffer() = static_cast<unsigned long long*>(buffer);
    return 0;
#else
    (void)buffer;
    return cudaErrorNotSupported;
#endif
}
extern "C" int nexrt_trace_layout(int* kinds, int* slots, int* words) {
    *kinds = kTraceKinds; *slots = kTraceSlots; *words = kTraceWords;
    return 0;
}
extern "C" int nexrt_set_gemv_mode(int mode) {
    gemv_mode_ref() = mode;
    return 0;
}
extern "C" int nexrt_set_gemv_threads(int threads) {
    if (threads != 256 && threads != 512) return cudaErrorInvalidValue;
    gemv_threads_ref() = threads;
    return 0;
}

extern "C" int nexrt_embed_gather(const void* embed, const void* ctl, void* x, void* status, int H, int vocab, int M, void* stream) {
    if (M < 1 || M > kMaxRows || H % 8) return cudaErrorInvalidValue;
    return launch(embed_gather_kernel, dim3(M), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(embed),
                  static_cast<const int*>(ctl), static_cast<__nv_bfloat16*>(x), static_cast<int*>(status), H, vocab, M);
}

extern "C" int nexrt_step_end(void* ctl, void* seq, unsigned int n_sites, void* mirror_host, void* mirror_gen, int words, void* stream) {
    if (words < 0 || words > 32) return cudaErrorInvalidValue;
    return launch(step_end_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), static_cast<int*>(ctl),
                  static_cast<unsigned int*>(seq), n_sites, static_cast<int*>(mirror_host), static_cast<unsigned int*>(mirror_gen), words);
}

// One empty kernel node of `grid` CTAs x `block` threads with `smem` bytes of dynamic shared memory (launched like every
// step kernel: programmatic dependent launch when it is switched on).  The fit latency(K) = a + b K over K such nodes
// separates the per-node cost of a captured graph from the work inside the nodes (the reference's `--scale` mode,
// nex_n2_5_pro/decode_engine.py:549-630).
extern "C" int nexrt_null_node(int grid, int block, int smem, unsigned long long body_ns, int early_release, void* clock_out, void* stream) {
    if (grid < 1 || block < 32 || block > 1024 || smem < 0 || smem > 200 * 1024) return cudaErrorInvalidValue;
    return launch(null_kernel, dim3(grid), dim3(block), static_cast<size_t>(smem), static_cast<cudaStream_t>(stream), body_ns, early_release,
                  static_cast<unsigned long long*>(clock_out));
}

extern "C" int nexrt_residual_add(void* x, const void* y, int n, void* stream) {
    return launch(residual_add_kernel, dim3((n + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream),
                  static_cast<__nv_bfloat16*>(x), static_cast<const float*>(y), n);
}
