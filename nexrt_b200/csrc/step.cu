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
    static int mode = 63;
    return mode;
}

int& pdl_enabled() {
    static int enabled = 1;
    return enabled;
}

// x[m] = embed[ids[m]] for the M rows named by the control block.  A negative id (the host
// learns of a failed step one replay late) is clamped to 0 so the speculative replay stays in
// bounds; an id beyond the vocabulary latches a status.
__global__ void __launch_bounds__(256) embed_gather_kernel(const __nv_bfloat16* __restrict__ embed, const int* __restrict__ ctl,
                                                           __nv_bfloat16* __restrict__ x, int* status, int H, int vocab, int M) {
    pdl_launch_dependents();
    pdl_wait();
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
}

// Last node of a step: advance the LL sequence base by the number of channel users of this
// graph, copy the control block into host-mapped memory, then publish the generation flag.
__global__ void __launch_bounds__(32) step_end_kernel(int* ctl, unsigned int* seq, unsigned int n_sites, int* mirror_host,
                                                      unsigned int* mirror_gen, int words) {
    pdl_launch_dependents();
    pdl_wait();
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
extern "C" int nexrt_version(void) { return 100; }
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

extern "C" int nexrt_residual_add(void* x, const void* y, int n, void* stream) {
    return launch(residual_add_kernel, dim3((n + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream),
                  static_cast<__nv_bfloat16*>(x), static_cast<const float*>(y), n);
}
