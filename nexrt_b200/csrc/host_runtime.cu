// Host-side runtime pieces that PyTorch does not provide: a peer-shareable device allocation
// (CUDA IPC: the fallback symmetric-memory substrate when NVSwitch multicast objects cannot be
// created), host-mapped pinned memory for the control-block mirror, and a tiny spin-wait on a
// host flag.
//
// The reference gets peer addresses and the multicast address from
// torch.distributed._symmetric_memory only and refuses to start without multicast
// (nex_n2_5_pro/gdn.py:178-198); its mirror allocates with cudaHostAlloc(mapped) through ctypes
// (nex_n2_5_pro/ctl_mirror.py:38-65).
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <thread>

#include "api.h"

extern "C" int nexrt_ipc_alloc(size_t bytes, void** ptr) {
    cudaError_t e = cudaMalloc(ptr, bytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    return static_cast<int>(cudaMemset(*ptr, 0, bytes));
}

extern "C" int nexrt_ipc_get_handle(void* ptr, void* handle64) {
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
    if (e != cudaSuccess) return static_cast<int>(e);
    static_assert(sizeof(h) == 64, "CUDA IPC handle is 64 bytes");
    std::memcpy(handle64, &h, sizeof(h));
    return 0;
}

extern "C" int nexrt_ipc_open(const void* handle64, void** ptr) {
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, sizeof(h));
    return static_cast<int>(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}

extern "C" int nexrt_ipc_close(void* ptr) { return static_cast<int>(cudaIpcCloseMemHandle(ptr)); }
extern "C" int nexrt_ipc_free(void* ptr) { return static_cast<int>(cudaFree(ptr)); }

// Pinned host memory that the device can write through `*dev` and the host can read through
// `*host` with no copy, event or synchronise call.
extern "C" int nexrt_host_mapped_alloc(size_t bytes, void** host, void** dev) {
    cudaError_t e = cudaHostAlloc(host, bytes, cudaHostAllocMapped);
    if (e != cudaSuccess) return static_cast<int>(e);
    std::memset(*host, 0, bytes);
    return static_cast<int>(cudaHostGetDevicePointer(dev, *host, 0));
}

extern "C" int nexrt_host_mapped_free(void* host) { return static_cast<int>(cudaFreeHost(host)); }

// Spin (with a short sleep) until *flag == want or the timeout passes.  Returns 0 on success,
// 1 on timeout.  Runs without the Python GIL because ctypes releases it around the call.
extern "C" int nexrt_host_wait_flag(const volatile int* flag, int want, double timeout_s) {
    const auto t0 = std::chrono::steady_clock::now();
    unsigned spins = 0;
    while (*flag != want) {
        if ((++spins & 0x3ff) == 0) {
            const double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            if (el > timeout_s) return 1;
            if (el > 0.002) std::this_thread::sleep_for(std::chrono::microseconds(20));
        }
    }
    std::atomic_thread_fence(std::memory_order_acquire);
    return 0;
}
