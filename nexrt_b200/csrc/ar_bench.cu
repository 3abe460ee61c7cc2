// The in-kernel all-reduce in isolation, and the latency floor it is judged against.
//
// Every reduce site of a decode step is the epilogue of a projection kernel (epilogue.cuh).  Two kernels here take that
// epilogue out of its producer so it can be timed alone:
//
//   ll_allreduce_bench_kernel   the production epilogue, unchanged (allreduce_residual), fed with partial sums that are
//                               already in memory: H / 16 CTAs of 256 threads, each reducing its 16 output rows of M
//                               token rows, exactly the geometry of the out-projection and expert-down kernels;
//   ll_pingpong_kernel          one thread on each of two ranks bouncing one tagged 8-byte packet: the one-hop
//                               store -> poll latency of the link, which no all-reduce over it can beat.
//
// The reference quotes its fused reduce kernels against NCCL only (nex_n2_5_pro/decode_engine.py:259-276); the ping-pong
// floor is the stricter yardstick.  Every wait is bounded by the channel's time budget and reports through the
// channel's status word.
#include "epilogue.cuh"

namespace nexrt {

__global__ void __launch_bounds__(256) ll_allreduce_bench_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ x, LLChannel ch,
                                                                 unsigned int site, int M, int H, unsigned long long* stamps) {
    extern __shared__ float res[];   // [M][16]
    const int row0 = blockIdx.x * 16;
    for (int idx = threadIdx.x; idx < M * 16; idx += blockDim.x) res[idx] = partial[static_cast<size_t>(idx / 16) * H + row0 + idx % 16];
    pdl_launch_dependents();
    pdl_wait();                      // the previous use of this inbox half has been read by every CTA of the previous launch
    __syncthreads();
    unsigned long long t0 = 0;
    if (stamps != nullptr && threadIdx.x == 0) t0 = globaltimer_ns();
    allreduce_residual(ch, site, res, M, row0, 16, H, x, false);
    __syncthreads();
    if (stamps != nullptr && threadIdx.x == 0) stamps[blockIdx.x] = globaltimer_ns() - t0;
}

__global__ void ll_seq_advance_kernel(unsigned int* seq, unsigned int n) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) *seq += n;
}

// Ranks a and b bounce `iters` packets; every other rank returns at once.  out[0] = elapsed ns, out[1] = round trips done.
__global__ void ll_pingpong_kernel(LLChannel ch, int a, int b, unsigned int tag0, int iters, int use_mc, unsigned long long* out) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    const int me = ch.rank;
    out[0] = 0;
    out[1] = 0;
    if (me != a && me != b) return;
    const int other = me == a ? b : a;
    const size_t off_out = static_cast<size_t>(me) * ch.slots;        // half 0, source = me, slot 0 (in the receiver's inbox)
    const unsigned long long* in = ch.local + static_cast<size_t>(other) * ch.slots;
    const bool mc = use_mc && ch.mc != nullptr;
    const unsigned long long t0 = globaltimer_ns();
    int done = 0;
    for (int i = 0; i < iters; ++i) {
        const unsigned int tag = (tag0 + static_cast<unsigned int>(i)) | 0x80000000u;
        const unsigned long long pkt = (static_cast<unsigned long long>(tag) << 32) | static_cast<unsigned int>(i);
        if (me == a) {
            if (mc) mc_st_u64(ch.mc + off_out, pkt);
            else st_sys_u64(ch.peer[other] + off_out, pkt);
        }
        const unsigned long long w0 = globaltimer_ns();
        unsigned int spins = 0;
        bool ok = true;
        while (static_cast<unsigned int>(ld_sys_u64(in) >> 32) != tag) {
            if ((++spins & 63u) == 0 && globaltimer_ns() - w0 > ch.budget_ns) { ok = false; break; }
        }
        if (!ok) { atomicCAS(ch.status, 0, kStatusReduceTimeout); break; }
        if (me == b) {
            if (mc) mc_st_u64(ch.mc + off_out, pkt);
            else st_sys_u64(ch.peer[other] + off_out, pkt);
        }
        ++done;
    }
    out[0] = globaltimer_ns() - t0;
    out[1] = static_cast<unsigned long long>(done);
}

}  // namespace nexrt

using namespace nexrt;

extern "C" int nexrt_ll_allreduce_bench(const void* partial, void* x, int M, int H, const NexrtLLChannel* ch, unsigned int site, void* stamps,
                                        void* stream) {
    if (ch == nullptr || M < 1 || M > kMaxRows || H % 16 || (ch->world > 1 && static_cast<size_t>(M) * H > ch->slots)) return cudaErrorInvalidValue;
    return launch(ll_allreduce_bench_kernel, dim3(H / 16), dim3(256), sizeof(float) * 16 * M, static_cast<cudaStream_t>(stream),
                  static_cast<const float*>(partial), static_cast<__nv_bfloat16*>(x), *ch, site, M, H, static_cast<unsigned long long*>(stamps));
}

extern "C" int nexrt_ll_seq_advance(void* seq, unsigned int n, void* stream) {
    return launch(ll_seq_advance_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), static_cast<unsigned int*>(seq), n);
}

extern "C" int nexrt_ll_pingpong(const NexrtLLChannel* ch, int a, int b, unsigned int tag0, int iters, int use_mc, void* out, void* stream) {
    if (ch == nullptr || a == b || a < 0 || b < 0 || a >= ch->world || b >= ch->world || iters < 1 || iters > (1 << 20)) return cudaErrorInvalidValue;
    return launch(ll_pingpong_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), *ch, a, b, tag0, iters, use_mc,
                  static_cast<unsigned long long*>(out));
}
