// LM head fused with vocab-parallel distributed top-k, the sampler and the accept / commit step.
//
// One launch per step does all of: final RMSNorm, the bf16 GEMV over this rank's vocabulary
// rows for 1..8 token rows, a per-CTA top-k (k <= 28) of its rows, and - in whichever CTA takes
// the last ticket - the merge of the per-CTA candidate lists, the exchange of this rank's
// top-k with every peer as self-tagged 8-byte packets over the LL channel, the merge of the
// world's candidates, temperature / top-k / top-p sampling with the position-keyed splitmix64
// generator, the prefix accept of speculative rows and the single-writer commit into the
// control block (committed_len is written last).
//
// Replaces the reference's LmHeadGemvRowRmsCta0Kernel, ProducerKernel, ReducerKernel and
// SamplerKernel (nex_n2_5_pro/kernels/head/nex_n2_5_pro_lmhead_gemv_ctypes.cu:39-85,
// …lmhead_topk_ctypes.cu:46-147, …lmhead_sampler_ctypes.cu:35-141), their M=4 / M=8 families
// (…m4_lmhead_gemm, m4_sampling:45-342, m8_lmhead_gemm, m8_sampling) and the greedy draft
// argmax exchanges (…mtp/nex_n2_5_pro_mtp_draft_argmax_ctypes.cu:86-151,
// …dflash/nex_n2_5_pro_dflash_argmax_ctypes.cu:35-114).  Candidates are 64-bit keys
// (order-preserving image of the fp32 logit in the high word, ~token id in the low word), so a
// plain integer max picks the largest logit and, on ties, the lowest token id.
#include "api.h"
#include "gemv.cuh"
#include "gemv_cta.cuh"
#include "ll.cuh"

namespace nexrt {

constexpr int kMaxTopK = 28;
constexpr int kExportWords = 64;   // per row: ids[28] | prob bits[28] | target | kept | pad

__device__ __forceinline__ unsigned int ordered_f32(float f) {
    if (f != f) return 0xffffffffu;                    // NaN wins so that the sampler reports it
    const unsigned int b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float unordered_f32(unsigned int o) {
    if (o == 0xffffffffu) return __uint_as_float(0x7fc00000u);
    return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}
__device__ __forceinline__ unsigned long long make_key(float v, int id) {
    return (static_cast<unsigned long long>(ordered_f32(v)) << 32) | static_cast<unsigned int>(~id);
}
__device__ __forceinline__ float key_val(unsigned long long k) { return unordered_f32(static_cast<unsigned int>(k >> 32)); }
__device__ __forceinline__ int key_id(unsigned long long k) { return static_cast<int>(~static_cast<unsigned int>(k)); }

__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long t = __shfl_xor_sync(0xffffffffu, v, o);
        v = t > v ? t : v;
    }
    return v;
}

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long v) {
    v += 0x9E3779B97F4A7C15ull;
    v = (v ^ (v >> 30)) * 0xBF58476D1CE4E5B9ull;
    v = (v ^ (v >> 27)) * 0x94D049BB133111EBull;
    return v ^ (v >> 31);
}
// uniform in [0,1) for an absolute position: hash(request seed, position), top 24 bits.
__device__ __forceinline__ float seeded_uniform(unsigned long long seed, unsigned int pos) {
    const unsigned long long h = splitmix64(seed ^ splitmix64(static_cast<unsigned long long>(pos)));
    return static_cast<float>(h >> 40) * (1.0f / 16777216.0f);
}

struct SamplingCfg {
    unsigned long long seed;
    float temperature, top_p;
    int top_k;
    int bad;
};
__device__ __forceinline__ SamplingCfg read_sampling(const unsigned long long* words) {
    SamplingCfg c;
    c.seed = words[0];
    c.temperature = __uint_as_float(static_cast<unsigned int>(words[1]));
    c.top_p = __uint_as_float(static_cast<unsigned int>(words[1] >> 32));
    const long long k = static_cast<long long>(words[2]);
    c.bad = !(k >= 1 && k <= kMaxTopK) || !(c.temperature >= 0.f) || !(c.top_p > 0.f && c.top_p <= 1.f) || isinf(c.temperature);
    c.top_k = c.bad ? 1 : static_cast<int>(k);
    return c;
}

// Sample one row from its k sorted candidates (descending).  Returns the token, or -1 and a status.
__device__ __forceinline__ int sample_row(const unsigned long long* keys, int k, const SamplingCfg& cfg, unsigned int pos, int* status,
                                          int* export_row) {
    float vals[kMaxTopK], probs[kMaxTopK];
    const float v0 = key_val(keys[0]);
    if (!(fabsf(v0) <= 3.0e38f)) { *status = kStatusNonFinite; return -1; }
    int kept = 1, pick = 0;
    if (cfg.temperature > 0.f && k > 1) {
        float sum = 0.f;
        for (int i = 0; i < k; ++i) {
            vals[i] = key_val(keys[i]);
            probs[i] = __expf((vals[i] - v0) / cfg.temperature);
            sum += probs[i];
        }
        float cum = 0.f;
        kept = k;
        for (int i = 0; i < k; ++i) {
            probs[i] /= sum;
            cum += probs[i];
            if (cum >= cfg.top_p) { kept = i + 1; break; }
        }
        float mass = 0.f;
        for (int i = 0; i < kept; ++i) mass += probs[i];
        if (!(mass > 0.f)) { *status = kStatusNonFinite; return -1; }
        const float u = seeded_uniform(cfg.seed, pos);
        float cdf = 0.f;
        pick = kept - 1;
        for (int i = 0; i < kept; ++i) {
            probs[i] /= mass;
            cdf += probs[i];
            if (cdf >= u) { pick = i; break; }
        }
        for (int i = pick + 1; i < kept; ++i) probs[i] /= mass;
    } else {
        probs[0] = 1.f;
    }
    const int token = key_id(keys[pick]);
    if (export_row) {
        for (int i = 0; i < kMaxTopK; ++i) {
            export_row[i] = i < k ? key_id(keys[i]) : -1;
            export_row[kMaxTopK + i] = i < kept ? __float_as_int(probs[i]) : 0;
        }
        export_row[2 * kMaxTopK] = token;
        export_row[2 * kMaxTopK + 1] = kept;
    }
    return token;
}

// Seeded forced-commit schedule: commit counts in [1, M] whose mean is mean10 / 10.
__device__ __forceinline__ int forced_schedule(unsigned int seed, unsigned int epoch, int mean10, int M) {
    const unsigned long long h = splitmix64((static_cast<unsigned long long>(seed) << 32) ^ epoch);
    const int base = mean10 / 10, frac = mean10 % 10;
    const int up = (static_cast<int>(h % 10) < frac) ? 1 : 0;
    int w = min(base - 1, M - base - (frac ? 1 : 0));
    if (w < 0) w = 0;
    const int jitter = static_cast<int>((h >> 8) % (2 * w + 1)) - w;
    return max(1, min(M, base + up + jitter));
}

// Accept / commit by one thread.  tok[j] is the target's token for the position after row j.
// `in` is a snapshot of the control block taken by one coalesced load at the start of the tail (shared memory): read word by
// word from global memory, this single-thread routine is a chain of L2 round trips.
__device__ __forceinline__ void commit_rows(int* ctl, const int* in, const int* tok, int M, int upstream_status) {
    const int C = in[kCtlCommittedLen];
    int status = in[kCtlStatus] | upstream_status;
    for (int j = 0; j < M; ++j)
        if (tok[j] < 0 && status == 0) status = kStatusNonFinite;
    const unsigned int epoch = static_cast<unsigned int>(in[kCtlStepEpoch]);
    if (status != 0) {
        // fail closed: nothing is committed anywhere
        ctl[kCtlStatus] = status;
        ctl[kCtlCommitCount] = 0;
        ctl[kCtlAccepted] = 0;
        ctl[kCtlPending] = -1;
        ctl[kCtlIds] = -1;
        for (int j = 0; j < kMaxRows; ++j) ctl[kCtlEmitted + j] = -1;
        ctl[kCtlStopPos] = -1;
        __threadfence();
        ctl[kCtlStepEpoch] = static_cast<int>(epoch + 1);
        return;
    }
    int accepted = 0;
    for (int j = 0; j + 1 < M; ++j)
        if (accepted == j && tok[j] == in[kCtlIds + j + 1]) accepted = j + 1;
    int forced = in[kCtlForcedCommit];
    if (in[kCtlForcedSeed] != 0) forced = forced_schedule(static_cast<unsigned int>(in[kCtlForcedSeed]), epoch, in[kCtlForcedMean10], M);
    if (forced > 0) accepted = min(forced, M) - 1;
    const int commit = accepted + 1;
    int emitted[kMaxRows];
    for (int j = 0; j < kMaxRows; ++j) emitted[j] = j < accepted ? in[kCtlIds + j + 1] : (j == accepted ? tok[accepted] : -1);
    const int eos = in[kCtlEos];
    int stop = -1;
    for (int j = 0; j < commit; ++j)
        if (stop < 0 && eos >= 0 && emitted[j] == eos) stop = j;
    for (int j = 0; j < kMaxRows; ++j) ctl[kCtlEmitted + j] = emitted[j];
    ctl[kCtlStopPos] = stop;
    ctl[kCtlAccepted] = accepted;
    ctl[kCtlCommitCount] = commit;
    ctl[kCtlPending] = tok[accepted];
    ctl[kCtlIds] = tok[accepted];
    ctl[kCtlStepEpoch] = static_cast<int>(epoch + 1);
    __threadfence();
    ctl[kCtlCommittedLen] = C + commit;   // published last
}

struct HeadArgs {
    const __nv_bfloat16* x;          // [M][H]
    const float* final_ln;           // [H] 1 + w
    const __nv_bfloat16* w;          // [V_local][H]
    float* logits_out;               // optional [M][V_local]
    const float* logits_in;          // optional [M][V_local]: logits computed beforehand (wide steps); skips the GEMV
    unsigned long long* cand;        // [M][n_cta][28]
    int* ticket;
    const unsigned long long* sampling;
    int* ctl;
    int* export_buf;                 // optional [M][64]
    int H, V_local, vocab_base, M;
    float eps;
    int mode, arg;                   // 1: sample + accept + commit; 2: greedy, row r -> ctl ids[arg + r]
    LLChannel ch;
    unsigned int site;
    size_t smem_bytes;               // dynamic shared memory of the launch (the last CTA stages the candidate lists in it)
};

template <int MB>
__global__ void __launch_bounds__(512, 1) lmhead_sample_kernel(HeadArgs a) {
    extern __shared__ __align__(16) float smem[];
    __shared__ float red[32];
    __shared__ int s_last;
    __shared__ int s_tok[kMaxRows];
    __shared__ int s_status;
    __shared__ unsigned long long s_top[kMaxRows][kMaxTopK];
    __shared__ int s_ctl[kCtlWords];
    TraceCta tr;
    tr.begin(kTrHead);
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    int v0, v1;
    cta_range(a.V_local, blockIdx.x, gridDim.x, &v0, &v1);
    const int nv = v1 - v0, nv_max = (a.V_local + gridDim.x - 1) / gridDim.x;
    const bool pre = a.logits_in != nullptr;
    if (nv && !pre) prefetch_l2_range(a.w + static_cast<size_t>(v0) * a.H, static_cast<size_t>(nv) * a.H * 2);
    constexpr int kTile = 256;                                                          // rows per GEMV tile
    const GemvGeom gg = gemv_geom(a.H / 8, blockDim.x);
    float* xs = smem;                                                                   // [MB][H]
    float* part = xs + static_cast<size_t>(MB) * a.H;                                   // [kTile][wpr][MB]
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(part + gemv_part_floats(kTile, MB, gg));   // [MB][nv_max]
    float* gs = reinterpret_cast<float*>(keys + static_cast<size_t>(MB) * nv_max);                                // [H] norm multiplier
    GemvCta<MB, (MB == 1 ? 8 : 4), PlainBf16> gemv0(PlainBf16{a.w, a.H}, v0, min(kTile, nv), a.H);
    if (!pre) {
        gemv0.preload();
        for (int i = threadIdx.x; i < a.H; i += blockDim.x) gs[i] = a.final_ln[i];
    }
    pdl_wait();
    tr.mark(1);
    const SamplingCfg cfg = read_sampling(a.sampling);
    const int K = a.mode == 2 ? 1 : cfg.top_k;
    for (int m0 = 0; m0 < a.M; m0 += MB) {
        const int mb = min(MB, a.M - m0);
        if (m0) __syncthreads();
        if (pre) {
            for (int idx = threadIdx.x; idx < nv * mb; idx += blockDim.x) {
                const int rl = idx % nv, m = idx / nv, row = v0 + rl;
                keys[m * nv_max + rl] = make_key(__ldcg(a.logits_in + static_cast<size_t>(m0 + m) * a.V_local + row), a.vocab_base + row);
            }
            __syncthreads();
        } else
            stage_rmsnorm_plain(xs, a.x + static_cast<size_t>(m0) * a.H, gs, mb, a.H, a.eps, red);
        for (int t0 = 0; t0 < nv && !pre; t0 += kTile) {
            const int nt = min(kTile, nv - t0);
            if (m0 == 0 && t0 == 0) gemv0.run(xs, part);
            else gemv_cta<MB, (MB == 1 ? 8 : 4)>(PlainBf16{a.w, a.H}, v0 + t0, nt, xs, a.H, part);
            __syncthreads();
            for (int idx = threadIdx.x; idx < nt * mb; idx += blockDim.x) {
                const int rl = idx / mb, m = idx % mb, row = v0 + t0 + rl;
                const float v = gemv_result(part, rl, m, MB, gg.wpr);
                keys[m * nv_max + t0 + rl] = make_key(v, a.vocab_base + row);
                if (a.logits_out) a.logits_out[static_cast<size_t>(m0 + m) * a.V_local + row] = v;
            }
            __syncthreads();
        }
        // per-CTA top-K of each row: warp m owns row m
        if (warp < mb) {
            unsigned long long* kr = keys + warp * nv_max;
            unsigned long long* out = a.cand + (static_cast<size_t>(m0 + warp) * gridDim.x + blockIdx.x) * kMaxTopK;
            for (int k = 0; k < K; ++k) {
                unsigned long long best = 0ull;
                for (int i = lane; i < nv; i += 32) best = kr[i] > best ? kr[i] : best;
                best = warp_max_u64(best);
                if (best != 0ull) {
                    const int local = key_id(best) - a.vocab_base - v0;
                    if ((local & 31) == lane) kr[local] = 0ull;
                }
                if (lane == 0) out[k] = best;
                __syncwarp();
            }
        }
    }
    tr.mark(2);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(a.ticket, 1) == static_cast<int>(gridDim.x) - 1);
    __syncthreads();
    if (!s_last) { tr.mark(3); return; }
    tr.mark(4);
    __threadfence();
    if (threadIdx.x == 0) s_status = cfg.bad ? kStatusBadConfig : 0;
    if (threadIdx.x < kCtlWords) s_ctl[threadIdx.x] = __ldcg(a.ctl + threadIdx.x);     // one coalesced load for everything the sampler and the commit read
    __syncthreads();
    // ---- last CTA: the per-CTA lists (each sorted descending) are staged in shared memory with one round of coalesced
    // loads - the GEMV's buffers are free now - and warp m merges row m's lists from there, `rows_fit` rows at a time
    const int n_lists = gridDim.x;
    LLCall call{0u, 0u};
    if (a.ch.world > 1) call = ll_begin(a.ch, a.site);
    unsigned long long* stage = reinterpret_cast<unsigned long long*>(smem);
    const int per_row = n_lists * K;
    const int rows_fit = max(1, min(nwarps, static_cast<int>(a.smem_bytes / (sizeof(unsigned long long) * per_row))));
    const bool staged = a.smem_bytes >= sizeof(unsigned long long) * per_row;
    for (int mbase = 0; mbase < a.M; mbase += rows_fit) {
    const int mcount = min(rows_fit, a.M - mbase);
    __syncthreads();
    if (staged) {
        for (int idx = threadIdx.x; idx < mcount * per_row; idx += blockDim.x) {
            const int mm = idx / per_row, rem = idx % per_row, li = rem / K, k = rem % K;
            stage[idx] = __ldcg(a.cand + (static_cast<size_t>(mbase + mm) * n_lists + li) * kMaxTopK + k);
        }
    }
    __syncthreads();
    tr.mark(5);
    for (int m = mbase + warp; m < mbase + mcount; m += nwarps) {
        const unsigned long long* lists = a.cand + static_cast<size_t>(m) * n_lists * kMaxTopK;
        const unsigned long long* srow = stage + static_cast<size_t>(m - mbase) * per_row;
        constexpr int kListsPerLane = 8;   // up to 256 CTAs
        int head[kListsPerLane];
#pragma unroll
        for (int i = 0; i < kListsPerLane; ++i) head[i] = 0;
        for (int k = 0; k < K; ++k) {
            unsigned long long best = 0ull;
            int bl = -1;
#pragma unroll
            for (int i = 0; i < kListsPerLane; ++i) {
                const int li = lane + 32 * i;
                if (li < n_lists && head[i] < K) {
                    const unsigned long long c = staged ? srow[li * K + head[i]] : __ldcg(lists + static_cast<size_t>(li) * kMaxTopK + head[i]);
                    if (c > best) { best = c; bl = i; }
                }
            }
            // 64-bit maximum over the warp on the warp-reduce unit: high words first, then the low words of the lanes that tie
            const unsigned int hi_max = redux_max_u32(static_cast<unsigned int>(best >> 32));
            const unsigned int lo_max = redux_max_u32(static_cast<unsigned int>(best >> 32) == hi_max ? static_cast<unsigned int>(best) : 0u);
            const unsigned long long win = (static_cast<unsigned long long>(hi_max) << 32) | lo_max;
            if (win != 0ull && best == win && bl >= 0) {
#pragma unroll
                for (int i = 0; i < kListsPerLane; ++i)
                    if (i == bl) head[i]++;
            }
            if (lane == 0) s_top[m][k] = win;
        }
        __syncwarp();
        if (a.ch.world > 1) {
            // exchange: 2 packets per candidate (high word, low word), then merge the world's lists
            for (int i = lane; i < K * 2; i += 32) {
                const unsigned long long key = s_top[m][i >> 1];
                ll_publish(a.ch, call, (static_cast<unsigned int>(m) * kMaxTopK) * 2 + i, static_cast<unsigned int>(i & 1 ? key : key >> 32));
            }
            // lane s < world owns the list of rank s
            unsigned long long mine[kMaxTopK];
            int hd = 0;
            const bool owner = lane < a.ch.world;
            if (owner) {
                for (int k = 0; k < K; ++k) {
                    if (lane == a.ch.rank) { mine[k] = s_top[m][k]; continue; }
                    unsigned int hi, lo;
                    ll_wait(a.ch, call, lane, (static_cast<unsigned int>(m) * kMaxTopK + k) * 2, &hi);
                    ll_wait(a.ch, call, lane, (static_cast<unsigned int>(m) * kMaxTopK + k) * 2 + 1, &lo);
                    mine[k] = (static_cast<unsigned long long>(hi) << 32) | lo;
                }
            }
            __syncwarp();
            for (int k = 0; k < K; ++k) {
                unsigned long long c = 0ull;
                if (owner && hd < K) {
#pragma unroll
                    for (int i = 0; i < kMaxTopK; ++i)
                        if (i == hd) c = mine[i];
                }
                const unsigned long long win = warp_max_u64(c);
                if (owner && win != 0ull && c == win) hd++;
                if (lane == 0) s_top[m][k] = win;
                __syncwarp();
            }
        }
        if (lane == 0) {
            int st = 0;
            int tok;
            if (a.mode == 2) {
                tok = s_top[m][0] == 0ull ? -1 : key_id(s_top[m][0]);
            } else {
                const unsigned int pos = static_cast<unsigned int>(s_ctl[kCtlCommittedLen] + m);
                tok = sample_row(s_top[m], K, cfg, pos, &st, a.export_buf ? a.export_buf + m * kExportWords : nullptr);
            }
            s_tok[m] = tok;
            if (st) atomicCAS(&s_status, 0, st);
        }
    }
    }
    __syncthreads();
    tr.mark(6);
    if (threadIdx.x == 0) {
        const int upstream = s_status | (a.ch.status ? *reinterpret_cast<volatile int*>(a.ch.status) : 0);
        if (a.mode == 2) {
            for (int m = 0; m < a.M; ++m) a.ctl[kCtlIds + a.arg + m] = s_tok[m];
            if (upstream) atomicOr(a.ctl + kCtlStatus, upstream);
        } else {
            commit_rows(a.ctl, s_ctl, s_tok, a.M, upstream);
        }
        *a.ticket = 0;
    }
    tr.mark(3);
}

// Sample row 0 from full fp32 logits [V] already in memory (first token after a prefill whose
// logits were produced elsewhere): one CTA, greedy or sampled, writes pending / ids[0].
__global__ void __launch_bounds__(1024) sample_logits_kernel(const float* logits, const unsigned long long* sampling, int* ctl, int V,
                                                             int position_base) {
    __shared__ unsigned long long s_w[32];
    __shared__ unsigned long long s_top[kMaxTopK];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const SamplingCfg cfg = read_sampling(sampling);
    unsigned long long prev = ~0ull;
    for (int k = 0; k < cfg.top_k; ++k) {
        unsigned long long best = 0ull;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const unsigned long long c = make_key(logits[i], i);
            if (c < prev && c > best) best = c;
        }
        best = warp_max_u64(best);
        if (lane == 0) s_w[warp] = best;
        __syncthreads();
        unsigned long long t = lane < static_cast<int>(blockDim.x >> 5) ? s_w[lane] : 0ull;
        t = warp_max_u64(t);
        prev = t;
        if (threadIdx.x == 0) s_top[k] = t;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        int st = cfg.bad ? kStatusBadConfig : 0;
        const int tok = st ? -1 : sample_row(s_top, cfg.top_k, cfg, static_cast<unsigned int>(position_base), &st, nullptr);
        if (st) atomicOr(ctl + kCtlStatus, st);
        ctl[kCtlPending] = tok;
        ctl[kCtlIds] = tok;
    }
}

}  // namespace nexrt

using namespace nexrt;

extern "C" int nexrt_lmhead_sample(const void* x, const void* final_ln, const void* w, void* logits_out, void* cand, void* ticket,
                                   const void* sampling, void* ctl, void* export_buf, int H, int V_local, int vocab_base, int M, float eps,
                                   int mode, int arg, const NexrtLLChannel* ch, unsigned int site, int n_cta, void* stream) {
    if (M < 1 || M > kMaxRows || H % 256 || n_cta > 256 || ch == nullptr || (mode != 1 && mode != 2)) return cudaErrorInvalidValue;
    if (ch->world > 1 && ch->slots < static_cast<unsigned int>(kMaxRows) * kMaxTopK * 2) return cudaErrorInvalidValue;
    HeadArgs a{};
    a.x = static_cast<const __nv_bfloat16*>(x); a.final_ln = static_cast<const float*>(final_ln); a.w = static_cast<const __nv_bfloat16*>(w);
    a.logits_out = static_cast<float*>(logits_out); a.cand = static_cast<unsigned long long*>(cand); a.ticket = static_cast<int*>(ticket);
    a.sampling = static_cast<const unsigned long long*>(sampling); a.ctl = static_cast<int*>(ctl); a.export_buf = static_cast<int*>(export_buf);
    a.H = H; a.V_local = V_local; a.vocab_base = vocab_base; a.M = M; a.eps = eps; a.mode = mode; a.arg = arg; a.ch = *ch; a.site = site;
    const int mb = M == 1 ? 1 : 4;
    const int nv_max = (V_local + n_cta - 1) / n_cta;
    const size_t smem = sizeof(float) * (static_cast<size_t>(mb) * H + gemv_part_floats(256, mb, gemv_geom(H / 8, gemv_threads()))) +
                        sizeof(unsigned long long) * static_cast<size_t>(mb) * nv_max + sizeof(float) * H;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    a.smem_bytes = smem;
    if (mb == 1) return launch(lmhead_sample_kernel<1>, dim3(n_cta), dim3(gemv_threads()), smem, st, a);
    return launch(lmhead_sample_kernel<4>, dim3(n_cta), dim3(gemv_threads()), smem, st, a);
}

// Same head on logits that were computed beforehand (the wide path of multi-row steps): logits_in [M][V_local] fp32.
extern "C" int nexrt_lmhead_sample_from_logits(const void* logits_in, void* cand, void* ticket, const void* sampling, void* ctl, void* export_buf, int H,
                                               int V_local, int vocab_base, int M, int mode, int arg, const NexrtLLChannel* ch, unsigned int site,
                                               int n_cta, void* stream) {
    if (M < 1 || M > kMaxRows || n_cta > 256 || ch == nullptr || (mode != 1 && mode != 2) || logits_in == nullptr) return cudaErrorInvalidValue;
    if (ch->world > 1 && ch->slots < static_cast<unsigned int>(kMaxRows) * kMaxTopK * 2) return cudaErrorInvalidValue;
    HeadArgs a{};
    a.logits_in = static_cast<const float*>(logits_in); a.cand = static_cast<unsigned long long*>(cand); a.ticket = static_cast<int*>(ticket);
    a.sampling = static_cast<const unsigned long long*>(sampling); a.ctl = static_cast<int*>(ctl); a.export_buf = static_cast<int*>(export_buf);
    a.H = H; a.V_local = V_local; a.vocab_base = vocab_base; a.M = M; a.mode = mode; a.arg = arg; a.ch = *ch; a.site = site;
    const int mb = M == 1 ? 1 : 4;
    const int nv_max = (V_local + n_cta - 1) / n_cta;
    const size_t smem = sizeof(float) * (static_cast<size_t>(mb) * H + gemv_part_floats(256, mb, gemv_geom(H / 8, gemv_threads()))) +
                        sizeof(unsigned long long) * static_cast<size_t>(mb) * nv_max + sizeof(float) * H;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    a.smem_bytes = smem;
    if (mb == 1) return launch(lmhead_sample_kernel<1>, dim3(n_cta), dim3(gemv_threads()), smem, st, a);
    return launch(lmhead_sample_kernel<4>, dim3(n_cta), dim3(gemv_threads()), smem, st, a);
}

extern "C" int nexrt_sample_logits(const void* logits, const void* sampling, void* ctl, int V, int position_base, void* stream) {
    return launch(sample_logits_kernel, dim3(1), dim3(1024), 0, static_cast<cudaStream_t>(stream), static_cast<const float*>(logits),
                  static_cast<const unsigned long long*>(sampling), static_cast<int*>(ctl), V, position_base);
}
