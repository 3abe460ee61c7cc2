// Glue kernels of the speculative runtimes (MTP draft chain, DFlash block draft).
//
//   mtp_prep        : bookkeeping between the verify step and the draft layer: base position and
//                     token ids of the next draft-layer pass (extend after a commit, first and second
//                     chained draft), written into the draft layer's own small control block.
//   mtp_preprocess  : embedding gather + the two pre-fc RMSNorms; emits this rank's window of
//                     cat[norm_e(emb(tok)) | norm_h(norm_f(hidden))] as fp32 for the fc projection.
//   row_select      : y_sel = x[commit_count - 1] (hidden of the last committed row).
//   dflash_noise    : rows of the block draft: embed[pending], embed[mask] x 7.
//   dflash_commit   : the 7 proposals become ids[1..7] of the next verify step.
//   feature_tap     : snapshot of the 8 residual rows at a tap layer.
//
// Counterparts in the reference: MtpPrepKernel / MtpRowSelectKernel / MtpStatusFoldKernel
// (nex_n2_5_pro/kernels/mtp/nex_n2_5_pro_mtp_glue_ctypes.cu:41-95), MtpPreprocessKernel
// (…mtp_preprocess_ctypes.cu:68-127), DfNoiseEmbedKernel / DfProposalCommitKernel
// (…dflash/nex_n2_5_pro_dflash_glue_ctypes.cu:43-93), M8FeatTapKernel
// (…embed/nex_n2_5_pro_m8_feature_tap_ctypes.cu:45-68).
#include "api.h"
#include "common.cuh"

namespace nexrt {

enum MtpPrepMode : int { kPrepExtend = 0, kPrepDraft1 = 1, kPrepDraft2 = 2 };

__global__ void __launch_bounds__(32) mtp_prep_kernel(const int* __restrict__ ctl, int* __restrict__ dctl, int mode, int rows) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x != 0) return;
    const int C = ctl[kCtlCommittedLen];
    if (mode == kPrepExtend) {
        const int commit = ctl[kCtlCommitCount];
        dctl[kCtlCommittedLen] = C - commit;
        dctl[kCtlCommitCount] = commit;
        for (int j = 0; j < rows; ++j) {
            const int t = j < commit ? ctl[kCtlEmitted + j] : 0;
            dctl[kCtlIds + j] = t < 0 ? 0 : t;
        }
    } else {
        const int k = mode == kPrepDraft1 ? 1 : 2;
        dctl[kCtlCommittedLen] = C + k - 1;
        dctl[kCtlCommitCount] = 1;
        const int t = ctl[kCtlIds + k];
        dctl[kCtlIds] = t < 0 ? 0 : t;
    }
    dctl[kCtlStatus] = 0;
}

// out[m][0 .. win) = window [win0, win0 + win) of cat[ rms(emb[tok_m]) * ge | rms(rms(h_m) * gf) * gh ].
// One CTA per row.  hidden_row < 0: row m of `hidden`; otherwise that fixed row for every m.
__global__ void __launch_bounds__(256) mtp_preprocess_kernel(const __nv_bfloat16* __restrict__ embed, const int* __restrict__ dctl,
                                                             const __nv_bfloat16* __restrict__ hidden, const float* __restrict__ ge,
                                                             const float* __restrict__ gf, const float* __restrict__ gh, float* __restrict__ out,
                                                             int H, int vocab, int win0, int win, float eps, int hidden_row) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x;
    int tok = dctl[kCtlIds + m];
    if (tok < 0 || tok >= vocab) tok = 0;
    const __nv_bfloat16* e = embed + static_cast<size_t>(tok) * H;
    const __nv_bfloat16* h = hidden + static_cast<size_t>(hidden_row < 0 ? m : hidden_row) * H;
    float se = 0.f, sh = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float a = __bfloat162float(e[i]), b = __bfloat162float(h[i]);
        se = fmaf(a, a, se);
        sh = fmaf(b, b, sh);
    }
    se = block_sum(se, red);
    sh = block_sum(sh, red);
    const float inv_e = rsqrtf(se / static_cast<float>(H) + eps), inv_f = rsqrtf(sh / static_cast<float>(H) + eps);
    // second norm of the hidden half needs the mean square of the once-normalised vector
    float s2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = __bfloat162float(h[i]) * inv_f * gf[i];
        s2 = fmaf(v, v, s2);
    }
    s2 = block_sum(s2, red);
    const float inv_h = rsqrtf(s2 / static_cast<float>(H) + eps);
    for (int i = threadIdx.x; i < win; i += blockDim.x) {
        const int c = win0 + i;
        float v;
        if (c < H) v = __bfloat162float(e[c]) * inv_e * ge[c];
        else v = __bfloat162float(h[c - H]) * inv_f * gf[c - H] * inv_h * gh[c - H];
        out[static_cast<size_t>(m) * win + i] = v;
    }
}

__global__ void __launch_bounds__(256) row_select_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ctl,
                                                         __nv_bfloat16* __restrict__ y, int H, int rows) {
    pdl_launch_dependents();
    pdl_wait();
    int r = ctl[kCtlCommitCount] - 1;
    r = r < 0 ? 0 : (r >= rows ? rows - 1 : r);
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * H);
    uint4* dst = reinterpret_cast<uint4*>(y);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

__global__ void __launch_bounds__(256) zero_rows_kernel(__nv_bfloat16* __restrict__ x, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = __float2bfloat16_rn(0.f);
}

// DFlash: row 0 = embed[pending], rows 1..rows-1 = embed[mask_id]; meta = {rows, committed_len}.
__global__ void __launch_bounds__(256) dflash_noise_kernel(const __nv_bfloat16* __restrict__ embed, const int* __restrict__ ctl,
                                                           __nv_bfloat16* __restrict__ noise, int* __restrict__ dctl, int H, int vocab, int mask_id) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x;
    int tok = m == 0 ? ctl[kCtlPending] : mask_id;
    if (tok < 0 || tok >= vocab) tok = 0;
    const uint4* src = reinterpret_cast<const uint4*>(embed + static_cast<size_t>(tok) * H);
    uint4* dst = reinterpret_cast<uint4*>(noise + static_cast<size_t>(m) * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
    if (m == 0 && threadIdx.x == 0) {
        dctl[kCtlCommittedLen] = ctl[kCtlCommittedLen];
        dctl[kCtlIds] = tok;
        dctl[kCtlStatus] = 0;
    }
}

// ids[1 .. rows-1] of the verify step = the draft's proposals (its rows 1 .. rows-1); ids[0] = pending.
__global__ void __launch_bounds__(32) dflash_commit_kernel(int* __restrict__ ctl, const int* __restrict__ dctl, int rows) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        ctl[kCtlIds] = ctl[kCtlPending];
        for (int j = 1; j < rows; ++j) ctl[kCtlIds + j] = dctl[kCtlIds + j];
        if (dctl[kCtlStatus] != 0) atomicOr(ctl + kCtlStatus, dctl[kCtlStatus]);
    }
}

// tap[m][col0 .. col0 + H) = x[m][0 .. H) for the rows of the step (tap rows are ld elements apart).
__global__ void __launch_bounds__(256) feature_tap_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ tap, int H, int ld,
                                                          int col0) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(m) * H);
    uint4* dst = reinterpret_cast<uint4*>(tap + static_cast<size_t>(m) * ld + col0);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

}  // namespace nexrt

using namespace nexrt;

extern "C" int nexrt_mtp_prep(const void* ctl, void* dctl, int mode, int rows, void* stream) {
    if (mode < 0 || mode > 2 || rows < 1 || rows > kMaxRows) return cudaErrorInvalidValue;
    return launch(mtp_prep_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), static_cast<const int*>(ctl), static_cast<int*>(dctl),
                  mode, rows);
}

extern "C" int nexrt_mtp_preprocess(const void* embed, const void* dctl, const void* hidden, const void* ge, const void* gf, const void* gh,
                                    void* out, int H, int vocab, int win0, int win, float eps, int hidden_row, int M, void* stream) {
    if (M < 1 || M > kMaxRows || win0 < 0 || win0 + win > 2 * H) return cudaErrorInvalidValue;
    return launch(mtp_preprocess_kernel, dim3(M), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(embed),
                  static_cast<const int*>(dctl), static_cast<const __nv_bfloat16*>(hidden), static_cast<const float*>(ge),
                  static_cast<const float*>(gf), static_cast<const float*>(gh), static_cast<float*>(out), H, vocab, win0, win, eps, hidden_row);
}

extern "C" int nexrt_row_select(const void* x, const void* ctl, void* y, int H, int rows, void* stream) {
    if (H % 8 || rows < 1 || rows > kMaxRows) return cudaErrorInvalidValue;
    return launch(row_select_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(x),
                  static_cast<const int*>(ctl), static_cast<__nv_bfloat16*>(y), H, rows);
}

extern "C" int nexrt_zero_rows(void* x, int n, void* stream) {
    return launch(zero_rows_kernel, dim3((n + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<__nv_bfloat16*>(x), n);
}

extern "C" int nexrt_dflash_noise(const void* embed, const void* ctl, void* noise, void* dctl, int H, int vocab, int mask_id, int rows,
                                  void* stream) {
    if (H % 8 || rows < 1 || rows > kMaxRows) return cudaErrorInvalidValue;
    return launch(dflash_noise_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(embed),
                  static_cast<const int*>(ctl), static_cast<__nv_bfloat16*>(noise), static_cast<int*>(dctl), H, vocab, mask_id);
}

extern "C" int nexrt_dflash_commit(void* ctl, const void* dctl, int rows, void* stream) {
    if (rows < 1 || rows > kMaxRows) return cudaErrorInvalidValue;
    return launch(dflash_commit_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), static_cast<int*>(ctl),
                  static_cast<const int*>(dctl), rows);
}

extern "C" int nexrt_feature_tap(const void* x, void* tap, int H, int ld, int col0, int M, void* stream) {
    if (H % 8 || ld % 8 || col0 % 8 || M < 1 || M > 128) return cudaErrorInvalidValue;   // one CTA per row: a prefill chunk taps up to 128 rows
    return launch(feature_tap_kernel, dim3(M), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(x),
                  static_cast<__nv_bfloat16*>(tap), H, ld, col0);
}
