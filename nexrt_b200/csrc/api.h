/* C ABI of libnexrt_b200: every launcher returns a cudaError_t as int (0 == success), takes raw
 * device pointers and a stream handle, allocates nothing and is safe to call while the stream
 * is being captured into a CUDA graph.  Same calling convention as the reference's per-kernel
 * `extern "C" int NexN25Pro…Launch(ptrs…, stream)` entry points (e.g. nex_n2_5_pro/kernels/
 * full_attn/nex_n2_5_pro_o_proj_reduce_ctypes.cu:299), but one library and run-time geometry.
 */
#pragma once

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* One LL packet channel (see ll.cuh).  Mirrored field by field in parallel/channel.py. */
typedef struct NexrtLLChannel {
    unsigned long long* local;    /* this rank's inbox: [2 halves][world][slots] 8-byte packets */
    unsigned long long* mc;       /* multicast alias of every rank's inbox, or NULL */
    unsigned long long* peer[8];  /* unicast address of each rank's inbox (peer[rank] == local) */
    const unsigned int* seq;      /* call sequence base, advanced by the last kernel of a step */
    int* status;                  /* sticky failure word, 0 == healthy */
    int world;
    int rank;
    unsigned int slots;           /* packets per (half, source rank) */
    unsigned int reserved;
    unsigned long long budget_ns; /* longest time one wait may take */
} NexrtLLChannel;

int nexrt_set_pdl(int enabled);
int nexrt_version(void);
int nexrt_set_gemv_threads(int threads);
int nexrt_set_event_ring(void* ring);  /* 8 x u64 device words: phase timestamps of the GDN front kernel, NULL = off */
int nexrt_set_attn_event_ring(void* ring);   /* 16 x u64 device words: phase timestamps of the attention decode kernel; null = off */
int nexrt_set_gemv_mode(int mode);   /* bit mask: 1 fronts, 2 out-proj, 4 expert up, 8 expert down, 16 router, 32 attention key loop on tensor cores; 64 attention decode as thread-block clusters, 128 clusters of 16 CTAs where the device can place them; 255 = everything (default), 0 = CUDA-core kernels */

/* step plumbing */
int nexrt_embed_gather(const void* embed, const void* ctl, void* x, void* status, int H, int vocab, int M, void* stream);
int nexrt_step_end(void* ctl, void* seq, unsigned int n_sites, void* mirror_host, void* mirror_gen, int words, void* stream);
int nexrt_residual_add(void* x, const void* y, int n, void* stream);

/* measurement plumbing */
unsigned long long nexrt_launch_count(void);   /* kernels launched through the library since it was loaded */
int nexrt_set_partial_out(void* buffer);       /* library-baseline arm: reduce sites store fp32 partial sums [8][H] here instead of exchanging them; NULL = normal */
int nexrt_set_trace(void* buffer);             /* timeline build only (returns non-zero otherwise): device buffer of nexrt_trace_layout() words, NULL = off */
int nexrt_trace_layout(int* kinds, int* slots, int* words);
int nexrt_null_node(int grid, int block, int smem, unsigned long long body_ns, int early_release, void* clock_out, void* stream);   /* empty kernel node that spins body_ns */

/* the all-reduce epilogue in isolation (partial [M][H] fp32 -> x [M][H] bf16, H / 16 CTAs; stamps: per-CTA ns or NULL), the
 * sequence advance that closes a batch of such calls, and a two-rank packet ping-pong (out: elapsed ns, round trips done) */
int nexrt_ll_allreduce_bench(const void* partial, void* x, int M, int H, const NexrtLLChannel* ch, unsigned int site, void* stamps, void* stream);
int nexrt_ll_seq_advance(void* seq, unsigned int n, void* stream);
int nexrt_ll_pingpong(const NexrtLLChannel* ch, int a, int b, unsigned int tag0, int iters, int use_mc, void* out, void* stream);

/* gated delta net */
int nexrt_gdn_front(const void* x, const void* in_ln, const void* front_w, const void* front_s, const void* ba_w, const void* conv_w,
                    const void* a_log, const void* dt_bias, const void* ctl, void* conv_ring, void* qkv, void* z, void* beta, void* g, int H,
                    int R, int C, int nv, int M, int conv_ring_len, float eps, int ba_rows_pad, int n_cta, void* stream);
int nexrt_gdn_core(const void* qkv, const void* beta, const void* g, const void* ctl, void* state_ring, void* out, int nqk, int nv, int M,
                   int state_ring_len, int C, void* stream);

/* gated full attention */
int nexrt_attn_front(const void* x, const void* in_ln, const void* w, const void* s, const void* ctl, void* q_raw, void* gate, void* k_raw,
                     void* v_cache, int H, int hd, int nq, int ngate, int kvh, int M, int cache_len, float eps, int n_cta, void* stream);
size_t nexrt_attn_decode_smem(int hd, int nq, int kvh, int M);
int nexrt_attn_decode(const void* q_raw, const void* gate, const void* k_raw, const void* qn, const void* kn, const void* inv_freq,
                      const void* rope_table, const void* ctl, void* k_cache, const void* v_cache, void* ws_acc, void* ws_ml, void* ticket, void* out, int hd, int nq,
                      int ngate, int kvh, int M, int cache_len, int rotary, int n_splits, float eps, int flags, int window, int ldq, int ldk,
                      int cp_size, int cp_rank, const NexrtLLChannel* ch, unsigned int site, void* stream);

/* output projection + all-reduce + residual.  mode 0: plain fp32 input; 1: GDN gated RMSNorm of
 * (in, z); 2: context-parallel merge of the partials waiting in `cp` followed by * sigmoid(gate).
 * Adding 4 to the mode makes x the reduced projection itself instead of adding it to x. */
int nexrt_oproj_allreduce(const void* in, const void* z, const void* gnorm_w, const void* w, const void* s, void* x, int H, int K, int M,
                          int mode, float eps, int hd, const NexrtLLChannel* ch, unsigned int site, const NexrtLLChannel* cp,
                          unsigned int cp_site, int n_cta, void* stream);

/* mixture of experts */
/* w holds E+1 rows; if it is padded with zero rows to rows_pad (a multiple of 16) and `partial`
 * ([4][M][rows_pad] floats) is given, the tensor-core form runs. */
int nexrt_moe_router(const void* x, const void* post_ln, const void* w, void* logits, void* ids, void* wts, void* ticket, void* partial,
                     int rows_pad, int H, int E, int topk, int M, float eps, int n_cta, void* planes, void* stream);   /* planes: optional e4m3 [3M][H] for the tcgen05 experts */
int nexrt_moe_l1(const void* x, const void* post_ln, const void* w13, const void* w13_s, const void* ids, void* gu, int H, int I, int S, int M,
                 float eps, int shared_expert, int n_cta, void* stream);
/* routed pair of the one-row step: the router stops at K-split partial logits [split][M][rows_pad]; the gate/up kernel adds
 * them, selects the experts in every CTA and leaves ids / weights / logits for the down projection */
int nexrt_moe_router_partial(const void* x, const void* post_ln, const void* w, void* partial, int rows_pad, int H, int E, int topk, int M,
                             float eps, void* planes, void* stream);
int nexrt_moe_router_partial_split(void);
int nexrt_moe_l1_routed(const void* x, const void* post_ln, const void* w13, const void* w13_s, const void* partial, int rows_pad, void* ids_out,
                        void* wts_out, void* logits_out, void* gu, const void* w2, const void* pf, unsigned long long pf_bytes, int H, int I,
                        int E, int topk, int M, float eps, void* stream);
int nexrt_attn_decode_merges_cp(int n_splits);   /* 1: the decode kernel chosen for this split count also merges the context-parallel partials */
int nexrt_moe_l2_allreduce(const void* gu, const void* ids, const void* wts, const void* w2, const void* w2_s, void* x, int H, int I, int S,
                           int M, const NexrtLLChannel* ch, unsigned int site, int n_cta, void* stream);

/* LM head, distributed top-k, sampler, accept / commit */
int nexrt_lmhead_sample(const void* x, const void* final_ln, const void* w, void* logits_out, void* cand, void* ticket, const void* sampling,
                        void* ctl, void* export_buf, int H, int V_local, int vocab_base, int M, float eps, int mode, int arg,
                        const NexrtLLChannel* ch, unsigned int site, int n_cta, void* stream);
int nexrt_sample_logits(const void* logits, const void* sampling, void* ctl, int V, int position_base, void* stream);

/* speculative-decoding glue (spec.cu) */
int nexrt_mtp_prep(const void* ctl, void* dctl, int mode, int rows, void* stream);
int nexrt_mtp_preprocess(const void* embed, const void* dctl, const void* hidden, const void* ge, const void* gf, const void* gh, void* out,
                         int H, int vocab, int win0, int win, float eps, int hidden_row, int M, void* stream);
int nexrt_row_select(const void* x, const void* ctl, void* y, int H, int rows, void* stream);
int nexrt_zero_rows(void* x, int n, void* stream);
int nexrt_dflash_noise(const void* embed, const void* ctl, void* noise, void* dctl, int H, int vocab, int mask_id, int rows, void* stream);
int nexrt_dflash_commit(void* ctl, const void* dctl, int rows, void* stream);
int nexrt_feature_tap(const void* x, void* tap, int H, int ld, int col0, int M, void* stream);

/* dense BF16 projection (dense.cu).  in_mode 0: bf16 rows + RMSNorm * gamma, 1: fp32 rows, 2: SwiGLU of
 * fp32 [gate | up], 3: bf16 rows as they are; ld_in = input row stride in elements (0: packed); out_mode 0: fp32 out, 1: all-reduce + residual add into bf16 x, 2: all-reduce + store. */
int nexrt_dense_bf16(const void* in, const void* gamma, const void* w, void* out, void* x, int R, int K, int M, int in_mode, int out_mode,
                     int ld_in, float eps, const NexrtLLChannel* ch, unsigned int site, void* stream);
int nexrt_kv_publish(const void* kv, int ld, int k_off, int v_off, const void* kn, const void* rope_table, const void* ctl, void* k_cache,
                     void* v_cache, int hd, int kvh, int M, int cache_len, int rotary, float eps, int ring, void* stream);

/* host runtime (host_runtime.cu) */
int nexrt_ipc_alloc(size_t bytes, void** ptr);
int nexrt_ipc_get_handle(void* ptr, void* handle64);
int nexrt_ipc_open(const void* handle64, void** ptr);
int nexrt_ipc_close(void* ptr);
int nexrt_ipc_free(void* ptr);
int nexrt_host_mapped_alloc(size_t bytes, void** host, void** dev);
int nexrt_host_mapped_free(void* host);
int nexrt_host_wait_flag(const volatile int* flag, int want, double timeout_s);

// ---- tensor-core GEMM (tcgen05 + TMEM + TMA) for many-row work; tc_gemm.cu ---------------------------------
// Y[T, R] = dequant(Xq, sx) * dequant(Wq, sw)^T.  Wq [R, K] e4m3 with row stride ldw, sw [ceil(R/128), K/128],
// Xq [T, K] e4m3, sx [T, K/128]; out_mode 0 fp32 store, 1 bf16 store, 2 fp32 accumulate.  K % 128 == 0, K <= 8192.
int nexrt_tc_gemm_fp8(const void* wq, const float* sw, int64_t ldw, const void* xq, const float* sx, void* y, int T, int R, int K, int ldy,
                      int out_mode, int* status, void* stream);
// Y[T, R] = X[T, K] * W[R, K]^T, bf16 operands (leading dimensions in elements), fp32 accumulation.  K % 64 == 0, K <= 4096.
int nexrt_tc_gemm_bf16(const void* w, int64_t ldw, const void* x, int64_t ldx, void* y, int T, int R, int K, int ldy, int out_mode, int* status,
                       void* stream);
// The same product with K split over ksplit CTAs per tile (fp32 partial planes of T * ldy elements, added by the consumer in
// plane order) and, with group_rows > 0, W stored as K / group_k matrices [group_rows, group_k] one after the other (expert
// down projections; sw [groups][group_rows / 128][group_k / 128], R == group_rows).  K / 128 / ksplit <= 64.
int nexrt_tc_gemm_fp8_ex(const void* wq, const float* sw, int64_t ldw, const void* xq, const float* sx, void* y, int T, int R, int K, int ldy,
                         int ksplit, int group_k, int group_rows, const int* used, int used_rows, int* status, void* stream);
/* used (optional, one int per group): plain matrix - row tiles of group m0 / used_rows with used == 0 are skipped (their
   output is left untouched); grouped K - the K blocks of unused groups are left out of the walk */
int nexrt_tc_gemm_bf16_ex(const void* w, int64_t ldw, const void* x, int64_t ldx, void* y, int T, int R, int K, int ldy, int ksplit, int* status,
                          void* stream);   /* K / 64 must divide into ksplit non-empty ranges of at most 64 blocks */
// Optional RMSNorm (gamma != null, stored as the full multiplier) then per-row, per-128-column e4m3 quantisation.
int nexrt_act_quant(const void* x, int x_fp32, int ldx, const float* gamma, float eps, void* xq, float* sx, int T, int K, int terms, void* stream);   /* xq / sx: terms planes of T rows */

// ---- glue kernels of the wide prefill path (prefill.cu) ---------------------------------------------------------
int nexrt_prefill_embed(const void* embed, const void* ids, void* x, void* status, int H, int vocab, int T, void* stream);
int nexrt_prefill_ctl(const void* ctl, void* table, int n_sub, int rows, void* stream);   /* table[j] = ctl with committed length + j * rows */
int nexrt_prefill_advance(void* ctl, int rows, void* seq, unsigned int n_sites, void* stream);   /* committed length += rows, LL sequence base += n_sites */
int nexrt_planes_allreduce_residual(void* x, const void* y, int64_t n, int ksplit, const NexrtLLChannel* ch, unsigned int site, void* stream);
int nexrt_norm_rows(const void* x, const void* gamma, void* xq, void* sx, void* xn, void* planes, int K, int T, float eps, int terms, void* stream);
int nexrt_gdn_gate_quant(const void* o, const void* z, const void* gnorm_w, void* xq, void* sx, int K, int T, float eps, int terms, void* stream);
int nexrt_moe_dense_act(const void* gu, const void* ids, const void* wts, void* hq, void* hs, int I, int S, int T, int n_total, int ksplit, int terms, void* stream);   /* gu: [ksplit][T][n_total * 2I] */
int nexrt_moe_mark_used(const void* ids, void* used, int n_ids, int n_total, void* stream);   /* used[e] = 1 for every routed expert id */
int nexrt_planes_residual(void* x, const void* y, void* sum_out, int64_t n, int ksplit, void* stream);
int nexrt_gdn_chunk(const void* pre, const void* xn, const void* ba_w, const void* conv_w, const void* a_log, const void* dt_bias, const void* ctl,
                    void* conv_ring, void* qkv, void* z, void* beta, void* g, void* state_ring, void* out, int H, int R, int C, int nv, int nqk, int T,
                    int conv_ring_len, int state_ring_len, int ksplit, void* stream);   /* conv + gates + delta rule of T rows after their q|k|v|z projection (pre: [ksplit][T][R]) */

// ---- experts of a multi-row step on tcgen05 (tc_moe.cu) -------------------------------------------------------
// Gate/up of every distinct expert named in ids [M][S] (streamed once each); planes is e4m3 scratch [3M][H].
int nexrt_tc_moe_l1(const void* x, const void* post_ln, const void* w13, const void* w13_s, const void* ids, void* gu, void* planes, int H, int I, int S,
                    int M, int n_experts_total, int ksplit, float eps, int planes_ready, int* status, void* stream);   /* gu: [ksplit][M][S][2I] partial planes */
// Down projection over each row's S experts + tensor-parallel all-reduce + residual in one kernel; planes is e4m3
// scratch [3M][S*I], descale fp32 scratch [M].
int nexrt_tc_moe_l2_allreduce(const void* gu, const void* ids, const void* wts, const void* w2, const void* w2_s, void* x, void* planes, void* descale,
                              int H, int I, int S, int M, int n_experts_total, int gu_ksplit, const NexrtLLChannel* ch, unsigned int site, int* status,
                              void* stream);

// ---- wide (multi-row) projections on tcgen05 ---------------------------------------------------------------------
int nexrt_rows_norm_split(const void* x, const void* gamma, void* planes, void* xn, int H, int M, float eps, void* stream);
int nexrt_tc_rows_gemm(const void* w, const void* w_s, const void* planes, void* out, const void* zero_ids, int R, int K, int M, int ksplit, int* status,
                       void* stream);   /* out: [ksplit][M][R] partial planes */
int nexrt_gdn_front_tail(const void* pre, const void* xn, const void* ba_w, const void* conv_w, const void* a_log, const void* dt_bias, const void* ctl,
                         void* conv_ring, void* qkv, void* z, void* beta, void* g, int H, int R, int C, int nv, int M, int conv_ring_len, int ksplit,
                         void* stream);

int nexrt_tc_router_logits(const void* x, const void* gamma, const void* w, void* planes, void* partial, const void* zero_ids, int rows, int rows_pad, int K,
                           int M, int ksplit, float eps, void* planes_e4m3, int* status, void* stream);   /* partial: [ksplit][M][rows_pad] */
int nexrt_moe_router_topk(const void* partial, int ksplit, int rows_pad, void* logits, void* ids, void* wts, int E, int topk, int M, void* stream);

int nexrt_lmhead_sample_from_logits(const void* logits_in, void* cand, void* ticket, const void* sampling, void* ctl, void* export_buf, int H, int V_local,
                                    int vocab_base, int M, int mode, int arg, const NexrtLLChannel* ch, unsigned int site, int n_cta, void* stream);

// Wide out-projection (multi-row steps): staging + split into planes, then tcgen05 GEMM with all-reduce epilogue.
int nexrt_oproj_stage_split(const void* in, const void* z, const void* gnorm_w, void* planes, void* descale, int K, int M, int mode, float eps, int hd,
                            const NexrtLLChannel* cp, unsigned int cp_site, void* stream);
int nexrt_tc_oproj_allreduce(const void* planes, const void* descale, const void* w, const void* w_s, void* x, const void* zero_ids, int H, int K, int M,
                             int overwrite, const NexrtLLChannel* ch, unsigned int site, int* status, void* stream);

int nexrt_attn_front_tail(const void* pre, const void* ctl, void* q_raw, void* gate, void* k_raw, void* v_cache, int hd, int nq, int ngate, int kvh, int M,
                          int cache_len, int ksplit, void* stream);   /* pre: [ksplit][M][R] partial planes of the rows GEMM */

#ifdef __cplusplus
}
#endif
