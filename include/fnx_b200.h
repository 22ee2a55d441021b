/* fnx_b200: C ABI of the B200 (sm_100a) speculative-decoding verify path.
 *
 * Drop-in boundary: these entry points stand where the reference engine's per-layer operator API stands
 * (engine/src/kernels.hpp, namespace fnx: free functions on raw device pointers and a stream, called only by the
 * window scheduler in engine/src/engine.cu and engine_common.cu).  The reference has no FFI of its own; a C ABI
 * is what a maintainer would bind from C++ (or any other host language) to swap this path in.  Each declaration
 * names the reference interface it replaces.
 *
 * Conventions (as the reference's, engine/src/kernels.hpp:1-2):
 *   - every pointer is DEVICE memory unless its name starts with h_; the caller owns every buffer;
 *   - activations are f32 rows; quantised weights are GGML IQ3_S, re-tiled once by fnx_iq3s_retile();
 *   - window scalars (first position, state slot) live in device memory so that captured graphs replay;
 *   - no entry point synchronises, allocates or reads results back: all are stream-capture safe, except where
 *     a comment says otherwise (fnx_engine_* set-up calls, fnx_engine_load_gguf, fnx_comm_*; fnx_gguf_* is host code);
 *     the prompt-sized products (fnx_dense_prompt, fnx_router_rows, fnx_moe_prefill, fnx_attn_prompt) encode their
 *     tensor maps on the host at each call and pass them by value: no device allocation, capture safe;
 *   - return value: 0 on success, a negative FNX_E_* code otherwise, with text from fnx_last_error();
 *     device-side conditions are OR-ed into the `err` word (FNX_ERR_* bits, the reference's bit values,
 *     engine/src/kernels.hpp:373-375), which the caller reads back with the window's results.
 */
#ifndef FNX_B200_H
#define FNX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* fnx_stream;   /* a cudaStream_t */

enum { FNX_OK = 0, FNX_E_ARG = -1, FNX_E_CUDA = -2, FNX_E_STATE = -3, FNX_E_UNAVAILABLE = -4 };
/* device error bits (engine/src/kernels.hpp:373-375): a wait gave up; a non-finite value; non-finite logits */
enum { FNX_ERR_TIMEOUT = 1, FNX_ERR_NONFINITE = 2, FNX_ERR_LOGITS = 16 };

enum { FNX_TOPK_N = 64,      /* sampler candidates per row (TOPK_N, engine/src/kernels.hpp:441) */
       FNX_MAX_ROWS = 32,    /* rows (tree nodes) of one verify window */
       FNX_JOB_TOK = 4,      /* activation rows of one expert job */
       FNX_DENSE_ROWS = 12,  /* activation rows of one fnx_dense call (three row groups of four) */
       FNX_LANE_ROWS = 5,    /* rows of one lane of a batched window */
       FNX_PENALTY_CAP = 4096, /* tokens of a penalty window (Engine::PEN_CAP of the reference's sampler) */
       FNX_ATTN_STATIC_MAX_SLOTS = 16384 };   /* (row, head, split) partials fnx_attn_static's built-in scratch holds */

const char* fnx_last_error(void);
int fnx_version(void);

/* ---------------------------------------------------------------------------------------------- IQ3_S weights
 * GGML block_iq3_s <-> the device tile layout (a bit permutation; same size).  Replaces the reference's load-time
 * re-layout of weights (split Q8_0 layout, engine/src/dense.cuh; expert slicing engine/src/model.cpp:1063-1069).
 * rows % 16 == 0, cols % 256 == 0. */
size_t fnx_iq3s_bytes(size_t rows, size_t cols);
int fnx_iq3s_retile(const void* ggml_blocks, void* tiles, size_t rows, size_t cols, fnx_stream st);
int fnx_iq3s_untile(const void* tiles, void* ggml_blocks, size_t rows, size_t cols, fnx_stream st);
/* tiles -> f32 [rows][cols] (tests and tools; fnx::conv::dequantize, engine/src/tensor_convert.hpp:143-326) */
int fnx_iq3s_dequant_tiles(const void* tiles, float* out, size_t rows, size_t cols, fnx_stream st);
/* deterministic fixture quantiser f32 -> GGML blocks (ggml's own quantiser is not part of the reference tree) */
int fnx_iq3s_quantize(const float* w, void* ggml_blocks, size_t n, fnx_stream st);
/* out[i] = sigma * N(0,1) from Philox4x32-10 keyed by (seed, stream_id), counter i / 4 */
int fnx_fill_normal(float* out, size_t n, float sigma, uint64_t seed, uint32_t stream_id, fnx_stream st);

/* ---------------------------------------------------------------------------------------------- dense GEMV
 * y[t][r] (+)= W[r] . xin[t] for t < T (T <= fnx_dense_rows(cols) per call: FNX_DENSE_ROWS up to 2048 columns, 8 beyond, where
 * three row groups' images no longer fit the block's shared memory), W an IQ3_S tile matrix; xin[t] = x[t], or
 * rmsnorm(x[t]) * norm_w when norm_w is not null.  Replaces q8s_gemv / mmvq / rms_norm_rows
 * (engine/src/kernels.hpp:49-52, 405-406).  rows % 16 == 0; cols in {256, 512, 1024, 2048, 4096}. */
int fnx_dense_rows(int cols);
int fnx_dense(const void* W, int rows, int cols, const float* x, int ldx, int T, const float* norm_w, float eps,
              float* y, int ldy, int accumulate, unsigned* err, fnx_stream st);
/* fnx_dense over rows whose quantised image a producer already left on the device (fnx_moe_combine_image): ximg = the image of
 * the call's T rows (fnx_dense_image_bytes(cols) bytes per FNX_DENSE_ROWS rows; 16-byte aligned), normed != 0 when it is the image of
 * rmsnorm(x) * norm_w.  The blocks copy the image instead of each quantising the rows (the reference quantises a row once
 * for all its consumers the same way: quantize_q8_1 / q8_twin, engine/src/kernels.hpp:49-52).  Same bits as fnx_dense. */
size_t fnx_dense_image_bytes(int cols);
int fnx_dense_image(const void* W, int rows, int cols, const void* ximg, int T, int normed, float eps, float* y, int ldy,
                    int accumulate, unsigned* err, fnx_stream st);

/* Tracing (FNX_PROF / k_prof_stamp, engine/src/engine.cu:1382-1529): while a device buffer of
 * [blocks][64] u64 is registered, block b of every IQ3_S matvec launch writes %globaltimer stamps of its phases
 * (start, set-up done, activations ready, then per step: weights landed, computed) to row b, count in word 0.
 * Null unregisters.  Synchronises. */
int fnx_debug_profile_buffer(void* dev_u64);

/* ---------------------------------------------------------------------------------------------- MoE
 * One expert job: expert `w` applied to n activation rows (Job, engine/src/kernels.hpp:18-23, with MAXT = 4 rows;
 * an expert picked by more rows gets several jobs). */
typedef struct {
    int w;                    /* expert index */
    int n;                    /* rows of the job, 1..FNX_JOB_TOK */
    int y[FNX_JOB_TOK];       /* activation rows (tokens) */
    int out[FNX_JOB_TOK];     /* output rows: pair t * K + k; the shared expert's T * K + t */
} fnx_job;

/* router_route (engine/src/kernels.hpp:294-296; simple form route :79): logits [T][E + 1] = Wr . xin (f32 weights,
 * row E the shared expert's gate), top-K by logit (ties: lower index), weights = softmax over the K; jobs for the
 * experts in [e_lo, e_hi) in first-pick order, then (add_shared != 0) one job of the shared expert (w = E) per 4
 * rows; njobs[0] = their number (njobs[1] is the launch's block counter: zero it once, it is left at zero).
 * xin = rmsnorm(x) * norm_w when norm_w is not null.  stats (may be null): stats[0] += routed jobs of this call,
 * stats[1] += 1 (how many distinct experts the windows touched: the roofline's byte count). */
int fnx_router_route(const float* Wr, const float* x, const float* norm_w, float eps, int T, int E, int H, int K,
                     int e_lo, int e_hi, int add_shared, float* logits, int* topi, float* topw, fnx_job* jobs,
                     int* njobs, unsigned long long* stats, unsigned* err, fnx_stream st);
/* the routing of any number of rows, for prompts (the prompt pass's router, engine/src/prefill.cu:653): logits, top K and
 * weights as fnx_router_route computes them, without a job list (fnx_moe_prefill groups the pairs itself).  With scratch
 * (fnx_router_rows_scratch_bytes(T, E, H) bytes) and 1,024 rows or more the logits are a tcgen05.mma product of the rows and the
 * weights split into f16 high and low parts (three products; the tensor core's truncating f32 accumulation leaves the logits
 * good to a few 1e-5, against ~1e-6 for the f32 walk that scratch = null keeps). */
size_t fnx_router_rows_scratch_bytes(int T, int E, int H);
int fnx_router_rows(const float* Wr, const float* x, const float* norm_w, float eps, int T, int E, int H, int K, float* logits,
                    int* topi, float* topw, void* scratch, unsigned* err, fnx_stream st);
/* moe_gate_up + SwiGLU (engine/src/kernels.hpp:319, :329; engine/src/moe.cuh:572-608): h[out][F] =
 * silu(Wg . xin) * (Wu . xin).  Wgu: expert e's [gate (F); up (F)] x H tile matrix at Wgu + (e - e_base) *
 * expert_stride; the shared expert (w == E) is read from Wsh. */
int fnx_moe_gate_up(const void* Wgu, size_t expert_stride, int e_base, const void* Wsh, int E, const fnx_job* jobs,
                    const int* njobs, int njobs_max, const float* x, const float* norm_w, float eps, int H, int F,
                    float* h, unsigned* err, fnx_stream st);
/* moe_down (engine/src/kernels.hpp:343): part[out][H] = Wd . h[out] */
int fnx_moe_down(const void* Wdn, size_t expert_stride, int e_base, const void* Wsh, int E, const fnx_job* jobs,
                 const int* njobs, int njobs_max, const float* h, int H, int F, float* part, unsigned* err,
                 fnx_stream st);
/* moe_combine (engine/src/kernels.hpp:83; the cross-card addend of ring_sum :396): out[t] (+)= sum over the picks in
 * [e_lo, e_hi) of topw * part[t K + k], + sigmoid(logits[t][E]) * part[T K + t] when add_shared */
int fnx_moe_combine(const float* part, const int* topi, const float* topw, const float* logits, int T, int E, int H,
                    int K, int e_lo, int e_hi, int add_shared, float* out, int accumulate, fnx_stream st);
/* fnx_moe_combine(part, ..., 0, E, 1, R, 1) that also leaves the image of rmsnorm(R[t]) * img_norm_w for fnx_dense_image
 * (ceil(T / FNX_DENSE_ROWS) * fnx_dense_image_bytes(H) bytes, 16-byte aligned: one image per FNX_DENSE_ROWS rows): the rows are quantised once, by the kernel that completes
 * them, instead of by every block of the next projection.  R gets the same bits as from fnx_moe_combine. */
int fnx_moe_combine_image(const float* part, const int* topi, const float* topw, const float* logits, int T, int E, int H,
                          int K, float* R, void* img_out, const float* img_norm_w, fnx_stream st);

/* Prompt-sized MoE block (moe_gate_up_mma / moe_down_mma, engine/src/kernels.hpp:328-330, with the job build of
 * engine/src/prefill.cu:288-377): out[t] (+)= the routed experts in [e_lo, e_hi) and (add_shared) the shared expert of
 * rmsnorm(x[t]) * norm_w, for any number of rows T, given the routing (topi, topw [T][K], logits [T][E + 1]).  The
 * (row, pick) pairs are grouped by expert into jobs of up to 256 rows whose products run on the tensor cores
 * (tcgen05.mma, f16 operands decoded from IQ3_S, f32 accumulators in tensor memory).  The job count stays on the device
 * (the grids cover its largest possible value; surplus blocks leave at once).  scratch: fnx_moe_prefill_scratch_bytes(T, K, E, H, F) bytes. */
size_t fnx_moe_prefill_scratch_bytes(int T, int K, int E, int H, int F);
/* fnx_dense for prompt-sized row counts (the prompt pass's projections, engine/src/prefill.cu; q8s_gemm / k_mmq,
 * engine/src/kernels.hpp:56-70): y[t][r] (+)= W[r] . xin[t] for any T on the same tensor-core kernel as the prompt MoE block
 * (weights decoded from IQ3_S to f16, activations rounded to f16 once per call, f32 accumulators in tensor memory).  x is
 * [T][cols] contiguous; rows % 16 == 0; cols % 256 == 0; scratch: fnx_dense_prompt_scratch_bytes(T, rows, cols) bytes.
 * From 1,024 rows on the matrix is decoded to f16 once and the product takes both operands by tensor copies. */
size_t fnx_dense_prompt_scratch_bytes(int T, int rows, int cols);
int fnx_dense_prompt(const void* W, int rows, int cols, const float* x, int T, const float* norm_w, float eps, float* y,
                     int ldy, int accumulate, void* scratch, unsigned* err, fnx_stream st);
int fnx_moe_prefill(const void* Wgu, size_t gu_stride, const void* Wdn, size_t dn_stride, const void* Wsh_gu,
                    const void* Wsh_dn, int e_base, int E, int K, int e_lo, int e_hi, int add_shared, const int* topi,
                    const float* topw, const float* logits, const float* x, const float* norm_w, float eps, int T, int H,
                    int F, float* out, int accumulate, void* scratch, unsigned* err, fnx_stream st);

/* ---------------------------------------------------------------------------------------------- attention
 * attn_prep_append (engine/src/kernels.hpp:259): per-head RMS norm, NEOX rotary on the first nrot dims at position
 * *pos0 + depth[t] (depth null: t), K and V rows stored as f16 at cache row *pos0 + t.
 * qg rows [nq][q (hd) | gate (hd)], k and v rows [nkv][hd], with row strides ldq, ldk, ldv floats;
 * caches [rows][nkv][hd] f16. */
int fnx_attn_prep_append(float* qg, int ldq, float* k, int ldk, const float* v, int ldv, const float* q_norm,
                         const float* k_norm, void* kc, void* vc, int T, int nq, int nkv, int hd, int nrot,
                         const int* pos0, const int* depth, float eps, float rope_base, fnx_stream st);
/* attn (engine/src/kernels.hpp:238): softmax(q k / sqrt(hd)) v sigmoid(gate) over cache rows [0, *pos0) and the
 * window rows on row t's path to the root (parent null: a chain, the reference's causal case).
 * out [T][nq][hd].  scratch: fnx_attn_scratch_bytes(T, nq, hd) bytes (attn_scratch_floats, :131). */
size_t fnx_attn_scratch_bytes(int T, int nq, int hd);
int fnx_attn(const float* qg, int ldq, const void* kc, const void* vc, float* out, int T, int nq, int nkv, int hd,
             const int* pos0, const int* parent, void* scratch, fnx_stream st);
/* the same for a prompt's rows (attn_prompt, engine/src/kernels.hpp:252): T rows of any number, a chain (row t sees every
 * position up to pos0 + t), no splits; the scores come from the f16-rounded queries alone (the window form adds their low
 * halves).  Where a KV head serves eight query heads of 256 dims: sixteen rows per block on tcgen05.mma, scores and sums in
 * tensor memory (a wait that gives up sets FNX_ERR_TIMEOUT in *err, which may be null); otherwise, or with use_mma_sync != 0:
 * twelve rows per block on mma.sync.  fnx_attn_prep_append takes such T when depth is null.
 * scratch: fnx_attn_prompt_scratch_bytes(T, nq, hd) bytes. */
size_t fnx_attn_prompt_scratch_bytes(int T, int nq, int hd);
int fnx_attn_prompt(const float* qg, int ldq, const void* kc, const void* vc, float* out, int T, int nq, int nkv, int hd,
                    const int* pos0, void* scratch, unsigned* err, int use_mma_sync, fnx_stream st);
/* fnx_attn without caller scratch and without any allocation (no counterpart in the reference, whose attn takes the
 * caller's buffer, engine/src/kernels.hpp:238): the split partials go to one file-scope device array of
 * FNX_ATTN_STATIC_MAX_SLOTS x (hd floats + 8 bytes) = 16.9 MB per device, for callers that may not allocate (a
 * memory-frozen serving process).  Same arguments, kernels and results as fnx_attn.
 * Limit: T * nq * splits <= FNX_ATTN_STATIC_MAX_SLOTS, where splits = SM count / nkv (148 / nkv on a B200): e.g. 13
 * rows of 16 heads over 2 KV heads; larger windows are rejected with FNX_E_ARG and a message naming the three factors.
 * Set-up: the first call on a device resolves the array's address with cudaGetSymbolAddress (return code checked) and
 * raises the kernel's shared-memory limit; neither belongs inside a stream capture, so call fnx_attn_static_setup()
 * (or one plain fnx_attn_static) once per device before capturing.  After set-up a call makes two kernel launches; its
 * only other runtime calls are cudaGetDevice and cudaGetLastError, which neither allocate nor synchronise.
 * Sharing: every call on a device uses the same array.  Nothing in it has to start at zero (each call overwrites
 * every slot it later reads), but two calls that overlap in time (different streams or host threads, same device)
 * race on it and give undefined results: serialise them on one stream, or use fnx_attn with separate scratch. */
int fnx_attn_static_setup(void);
int fnx_attn_static(const float* qg, int ldq, const void* kc, const void* vc, float* out, int T, int nq, int nkv, int hd,
                    const int* pos0, const int* parent, fnx_stream st);

/* Batched lanes of attention (enqueue_rows, engine/src/engine.cu:1936): lane j = rows [lane_row0[j], lane_row0[j + 1]) of
 * the window (at most FNX_LANE_ROWS rows), a chain of sequence lane_seq[j] at position pos[lane_seq[j]], reading and
 * appending that sequence's caches at kc_base / vc_base + seq * seq_stride_rows rows.  Same kernels' bodies and results as
 * the single-sequence calls. */
/* (in the lanes forms a lane whose lane_seq entry is negative is skipped: its rows are computed elsewhere, e.g. by the
 * expert-parallel rank that holds that sequence's caches and states) */
int fnx_attn_prep_append_lanes(float* qg, int ldq, float* k, int ldk, const float* v, int ldv, const float* q_norm,
                               const float* k_norm, void* kc_base, void* vc_base, size_t seq_stride_rows, int n_lanes,
                               int max_lane_rows, int nq, int nkv, int hd, int nrot, const int* pos, const int* lane_seq,
                               const int* lane_row0, float eps, float rope_base, fnx_stream st);
int fnx_attn_lanes(const float* qg, int ldq, const void* kc_base, const void* vc_base, size_t seq_stride_rows, float* out,
                   int T, int n_lanes, int nq, int nkv, int hd, const int* pos, const int* lane_seq, const int* lane_row0,
                   void* scratch, fnx_stream st);

/* ---------------------------------------------------------------------------------------------- gated DeltaNet
 * gdn_core (engine/src/kernels.hpp:97-99).  State and conv-history rings of NS slots replace snap / hsnap + the
 * commit copy: the window starts from slot *cur; row t starts from its parent's result and writes slot
 * (*cur + 1 + t) % NS.  S_pool [NS][nv][hs][hs] f32, hist_pool [NS][3][(2 nk + nv) hs] f32; y [T][nv hs].
 * qkvz rows [q | k | v | z] with stride ldx floats, ab rows [alpha (nv) | beta (nv)] with stride ldab. */
int fnx_gdn_core(const float* qkvz, int ldx, const float* ab, int ldab, float* hist_pool, const float* convw, const float* dt,
                 const float* a, const float* nw, float* S_pool, const int* cur, int NS, const int* parent, float* y,
                 int nk, int nv, int hs, int T, float eps, fnx_stream st);

/* Batched lanes of gdn_core (gdn_core_segs, engine/src/kernels.cu:2112-2156; GdnLanes, engine/src/kernels.hpp:103-110):
 * lane j is a chain from slot cur[lane_seq[j]] of that sequence's rings at hist_pool + seq * hist_seq_stride floats and
 * S_pool + seq * s_seq_stride floats. */
/* the same over a prompt's T rows (any T), a chain of which every row is kept (gdn_prompt, engine/src/kernels.cu:2158), in three
 * launches: conv + SiLU, q / k norms and gates of every row at once; the delta rule with the state in registers from the
 * first row to the last; the gated norm of every row at once.  Starts from state slot `cur` (a host value here) and leaves the
 * last row's state and conv history in slot (cur + T) % NS: the caller advances its slot index by T.
 * scratch: fnx_gdn_prompt_scratch_bytes(T, nk, nv, hs) bytes. */
size_t fnx_gdn_prompt_scratch_bytes(int T, int nk, int nv, int hs);
int fnx_gdn_prompt(const float* qkvz, int ldx, const float* ab, int ldab, float* hist_pool, const float* convw, const float* dt,
                   const float* a, const float* nw, float* S_pool, int cur, int NS, float* y, int nk, int nv, int hs, int T,
                   float eps, void* scratch, fnx_stream st);
int fnx_gdn_core_lanes(const float* qkvz, int ldx, const float* ab, int ldab, float* hist_pool, size_t hist_seq_stride,
                       const float* convw, const float* dt, const float* a, const float* nw, float* S_pool,
                       size_t s_seq_stride, const int* cur, int NS, const int* lane_seq, const int* lane_row0, int n_lanes,
                       int max_lane_rows, float* y, int nk, int nv, int hs, float eps, fnx_stream st);

/* ---------------------------------------------------------------------------------------------- commit
 * Engine::commit at operator level (engine/src/engine_common.cu:710-754; its copies, copy_many, engine/src/kernels.hpp:429):
 * keeps the window rows path[0..n) (device array, increasing, path[0] = 0).  The kept rows' K and V move to consecutive
 * cache rows *pos0 .. *pos0 + n of every attention layer (k_caches / v_caches: device arrays of n_attn_layers cache
 * pointers, rows of row_halves f16), the DeltaNet rings advance to the last kept row's slot (*cur = (*cur + 1 +
 * path[n - 1]) % NS: the states themselves do not move), and *pos0 += n.  A chain kept as a prefix copies nothing. */
int fnx_commit(void* const* k_caches, void* const* v_caches, int n_attn_layers, int row_halves, const int* path, int n,
               int* pos0, int* cur, int NS, fnx_stream st);

/* ---------------------------------------------------------------------------------------------- head
 * argmax (engine/src/kernels.hpp:433): per-row maximum, ties to the lower index; err bit 16 on a non-finite logit */
int fnx_argmax(const float* logits, int T, int V, int* best_i, float* best_v, unsigned* err, fnx_stream st);
/* the same over a reduced vocabulary: best_i[t] = map[row] (the draft vocabulary's token ids, Mtp::vocab) */
int fnx_argmax_mapped(const float* logits, int T, int V, const int* map, int* best_i, float* best_v, unsigned* err,
                      fnx_stream st);
/* top_tokens (engine/src/kernels.hpp:445) without penalties: the 64 highest per row, logit descending, id ascending */
int fnx_top_tokens(const float* logits, int T, int V, float* out_v, int* out_i, fnx_stream st);
/* The sampler's logit changes before the candidates are taken (the first half of k_topk_rows, engine/src/topk.cuh:30-45, with
 * the rows' penalty windows of engine/src/session.cpp:88-98, 581-585), in place on logits [T][V]: per row the logit_bias
 * list added (bias_tok each once), then over the row's penalty window (the last last_n tokens of ctx[0 .. *ctx_n) followed by
 * window rows tok[0 .. row]) each token once: l = l <= 0 ? l * repeat : l / repeat, then l -= count * freq + present.
 * last_n = 0: the bias only (ctx, ctx_n, tok may be null). */
int fnx_logit_adjust(float* logits, int T, int V, const int* ctx, const int* ctx_n, const int* tok, int last_n, float repeat, float freq,
                     float present, const int* bias_tok, const float* bias_val, int bias_n, fnx_stream st);
/* embed rows: R[t] = f16 table[tok[t]] (the reference embeds on the host, engine_common.cu:955) */
int fnx_embed_rows(const void* table_f16, const int* tok, int T, int H, float* R, fnx_stream st);
/* The draft (MTP) layer's input rows, the one step of mtp_enqueue that no other layer has (engine/src/engine.cu:2103-2113):
 * R[t] = fc_hid . (rmsnorm(h[t]) * hnorm) + fc_emb . (rmsnorm(table[tok[t]]) * enorm), t < T; fc_hid and fc_emb H x H IQ3_S tile
 * matrices, h the main model's rows ahead of its output norm (row stride ldh), tok the tokens that follow them, emb [T][H]
 * scratch that receives the embedding rows.  The rest of a draft call is the attention block (fnx_dense, fnx_attn_prep_append,
 * fnx_attn), the MoE block (fnx_router_route, fnx_moe_gate_up, fnx_moe_down, fnx_moe_combine) and the head (fnx_dense,
 * fnx_argmax) on R, as for any layer; fnx_engine_draft is that composition.  Capture-safe; allocates nothing. */
int fnx_mtp_input(const void* fc_hid, const void* fc_emb, const void* table_f16, const float* hnorm, const float* enorm, float eps,
                  const float* h, int ldh, const int* tok, int T, int H, float* emb, float* R, unsigned* err, fnx_stream st);
/* rms_norm_rows (engine/src/kernels.hpp:406) */
int fnx_rmsnorm(const float* x, const float* w, float* y, int rows, int n, float eps, fnx_stream st);

/* ---------------------------------------------------------------------------------------------- drafting, acceptance
 * lookup_drafts (engine/src/session.cpp:428-447) on the GPU: ctx[0 .. *n) tokens; out[0 .. out_n[0]) drafts,
 * out_n[1] = match start or -1.  d1: device scalar (the draft layer's first token, < 0: any). */
int fnx_lookup_draft(const int* ctx, const int* n, int lk, const int* d1, int* out, int* out_n, fnx_stream st);
/* greedy acceptance over a tree (chain rule engine/src/session.cpp:573): result[0] = n, result[1 .. 1 + n) = the
 * accepted node path, result[1 + FNX_MAX_ROWS ..] = the emitted tokens */
int fnx_accept_greedy(const int* tok, const int* parent, const int* best, int T, int* result, fnx_stream st);
typedef struct {
    float temperature, top_p, min_p;
    int top_k;
} fnx_sampling;
/* speculative sampling over a chain (engine/src/session.cpp:575-612, make_dist :41-75, draw :77-84) with
 * Philox4x32-10 uniforms addressed (seed, seq, step, slot).  cand_* [T][64] from fnx_top_tokens; q_* the draft
 * distributions ([T-1][64], q_n[j] = 0: a fixed draft; all null: every draft fixed). result as fnx_accept_greedy's. */
int fnx_accept_sample(const float* cand_v, const int* cand_i, const int* tok, int T, fnx_sampling s, const int* q_ids,
                      const double* q_p, const int* q_n, uint64_t seed, uint32_t seq, const uint32_t* step,
                      int* result, fnx_stream st);
/* Batched lanes of the two rules: lane j's chain is rows [lane_row0[j], lane_row0[j + 1]); result [n_lanes][1 + 2
 * FNX_MAX_ROWS]; the sampling rule draws sequence lane_seq[j]'s uniforms at window steps[lane_seq[j]], drafts fixed. */
int fnx_accept_greedy_lanes(const int* tok, const int* best, const int* lane_row0, int n_lanes, int* result, fnx_stream st);
int fnx_accept_sample_lanes(const float* cand_v, const int* cand_i, const int* tok, fnx_sampling s, uint64_t seed,
                            const int* lane_seq, const int* lane_row0, int n_lanes, int max_lane_rows,
                            const uint32_t* steps, int* result, fnx_stream st);

/* ---------------------------------------------------------------------------------------------- engine
 * The thin window scheduler: Engine::verify / commit / draft (engine/src/engine.hpp:50-229) for the synthetic
 * Qwen3-Next-style model, one CUDA graph per window shape.  Set-up calls allocate and synchronise. */
typedef struct {
    int n_layer, hidden, n_expert, top_k, ffn;          /* 48, 2048, 512, 10, 512 */
    int n_q_head, n_kv_head, head_dim, n_rot;           /* 16, 2, 256, 64 */
    int gdn_k_head, gdn_v_head, gdn_head_dim;           /* 16, 32, 128 */
    int vocab, max_ctx, max_rows;                       /* 151936, context rows, rows per window <= FNX_MAX_ROWS */
    int attn_every;                                     /* 4: layer l is attention when (l + 1) % 4 == 0 */
    int ep_rank, ep_size;                               /* expert-parallel shard of this process */
    int n_seq;                                          /* independent sequences (lanes) held */
    float eps, rope_base;
    int draft_vocab;                                    /* 0: the draft layer's head is the main head over the whole vocabulary;
                                                         * else (a multiple of 16, <= vocab) the rows of the draft layer's own head
                                                         * over a draft vocabulary (Mtp::vocab, engine/src/model.hpp:252: head row
                                                         * -> token id; the reference ships 40,525 and 49,146 ids) */
} fnx_model_config;
typedef struct fnx_engine fnx_engine;

int fnx_engine_create(const fnx_model_config* cfg, fnx_engine** out);
void fnx_engine_destroy(fnx_engine* e);
/* random-init weights: every matrix N(0, sigma) -> IQ3_S; norm weights 1; router f32 N(0, sigma) */
int fnx_engine_init_synthetic(fnx_engine* e, uint64_t seed, float sigma);
/* bytes of weights + state this engine holds on its GPU */
size_t fnx_engine_device_bytes(const fnx_engine* e);
/* the engine's tensors by name, for tests and loaders: device pointer and byte size (0 if unknown) */
void* fnx_engine_tensor(fnx_engine* e, const char* name, size_t* bytes);
/* resets sequence `seq` to an empty context */
int fnx_engine_reset(fnx_engine* e, int seq);
/* Engine::verify: runs the T window rows (h_tok, h_parent host arrays; parent null = chain) of sequence `seq`
 * through the model; leaves logits, per-row argmax and the acceptance result on the device and, when h_result is
 * not null, copies the greedy acceptance result back (synchronises).  Does not commit. */
int fnx_engine_verify(fnx_engine* e, int seq, const int* h_tok, const int* h_parent, int T, int* h_result);
/* Engine::prefill (the prompt pass, engine/src/prefill.cu): reads n prompt tokens into sequence `seq` and leaves the engine
 * as after verifying and keeping them (caches, states, context, the last token's logits and emitted token), but on the
 * prompt-sized kernels: the first n - 1 tokens go chunk by chunk and layer by layer through tensor-core projections and
 * experts, chained DeltaNet windows and window attention; the last token through a one-row window.  Activations are rounded
 * to f16 where the window path uses two int8 levels, so the states agree with the window path to the parity tolerance, not
 * bit for bit.  Single rank only (FNX_E_ARG on an expert-parallel engine).  Synchronises. */
int fnx_engine_prompt(fnx_engine* e, int seq, const int* h_tok, int n);
/* Tracing of the prompt pass (the reference's FNX_PROF idea, engine/src/engine.cu:1382-1529): with on != 0 the following
 * fnx_engine_prompt calls time their phases with events (a synchronisation per chunk); h_phase_ms6, when not null, receives the
 * last timed prompt's device ms: input projections, attention, DeltaNet, output projections, router, experts. */
int fnx_engine_prompt_timing(fnx_engine* e, int on, float* h_phase_ms6);
/* Engine::commit: keeps the n accepted rows h_path[0..n) of the last window of `seq`.  The window buffers (tokens,
 * acceptance result, residual rows) are shared by the engine's sequences: commit (and draft) sequence A before verifying
 * sequence B; a commit or draft for a sequence other than the one verified last returns FNX_E_STATE. */
int fnx_engine_commit(fnx_engine* e, int seq, const int* h_path, int n);
/* Engine::draft: the MTP layer on the rows kept by the last commit, then k - 1 chained single-row calls;
 * h_drafts receives k tokens */
int fnx_engine_draft(fnx_engine* e, int seq, int k, int* h_drafts);
/* the device time of the last verify / draft graph launch in milliseconds (CUDA events on the engine's stream) */
float fnx_engine_last_ms(const fnx_engine* e);
/* the device error word (FNX_ERR_* bits) of the last window; synchronises.  fnx_engine_verify clears the word when it
 * starts a window, and returns FNX_E_STATE with the bits when it copies a result back. */
int fnx_engine_error_bits(fnx_engine* e, unsigned* h_bits);
/* Acceptance rule of the following windows: null = greedy (the default); else the sampling rule of
 * engine/src/session.cpp:575-612 over each row's 64 best tokens with Philox uniforms addressed (seed, seq, window, slot);
 * drafts count as fixed (q = 1), windows must be chains.  Resets the per-sequence window counters. */
int fnx_engine_set_sampling(fnx_engine* e, const fnx_sampling* s, uint64_t seed);
/* The sampler's logit changes of the following single-sequence windows (fnx_logit_adjust on every window's logits before the
 * acceptance rule, greedy or sampling, looks at them): a request's logit_bias (host arrays, copied) and its penalties over
 * each row's penalty window (Sampling's pen_* and bias, engine/src/session.hpp:17-26; applied as engine/src/session.cpp:566-585).
 * null, or neither a window nor a list: none (the default).  Penalty windows need chain windows.  Batched lane windows and the
 * draft layer's own logits are not changed.  Drops the captured graphs. */
typedef struct {
    float repeat, freq, present;   /* 1, 0, 0 change nothing */
    int last_n;                    /* tokens of the penalty window, 0: no penalties */
    const int* bias_tok;           /* logit_bias: each token once */
    const float* bias_val;
    int bias_n;
} fnx_logit_rules;
int fnx_engine_set_logit_rules(fnx_engine* e, const fnx_logit_rules* r);
/* lookup_drafts (engine/src/session.cpp:428-447) over the sequence's own context on the device (committed tokens and
 * the pending one; root >= 0 replaces the pending token, for a caller that starts the next window from another token):
 * up to lk drafts into h_out, their number into h_n; d1 >= 0 keeps only a match whose first draft is d1. */
int fnx_engine_lookup(fnx_engine* e, int seq, int lk, int d1, int root, int* h_out, int* h_n);
/* The lane planner (plan_rows, engine/src/batch_plan.hpp:63-132): host arithmetic.  Lane i offers up to avail[i] drafts;
 * reach[i * (FNX_LANE_ROWS - 1) + j] is the chance that its drafts 0..j all stand (non-increasing in j); chain[i] != 0: a
 * draft-layer chain, whose drafts after the first cost chain_ms each.  A window's rows past the lanes' first cost row_lo each
 * up to the knee'th row of the window and row_hi past it, on top of base_ms.  drafts[i] receives the counts with the most
 * expected tokens per ms (exact), at most max_rows - n_lanes in all and FNX_LANE_ROWS - 1 per lane; rate_out (optional) that
 * rate.  Feed the result to fnx_engine_verify_lanes_rows (rows = 1 + drafts). */
typedef struct {
    double row_lo, row_hi, chain_ms;
    int knee;
} fnx_row_cost;
int fnx_plan_rows(int n_lanes, const int* avail, const double* reach, const int* chain, int max_rows, double base_ms,
                  const fnx_row_cost* cost, int* drafts, double* rate_out);
/* Sequence-state cache (Engine::save_state / load_state / state_bytes, engine/src/engine_common.cu:629-688): a committed
 * sequence's DeltaNet states, conv histories, context tokens and, with kv, its cache rows [0, pos), copied to host memory the
 * caller owns (fnx_engine_state_bytes(e, seq, kv) bytes) and put back later into the same or another sequence.  Without kv
 * the image is a checkpoint of the same sequence: it can only be loaded while the engine still holds those rows' K/V (the
 * tokens are compared).  Neither call may fall between a window and its commit (FNX_E_ARG); after a load the sequence stands
 * at the saved position with no window pending (verify next; drafts need a window first).  Both synchronise. */
size_t fnx_engine_state_bytes(fnx_engine* e, int seq, int kv);
int fnx_engine_save_state(fnx_engine* e, int seq, int kv, void* host, size_t bytes);
int fnx_engine_load_state(fnx_engine* e, int seq, const void* host, size_t bytes);
/* Batched lanes (Engine::verify_rows / commit_rows / draft_rows, engine/src/engine_common.cu:1234-1684; GdnLanes,
 * engine/src/kernels.hpp:103-110): one window holds `rows` <= FNX_LANE_ROWS rows of each of n_lanes distinct sequences
 * (n_lanes * rows <= max_rows), every lane a chain continuing its own sequence.  Projections, router, experts and head run
 * over all rows at once (an expert picked by rows of several lanes is read once); attention, DeltaNet, acceptance and
 * commit go by lane with that sequence's position, caches and state.  A lane's results are bit-identical to the same rows
 * run through fnx_engine_verify on that sequence alone.
 * h_tok [n_lanes][rows]; h_results [n_lanes][1 + 2 FNX_MAX_ROWS] (per lane as fnx_engine_verify's result).
 * commit_lanes keeps the first h_keep[j] rows of lane j (chains are kept as prefixes); draft_lanes runs the MTP layer on
 * every lane's kept rows and k - 1 chained calls of one row per lane, h_drafts [n_lanes][k]. */
int fnx_engine_verify_lanes(fnx_engine* e, int n_lanes, const int* h_seqs, const int* h_tok, int rows, int* h_results);
/* the same with each lane's own row count (h_rows[j] in 1..FNX_LANE_ROWS; h_tok holds the lanes' rows one after another): the
 * windows a planner lays out, where a lane carries as many drafts as are worth their rows */
int fnx_engine_verify_lanes_rows(fnx_engine* e, int n_lanes, const int* h_seqs, const int* h_rows, const int* h_tok,
                                 int* h_results);
int fnx_engine_commit_lanes(fnx_engine* e, int n_lanes, const int* h_seqs, const int* h_keep);
int fnx_engine_draft_lanes(fnx_engine* e, int n_lanes, const int* h_seqs, int k, int* h_drafts);
/* Places sequence `seq` at position `pos` as if that many tokens had been read, without reading them: its K/V rows and
 * DeltaNet state keep whatever they hold (fill them through fnx_engine_tensor).  For throughput measurements at long
 * contexts; results afterwards are a function of that memory, not of a token history. */
int fnx_engine_set_position(fnx_engine* e, int seq, int pos);
/* counters since creation: [0] kernels launched through graphs, [1] routed expert jobs, [2] router calls */
int fnx_engine_counters(fnx_engine* e, unsigned long long* h_out3);
int fnx_engine_pos(const fnx_engine* e, int seq);
fnx_stream fnx_engine_stream(fnx_engine* e);
/* the configuration the engine was made with */
int fnx_engine_config(const fnx_engine* e, fnx_model_config* out);

/* ---------------------------------------------------------------------------------------------- model files
 * GGUF reader (fnx::Gguf, engine/src/gguf.hpp:47-95): maps a model file (and the other "-0000N-of-0000M" shards beside a
 * first shard), indexes its tensors by name and keeps the first shard's metadata.  Host only: none of these calls
 * touches a GPU.  Tensor data stays in the mapping (pointers are valid until fnx_gguf_close). */
typedef struct fnx_gguf fnx_gguf;
typedef struct {
    const char* name;
    uint32_t type;        /* ggml type id: 0 F32, 1 F16, 8 Q8_0, 21 IQ3_S, 26 I32, 30 BF16, ... */
    int n_dims;
    int64_t ne[4];        /* ne[0] = weights per row; unused extents are 1 */
    const void* data;
    size_t bytes;
    int shard;
    uint64_t offset;      /* of the data in its shard's file */
} fnx_gguf_tensor;
int fnx_gguf_open(const char* path, fnx_gguf** out);
void fnx_gguf_close(fnx_gguf* g);
int fnx_gguf_count(const fnx_gguf* g);
int fnx_gguf_shards(const fnx_gguf* g);
int fnx_gguf_tensor_at(const fnx_gguf* g, int i, fnx_gguf_tensor* out);
/* these four return 1 when the tensor / key exists (and fill the output), else 0 */
int fnx_gguf_find(const fnx_gguf* g, const char* name, fnx_gguf_tensor* out);
int fnx_gguf_num(const fnx_gguf* g, const char* key, double* out);                 /* an integer, float or bool key */
int fnx_gguf_str(const fnx_gguf* g, const char* key, char* buf, size_t cap);
int fnx_gguf_int_array(const fnx_gguf* g, const char* key, int64_t* out, size_t cap, size_t* n);
/* rows [row0, row0 + n_rows) of a tensor as f32 (fnx::conv::dequantize, engine/src/tensor_convert.hpp:143-326): F32, F16,
 * BF16, Q8_0 and IQ3_S; FNX_E_UNAVAILABLE for other types */
int fnx_gguf_rows_f32(const fnx_gguf_tensor* t, int64_t row0, int64_t n_rows, float* out);
/* the architecture fields of a configuration from the file's metadata (the keys checked at engine/src/model.cpp:1481-1506)
 * and tensor shapes; max_ctx, max_rows, n_seq, ep_rank and ep_size are the caller's and stay as they are */
int fnx_gguf_model_config(const fnx_gguf* g, fnx_model_config* cfg);
/* Fills an engine's weights from the file (llama.cpp's tensor names for this architecture; the load of
 * engine/src/model.cpp:932-1097 with the expert slicing of :1063-1069).  IQ3_S tensors are re-tiled bit for bit; matrices of
 * another type are quantised to IQ3_S on the GPU and counted in *h_converted (may be null).  Synchronises. */
int fnx_engine_load_gguf(fnx_engine* e, const fnx_gguf* g, int* h_converted);

/* ---------------------------------------------------------------------------------------------- expert-parallel sum
 * ring_sum (engine/src/kernels.hpp:396) over NCCL: in-place sum of x[count] f32 across the communicator. */
int fnx_comm_unique_id(void* h_id128);
int fnx_engine_comm_init(fnx_engine* e, const void* h_id128, int rank, int size);
int fnx_allreduce(fnx_engine* e, float* x, size_t count, fnx_stream st);
/* The same sum without NCCL, fused with the combine: every rank stores its routed addend straight into every peer's
 * landing buffer over NVLink (plain peer stores + one release flag per peer), then adds the ranks' planes in rank order
 * after a bounded wait (FNX_ERR_TIMEOUT).  fnx_engine_ep_handles: this rank's two CUDA IPC handles (128 bytes);
 * exchange them between the ranks' processes by any means, then fnx_engine_ep_open(all ranks' handles, [size][128]).
 * Replaces the reference's pinned-host sum exchange (ring_sum, engine/src/kernels.hpp:396). */
int fnx_engine_ep_handles(fnx_engine* e, void* h_out128);
int fnx_engine_ep_open(fnx_engine* e, const void* h_all, int rank, int size);
/* polls a wait for a peer's flag makes before it gives up with FNX_ERR_TIMEOUT (default 2,000,000, about a second).
 * Drops the captured graphs. */
int fnx_engine_set_wait_limit(fnx_engine* e, unsigned polls);
/* Diagnostic: maps every peer of an expert-parallel engine to this rank's own landing buffer, so that the other ranks'
 * flags never arrive: each window's first exchange then runs out its bounded wait, the window returns FNX_E_STATE with
 * FNX_ERR_TIMEOUT set, and the context stays usable.  Checks on one GPU, without any fault, that a missing peer cannot hang
 * a rank (the reference's ring_sum has the same bounded wait, engine/src/kernels.hpp:373). */
int fnx_engine_ep_open_loopback(fnx_engine* e);

#ifdef __cplusplus
}
#endif
#endif
