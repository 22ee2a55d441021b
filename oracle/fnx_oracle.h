/* CPU oracle for the speculative-decoding verify path.
 *
 * TEST INFRASTRUCTURE ONLY: this is the checker the CUDA path is compared with (and the timed
 * CPU baseline of the benchmark).  Nothing in the shipped library links, loads or calls it.
 *
 * Every function restates, in plain C with double accumulators, the arithmetic of one operator
 * of the reference engine (Megla123/qwen3.8-flash-next-2x-p100); the reference file:line each one
 * follows is given beside its definition in fnx_oracle.c.
 *
 * Pin status: IQ3_S decoding is pinned bit-for-bit against the reference's own host dequantiser
 * (engine/src/tensor_convert.hpp, compiled from where it lies into oracle/_ref) and against
 * gguf-py; make_dist / draw / lookup_drafts are pinned against engine/src/session.cpp compiled the
 * same way.  The reference has no stored vectors for its CUDA operators (router, experts, attention,
 * DeltaNet): for those this oracle is "parity unpinned" beyond the reference's own procedural checks
 * (selftest.cu tolerances), which the tests restate.
 */
#ifndef FNX_ORACLE_H
#define FNX_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FNX_O_IQ3S_BLOCK_BYTES 110
#define FNX_O_QK 256
#define FNX_O_TOPN 64

/* ---- fp16 ---- */
float fnx_o_h2f(uint16_t h);
uint16_t fnx_o_f2h(float x);

/* ---- IQ3_S ---- */
const uint32_t* fnx_o_iq3s_grid(void);
void fnx_o_iq3s_dequant(const uint8_t* blocks, size_t nblocks, float* out);
/* deterministic fixture quantiser (NOT ggml's): n a multiple of 256 */
void fnx_o_iq3s_quantize(const float* w, size_t n, uint8_t* blocks);
/* y[t*ldy + r] = W[r] . x[t*ldx ..], W rows of `cols` IQ3_S weights */
void fnx_o_iq3s_gemv(const uint8_t* W, int rows, int cols, const float* x, int ldx, int T, float* y, int ldy);

/* ---- small dense pieces ---- */
void fnx_o_rmsnorm(const float* x, const float* w, float* y, int rows, int n, float eps);
void fnx_o_gemv_f32(const float* W, int rows, int cols, const float* x, int T, float* y);

/* ---- MoE ---- */
void fnx_o_router(const float* Wr, const float* x, int T, int E, int H, int K, float* logits, int* topi, float* topw);
/* experts e_lo <= e < e_hi only (expert-parallel partial sum); shared expert added when add_shared != 0 */
void fnx_o_moe(const float* Wr, const uint8_t* Wgu, const uint8_t* Wdn, const uint8_t* Wsh_gu, const uint8_t* Wsh_dn,
               const float* x, int T, int E, int H, int F, int K, int e_lo, int e_hi, int add_shared, float* out,
               float* logits, int* topi, float* topw);

/* ---- attention ---- */
void fnx_o_attn_prep_append(float* qg, float* k, const float* v, const float* qn, const float* kn, uint16_t* kc,
                            uint16_t* vc, int T, int nq, int nkv, int hd, int nrot, int pos0, const int* depth,
                            float eps, float rope_base);
void fnx_o_attn(const float* qg, const uint16_t* kc, const uint16_t* vc, float* out, int T, int nq, int nkv, int hd,
                int pos0, const int* parent);

/* ---- gated DeltaNet ---- */
void fnx_o_gdn_core(const float* qkvz, const float* ab, float* hist_pool, const float* convw, const float* dt,
                    const float* a, const float* nw, float* S_pool, int cur, int NS, const int* parent, float* y,
                    int nk, int nv, int hs, int T, float eps);

/* ---- head ---- */
void fnx_o_argmax(const float* logits, int T, int V, int* best_i, float* best_v);
void fnx_o_top_tokens(const float* logits, int T, int V, int n, float* out_v, int* out_i);
void fnx_o_logit_adjust(float* logits, int T, int V, const int* ctx, int ctx_n, const int* tok, int last_n, float repeat, float freq,
                        float present, const int* bias_tok, const float* bias_val, int bias_n);

/* ---- drafting and acceptance ---- */
int fnx_o_lookup(const int* ctx, int n, int lk, int d1, int* out, int* match);
void fnx_o_philox4x32(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]);
int fnx_o_threads(int n);
double fnx_o_uniform(uint64_t seed, uint32_t seq, uint32_t step, uint32_t slot);
typedef struct {
    float temperature, top_p, min_p;
    int top_k;
} fnx_o_sampling;
/* returns how many entries are kept; ids/p sized n */
int fnx_o_make_dist(const float* cand_v, const int* cand_i, int n, const fnx_o_sampling* s, int* ids, double* p);
int fnx_o_draw(const int* ids, const double* p, int n, double u);
/* greedy over a tree of T rows: tok[i] row tokens, parent[i], best[i] = argmax of row i.  Writes the accepted
 * node path (path[0] = 0) and the emitted tokens; returns n = number of emitted tokens (1 + accepted drafts). */
int fnx_o_accept_greedy(const int* tok, const int* parent, const int* best, int T, int* path, int* emitted);
/* stochastic chain acceptance; q_n[j] = 0 means draft j+1 is fixed.  Returns n. */
int fnx_o_accept_sample(const float* cand_v, const int* cand_i, const int* tok, int T, const fnx_o_sampling* s,
                        const int* q_ids, const double* q_p, const int* q_n, uint64_t seed, uint32_t seq,
                        uint32_t step, int* emitted);

#ifdef __cplusplus
}
#endif
#endif
