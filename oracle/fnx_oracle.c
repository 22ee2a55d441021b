/* CPU oracle (test infrastructure; see fnx_oracle.h).  Plain C, double accumulators, OpenMP over
 * independent outputs only (no parallel reductions), so results do not depend on the thread count. */
#include "fnx_oracle.h"

#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <stdlib.h>
#include <string.h>

#include "iq3s_grid.h"

/* ------------------------------------------------------------------------------------------------ fp16
 * IEEE binary16 <-> binary32, round to nearest even: the conversions the reference's host code uses
 * (engine/src/tensor_convert.hpp:23-52). */
float fnx_o_h2f(uint16_t h) {
    const uint32_t s = (h >> 15) & 1u, e = (h >> 10) & 31u, m = h & 1023u;
    float f;
    if (e == 0) f = ldexpf((float) m, -24);
    else if (e == 31) f = m ? NAN : INFINITY;
    else f = ldexpf((float) (m + 1024u), (int) e - 25);
    return s ? -f : f;
}

uint16_t fnx_o_f2h(float x) {
    uint32_t b;
    memcpy(&b, &x, 4);
    const uint32_t s = (b >> 16) & 0x8000u, e = (b >> 23) & 0xFFu, m = b & 0x7FFFFFu;
    if (e == 0xFF) return (uint16_t) (s | 0x7C00u | (m ? 0x200u : 0u));
    const int ne = (int) e - 127 + 15;
    if (ne >= 31) return (uint16_t) (s | 0x7C00u);
    if (ne <= 0) {
        if (ne < -10) return (uint16_t) s;
        const uint32_t mm = (m | 0x800000u) >> (1 - ne);
        uint32_t r = mm >> 13;
        const uint32_t rem = mm & 0x1FFFu;
        if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) ++r;
        return (uint16_t) (s | r);
    }
    uint32_t r = ((uint32_t) ne << 10) | (m >> 13);
    const uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) ++r;
    return (uint16_t) (s | r);
}

/* ------------------------------------------------------------------------------------------------ IQ3_S */
static const uint32_t k_grid[512] = {FNX_IQ3S_GRID_VALUES};

const uint32_t* fnx_o_iq3s_grid(void) { return k_grid; }

/* One 110-byte block -> 256 floats.  Layout and arithmetic of ggml's dequantize_row_iq3_s as the
 * reference restates it at engine/src/tensor_convert.hpp:295-322 (second statement of the same bits:
 * engine/src/moe_mma_iq.cuh:146-185): d f16 @0, qs[64] @2, qh[8] @66, signs[32] @74, scales[4] @106.
 * Sub-block ib (32 weights): scale nibble ib, index k = qs[8 ib + k] | bit k of qh[ib] << 8,
 * weight 8 l + j negative when bit j of signs[4 ib + l] is set.  Value = (d (1 + 2 s)) * g * (+-1), in
 * float, in that order of multiplication. */
static void dequant_block(const uint8_t* p, float* o) {
    uint16_t dh;
    memcpy(&dh, p, 2);
    const float d = fnx_o_h2f(dh);
    const uint8_t *qs = p + 2, *qh = p + 66, *signs = p + 74, *scales = p + 106;
    for (int ib = 0; ib < 8; ++ib) {
        const int nib = (scales[ib / 2] >> (4 * (ib & 1))) & 0xF;
        const float db = d * (float) (1 + 2 * nib);
        for (int l = 0; l < 4; ++l) {
            for (int half = 0; half < 2; ++half) {
                const int k = 2 * l + half;
                const uint32_t g = k_grid[qs[8 * ib + k] | (((qh[ib] >> k) & 1) << 8)];
                for (int j = 0; j < 4; ++j) {
                    const float sg = (signs[4 * ib + l] >> (4 * half + j)) & 1 ? -1.f : 1.f;
                    o[32 * ib + 8 * l + 4 * half + j] = db * (float) ((g >> (8 * j)) & 255u) * sg;
                }
            }
        }
    }
}

void fnx_o_iq3s_dequant(const uint8_t* blocks, size_t nblocks, float* out) {
#pragma omp parallel for schedule(static)
    for (long long b = 0; b < (long long) nblocks; ++b)
        dequant_block(blocks + (size_t) b * FNX_O_IQ3S_BLOCK_BYTES, out + (size_t) b * FNX_O_QK);
}

/* Fixture quantiser.  ggml's quantize_row_iq3_s is not part of the reference tree (third_party/ggml holds
 * only LICENSE and VERSION.txt), so test weights are encoded by this deterministic search instead; both
 * the oracle and the CUDA path consume the resulting bytes, so its quality does not enter any parity claim.
 *   d = f16(amax / 465); per sub-block three scale candidates around amax_sb / (15 d); per 4-weight group the
 *   codebook row nearest (squared error, 1/16-unit fixed point, ties -> lower index) to |w| / (d (1 + 2 s)).
 * Every float step is a single IEEE operation and the search is integer, so the CUDA twin is bit-identical. */
static void quantize_block(const float* w, uint8_t* p) {
    memset(p, 0, FNX_O_IQ3S_BLOCK_BYTES);
    float amax = 0.f;
    for (int i = 0; i < 256; ++i) amax = fmaxf(amax, fabsf(w[i]));
    const uint16_t dh = fnx_o_f2h(amax / 465.0f);
    const float d = fnx_o_h2f(dh);
    if (!(d > 0.f)) return;
    memcpy(p, &dh, 2);
    uint8_t *qs = p + 2, *qh = p + 66, *signs = p + 74, *scales = p + 106;
    for (int ib = 0; ib < 8; ++ib) {
        const float* ws = w + 32 * ib;
        float am = 0.f;
        for (int i = 0; i < 32; ++i) am = fmaxf(am, fabsf(ws[i]));
        const float t0 = (am / (15.0f * d) - 1.0f) * 0.5f;
        int s0 = (int) rintf(t0);
        if (s0 < 0) s0 = 0;
        if (s0 > 15) s0 = 15;
        long long best_err = -1;
        int best_s = 0;
        uint16_t best_idx[8] = {0};
        for (int c = -1; c <= 1; ++c) {
            const int s = s0 + c;
            if (s < 0 || s > 15) continue;
            const float sc = d * (float) (1 + 2 * s);
            long long err = 0;
            uint16_t idx[8];
            for (int gidx = 0; gidx < 8; ++gidx) {
                int mi[4];
                for (int j = 0; j < 4; ++j) {
                    const float t = fabsf(ws[4 * gidx + j]) / sc;
                    int v = (int) rintf(t * 16.0f);
                    if (v > 272) v = 272;
                    mi[j] = v;
                }
                int be = 0x7fffffff, bi = 0;
                for (int e = 0; e < 512; ++e) {
                    const uint32_t g = k_grid[e];
                    int ee = 0;
                    for (int j = 0; j < 4; ++j) {
                        const int df = mi[j] - 16 * (int) ((g >> (8 * j)) & 255u);
                        ee += df * df;
                    }
                    if (ee < be) { be = ee; bi = e; }
                }
                idx[gidx] = (uint16_t) bi;
                err += be;
            }
            err *= (long long) (1 + 2 * s) * (1 + 2 * s);
            if (best_err < 0 || err < best_err) {
                best_err = err;
                best_s = s;
                memcpy(best_idx, idx, sizeof idx);
            }
        }
        scales[ib / 2] |= (uint8_t) (best_s << (4 * (ib & 1)));
        for (int k = 0; k < 8; ++k) {
            qs[8 * ib + k] = (uint8_t) (best_idx[k] & 255);
            qh[ib] |= (uint8_t) (((best_idx[k] >> 8) & 1) << k);
        }
        for (int l = 0; l < 4; ++l)
            for (int j = 0; j < 8; ++j)
                if (ws[8 * l + j] < 0.f) signs[4 * ib + l] |= (uint8_t) (1u << j);
    }
}

void fnx_o_iq3s_quantize(const float* w, size_t n, uint8_t* blocks) {
#pragma omp parallel for schedule(static)
    for (long long b = 0; b < (long long) (n / 256); ++b)
        quantize_block(w + (size_t) b * 256, blocks + (size_t) b * FNX_O_IQ3S_BLOCK_BYTES);
}

/* Dense IQ3_S matrix times T activation rows: the result the reference's quantised GEMV kernels approximate
 * (k_mmvq engine/src/kernels.cu:192-228, k_q8s engine/src/dense.cuh:211), here without requantising the
 * activations: dequantised weight (float) times float activation, summed in double. */
void fnx_o_iq3s_gemv(const uint8_t* W, int rows, int cols, const float* x, int ldx, int T, float* y, int ldy) {
    const int nb = cols / 256;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        float wrow[256];
        double acc[64];
        for (int t = 0; t < T; ++t) acc[t] = 0.0;
        for (int b = 0; b < nb; ++b) {
            dequant_block(W + ((size_t) r * nb + b) * FNX_O_IQ3S_BLOCK_BYTES, wrow);
            for (int t = 0; t < T; ++t) {
                const float* xt = x + (size_t) t * ldx + b * 256;
                double s = 0.0;
                for (int i = 0; i < 256; ++i) s += (double) wrow[i] * (double) xt[i];
                acc[t] += s;
            }
        }
        for (int t = 0; t < T; ++t) y[(size_t) t * ldy + r] = (float) acc[t];
    }
}

/* ------------------------------------------------------------------------------------------------ small pieces */
/* y = x / sqrt(mean(x^2) + eps) * w  (k_rms_norm_rows, engine/src/kernels.hpp:405-406) */
void fnx_o_rmsnorm(const float* x, const float* w, float* y, int rows, int n, float eps) {
    for (int r = 0; r < rows; ++r) {
        double ss = 0.0;
        for (int i = 0; i < n; ++i) ss += (double) x[(size_t) r * n + i] * x[(size_t) r * n + i];
        const double sc = 1.0 / sqrt(ss / n + (double) eps);
        for (int i = 0; i < n; ++i) y[(size_t) r * n + i] = (float) (x[(size_t) r * n + i] * sc * w[i]);
    }
}

/* y[t][r] = W[r] . x[t], float weights (gemv_f32, engine/src/kernels.hpp:53-54) */
void fnx_o_gemv_f32(const float* W, int rows, int cols, const float* x, int T, float* y) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r)
        for (int t = 0; t < T; ++t) {
            double s = 0.0;
            for (int i = 0; i < cols; ++i) s += (double) W[(size_t) r * cols + i] * (double) x[(size_t) t * cols + i];
            y[(size_t) t * rows + r] = (float) s;
        }
}

static double sigm(double x) { return 1.0 / (1.0 + exp(-x)); }
static double silu(double x) { return x / (1.0 + exp(-x)); }

/* ------------------------------------------------------------------------------------------------ MoE routing
 * logits rows of E + 1 = Wr [E + 1][H] . x (row E: the shared expert's gate), the K largest of the first E by
 * logit (ties: the lower index), weights the softmax over the selected, i.e. the full softmax renormalised
 * (k_topk engine/src/kernels.cu:338-378; fused form engine/src/moe.cuh:382-411; router_route contract
 * engine/src/kernels.hpp:277-282). */
void fnx_o_router(const float* Wr, const float* x, int T, int E, int H, int K, float* logits, int* topi, float* topw) {
    fnx_o_gemv_f32(Wr, E + 1, H, x, T, logits);
    for (int t = 0; t < T; ++t) {
        const float* l = logits + (size_t) t * (E + 1);
        char* used = (char*) calloc((size_t) E, 1);
        for (int k = 0; k < K; ++k) {
            int bi = -1;
            for (int e = 0; e < E; ++e)
                if (!used[e] && (bi < 0 || l[e] > l[bi])) bi = e;
            used[bi] = 1;
            topi[t * K + k] = bi;
        }
        free(used);
        const double mx = l[topi[t * K]];
        double z = 0.0;
        for (int k = 0; k < K; ++k) z += exp((double) l[topi[t * K + k]] - mx);
        for (int k = 0; k < K; ++k) topw[t * K + k] = (float) (exp((double) l[topi[t * K + k]] - mx) / z);
    }
}

/* One expert on one activation row: gate|up rows stacked [gate (F); up (F)] (engine/src/model.hpp:166),
 * h = silu(g) u (engine/src/moe.cuh:631-640), down rows of F (engine/src/moe.cuh:613-658). */
static void expert_row(const uint8_t* Wgu, const uint8_t* Wdn, const float* x, int H, int F, float* gu, float* h, float* part) {
    fnx_o_iq3s_gemv(Wgu, 2 * F, H, x, H, 1, gu, 2 * F);
    for (int i = 0; i < F; ++i) h[i] = (float) (silu((double) gu[i]) * (double) gu[F + i]);
    fnx_o_iq3s_gemv(Wdn, H, F, h, F, 1, part, H);
}

/* The MoE block: out[t] = sum_k topw[t][k] part[t K + k] + sigmoid(logit[t][E]) shared[t]
 * (k_combine engine/src/kernels.cu:412-419; ring_x :909-918).  With an expert range the sum keeps only the
 * picks in [e_lo, e_hi): one expert-parallel rank's addend. */
void fnx_o_moe(const float* Wr, const uint8_t* Wgu, const uint8_t* Wdn, const uint8_t* Wsh_gu, const uint8_t* Wsh_dn,
               const float* x, int T, int E, int H, int F, int K, int e_lo, int e_hi, int add_shared, float* out,
               float* logits, int* topi, float* topw) {
    fnx_o_router(Wr, x, T, E, H, K, logits, topi, topw);
    const size_t gu_bytes = (size_t) 2 * F * (H / 256) * FNX_O_IQ3S_BLOCK_BYTES;
    const size_t dn_bytes = (size_t) H * (F / 256) * FNX_O_IQ3S_BLOCK_BYTES;
    float* gu = (float*) malloc(sizeof(float) * 2 * F);
    float* h = (float*) malloc(sizeof(float) * F);
    float* part = (float*) malloc(sizeof(float) * H);
    double* acc = (double*) malloc(sizeof(double) * H);
    for (int t = 0; t < T; ++t) {
        for (int i = 0; i < H; ++i) acc[i] = 0.0;
        for (int k = 0; k < K; ++k) {
            const int e = topi[t * K + k];
            if (e < e_lo || e >= e_hi) continue;
            expert_row(Wgu + (size_t) e * gu_bytes, Wdn + (size_t) e * dn_bytes, x + (size_t) t * H, H, F, gu, h, part);
            for (int i = 0; i < H; ++i) acc[i] += (double) topw[t * K + k] * (double) part[i];
        }
        if (add_shared) {
            expert_row(Wsh_gu, Wsh_dn, x + (size_t) t * H, H, F, gu, h, part);
            const double g = sigm((double) logits[(size_t) t * (E + 1) + E]);
            for (int i = 0; i < H; ++i) acc[i] += g * (double) part[i];
        }
        for (int i = 0; i < H; ++i) out[(size_t) t * H + i] = (float) acc[i];
    }
    free(gu);
    free(h);
    free(part);
    free(acc);
}

/* ------------------------------------------------------------------------------------------------ attention
 * Per (row, head): RMS norm with the head-dim weight, NEOX rotary on dims [0, nrot) in pairs (i, i + nrot/2)
 * with angle pos * base^(-2 i / nrot) (norm_rope engine/src/kernels.cu:513-530; unit frequency
 * engine/src/rope.hpp:33-35, unscaled), then the K and V rows stored as f16, round to nearest
 * (k_attn_prep_append engine/src/kernels.cu:1880-1910; k_kv_append :1850-1875).
 * Window row i takes rotary position pos0 + depth[i] and cache row pos0 + i; for a chain depth[i] = i, the
 * reference's case.  qg rows: [nq][q (hd) | gate (hd)]. */
static void norm_rope_row(float* x, const float* w, int hd, int nrot, int pos, float eps, float base) {
    double ss = 0.0;
    for (int i = 0; i < hd; ++i) ss += (double) x[i] * x[i];
    const double sc = 1.0 / sqrt(ss / hd + (double) eps);
    for (int i = 0; i < hd; ++i) x[i] = (float) (x[i] * sc * w[i]);
    for (int i = 0; i < nrot / 2; ++i) {
        const float fe = powf(base, -2.0f * (float) i / (float) nrot);
        const float theta = (float) pos * fe;
        const float sn = sinf(theta), cs = cosf(theta);
        const float x0 = x[i], x1 = x[i + nrot / 2];
        x[i] = x0 * cs - x1 * sn;
        x[i + nrot / 2] = x0 * sn + x1 * cs;
    }
}

void fnx_o_attn_prep_append(float* qg, float* k, const float* v, const float* qn, const float* kn, uint16_t* kc,
                            uint16_t* vc, int T, int nq, int nkv, int hd, int nrot, int pos0, const int* depth,
                            float eps, float rope_base) {
    for (int t = 0; t < T; ++t) {
        const int pos = pos0 + (depth ? depth[t] : t);
        for (int h = 0; h < nq; ++h) norm_rope_row(qg + ((size_t) t * nq + h) * 2 * hd, qn, hd, nrot, pos, eps, rope_base);
        for (int h = 0; h < nkv; ++h) norm_rope_row(k + ((size_t) t * nkv + h) * hd, kn, hd, nrot, pos, eps, rope_base);
        for (int i = 0; i < nkv * hd; ++i) {
            kc[(size_t) (pos0 + t) * nkv * hd + i] = fnx_o_f2h(k[(size_t) t * nkv * hd + i]);
            vc[(size_t) (pos0 + t) * nkv * hd + i] = fnx_o_f2h(v[(size_t) t * nkv * hd + i]);
        }
    }
}

/* softmax(q . k / sqrt(hd)) v over the cache rows a window row may see, times sigmoid(gate)
 * (k_attn_part engine/src/kernels.cu:558-643; combine `acc / z * sigmoid(gate)` :786-803).  Row i sees cache
 * rows [0, pos0) and the window rows on its path to the root, itself included (parent[0] = -1); for a chain
 * that is rows [0, pos0 + i], the reference's causal case.  K and V are read from the f16 cache. */
void fnx_o_attn(const float* qg, const uint16_t* kc, const uint16_t* vc, float* out, int T, int nq, int nkv, int hd,
                int pos0, const int* parent) {
    const int qpk = nq / nkv;
    const double scale = 1.0 / sqrt((double) hd);
#pragma omp parallel for schedule(static) collapse(2)
    for (int t = 0; t < T; ++t)
        for (int h = 0; h < nq; ++h) {
            const int kvh = h / qpk;
            const float* q = qg + ((size_t) t * nq + h) * 2 * hd;
            const float* gate = q + hd;
            char see[64] = {0};
            for (int a = t; a >= 0; a = parent ? parent[a] : a - 1) see[a] = 1;
            const int n = pos0 + T;
            double* sc = (double*) malloc(sizeof(double) * (size_t) n);
            double mx = -INFINITY;
            for (int p = 0; p < n; ++p) {
                if (p >= pos0 && !see[p - pos0]) { sc[p] = -INFINITY; continue; }
                const uint16_t* kr = kc + ((size_t) p * nkv + kvh) * hd;
                double s = 0.0;
                for (int d = 0; d < hd; ++d) s += (double) q[d] * (double) fnx_o_h2f(kr[d]);
                sc[p] = s * scale;
                if (sc[p] > mx) mx = sc[p];
            }
            double z = 0.0;
            double* acc = (double*) calloc((size_t) hd, sizeof(double));
            for (int p = 0; p < n; ++p) {
                if (sc[p] == -INFINITY) continue;
                const double w = exp(sc[p] - mx);
                z += w;
                const uint16_t* vr = vc + ((size_t) p * nkv + kvh) * hd;
                for (int d = 0; d < hd; ++d) acc[d] += w * (double) fnx_o_h2f(vr[d]);
            }
            for (int d = 0; d < hd; ++d) out[((size_t) t * nq + h) * hd + d] = (float) (acc[d] / z * sigm((double) gate[d]));
            free(acc);
            free(sc);
        }
}

/* ------------------------------------------------------------------------------------------------ gated DeltaNet
 * The recurrent layer's core over a window (unfused statement engine/src/kernels.cu:422-506; fused kernel
 * engine/src/gdn_core.cuh:20-225).  qkvz rows [q (nk hs) | k (nk hs) | v (nv hs) | z (nv hs)], ab rows
 * [alpha (nv) | beta (nv)].  Per row: causal conv over the 3 previous rows and itself on the q|k|v channels
 * then SiLU (k_gdn_conv :422-432), L2 norm of each q and k head with eps 1e-6 (:435-442), decay
 * exp(softplus(alpha + dt) a) and beta = sigmoid(b) (:444-453; applied :472), the delta rule on the head's
 * state S[key][value] with value head lv reading key head lv % nk (:457-492), output o = S^T q / sqrt(hs), then
 * o rsqrt(mean o^2 + eps) w sigmoid(z) (:495-505).
 * States and conv histories live in rings of NS slots: the window starts from slot `cur`; row i starts from its
 * parent's result (slot cur for the root) and leaves the state after it, and the 3-row history that keeping it
 * would leave, in slot (cur + 1 + i) % NS.  These are the reference's snap / hsnap buffers
 * (engine/src/gdn_core.cuh:13-14, 91-98, 172-176) with the commit copy (engine/src/engine_common.cu:710-754)
 * turned into a change of `cur`; for a chain parent[i] = i - 1. */
void fnx_o_gdn_core(const float* qkvz, const float* ab, float* hist_pool, const float* convw, const float* dt,
                    const float* a, const float* nw, float* S_pool, int cur, int NS, const int* parent, float* y,
                    int nk, int nv, int hs, int T, float eps) {
    const int ch = (2 * nk + nv) * hs, stride = ch + nv * hs;
    const size_t hsz = (size_t) 3 * ch, ssz = (size_t) nv * hs * hs;
    float* conv = (float*) malloc(sizeof(float) * (size_t) T * ch);
    for (int t = 0; t < T; ++t) {
        const int par = parent ? parent[t] : t - 1;
        const float* hin = hist_pool + (size_t) (par < 0 ? cur : (cur + 1 + par) % NS) * hsz;
        float* hout = hist_pool + (size_t) ((cur + 1 + t) % NS) * hsz;
        for (int c = 0; c < ch; ++c) {
            const float xin = qkvz[(size_t) t * stride + c];
            const float w0 = convw[c * 4], w1 = convw[c * 4 + 1], w2 = convw[c * 4 + 2], w3 = convw[c * 4 + 3];
            const float h0 = hin[c], h1 = hin[ch + c], h2 = hin[2 * ch + c];
            const double s = (double) w0 * h0 + (double) w1 * h1 + (double) w2 * h2 + (double) w3 * xin;
            conv[(size_t) t * ch + c] = (float) silu(s);
            hout[c] = h1;
            hout[ch + c] = h2;
            hout[2 * ch + c] = xin;
        }
        for (int h = 0; h < 2 * nk; ++h) {
            float* xh = conv + (size_t) t * ch + h * hs;
            double ss = 0.0;
            for (int i = 0; i < hs; ++i) ss += (double) xh[i] * xh[i];
            const double sc = 1.0 / sqrt(ss + 1e-6);
            for (int i = 0; i < hs; ++i) xh[i] = (float) (xh[i] * sc);
        }
    }
    const double oscale = 1.0 / sqrt((double) hs);
#pragma omp parallel for schedule(static)
    for (int lv = 0; lv < nv; ++lv) {
        const int kh = lv % nk;
        double* kv = (double*) malloc(sizeof(double) * hs);
        double* o = (double*) malloc(sizeof(double) * hs);
        for (int t = 0; t < T; ++t) {
            const int par = parent ? parent[t] : t - 1;
            const float* Sin = S_pool + (size_t) (par < 0 ? cur : (cur + 1 + par) % NS) * ssz + (size_t) lv * hs * hs;
            float* Sout = S_pool + (size_t) ((cur + 1 + t) % NS) * ssz + (size_t) lv * hs * hs;
            const float* q = conv + (size_t) t * ch + kh * hs;
            const float* k = conv + (size_t) t * ch + nk * hs + kh * hs;
            const float* v = conv + (size_t) t * ch + 2 * nk * hs + lv * hs;
            const float* z = qkvz + (size_t) t * stride + ch + lv * hs;
            const double xg = (double) ab[(size_t) t * 2 * nv + lv] + (double) dt[lv];
            const double sp = xg > 20.0 ? xg : log1p(exp(xg));
            const double g = exp(sp * (double) a[lv]);
            const double beta = sigm((double) ab[(size_t) t * 2 * nv + nv + lv]);
            for (int c = 0; c < hs; ++c) kv[c] = 0.0;
            for (int r = 0; r < hs; ++r)
                for (int c = 0; c < hs; ++c) kv[c] += (double) Sin[(size_t) r * hs + c] * (double) k[r];
            for (int c = 0; c < hs; ++c) o[c] = 0.0;
            for (int r = 0; r < hs; ++r)
                for (int c = 0; c < hs; ++c) {
                    const double delta = ((double) v[c] - g * kv[c]) * beta;
                    const float sn = (float) (g * (double) Sin[(size_t) r * hs + c] + (double) k[r] * delta);
                    Sout[(size_t) r * hs + c] = sn;
                    o[c] += (double) sn * (double) q[r];
                }
            double ms = 0.0;
            for (int c = 0; c < hs; ++c) { o[c] *= oscale; ms += o[c] * o[c]; }
            const double rs = 1.0 / sqrt(ms / hs + (double) eps);
            for (int c = 0; c < hs; ++c)
                y[(size_t) t * nv * hs + lv * hs + c] = (float) (o[c] * rs * (double) nw[c] * sigm((double) z[c]));
        }
        free(kv);
        free(o);
    }
    free(conv);
}

/* ------------------------------------------------------------------------------------------------ head
 * Per-row maximum, ties to the lower index (k_argmax key `(fkey(v) << 32) | ~i`, engine/src/kernels.cu:1056-1083). */
void fnx_o_argmax(const float* logits, int T, int V, int* best_i, float* best_v) {
    for (int t = 0; t < T; ++t) {
        const float* l = logits + (size_t) t * V;
        int bi = 0;
        for (int i = 1; i < V; ++i)
            if (l[i] > l[bi]) bi = i;
        best_i[t] = bi;
        if (best_v) best_v[t] = l[bi];
    }
}

/* The sampler's logit changes before the candidates are taken: the logit_bias list added, then llama.cpp's penalties
 * stage as the reference applies it (k_topk_rows, engine/src/topk.cuh:30-45: repeat multiplies a non-positive logit and
 * divides a positive one, then frequency x count and presence once per token of the window), with row j's penalty
 * window the last last_n tokens of the sequence followed by window rows 0..j (engine/src/session.cpp:88-98, 581-585;
 * ctx holds the kept tokens, tok the window's rows, tok[0] the token the sequence ends in). */
void fnx_o_logit_adjust(float* logits, int T, int V, const int* ctx, int ctx_n, const int* tok, int last_n, float repeat, float freq,
                        float present, const int* bias_tok, const float* bias_val, int bias_n) {
    for (int t = 0; t < T; ++t) {
        float* l = logits + (size_t) t * V;
        for (int i = 0; i < bias_n; ++i)
            if (bias_tok[i] >= 0 && bias_tok[i] < V) l[bias_tok[i]] += bias_val[i];
        if (last_n <= 0) continue;
        const int len = ctx_n + t + 1, start = len > last_n ? len - last_n : 0;
        for (int i = start; i < len; ++i) {
            const int a = i < ctx_n ? ctx[i] : tok[i - ctx_n];
            if (a < 0 || a >= V) continue;
            int seen = 0, cnt = 0;
            for (int j = start; j < len; ++j) {
                const int b = j < ctx_n ? ctx[j] : tok[j - ctx_n];
                if (b == a) {
                    if (j < i) seen = 1;
                    ++cnt;
                }
            }
            if (seen) continue;   /* each token once */
            float v = l[a];
            v = v <= 0.f ? v * repeat : v / repeat;
            l[a] = v - (float) cnt * freq - present;
        }
    }
}

/* The n highest logits per row, logit descending, id ascending on ties (top_tokens contract
 * engine/src/kernels.hpp:437-441; k_topk_rows engine/src/topk.cuh:17-155), without penalties or bias. */
void fnx_o_top_tokens(const float* logits, int T, int V, int n, float* out_v, int* out_i) {
    for (int t = 0; t < T; ++t) {
        const float* l = logits + (size_t) t * V;
        int cnt = 0;
        for (int i = 0; i < V; ++i) {
            /* insertion into the sorted list of the best so far */
            if (cnt == n && !(l[i] > out_v[t * n + n - 1])) continue;
            int p = cnt < n ? cnt : n - 1;
            while (p > 0 && l[i] > out_v[t * n + p - 1]) {
                out_v[t * n + p] = out_v[t * n + p - 1];
                out_i[t * n + p] = out_i[t * n + p - 1];
                --p;
            }
            out_v[t * n + p] = l[i];
            out_i[t * n + p] = i;
            if (cnt < n) ++cnt;
        }
    }
}

/* ------------------------------------------------------------------------------------------------ prompt lookup
 * The 3-gram drafter (lookup_drafts engine/src/session.cpp:428-447; LOOKUP_N = LOOKUP_MIN = 3 at :17-18): the
 * latest earlier start s with ctx[s .. s+3) equal to the last three tokens; only that occurrence is looked at; it
 * must be followed by d1 (when d1 >= 0); the run's length m counts backward agreement before the 3-gram, capped
 * at lk; k = min(lk, max(3, m)) tokens after the match are offered.  Returns the count, *match = s or -1. */
int fnx_o_lookup(const int* ctx, int n, int lk, int d1, int* out, int* match) {
    if (match) *match = -1;
    if (lk == 0 || n <= 3) return 0;
    const int n0 = n - 3;
    for (int s = n0 - 1; s >= 0; --s) {
        if (ctx[s] != ctx[n0] || ctx[s + 1] != ctx[n0 + 1] || ctx[s + 2] != ctx[n0 + 2]) continue;
        int cnt = 0;
        if (s + 3 < n && (d1 < 0 || ctx[s + 3] == d1)) {
            int m = 3;
            while (m < lk && (m - 3) < s && ctx[s - 1 - (m - 3)] == ctx[n0 - 1 - (m - 3)]) ++m;
            const int mm = m > 3 ? m : 3;
            const int k = lk < mm ? lk : mm;
            const int end = s + 3 + k < n ? s + 3 + k : n;
            for (int i = s + 3; i < end; ++i) out[cnt++] = ctx[i];
            if (match) *match = s;
        }
        return cnt;
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------------ Philox4x32-10
 * The counter-based generator of Salmon et al. (SC'11), 10 rounds, as published.  The reference draws its
 * uniforms from std::mt19937_64 on the host (engine/src/session.cpp:497-498); the CUDA path needs a generator
 * both sides can index, so a uniform is addressed by (seed, sequence, step, slot) and both sides consume slots in
 * the reference's order. */
void fnx_o_philox4x32(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
    uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3], k0 = key[0], k1 = key[1];
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t) 0xD2511F53u * c0, p1 = (uint64_t) 0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t) (p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t) p1;
        const uint32_t n2 = (uint32_t) (p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t) p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

/* 53-bit uniform in [0, 1) from words 0 and 1 of the block at counter (slot, step, seq, 0) */
/* the OpenMP team of the loops above: n > 0 sets it (a launcher may have exported OMP_NUM_THREADS=1); returns the size in use */
int fnx_o_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void) n;
    return 1;
#endif
}

double fnx_o_uniform(uint64_t seed, uint32_t seq, uint32_t step, uint32_t slot) {
    const uint32_t ctr[4] = {slot, step, seq, 0u}, key[2] = {(uint32_t) seed, (uint32_t) (seed >> 32)};
    uint32_t o[4];
    fnx_o_philox4x32(ctr, key, o);
    const uint64_t hi = o[0] >> 5, lo = o[1] >> 6;
    return (double) ((hi << 26) | lo) * (1.0 / 9007199254740992.0);
}

/* ------------------------------------------------------------------------------------------------ sampling
 * The sampler's distribution over a row's candidates (logit descending): top-k, then top-p on the softmax at
 * temperature 1, then min-p, then the softmax at the temperature, all in double (make_dist
 * engine/src/session.cpp:41-75). */
int fnx_o_make_dist(const float* cand_v, const int* cand_i, int n, const fnx_o_sampling* s, int* ids, double* p) {
    const int k = (s->top_k <= 0 || s->top_k > n) ? n : s->top_k;
    int keep = k;
    const double mx = cand_v[0];
    if (s->top_p < 1.f) {
        double sum = 0.0;
        for (int i = 0; i < k; ++i) sum += exp((double) cand_v[i] - mx);
        double cum = 0.0;
        for (int i = 0; i < k; ++i) {
            cum += exp((double) cand_v[i] - mx) / sum;
            if (cum >= (double) s->top_p) { keep = i + 1; break; }
        }
    }
    if (s->min_p > 0.f) {
        const float thresh = cand_v[0] + logf(s->min_p);
        for (int i = 1; i < keep; ++i)
            if (cand_v[i] < thresh) { keep = i; break; }
    }
    const double inv_t = 1.0 / s->temperature, smx = cand_v[0] * inv_t;
    double sum = 0.0;
    for (int i = 0; i < keep; ++i) {
        ids[i] = cand_i[i];
        p[i] = exp(cand_v[i] * inv_t - smx);
        sum += p[i];
    }
    for (int i = 0; i < keep; ++i) p[i] /= sum;
    return keep;
}

/* inverse-CDF draw (draw, engine/src/session.cpp:77-84) */
int fnx_o_draw(const int* ids, const double* p, int n, double u) {
    double cum = 0.0;
    for (int i = 0; i < n; ++i) {
        cum += p[i];
        if (u < cum) return ids[i];
    }
    return ids[n - 1];
}

static double dist_prob(const int* ids, const double* p, int n, int id) {
    for (int i = 0; i < n; ++i)
        if (ids[i] == id) return p[i];
    return 0.0;
}

/* Greedy acceptance.  Chain rule of the reference: keep drafts while rows[n] == o[n - 1]
 * (engine/src/session.cpp:573).  On a tree the same rule walks from the root to the child whose token is the
 * current node's argmax (the first such child in row order). */
int fnx_o_accept_greedy(const int* tok, const int* parent, const int* best, int T, int* path, int* emitted) {
    int cur = 0, n = 0;
    for (;;) {
        path[n] = cur;
        emitted[n] = best[cur];
        ++n;
        int next = -1;
        for (int c = cur + 1; c < T; ++c)
            if ((parent ? parent[c] : c - 1) == cur && tok[c] == best[cur]) { next = c; break; }
        if (next < 0) break;
        cur = next;
    }
    return n;
}

/* Speculative sampling over a chain (engine/src/session.cpp:575-612): draft j+1 stands when u q(d) < p(d) (a
 * fixed draft: q = 1); otherwise row j's token is drawn from max(0, p - q) normalised (from p when that mass is
 * <= 1e-12) and the window ends; all standing: one more token from the last row.  Uniforms are consumed in the
 * reference's order, slot 0, 1, 2, ... of (seed, seq, step). */
int fnx_o_accept_sample(const float* cand_v, const int* cand_i, const int* tok, int T, const fnx_o_sampling* s,
                        const int* q_ids, const double* q_p, const int* q_n, uint64_t seed, uint32_t seq,
                        uint32_t step, int* emitted) {
    uint32_t slot = 0;
    int ids[FNX_O_TOPN];
    double p[FNX_O_TOPN], p0[FNX_O_TOPN];
    int n;
    for (n = 0; n < T; ++n) {
        const int m = fnx_o_make_dist(cand_v + (size_t) n * FNX_O_TOPN, cand_i + (size_t) n * FNX_O_TOPN, FNX_O_TOPN, s, ids, p);
        if (n + 1 < T) {
            const int dr = tok[n + 1];
            const int qn = q_n ? q_n[n] : 0;
            const int* qi = q_ids ? q_ids + (size_t) n * FNX_O_TOPN : 0;
            const double* qp = q_p ? q_p + (size_t) n * FNX_O_TOPN : 0;
            const int fixed = qn == 0;
            const double u = fnx_o_uniform(seed, seq, step, slot++);
            if (u * (fixed ? 1.0 : dist_prob(qi, qp, qn, dr)) < dist_prob(ids, p, m, dr)) {
                emitted[n] = dr;
                continue;
            }
            memcpy(p0, p, sizeof(double) * (size_t) m);
            double rest = 0.0;
            for (int i = 0; i < m; ++i) {
                const double qv = fixed ? (ids[i] == dr ? 1.0 : 0.0) : dist_prob(qi, qp, qn, ids[i]);
                p[i] = p[i] - qv > 0.0 ? p[i] - qv : 0.0;
                rest += p[i];
            }
            if (rest > 1e-12) for (int i = 0; i < m; ++i) p[i] /= rest;
            else memcpy(p, p0, sizeof(double) * (size_t) m);
        }
        emitted[n] = fnx_o_draw(ids, p, m, fnx_o_uniform(seed, seq, step, slot++));
        ++n;
        break;
    }
    return n;
}
