// The window scheduler: a thin re-creation of Engine::verify / commit / draft (engine/src/engine.hpp:50-229;
// enqueue engine/src/engine.cu:1760-1848, ffn_half :1569-1757, mtp_enqueue :2095-2133; verify
// engine/src/engine_common.cu:913-1056, commit :710-754, draft :1569-1684) for the synthetic Qwen3-Next-style model:
// pre-norm residual blocks (RMS norm, eps 1e-6) instead of hyper-connections, every attn_every-th layer gated
// attention and the others gated DeltaNet, a top-k MoE with a sigmoid-gated shared expert in every layer, one
// MTP draft layer that shares the head.  One host thread drives one GPU; every window shape is captured once
// into a CUDA graph (the reference captures one graph per row count too, engine_common.cu:994-1003), window
// scalars live in device memory, and expert-parallel ranks add their partial sums with one all-reduce per layer.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstring>
#include <cmath>
#include <map>
#include <string>
#include <vector>

#include "fnx_common.cuh"
#include "iq3s_tile.h"
#include "mmv_core.cuh"

namespace fnxb {

// ---- NCCL through dlopen: the library has no link-time dependency on it; single-GPU use never loads it
struct NcclId { char b[128]; };
struct Nccl {
    void* lib = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, NcclId, int) = nullptr;   // ncclUniqueId: 128 bytes, passed by value
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};

static Nccl* nccl() {
    static Nccl n;
    static bool tried = false;
    if (!tried) {
        tried = true;
        n.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!n.lib) n.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (n.lib) {
            n.GetUniqueId = (int (*)(void*)) dlsym(n.lib, "ncclGetUniqueId");
            n.CommInitRank = (int (*)(void**, int, NcclId, int)) dlsym(n.lib, "ncclCommInitRank");
            n.AllReduce = (int (*)(const void*, void*, size_t, int, int, void*, cudaStream_t)) dlsym(n.lib, "ncclAllReduce");
            n.CommDestroy = (int (*)(void*)) dlsym(n.lib, "ncclCommDestroy");
            n.GetErrorString = (const char* (*) (int) ) dlsym(n.lib, "ncclGetErrorString");
        }
    }
    return n.lib && n.GetUniqueId && n.CommInitRank && n.AllReduce ? &n : nullptr;
}

struct LayerW {
    bool attn = false;
    float *norm1 = nullptr, *norm2 = nullptr;
    // mixer
    uint8_t *w_in = nullptr, *w_out = nullptr;   // attention: [q|gate per head; k; v] x H and H x (nq hd); DeltaNet: [q|k|v|z|alpha|beta] x H and H x (nv hs)
    int in_rows = 0;
    float *qn = nullptr, *kn = nullptr;          // attention head norms
    __half *kc = nullptr, *vc = nullptr;         // [n_seq][cache_rows][nkv hd]
    float *convw = nullptr, *dt = nullptr, *a = nullptr, *gnorm = nullptr;
    float *S_pool = nullptr, *hist_pool = nullptr;   // [n_seq][NS]...
    // MoE
    float* wr = nullptr;
    uint8_t *wgu = nullptr, *wdn = nullptr, *wsh_gu = nullptr, *wsh_dn = nullptr;
};

struct SeqState {
    int pos = 0, cur = 0;
    uint32_t step = 0;   // windows verified under the sampling rule (the Philox step of the next one)
    int last_T = 0;              // rows of the last verify window
    int kept = 0;                // rows kept by the last commit
    int kept_pos0 = 0;           // position of the first kept row
};

}  // namespace fnxb

using namespace fnxb;

struct fnx_engine {
    fnx_model_config c{};
    cudaStream_t st = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    float last_ms = 0.f;
    size_t bytes = 0;
    std::vector<void*> owned;
    std::map<std::string, std::pair<void*, size_t>> tensors;
    std::vector<LayerW> layers;
    LayerW mtp;
    float *mtp_hnorm = nullptr, *mtp_enorm = nullptr, *mtp_onorm = nullptr, *out_norm = nullptr;
    uint8_t *mtp_fc_hid = nullptr, *mtp_fc_emb = nullptr, *head = nullptr;
    __half* embed = nullptr;
    std::vector<SeqState> seqs;
    int NS = 0, cache_rows = 0, E_local = 0, e_lo = 0, e_hi = 0;
    size_t gu_bytes = 0, dn_bytes = 0;
    // window buffers
    float *R = nullptr, *Rm = nullptr, *Rsrc = nullptr, *Emb = nullptr, *proj = nullptr, *mix = nullptr, *logits = nullptr;
    float *rlogits = nullptr, *topw = nullptr, *hbuf = nullptr, *part = nullptr, *moe_out = nullptr, *best_v = nullptr, *cand_v = nullptr;
    int *topi = nullptr, *njobs = nullptr, *best_i = nullptr, *result = nullptr, *d_tok = nullptr, *d_parent = nullptr, *d_depth = nullptr;
    int *d_pos = nullptr, *d_cur = nullptr, *d_ctx = nullptr, *d_ctx_n = nullptr, *d_path = nullptr, *d_mtok = nullptr, *d_mpos = nullptr;
    int *cand_i = nullptr, *d_drafts = nullptr, *d_mpos_base = nullptr;
    int last_seq = -1;          // the sequence whose window the shared window buffers (tokens, result, residual rows) hold
    // batched lanes: device tables of the last lane window (sequence and first row per lane, rows kept per lane), one result
    // row per lane, the draft layer's positions per sequence and its own lane table
    int *d_lane_seq = nullptr, *d_lane_row0 = nullptr, *d_keep = nullptr, *d_results = nullptr, *d_mpos_seq = nullptr, *d_mlane_row0 = nullptr,
        *d_ident_row0 = nullptr, *d_ldrafts = nullptr;
    float* Rlast = nullptr;     // the lanes' last draft-layer rows, compact, for the head
    std::vector<int> lane_seqs; // the sequences of the last lane window, in lane order (empty: the last window was not batched)
    std::vector<int> lane_rows;   // rows of each lane of the last lanes window
    fnx_job* jobs = nullptr;
    unsigned* err = nullptr;
    void* att_scratch = nullptr;
    // the image of the new residual rows that the combine leaves for the next projection (single rank; one per FNX_DENSE_ROWS rows)
    uint8_t* d_img = nullptr;
    bool use_img = true;
    // the prompt pass (fnx_engine_prompt): buffers for a chunk of prompt_chunk rows, made at its first call
    int prompt_chunk = 40960;
    float *pR = nullptr, *pproj = nullptr, *pmix = nullptr, *plogits = nullptr, *ptopw = nullptr;
    int *ptopi = nullptr, *d_ptok = nullptr;
    int prompt_attn_mma_sync = 0;   // FNX_ATTN_PROMPT_MMA=1: the prompt pass's attention on mma.sync (the comparison form)
    bool prompt_timing = false;     // fnx_engine_prompt_timing: time the prompt pass's phases with events
    float prompt_phase_ms[6] = {0, 0, 0, 0, 0, 0};   // the last timed prompt: in-proj, attention, DeltaNet, out-proj, router, experts
    void *p_router_scratch = nullptr, *p_moe_scratch = nullptr, *p_dense_scratch = nullptr, *p_gdn_scratch = nullptr, *p_attn_scratch = nullptr;
    // the draft layer's own head over a draft vocabulary (config draft_vocab > 0): dvn rows, row -> token id in d_dvocab;
    // otherwise the main head and no map
    uint8_t* mtp_head = nullptr;
    int* d_dvocab = nullptr;
    int dvn = 0;
    int *h_stage = nullptr;      // pinned host staging
    std::map<uint64_t, cudaGraphExec_t> graphs;
    std::map<int, std::pair<__half**, __half**>> commit_tables;   // per sequence: device tables of its K and V caches
    void* comm = nullptr;
    int proj_ld = 0;
    unsigned long long* d_stats = nullptr;
    // expert-parallel exchange over peer memory (fnx_engine_ep_open): this rank's landing buffer [2 slots][ranks][MAXR][H]
    // and arrival flags [2][ranks]; device arrays of every rank's buffer and flags; sequence counters of the two kernels
    float* xbuf = nullptr;
    unsigned* xflag = nullptr;
    float** d_peer_x = nullptr;
    unsigned** d_peer_flag = nullptr;
    unsigned* d_xseq = nullptr;   // [0] sends so far, [1] receives so far, [2] send block counter, [3] receive block counter
    std::vector<void*> ipc_opened;
    bool ep_peers = false;
    // lanes windows on expert-parallel ranks: each rank runs the mixers (attention, DeltaNet) of its own sequences only
    // (sequence % ranks == rank) and the mixers' output rows are gathered over the same peer memory: a second region of the
    // landing buffer ([2 slots][MAXR][mixer width], after the expert planes) with its own flags ([2][ranks], after the
    // experts') and sequence counters (d_xseq[4..7])
    bool ep_one_kernel = true;    // the per-layer sum as one kernel (k_ep_exchange) instead of k_ep_send + k_ep_recv
    bool dp_mixers = true;
    size_t x_off_rows = 0;        // floats before the rows region
    int mix_width = 0;
    int* d_lane_own = nullptr;    // the lane table the mixers see: the lane's sequence, or -1 for another rank's lane
    unsigned wait_limit = 2000000u;   // polls a peer-flag wait makes before it gives up with FNX_ERR_TIMEOUT
    // stochastic acceptance (fnx_engine_set_sampling): off = greedy windows
    bool sampling_on = false;
    fnx_sampling sampling{};
    uint64_t sample_seed = 0;
    uint32_t* d_step = nullptr;   // [n_seq] windows sampled so far (the Philox step)
    // the sampler's logit changes before acceptance (fnx_engine_set_logit_rules): off = none
    bool rules_on = false;
    fnx_logit_rules rules{};
    int* d_bias_tok = nullptr;
    float* d_bias_val = nullptr;
    int bias_cap = 0;
    int* d_lk = nullptr;          // lookup: [0, MAX_ROWS) drafts, [MAX_ROWS, +2) count and match, +2 the first-draft filter, +3 the context length
    unsigned long long launches = 0;
    std::map<uint64_t, unsigned> graph_kernels;
};

namespace fnxb {

template <typename T>
static int dalloc(fnx_engine* e, T** p, size_t count, const char* name = nullptr) {
    void* q = nullptr;
    const size_t bytes = count * sizeof(T);
    FNX_CUDA_OK(cudaMalloc(&q, bytes ? bytes : 16));
    FNX_CUDA_OK(cudaMemset(q, 0, bytes ? bytes : 16));
    e->owned.push_back(q);
    e->bytes += bytes;
    *p = (T*) q;
    if (name) e->tensors[name] = {q, bytes};
    return FNX_OK;
}

static int round_up(int v, int m) { return (v + m - 1) / m * m; }

__global__ void k_fill_const(float* p, size_t n, float v) {
    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}
__global__ void k_f32_to_f16(const float* x, __half* y, size_t n) {
    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __float2half_rn(x[i]);
}
__global__ void k_gdn_params(float* dt, float* a, int nv) {
    const int h = blockIdx.x * blockDim.x + threadIdx.x;
    if (h < nv) {
        dt[h] = 0.1f * (float) ((h % 5) - 2);
        a[h] = -(0.5f + (float) (h % 8) / 8.0f);
    }
}
// dst[j] = src[idx[j]] rows of n floats
__global__ void k_gather_rows(float* __restrict__ dst, const float* __restrict__ src, const int* __restrict__ idx, int n) {
    const int j = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[(size_t) j * n + i] = src[(size_t) idx[j] * n + i];
}
__global__ void k_add_rows(float* __restrict__ dst, const float* __restrict__ src, size_t n) {
    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] += src[i];
}
// ---- expert-parallel sum over NVLink peer memory, fused with the combine (replaces combine + ncclAllReduce + add)
// Send: this rank's routed addend a[t][h] = sum over its experts' picks of topw * part, stored straight into EVERY
// rank's landing buffer (slot = sequence parity, plane = this rank); the last block to finish releases one flag per
// peer.  Receive: waits (bounded) until every rank's flag of the slot shows the sequence, then R += the planes in rank
// order (the same order on every rank: identical sums) + the local shared expert.  Two slots suffice: a rank sends
// sequence n + 2 only after it has received everyone's n + 1, which they sent after reading n.
__global__ void k_ep_send(const float* __restrict__ part, const int* __restrict__ topi, const float* __restrict__ topw, int T, int H, int K, int e_lo,
                          int e_hi, float* const* __restrict__ peer_x, unsigned* const* __restrict__ peer_flag, int rank, int R, int maxr,
                          unsigned* __restrict__ seqs) {
    const int t = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned seq = seqs[0];
    const int slot = (int) (seq & 1u);
    if (i < H) {
        float s = 0.f;
        for (int k = 0; k < K; ++k) {
            const int e = topi[t * K + k];
            if (e >= e_lo && e < e_hi) s = fmaf(topw[t * K + k], part[((size_t) t * K + k) * H + i], s);
        }
        const size_t off = (((size_t) slot * R + rank) * maxr + t) * H + i;
        for (int r = 0; r < R; ++r) peer_x[r][off] = s;
    }
    __threadfence_system();
    __syncthreads();
    __shared__ bool last;
    if (threadIdx.x == 0) last = atomicAdd(&seqs[2], 1u) == gridDim.x * gridDim.y - 1;
    __syncthreads();
    if (last && threadIdx.x < R) {
        __threadfence_system();
        unsigned* f = peer_flag[threadIdx.x] + slot * R + rank;
        const unsigned v = seq + 1u;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(v) : "memory");
    }
    if (last && threadIdx.x == 0) {
        seqs[2] = 0;
        seqs[0] = seq + 1u;
    }
}

__global__ void k_ep_recv(const float* __restrict__ xbuf, const unsigned* __restrict__ xflag, const float* __restrict__ part,
                          const float* __restrict__ logits, int T, int E, int H, int K, int R, int maxr, float* __restrict__ out,
                          unsigned* __restrict__ seqs, unsigned* __restrict__ err, unsigned wait_limit) {
    const int t = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned seq = seqs[1];
    const int slot = (int) (seq & 1u);
    __shared__ bool ok;
    if (threadIdx.x == 0) {
        // once a wait has given up (here or anywhere: the bit is sticky) nothing waits again: the window is lost anyway and
        // the remaining exchanges must not each run out their limit
        bool all = false;
        const bool gave_up = (*(volatile unsigned*) err & (unsigned) FNX_ERR_TIMEOUT) != 0;
        for (unsigned it = 0; it < wait_limit && !all && !gave_up; ++it) {
            all = true;
            for (int r = 0; r < R; ++r) {
                unsigned v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(xflag + slot * R + r) : "memory");
                all = all && v == seq + 1u;
            }
        }
        if (!all) atomicOr(err, (unsigned) FNX_ERR_TIMEOUT);
        ok = all;
    }
    __syncthreads();
    if (i < H && ok) {
        float s = 0.f;
        for (int r = 0; r < R; ++r) s += __ldcv(xbuf + (((size_t) slot * R + r) * maxr + t) * H + i);
        s += sigmoidf_(logits[(size_t) t * (E + 1) + E]) * part[((size_t) T * K + t) * H + i];
        out[(size_t) t * H + i] += s;
    }
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(&seqs[3], 1u) == gridDim.x * gridDim.y - 1) {
        seqs[3] = 0;
        seqs[1] = seq + 1u;
    }
}

__global__ void k_plus_one(int* dst, const int* src) { *dst = *src + 1; }
// depth of every window row from the parent array (parent null: a chain)
__global__ void k_depths(const int* __restrict__ parent, int* __restrict__ depth, int T) {
    const int t = threadIdx.x;
    if (t >= T) return;
    int d = 0;
    for (int a = parent ? parent[t] : t - 1; a >= 0; a = parent ? parent[a] : a - 1) ++d;
    depth[t] = d;
}
// commit: the kept rows' K and V move to consecutive cache rows (a no-op for a chain), the kept rows' tokens join
// the context followed by the token the window emitted last (the next window's first row, as the reference's ctx
// keeps it, engine/src/session.cpp:501), the state slot advances.  One block per attention layer + one for the
// bookkeeping.
__global__ void k_commit(__half* const* __restrict__ kcs, __half* const* __restrict__ vcs, int nlayer, int row_halves,
                         const int* __restrict__ path, const int* __restrict__ tok, const int* __restrict__ emitted, int n,
                         int* __restrict__ pos, int* __restrict__ cur, int NS, int* __restrict__ ctx, int* __restrict__ ctx_n) {
    const int l = blockIdx.x, p0 = *pos;
    if (l < nlayer) {
        for (int j = 0; j < n; ++j) {
            const int src = path[j];
            if (src == j) continue;   // path is increasing, so row j's source is never overwritten before it is read
            for (int i = threadIdx.x; i < row_halves; i += blockDim.x) {
                kcs[l][(size_t) (p0 + j) * row_halves + i] = kcs[l][(size_t) (p0 + src) * row_halves + i];
                vcs[l][(size_t) (p0 + j) * row_halves + i] = vcs[l][(size_t) (p0 + src) * row_halves + i];
            }
            __syncthreads();
        }
        return;
    }
    if (threadIdx.x == 0) {
        if (ctx) {
            const int cn = *ctx_n;
            for (int j = 0; j < n; ++j) ctx[cn + j] = tok[path[j]];
            ctx[cn + n] = emitted[n - 1];
            *ctx_n = cn + n;
        }
        *cur = (*cur + 1 + path[n - 1]) % NS;
    }
}
__global__ void k_advance_pos(int* pos, int n) { *pos += n; }
// the prompt pass: the chunk's tokens joining the context; position and state slot afterwards
__global__ void k_prompt_context(int* ctx, const int* ctx_n, const int* tok, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) ctx[*ctx_n + i] = tok[i];
}
__global__ void k_prompt_advance(int* pos, int* cur, int* ctx_n, int n, int NS) {
    *pos += n;
    *cur = (*cur + n) % NS;
    *ctx_n += n;
}
// a synthetic draft vocabulary: dv token ids spread evenly over the vocabulary, ascending
__global__ void k_fill_dvocab(int* map, int dv, int V) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < dv) map[r] = (int) ((long long) r * V / dv);
}

struct Dims {
    int H, E, K, F, nq, nkv, hd, nrot, nk, nv, hs, V, MAXR, q_rows, kv_rows, attn_in, gdn_ch, gdn_in, P;
};
static Dims dims(const fnx_model_config& c) {
    Dims d;
    d.H = c.hidden; d.E = c.n_expert; d.K = c.top_k; d.F = c.ffn;
    d.nq = c.n_q_head; d.nkv = c.n_kv_head; d.hd = c.head_dim; d.nrot = c.n_rot;
    d.nk = c.gdn_k_head; d.nv = c.gdn_v_head; d.hs = c.gdn_head_dim; d.V = c.vocab; d.MAXR = c.max_rows;
    d.q_rows = d.nq * 2 * d.hd;
    d.kv_rows = d.nkv * d.hd;
    const int tile_rows = 16 * (16 / (c.hidden / 256));   // output rows per step of the dense kernel at K = hidden
    d.attn_in = round_up(d.q_rows + 2 * d.kv_rows, tile_rows);
    d.gdn_ch = (2 * d.nk + d.nv) * d.hs;
    d.gdn_in = round_up(d.gdn_ch + d.nv * d.hs + 2 * d.nv, tile_rows);
    d.P = d.MAXR * d.K + d.MAXR;   // expert output rows: pairs + the shared expert's
    return d;
}

// an IQ3_S tile matrix of N(0, sigma) weights: generate, quantise, re-tile, in chunks of whole 16-row tiles
static int synth_iq3s(fnx_engine* e, uint8_t* dst, size_t rows, size_t cols, float sigma, uint64_t seed, uint32_t stream_id, float* tmp_f,
                      uint8_t* tmp_g, size_t tmp_weights) {
    size_t chunk_rows = tmp_weights / cols / 16 * 16;
    if (chunk_rows == 0) return fail(FNX_E_ARG, "synthetic init: staging buffer too small for %zu columns", cols);
    uint32_t sub = 0;
    for (size_t r0 = 0; r0 < rows; r0 += chunk_rows, ++sub) {
        const size_t nr = rows - r0 < chunk_rows ? rows - r0 : chunk_rows;
        FNX_TRY(fnx_fill_normal(tmp_f, nr * cols, sigma, seed, stream_id + sub, e->st));
        FNX_TRY(fnx_iq3s_quantize(tmp_f, tmp_g, nr * cols, e->st));
        FNX_TRY(fnx_iq3s_retile(tmp_g, dst + iq3s_bytes(r0, cols), nr, cols, e->st));
    }
    return FNX_OK;
}

static int alloc_layer(fnx_engine* e, LayerW& L, bool attn, const std::string& pre) {
    const Dims d = dims(e->c);
    const int ns = e->c.n_seq;
    L.attn = attn;
    FNX_TRY(dalloc(e, &L.norm1, d.H, (pre + "norm1").c_str()));
    FNX_TRY(dalloc(e, &L.norm2, d.H, (pre + "norm2").c_str()));
    if (attn) {
        L.in_rows = d.attn_in;
        FNX_TRY(dalloc(e, &L.w_in, iq3s_bytes(d.attn_in, d.H), (pre + "w_in").c_str()));
        FNX_TRY(dalloc(e, &L.w_out, iq3s_bytes(d.H, d.nq * d.hd), (pre + "w_out").c_str()));
        FNX_TRY(dalloc(e, &L.qn, d.hd, (pre + "q_norm").c_str()));
        FNX_TRY(dalloc(e, &L.kn, d.hd, (pre + "k_norm").c_str()));
        FNX_TRY(dalloc(e, &L.kc, (size_t) ns * e->cache_rows * d.kv_rows, (pre + "k_cache").c_str()));
        FNX_TRY(dalloc(e, &L.vc, (size_t) ns * e->cache_rows * d.kv_rows, (pre + "v_cache").c_str()));
    } else {
        L.in_rows = d.gdn_in;
        FNX_TRY(dalloc(e, &L.w_in, iq3s_bytes(d.gdn_in, d.H), (pre + "w_in").c_str()));
        FNX_TRY(dalloc(e, &L.w_out, iq3s_bytes(d.H, d.nv * d.hs), (pre + "w_out").c_str()));
        FNX_TRY(dalloc(e, &L.convw, (size_t) d.gdn_ch * 4, (pre + "conv_w").c_str()));
        FNX_TRY(dalloc(e, &L.dt, d.nv, (pre + "dt").c_str()));
        FNX_TRY(dalloc(e, &L.a, d.nv, (pre + "a").c_str()));
        FNX_TRY(dalloc(e, &L.gnorm, d.hs, (pre + "g_norm").c_str()));
        FNX_TRY(dalloc(e, &L.S_pool, (size_t) ns * e->NS * d.nv * d.hs * d.hs, (pre + "state").c_str()));
        FNX_TRY(dalloc(e, &L.hist_pool, (size_t) ns * e->NS * 3 * d.gdn_ch, (pre + "conv_hist").c_str()));
    }
    FNX_TRY(dalloc(e, &L.wr, (size_t) (d.E + 1) * d.H, (pre + "router").c_str()));
    FNX_TRY(dalloc(e, &L.wgu, e->gu_bytes * e->E_local, (pre + "experts_gu").c_str()));
    FNX_TRY(dalloc(e, &L.wdn, e->dn_bytes * e->E_local, (pre + "experts_dn").c_str()));
    FNX_TRY(dalloc(e, &L.wsh_gu, e->gu_bytes, (pre + "shared_gu").c_str()));
    FNX_TRY(dalloc(e, &L.wsh_dn, e->dn_bytes, (pre + "shared_dn").c_str()));
    return FNX_OK;
}

static int fill_const(fnx_engine* e, float* p, size_t n, float v) {
    k_fill_const<<<(unsigned) ((n + 255) / 256), 256, 0, e->st>>>(p, n, v);
    FNX_LAUNCH_OK("fill_const");
    return FNX_OK;
}

static int init_layer(fnx_engine* e, LayerW& L, int li, uint64_t seed, float sigma, float* tf, uint8_t* tg, size_t tw) {
    const Dims d = dims(e->c);
    auto sid = [&](int kind, int ex) { return (uint32_t) (((li * 16 + kind) << 12) | ex); };
    FNX_TRY(fill_const(e, L.norm1, d.H, 1.0f));
    FNX_TRY(fill_const(e, L.norm2, d.H, 1.0f));
    FNX_TRY(synth_iq3s(e, L.w_in, L.in_rows, d.H, sigma, seed, sid(0, 0), tf, tg, tw));
    if (L.attn) {
        FNX_TRY(synth_iq3s(e, L.w_out, d.H, d.nq * d.hd, sigma, seed, sid(1, 0), tf, tg, tw));
        FNX_TRY(fill_const(e, L.qn, d.hd, 1.0f));
        FNX_TRY(fill_const(e, L.kn, d.hd, 1.0f));
    } else {
        FNX_TRY(synth_iq3s(e, L.w_out, d.H, d.nv * d.hs, sigma, seed, sid(1, 0), tf, tg, tw));
        FNX_TRY(fnx_fill_normal(L.convw, (size_t) d.gdn_ch * 4, 0.5f, seed, sid(2, 0), e->st));
        k_gdn_params<<<(d.nv + 63) / 64, 64, 0, e->st>>>(L.dt, L.a, d.nv);
        FNX_LAUNCH_OK("gdn_params");
        FNX_TRY(fill_const(e, L.gnorm, d.hs, 1.0f));
    }
    FNX_TRY(fnx_fill_normal(L.wr, (size_t) (d.E + 1) * d.H, sigma, seed, sid(3, 0), e->st));
    for (int x = 0; x < e->E_local; ++x) {
        const int ge = e->e_lo + x;   // the global expert: every rank draws the same weights for it
        FNX_TRY(synth_iq3s(e, L.wgu + (size_t) x * e->gu_bytes, 2 * d.F, d.H, sigma, seed, sid(4, ge), tf, tg, tw));
        FNX_TRY(synth_iq3s(e, L.wdn + (size_t) x * e->dn_bytes, d.H, d.F, sigma, seed, sid(5, ge), tf, tg, tw));
    }
    FNX_TRY(synth_iq3s(e, L.wsh_gu, 2 * d.F, d.H, sigma, seed, sid(6, 0), tf, tg, tw));
    FNX_TRY(synth_iq3s(e, L.wsh_dn, d.H, d.F, sigma, seed, sid(7, 0), tf, tg, tw));
    return FNX_OK;
}

// ---- the exchange as one kernel: one warp per (256-column block, row) computes the rank's routed addend for its 8 columns a
// lane, stores it into every rank's plane, releases a flag of its own per peer, waits (bounded) for the same block's flag from
// every rank, adds the planes in rank order and the local shared expert into the residual, and (img_out) leaves the new rows'
// image for the next projection.  Against k_ep_send + k_ep_recv: no kernel boundary and no arrival counter between the sending
// and the receiving half, and the flags are per block, so a block never waits for rows it does not read.
// flags: xflag + flag_off, [2 slots][ranks][blocks]; seqs[8] = exchanges so far, seqs[9] = the blocks' arrival count.
__global__ void __launch_bounds__(32) k_ep_exchange(const float* __restrict__ part, const int* __restrict__ topi, const float* __restrict__ topw,
                                                    const float* __restrict__ logits, int T, int E, int H, int K, int e_lo, int e_hi,
                                                    float* const* __restrict__ peer_x, unsigned* const* __restrict__ peer_flag, size_t flag_off,
                                                    const float* __restrict__ xbuf, const unsigned* __restrict__ xflag, int rank, int R, int maxr,
                                                    float* __restrict__ out, unsigned* __restrict__ seqs, unsigned* __restrict__ err,
                                                    unsigned wait_limit, uint8_t* __restrict__ img_out, const float* __restrict__ img_norm_w,
                                                    size_t img_stride) {
    const int blk = blockIdx.x, t = blockIdx.y, lane = threadIdx.x, KB = H / 256;
    const int nblk = gridDim.x * gridDim.y, bid = t * gridDim.x + blk;
    const size_t col = (size_t) blk * 256 + lane * 8;
    const unsigned seq = seqs[8];
    const int slot = (int) (seq & 1u);
    // ---- this rank's addend (the sum k_ep_send makes: fmaf over the picks of this rank's experts, in pick order)
    float s[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i] = 0.f;
    for (int k = 0; k < K; ++k) {
        const int e = topi[t * K + k];
        if (e < e_lo || e >= e_hi) continue;
        const float w = topw[t * K + k];
        const float4* src = reinterpret_cast<const float4*>(part + ((size_t) t * K + k) * H + col);
        const float4 a0 = src[0], a1 = src[1];
        s[0] = fmaf(w, a0.x, s[0]); s[1] = fmaf(w, a0.y, s[1]); s[2] = fmaf(w, a0.z, s[2]); s[3] = fmaf(w, a0.w, s[3]);
        s[4] = fmaf(w, a1.x, s[4]); s[5] = fmaf(w, a1.y, s[5]); s[6] = fmaf(w, a1.z, s[6]); s[7] = fmaf(w, a1.w, s[7]);
    }
    const size_t off = (((size_t) slot * R + rank) * maxr + t) * H + col;
    for (int r = 0; r < R; ++r) {
        float4* dst = reinterpret_cast<float4*>(peer_x[r] + off);
        dst[0] = make_float4(s[0], s[1], s[2], s[3]);
        dst[1] = make_float4(s[4], s[5], s[6], s[7]);
    }
    __threadfence_system();
    __syncwarp();
    if (lane < R) {
        unsigned* f = peer_flag[lane] + flag_off + ((size_t) slot * R + rank) * nblk + bid;
        const unsigned v = seq + 1u;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(v) : "memory");
    }
    // ---- every rank's slice of this block (bounded; once a wait has given up nothing waits again)
    bool mine = true;
    if (lane < R) {
        const unsigned* f = xflag + flag_off + ((size_t) slot * R + lane) * nblk + bid;
        const bool gave_up = (*(volatile unsigned*) err & (unsigned) FNX_ERR_TIMEOUT) != 0;
        mine = false;
        for (unsigned it = 0; it < wait_limit && !mine && !gave_up; ++it) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            mine = v == seq + 1u;
        }
    }
    const bool all = __all_sync(0xffffffffu, mine);
    if (!all && lane == 0) atomicOr(err, (unsigned) FNX_ERR_TIMEOUT);
    if (all) {
        QuantTask q[QUANT_BATCH];
        float v[QUANT_BATCH][8], nw[QUANT_BATCH][8];
#pragma unroll
        for (int j = 0; j < QUANT_BATCH; ++j) {
            q[j].src = nullptr;
            q[j].t = q[j].blk = 0;
        }
        q[0].src = out + (size_t) t * H + (size_t) blk * 256;
        q[0].t = t % FNX_DENSE_ROWS;
        q[0].blk = blk;
        quant_fetch(q[0], img_out ? img_norm_w : nullptr, lane, v[0], nw[0]);
        float a[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = 0.f;
        for (int r = 0; r < R; ++r) {   // in rank order on every rank: identical sums everywhere
            const float4* src = reinterpret_cast<const float4*>(xbuf + (((size_t) slot * R + r) * maxr + t) * H + col);
            const float4 a0 = __ldcv(src), a1 = __ldcv(src + 1);
            a[0] += a0.x; a[1] += a0.y; a[2] += a0.z; a[3] += a0.w;
            a[4] += a1.x; a[5] += a1.y; a[6] += a1.z; a[7] += a1.w;
        }
        {
            const float4* src = reinterpret_cast<const float4*>(part + ((size_t) T * K + t) * H + col);
            const float4 a0 = src[0], a1 = src[1];
            const float g = sigmoidf_(logits[(size_t) t * (E + 1) + E]);
            a[0] += g * a0.x; a[1] += g * a0.y; a[2] += g * a0.z; a[3] += g * a0.w;
            a[4] += g * a1.x; a[5] += g * a1.y; a[6] += g * a1.z; a[7] += g * a1.w;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) v[0][i] += a[i];
        float* dst = out + (size_t) t * H + col;
        *reinterpret_cast<float4*>(dst) = make_float4(v[0][0], v[0][1], v[0][2], v[0][3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(v[0][4], v[0][5], v[0][6], v[0][7]);
        if (img_out) {
            const int t0 = t - t % FNX_DENSE_ROWS, nt = min((int) FNX_DENSE_ROWS, T - t0), NG = (nt + 3) / 4;
            uint2* cells = reinterpret_cast<uint2*>(img_out + (size_t) (t0 / FNX_DENSE_ROWS) * img_stride);
            float* scales = reinterpret_cast<float*>(cells + (size_t) NG * (H / 32) * 32);
            float* rs = scales + (size_t) NG * KB * 8;
            quant_finish(q, v, nw, H, img_norm_w, cells, scales, rs, lane);
            if (t == t0 + nt - 1)
                for (int td = nt; td < 4 * NG; ++td) {
                    const int ng = td >> 2, n = td & 3;
                    for (int i = lane; i < 64; i += 32) {
                        const int sbG = blk * 8 + (i >> 3), lvl = (i >> 2) & 1, qq = i & 3;
                        cells[((size_t) (ng * (H / 32) + sbG) * 8 + n + 4 * lvl) * 4 + qq] = make_uint2(0u, 0u);
                    }
                    if (lane < 2) scales[(size_t) (ng * KB + blk) * 8 + n + 4 * lane] = 0.f;
                    if (lane == 2) rs[td * 16 + blk] = 0.f;
                }
        }
    }
    __syncwarp();
    if (lane == 0 && atomicAdd(&seqs[9], 1u) == (unsigned) nblk - 1u) {
        seqs[9] = 0;
        seqs[8] = seq + 1u;
    }
}

// ---- the gather of the mixers' output rows among expert-parallel ranks (lanes windows): every rank stores the rows of its
// own lanes into every peer's rows region, the last block releases one flag per peer; the receiving kernel waits for every
// other rank's flag (bounded) and copies their lanes' rows into the local buffer.
__global__ void k_dp_send(const float* __restrict__ mix, int width, const int* __restrict__ lane_own, const int* __restrict__ lane_row0, int n_lanes,
                          float* const* __restrict__ peer_x, size_t x_off, unsigned* const* __restrict__ peer_flag, int rank, int R, int maxr,
                          unsigned* __restrict__ seqs) {
    const int lane = blockIdx.y;
    const unsigned seq = seqs[4];
    const int slot = (int) (seq & 1u);
    if (lane_own[lane] >= 0) {
        const int r0 = lane_row0[lane], nr = lane_row0[lane + 1] - r0;
        const size_t n4 = (size_t) nr * width / 4;
        const float4* src = reinterpret_cast<const float4*>(mix + (size_t) r0 * width);
        for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t) gridDim.x * blockDim.x) {
            const float4 v = src[i];
            for (int r = 0; r < R; ++r)
                if (r != rank) reinterpret_cast<float4*>(peer_x[r] + x_off + ((size_t) slot * maxr + r0) * width)[i] = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    __shared__ bool last;
    if (threadIdx.x == 0) last = atomicAdd(&seqs[6], 1u) == gridDim.x * gridDim.y - 1;
    __syncthreads();
    if (last && threadIdx.x < R) {
        __threadfence_system();
        unsigned* f = peer_flag[threadIdx.x] + 2 * R + slot * R + rank;
        const unsigned v = seq + 1u;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(v) : "memory");
    }
    if (last && threadIdx.x == 0) {
        seqs[6] = 0;
        seqs[4] = seq + 1u;
    }
}
__global__ void k_dp_recv(const float* __restrict__ xrows, const unsigned* __restrict__ xflag, float* __restrict__ mix, int width,
                          const int* __restrict__ lane_own, const int* __restrict__ lane_row0, int n_lanes, int rank, int R, int maxr,
                          unsigned* __restrict__ seqs, unsigned* __restrict__ err, unsigned wait_limit) {
    const int lane = blockIdx.y;
    const unsigned seq = seqs[5];
    const int slot = (int) (seq & 1u);
    __shared__ bool ok;
    if (threadIdx.x == 0) {
        bool all = false;
        const bool gave_up = (*(volatile unsigned*) err & (unsigned) FNX_ERR_TIMEOUT) != 0;
        for (unsigned it = 0; it < wait_limit && !all && !gave_up; ++it) {
            all = true;
            for (int r = 0; r < R; ++r) {
                if (r == rank) continue;
                unsigned v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(xflag + 2 * R + slot * R + r) : "memory");
                all = all && v == seq + 1u;
            }
        }
        if (!all) atomicOr(err, (unsigned) FNX_ERR_TIMEOUT);
        ok = all;
    }
    __syncthreads();
    if (ok && lane_own[lane] < 0) {
        const int r0 = lane_row0[lane], nr = lane_row0[lane + 1] - r0;
        const size_t n4 = (size_t) nr * width / 4;
        const float4* src = reinterpret_cast<const float4*>(xrows + ((size_t) slot * maxr + r0) * width);
        float4* dst = reinterpret_cast<float4*>(mix + (size_t) r0 * width);
        for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t) gridDim.x * blockDim.x) dst[i] = __ldcv(src + i);
    }
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(&seqs[7], 1u) == gridDim.x * gridDim.y - 1) {
        seqs[7] = 0;
        seqs[5] = seq + 1u;
    }
}

// ---- one MoE block on T rows of residual R: R += experts(rmsnorm(R))
// next_norm: the norm weights of the projection that reads R next; with them (single rank) the combine leaves that projection's
// image of the rows in e->d_img and *img_ready is set
static int enqueue_moe(fnx_engine* e, const LayerW& L, float* R, int T, const float* next_norm = nullptr, bool* img_ready = nullptr) {
    const Dims d = dims(e->c);
    const bool ep = e->c.ep_size > 1;
    if (img_ready) *img_ready = false;
    FNX_TRY(fnx_router_route(L.wr, R, L.norm2, e->c.eps, T, d.E, d.H, d.K, e->e_lo, e->e_hi, 1, e->rlogits, e->topi, e->topw, e->jobs, e->njobs,
                             e->d_stats, e->err, e->st));
    const int njobs_max = T * d.K + (T + FNX_JOB_TOK - 1) / FNX_JOB_TOK;
    FNX_TRY(fnx_moe_gate_up(L.wgu, e->gu_bytes, e->e_lo, L.wsh_gu, d.E, e->jobs, e->njobs, njobs_max, R, L.norm2, e->c.eps, d.H, d.F, e->hbuf,
                            e->err, e->st));
    FNX_TRY(fnx_moe_down(L.wdn, e->dn_bytes, e->e_lo, L.wsh_dn, d.E, e->jobs, e->njobs, njobs_max, e->hbuf, d.H, d.F, e->part, e->err, e->st));
    if (!ep && next_norm && e->use_img) {
        if (img_ready) *img_ready = true;
        return fnx_moe_combine_image(e->part, e->topi, e->topw, e->rlogits, T, d.E, d.H, d.K, R, e->d_img, next_norm, e->st);
    }
    if (!ep) return fnx_moe_combine(e->part, e->topi, e->topw, e->rlogits, T, d.E, d.H, d.K, 0, d.E, 1, R, 1, e->st);
    if (e->ep_peers && e->ep_one_kernel && d.H % 256 == 0) {
        const bool img = next_norm && e->use_img;
        if (img_ready) *img_ready = img;
        k_ep_exchange<<<dim3(d.H / 256, T), 32, 0, e->st>>>(e->part, e->topi, e->topw, e->rlogits, T, d.E, d.H, d.K, e->e_lo, e->e_hi, e->d_peer_x, e->d_peer_flag,
                                                             (size_t) 4 * e->c.ep_size, e->xbuf, e->xflag, e->c.ep_rank, e->c.ep_size, d.MAXR, R, e->d_xseq, e->err,
                                                             e->wait_limit, img ? e->d_img : nullptr, next_norm, fnx_dense_image_bytes(d.H));
        FNX_LAUNCH_OK("k_ep_exchange");
        return FNX_OK;
    }
    if (e->ep_peers) {
        const dim3 grid((d.H + 255) / 256, T);
        k_ep_send<<<grid, 256, 0, e->st>>>(e->part, e->topi, e->topw, T, d.H, d.K, e->e_lo, e->e_hi, e->d_peer_x, e->d_peer_flag, e->c.ep_rank,
                                             e->c.ep_size, d.MAXR, e->d_xseq);
        FNX_LAUNCH_OK("k_ep_send");
        k_ep_recv<<<grid, 256, 0, e->st>>>(e->xbuf, e->xflag, e->part, e->rlogits, T, d.E, d.H, d.K, e->c.ep_size, d.MAXR, R, e->d_xseq, e->err, e->wait_limit);
        FNX_LAUNCH_OK("k_ep_recv");
        return FNX_OK;
    }
    // expert parallel: this rank's routed addend, summed across ranks, then the (replicated) shared expert
    FNX_TRY(fnx_moe_combine(e->part, e->topi, e->topw, e->rlogits, T, d.E, d.H, d.K, e->e_lo, e->e_hi, 0, e->moe_out, 0, e->st));
    FNX_TRY(fnx_allreduce(e, e->moe_out, (size_t) T * d.H, e->st));
    k_add_rows<<<(unsigned) (((size_t) T * d.H + 255) / 256), 256, 0, e->st>>>(R, e->moe_out, (size_t) T * d.H);
    FNX_LAUNCH_OK("moe add");
    return fnx_moe_combine(e->part, e->topi, e->topw, e->rlogits, T, d.E, d.H, d.K, 0, 0, 1, R, 1, e->st);
}

// dense projection of up to MAXR rows in calls of fnx_dense_rows(cols) rows
// (img: the rows' image in e->d_img is that of x normed by norm_w: the blocks copy it instead of quantising the rows)
static int enqueue_dense(fnx_engine* e, const uint8_t* W, int rows, int cols, const float* x, int ldx, int T, const float* norm_w, float* y, int ldy,
                         int accumulate, bool img = false) {
    const int per = img ? FNX_DENSE_ROWS : fnx_dense_rows(cols);   // (an image holds FNX_DENSE_ROWS rows: its products have <= 2048 columns)
    for (int t0 = 0; t0 < T; t0 += per) {
        const int nt = T - t0 < per ? T - t0 : per;
        if (img) {
            FNX_TRY(fnx_dense_image(W, rows, cols, e->d_img + (size_t) (t0 / FNX_DENSE_ROWS) * fnx_dense_image_bytes(cols), nt, norm_w != nullptr, e->c.eps,
                                    y + (size_t) t0 * ldy, ldy, accumulate, e->err, e->st));
            continue;
        }
        FNX_TRY(fnx_dense(W, rows, cols, x + (size_t) t0 * ldx, ldx, nt, norm_w, e->c.eps, y + (size_t) t0 * ldy, ldy, accumulate, e->err, e->st));
    }
    return FNX_OK;
}

static int enqueue_attention(fnx_engine* e, const LayerW& L, float* R, int T, int seq, const int* d_parent, const int* d_depth, const int* d_pos,
                             bool img = false) {
    const Dims d = dims(e->c);
    FNX_TRY(enqueue_dense(e, L.w_in, L.in_rows, d.H, R, d.H, T, L.norm1, e->proj, e->proj_ld, 0, img));
    __half* kc = L.kc + (size_t) seq * e->cache_rows * d.kv_rows;
    __half* vc = L.vc + (size_t) seq * e->cache_rows * d.kv_rows;
    float* qg = e->proj;
    float* k = e->proj + d.q_rows;
    float* v = k + d.kv_rows;
    FNX_TRY(fnx_attn_prep_append(qg, e->proj_ld, k, e->proj_ld, v, e->proj_ld, L.qn, L.kn, kc, vc, T, d.nq, d.nkv, d.hd, d.nrot, d_pos, d_depth,
                                 e->c.eps, e->c.rope_base, e->st));
    FNX_TRY(fnx_attn(qg, e->proj_ld, kc, vc, e->mix, T, d.nq, d.nkv, d.hd, d_pos, d_parent, e->att_scratch, e->st));
    return enqueue_dense(e, L.w_out, d.H, d.nq * d.hd, e->mix, d.nq * d.hd, T, nullptr, R, d.H, 1);
}

static int enqueue_gdn(fnx_engine* e, const LayerW& L, float* R, int T, int seq, const int* d_parent, bool img = false) {
    const Dims d = dims(e->c);
    FNX_TRY(enqueue_dense(e, L.w_in, L.in_rows, d.H, R, d.H, T, L.norm1, e->proj, e->proj_ld, 0, img));
    float* S = L.S_pool + (size_t) seq * e->NS * d.nv * d.hs * d.hs;
    float* hist = L.hist_pool + (size_t) seq * e->NS * 3 * d.gdn_ch;
    FNX_TRY(fnx_gdn_core(e->proj, e->proj_ld, e->proj + d.gdn_ch + d.nv * d.hs, e->proj_ld, hist, L.convw, L.dt, L.a, L.gnorm, S, e->d_cur + seq,
                         e->NS, d_parent, e->mix, d.nk, d.nv, d.hs, T, e->c.eps, e->st));
    return enqueue_dense(e, L.w_out, d.H, d.nv * d.hs, e->mix, d.nv * d.hs, T, nullptr, R, d.H, 1);
}

// the whole verify window: embed, layers, head, argmax, greedy acceptance
static int enqueue_verify(fnx_engine* e, int seq, int T, bool tree) {
    const Dims d = dims(e->c);
    const int* par = tree ? e->d_parent : nullptr;
    k_depths<<<1, 32, 0, e->st>>>(par, e->d_depth, T);
    FNX_LAUNCH_OK("depths");
    FNX_TRY(fnx_embed_rows(e->embed, e->d_tok, T, d.H, e->R, e->st));
    bool img = false;   // the rows' image for the next projection is ready (left by the layer before)
    for (size_t l = 0; l < e->layers.size(); ++l) {
        const LayerW& L = e->layers[l];
        if (L.attn) FNX_TRY(enqueue_attention(e, L, e->R, T, seq, par, e->d_depth, e->d_pos + seq, img));
        else FNX_TRY(enqueue_gdn(e, L, e->R, T, seq, par, img));
        FNX_TRY(enqueue_moe(e, L, e->R, T, l + 1 < e->layers.size() ? e->layers[l + 1].norm1 : e->out_norm, &img));
    }
    FNX_TRY(enqueue_dense(e, e->head, d.V, d.H, e->R, d.H, T, e->out_norm, e->logits, d.V, 0, img));
    if (e->rules_on)   // the request's logit_bias and penalties, before either rule looks at the logits
        FNX_TRY(fnx_logit_adjust(e->logits, T, d.V, e->d_ctx + (size_t) seq * e->cache_rows, e->d_ctx_n + seq, e->d_tok, e->rules.last_n, e->rules.repeat,
                                 e->rules.freq, e->rules.present, e->d_bias_tok, e->d_bias_val, e->rules.bias_n, e->st));
    if (e->sampling_on) {   // the sampling rule over the rows' 64 best tokens, uniforms addressed (seed, sequence, window, slot)
        FNX_TRY(fnx_top_tokens(e->logits, T, d.V, e->cand_v, e->cand_i, e->st));
        FNX_TRY(fnx_accept_sample(e->cand_v, e->cand_i, e->d_tok, T, e->sampling, nullptr, nullptr, nullptr, e->sample_seed, (uint32_t) seq, e->d_step + seq,
                                  e->result, e->st));
        return FNX_OK;
    }
    FNX_TRY(fnx_argmax(e->logits, T, d.V, e->best_i, e->best_v, e->err, e->st));
    return fnx_accept_greedy(e->d_tok, par, e->best_i, T, e->result, e->st);
}

// one MTP call on T rows: Rm = fc_hid(rms(src)) + fc_emb(rms(emb(tok))), the draft block, the head on the last row
static int enqueue_mtp(fnx_engine* e, int seq, int T, const float* src) {
    const Dims d = dims(e->c);
    FNX_TRY(fnx_mtp_input(e->mtp_fc_hid, e->mtp_fc_emb, e->embed, e->mtp_hnorm, e->mtp_enorm, e->c.eps, src, d.H, e->d_mtok, T, d.H, e->Emb, e->Rm, e->err, e->st));
    FNX_TRY(enqueue_attention(e, e->mtp, e->Rm, T, seq, nullptr, nullptr, e->d_mpos));
    FNX_TRY(enqueue_moe(e, e->mtp, e->Rm, T));
    return fnx_dense(e->mtp_head ? e->mtp_head : e->head, e->dvn, d.H, e->Rm + (size_t) (T - 1) * d.H, d.H, 1, e->mtp_onorm, e->c.eps, e->logits, e->dvn, 0,
                     e->err, e->st);
}

// ------------------------------------------------------------------------------------------------ batched lanes
// Several sequences' rows in one window (Engine::verify_rows / commit_rows / draft_rows, engine/src/engine_common.cu:1234-1684):
// lane j = rows [row0[j], row0[j + 1]) of sequence lane_seq[j], a chain.  Projections, router, experts and head run over all
// rows at once (an expert picked by rows of several lanes is read once); attention, DeltaNet, acceptance and commit go by
// lane, each with its own sequence's position, caches and state rings.

// lanes kept as prefixes of their chains: the kept tokens and the emitted one join each sequence's context, positions and
// state slots advance
__global__ void k_commit_lanes(const int* __restrict__ lane_seq, const int* __restrict__ lane_row0, const int* __restrict__ keep,
                               const int* __restrict__ tok, const int* __restrict__ results, int* __restrict__ pos, int* __restrict__ cur, int NS,
                               int* __restrict__ ctx, size_t ctx_stride, int* __restrict__ ctx_n, int L) {
    const int lane = threadIdx.x;
    if (lane >= L) return;
    const int seq = lane_seq[lane], row0 = lane_row0[lane], n = keep[lane];
    const int* res = results + (size_t) lane * (1 + 2 * FNX_MAX_ROWS);
    int* c = ctx + (size_t) seq * ctx_stride;
    const int cn = ctx_n[seq];
    for (int j = 0; j < n; ++j) c[cn + j] = tok[row0 + j];
    c[cn + n] = res[1 + FNX_MAX_ROWS + n - 1];
    ctx_n[seq] = cn + n;
    cur[seq] = (cur[seq] + n) % NS;
    pos[seq] += n;
}
// the draft layer's first call: its rows are the lanes' kept rows (source rows and the tokens they emitted)
__global__ void k_mtp_gather_lanes(float* __restrict__ dst, const float* __restrict__ src, int* __restrict__ mtok, const int* __restrict__ results,
                                   const int* __restrict__ row0v, const int* __restrict__ row0m, int L, int H) {
    const int r = blockIdx.y;   // draft-layer row
    int lane = 0;
    while (lane + 1 < L && r >= row0m[lane + 1]) ++lane;
    if (r >= row0m[L]) return;
    const int j = r - row0m[lane];
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < H) dst[(size_t) r * H + i] = src[(size_t) (row0v[lane] + j) * H + i];
    if (i == 0) mtok[r] = results[(size_t) lane * (1 + 2 * FNX_MAX_ROWS) + 1 + FNX_MAX_ROWS + j];
}
// dst[lane] = src[last row of lane]
__global__ void k_last_rows(float* __restrict__ dst, const float* __restrict__ src, const int* __restrict__ row0, int H) {
    const int lane = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < H) dst[(size_t) lane * H + i] = src[(size_t) (row0[lane + 1] - 1) * H + i];
}
// the draft layer's positions advance per lane: by the rows of its first call, then by one
__global__ void k_mtp_advance_lanes(int* __restrict__ mpos, const int* __restrict__ lane_seq, const int* __restrict__ row0m, int L, int first) {
    const int lane = threadIdx.x;
    if (lane < L) mpos[lane_seq[lane]] += first ? row0m[lane + 1] - row0m[lane] : 1;
}
__global__ void k_mtp_set_pos_lanes(int* __restrict__ mpos, const int* __restrict__ lane_seq, const int* __restrict__ base, int L) {
    const int lane = threadIdx.x;
    if (lane < L) mpos[lane_seq[lane]] = base[lane];
}
__global__ void k_scatter_drafts(int* __restrict__ out, const int* __restrict__ best, int L, int k, int j) {
    const int lane = threadIdx.x;
    if (lane < L) out[lane * k + j] = best[lane];
}

// mixer of one layer over the lanes' rows: R += out_proj(mixer(in_proj(rmsnorm(R))))
// the gather of the mixers' rows among the ranks (every rank ran its own sequences' lanes only)
static int enqueue_dp_gather(fnx_engine* e, int width, int n_lanes, const int* d_row0) {
    const Dims d = dims(e->c);
    const dim3 grid(8, n_lanes);
    k_dp_send<<<grid, 256, 0, e->st>>>(e->mix, width, e->d_lane_own, d_row0, n_lanes, e->d_peer_x, e->x_off_rows, e->d_peer_flag, e->c.ep_rank, e->c.ep_size, d.MAXR,
                                         e->d_xseq);
    FNX_LAUNCH_OK("k_dp_send");
    k_dp_recv<<<grid, 256, 0, e->st>>>(e->xbuf + e->x_off_rows, e->xflag, e->mix, width, e->d_lane_own, d_row0, n_lanes, e->c.ep_rank, e->c.ep_size, d.MAXR, e->d_xseq,
                                         e->err, e->wait_limit);
    FNX_LAUNCH_OK("k_dp_recv");
    return FNX_OK;
}

static int enqueue_mixer_lanes(fnx_engine* e, const LayerW& L, float* R, int T, int n_lanes, int max_lane_rows, const int* d_lane_seq, const int* d_row0,
                               const int* d_pos, bool img = false) {
    const Dims d = dims(e->c);
    // expert-parallel ranks with the peer-memory exchange open: every rank runs its own sequences' lanes (d_lane_own holds -1
    // for the others', which the lane kernels skip) and the output rows are gathered before the output projection
    const bool dp = e->c.ep_size > 1 && e->ep_peers && e->dp_mixers;
    const int* lanes = dp ? e->d_lane_own : d_lane_seq;
    FNX_TRY(enqueue_dense(e, L.w_in, L.in_rows, d.H, R, d.H, T, L.norm1, e->proj, e->proj_ld, 0, img));
    if (L.attn) {
        float* qg = e->proj;
        float* k = e->proj + d.q_rows;
        float* v = k + d.kv_rows;
        FNX_TRY(fnx_attn_prep_append_lanes(qg, e->proj_ld, k, e->proj_ld, v, e->proj_ld, L.qn, L.kn, L.kc, L.vc, (size_t) e->cache_rows, n_lanes, max_lane_rows, d.nq,
                                           d.nkv, d.hd, d.nrot, d_pos, lanes, d_row0, e->c.eps, e->c.rope_base, e->st));
        FNX_TRY(fnx_attn_lanes(qg, e->proj_ld, L.kc, L.vc, (size_t) e->cache_rows, e->mix, T, n_lanes, d.nq, d.nkv, d.hd, d_pos, lanes, d_row0, e->att_scratch, e->st));
        if (dp) FNX_TRY(enqueue_dp_gather(e, d.nq * d.hd, n_lanes, d_row0));
        return enqueue_dense(e, L.w_out, d.H, d.nq * d.hd, e->mix, d.nq * d.hd, T, nullptr, R, d.H, 1);
    }
    FNX_TRY(fnx_gdn_core_lanes(e->proj, e->proj_ld, e->proj + d.gdn_ch + d.nv * d.hs, e->proj_ld, L.hist_pool, (size_t) e->NS * 3 * d.gdn_ch, L.convw, L.dt, L.a, L.gnorm,
                               L.S_pool, (size_t) e->NS * d.nv * d.hs * d.hs, e->d_cur, e->NS, lanes, d_row0, n_lanes, max_lane_rows, e->mix, d.nk, d.nv, d.hs,
                               e->c.eps, e->st));
    if (dp) FNX_TRY(enqueue_dp_gather(e, d.nv * d.hs, n_lanes, d_row0));
    return enqueue_dense(e, L.w_out, d.H, d.nv * d.hs, e->mix, d.nv * d.hs, T, nullptr, R, d.H, 1);
}

static int enqueue_verify_lanes(fnx_engine* e, int n_lanes, int rows, int T) {   // rows: the longest lane's; T: rows in all
    const Dims d = dims(e->c);
    FNX_TRY(fnx_embed_rows(e->embed, e->d_tok, T, d.H, e->R, e->st));
    bool img = false;
    for (size_t l = 0; l < e->layers.size(); ++l) {
        const LayerW& L = e->layers[l];
        FNX_TRY(enqueue_mixer_lanes(e, L, e->R, T, n_lanes, rows, e->d_lane_seq, e->d_lane_row0, e->d_pos, img));
        FNX_TRY(enqueue_moe(e, L, e->R, T, l + 1 < e->layers.size() ? e->layers[l + 1].norm1 : e->out_norm, &img));
    }
    FNX_TRY(enqueue_dense(e, e->head, d.V, d.H, e->R, d.H, T, e->out_norm, e->logits, d.V, 0, img));
    if (e->sampling_on) {
        FNX_TRY(fnx_top_tokens(e->logits, T, d.V, e->cand_v, e->cand_i, e->st));
        return fnx_accept_sample_lanes(e->cand_v, e->cand_i, e->d_tok, e->sampling, e->sample_seed, e->d_lane_seq, e->d_lane_row0, n_lanes, rows, e->d_step,
                                       e->d_results, e->st);
    }
    FNX_TRY(fnx_argmax(e->logits, T, d.V, e->best_i, e->best_v, e->err, e->st));
    return fnx_accept_greedy_lanes(e->d_tok, e->best_i, e->d_lane_row0, n_lanes, e->d_results, e->st);
}

// one draft-layer call over lanes (rows per the table d_row0, Tm in all, at most max_rows per lane); the lanes' last rows go
// through the head and their best tokens land in best_i[0 .. n_lanes)
static int enqueue_mtp_lanes(fnx_engine* e, int n_lanes, int Tm, int max_rows, const int* d_row0, const float* src) {
    const Dims d = dims(e->c);
    FNX_TRY(fnx_mtp_input(e->mtp_fc_hid, e->mtp_fc_emb, e->embed, e->mtp_hnorm, e->mtp_enorm, e->c.eps, src, d.H, e->d_mtok, Tm, d.H, e->Emb, e->Rm, e->err, e->st));
    FNX_TRY(enqueue_mixer_lanes(e, e->mtp, e->Rm, Tm, n_lanes, max_rows, e->d_lane_seq, d_row0, e->d_mpos_seq));
    FNX_TRY(enqueue_moe(e, e->mtp, e->Rm, Tm));
    k_last_rows<<<dim3((d.H + 255) / 256, n_lanes), 256, 0, e->st>>>(e->Rlast, e->Rm, d_row0, d.H);
    FNX_LAUNCH_OK("draft last rows");
    FNX_TRY(enqueue_dense(e, e->mtp_head ? e->mtp_head : e->head, e->dvn, d.H, e->Rlast, d.H, n_lanes, e->mtp_onorm, e->logits, e->dvn, 0));
    return fnx_argmax_mapped(e->logits, n_lanes, e->dvn, e->d_dvocab, e->best_i, nullptr, e->err, e->st);
}

template <typename F>
static int run_graph(fnx_engine* e, uint64_t key, F&& enqueue) {
    auto it = e->graphs.find(key);
    if (it == e->graphs.end()) {
        // a first, uncaptured run: it sets the kernels' launch attributes and is harmless, since a window changes no
        // committed state (cache rows past the position, state slots other than the current one)
        FNX_TRY(enqueue());
        FNX_CUDA_OK(cudaStreamSynchronize(e->st));
        cudaGraph_t g = nullptr;
        FNX_CUDA_OK(cudaStreamBeginCapture(e->st, cudaStreamCaptureModeRelaxed));
        const int rc = enqueue();
        const cudaError_t ce = cudaStreamEndCapture(e->st, &g);
        if (rc != FNX_OK) {
            if (g) cudaGraphDestroy(g);
            return rc;
        }
        if (ce != cudaSuccess) return fail(FNX_E_CUDA, "graph capture: %s", cudaGetErrorString(ce));
        size_t nn = 0;
        FNX_CUDA_OK(cudaGraphGetNodes(g, nullptr, &nn));
        std::vector<cudaGraphNode_t> nodes(nn);
        FNX_CUDA_OK(cudaGraphGetNodes(g, nodes.data(), &nn));
        unsigned nk = 0;
        for (size_t i = 0; i < nn; ++i) {
            cudaGraphNodeType ty;
            if (cudaGraphNodeGetType(nodes[i], &ty) == cudaSuccess && ty == cudaGraphNodeTypeKernel) ++nk;
        }
        e->graph_kernels[key] = nk;
        cudaGraphExec_t x = nullptr;
        FNX_CUDA_OK(cudaGraphInstantiate(&x, g, 0));
        cudaGraphDestroy(g);
        it = e->graphs.emplace(key, x).first;
    }
    FNX_CUDA_OK(cudaEventRecord(e->ev0, e->st));
    FNX_CUDA_OK(cudaGraphLaunch(it->second, e->st));
    e->launches += e->graph_kernels[key];
    FNX_CUDA_OK(cudaEventRecord(e->ev1, e->st));
    return FNX_OK;
}

}  // namespace fnxb

extern "C" int fnx_commit(void* const* k_caches, void* const* v_caches, int n_attn_layers, int row_halves, const int* path, int n, int* pos0, int* cur,
                          int NS, fnx_stream st) {
    FNX_REQUIRE(path && pos0 && cur && (n_attn_layers == 0 || (k_caches && v_caches)), "fnx_commit: null pointer");
    FNX_REQUIRE(n >= 1 && n <= FNX_MAX_ROWS && n_attn_layers >= 0 && row_halves >= 0 && NS >= 2, "fnx_commit: %d rows, %d layers, %d slots", n, n_attn_layers, NS);
    k_commit<<<n_attn_layers + 1, 256, 0, as_stream(st)>>>((__half* const*) k_caches, (__half* const*) v_caches, n_attn_layers, row_halves, path, nullptr, nullptr, n,
                                                             pos0, cur, NS, nullptr, nullptr);
    FNX_LAUNCH_OK("fnx_commit");
    k_advance_pos<<<1, 1, 0, as_stream(st)>>>(pos0, n);
    FNX_LAUNCH_OK("fnx_commit (position)");
    return FNX_OK;
}

extern "C" int fnx_engine_create(const fnx_model_config* cfg, fnx_engine** out) {
    FNX_REQUIRE(cfg && out, "fnx_engine_create: null pointer");
    const fnx_model_config& c = *cfg;
    FNX_REQUIRE(c.hidden % 256 == 0 && c.hidden <= 4096 && c.ffn % 256 == 0, "engine: hidden %d / ffn %d must be multiples of 256", c.hidden, c.ffn);
    FNX_REQUIRE(c.max_rows >= 1 && c.max_rows <= FNX_MAX_ROWS, "engine: max_rows %d (1..%d)", c.max_rows, FNX_MAX_ROWS);
    FNX_REQUIRE(c.ep_size >= 1 && c.ep_rank >= 0 && c.ep_rank < c.ep_size && c.n_expert % c.ep_size == 0, "engine: expert-parallel rank %d of %d over %d experts",
                c.ep_rank, c.ep_size, c.n_expert);
    FNX_REQUIRE(c.n_seq >= 1 && c.n_layer >= 1 && c.attn_every >= 1, "engine: bad sequence / layer counts");
    FNX_REQUIRE(c.vocab % (16 * (16 / (c.hidden / 256))) == 0, "engine: vocabulary %d is not a whole number of head tiles", c.vocab);
    FNX_REQUIRE(c.draft_vocab >= 0 && c.draft_vocab <= c.vocab && c.draft_vocab % 16 == 0, "engine: draft vocabulary %d (0, or a multiple of 16 up to %d)",
                c.draft_vocab, c.vocab);
    fnx_engine* e = new fnx_engine();
    e->c = c;
    const Dims d = dims(c);
    e->NS = c.max_rows + 1;
    e->cache_rows = c.max_ctx + c.max_rows;
    e->E_local = c.n_expert / c.ep_size;
    e->e_lo = c.ep_rank * e->E_local;
    e->e_hi = e->e_lo + e->E_local;
    e->gu_bytes = iq3s_bytes((size_t) 2 * d.F, d.H);
    e->dn_bytes = iq3s_bytes((size_t) d.H, d.F);
    e->seqs.resize(c.n_seq);
    int rc = FNX_OK;
    auto body = [&]() -> int {
        FNX_CUDA_OK(cudaStreamCreateWithFlags(&e->st, cudaStreamNonBlocking));
        FNX_CUDA_OK(cudaEventCreate(&e->ev0));
        FNX_CUDA_OK(cudaEventCreate(&e->ev1));
        e->layers.resize(c.n_layer);
        for (int l = 0; l < c.n_layer; ++l) FNX_TRY(alloc_layer(e, e->layers[l], (l + 1) % c.attn_every == 0, "l" + std::to_string(l) + "."));
        FNX_TRY(alloc_layer(e, e->mtp, true, "mtp."));
        FNX_TRY(dalloc(e, &e->mtp_hnorm, d.H, "mtp.h_norm"));
        FNX_TRY(dalloc(e, &e->mtp_enorm, d.H, "mtp.e_norm"));
        FNX_TRY(dalloc(e, &e->mtp_onorm, d.H, "mtp.out_norm"));
        FNX_TRY(dalloc(e, &e->out_norm, d.H, "out_norm"));
        FNX_TRY(dalloc(e, &e->mtp_fc_hid, iq3s_bytes(d.H, d.H), "mtp.fc_hid"));
        FNX_TRY(dalloc(e, &e->mtp_fc_emb, iq3s_bytes(d.H, d.H), "mtp.fc_emb"));
        FNX_TRY(dalloc(e, &e->head, iq3s_bytes(d.V, d.H), "head"));
        e->dvn = d.V;
        if (c.draft_vocab > 0) {
            e->dvn = c.draft_vocab;
            FNX_TRY(dalloc(e, &e->mtp_head, iq3s_bytes(e->dvn, d.H), "mtp.head"));
            FNX_TRY(dalloc(e, &e->d_dvocab, (size_t) e->dvn, "mtp.vocab"));
        }
        FNX_TRY(dalloc(e, &e->embed, (size_t) d.V * d.H, "embed"));
        e->proj_ld = d.attn_in > d.gdn_in ? d.attn_in : d.gdn_in;
        const int mixw = d.nq * d.hd > d.nv * d.hs ? d.nq * d.hd : d.nv * d.hs;
        FNX_TRY(dalloc(e, &e->R, (size_t) d.MAXR * d.H, "buf.R"));
        FNX_TRY(dalloc(e, &e->Rm, (size_t) d.MAXR * d.H, "buf.Rm"));
        FNX_TRY(dalloc(e, &e->Rsrc, (size_t) d.MAXR * d.H, "buf.Rsrc"));
        FNX_TRY(dalloc(e, &e->Emb, (size_t) d.MAXR * d.H, "buf.Emb"));
        FNX_TRY(dalloc(e, &e->proj, (size_t) d.MAXR * e->proj_ld, "buf.proj"));
        FNX_TRY(dalloc(e, &e->mix, (size_t) d.MAXR * mixw, "buf.mix"));
        FNX_TRY(dalloc(e, &e->logits, (size_t) d.MAXR * d.V, "buf.logits"));
        FNX_TRY(dalloc(e, &e->rlogits, (size_t) d.MAXR * (d.E + 1), "buf.router_logits"));
        FNX_TRY(dalloc(e, &e->topi, (size_t) d.MAXR * d.K, "buf.topi"));
        FNX_TRY(dalloc(e, &e->topw, (size_t) d.MAXR * d.K, "buf.topw"));
        FNX_TRY(dalloc(e, &e->jobs, (size_t) d.P + 8, "buf.jobs"));
        FNX_TRY(dalloc(e, &e->njobs, 2, "buf.njobs"));
        FNX_TRY(dalloc(e, &e->hbuf, (size_t) d.P * d.F, "buf.h"));
        FNX_TRY(dalloc(e, &e->part, (size_t) d.P * d.H, "buf.part"));
        FNX_TRY(dalloc(e, &e->moe_out, (size_t) d.MAXR * d.H, "buf.moe_out"));
        FNX_TRY(dalloc(e, &e->d_img, (size_t) ((d.MAXR + FNX_DENSE_ROWS - 1) / FNX_DENSE_ROWS) * fnx_dense_image_bytes(d.H)));
        if (const char* nf = getenv("FNX_NO_IMAGE")) e->use_img = nf[0] != '1';
        if (d.H > 2048) e->use_img = false;   // (an image's product takes FNX_DENSE_ROWS rows a call, which wider rows do not fit)
        if (c.ep_size > 1) {
            e->mix_width = mixw;
            e->x_off_rows = (size_t) 2 * c.ep_size * d.MAXR * d.H;
            FNX_TRY(dalloc(e, &e->xbuf, e->x_off_rows + (size_t) 2 * d.MAXR * mixw, "buf.ep_x"));
            // flags: [2][ranks] of the two-kernel exchange, [2][ranks] of the rows gather, [2][ranks][blocks] of the one-kernel exchange
            FNX_TRY(dalloc(e, &e->xflag, (size_t) 4 * c.ep_size + (size_t) 2 * c.ep_size * d.MAXR * (d.H / 256 + 1), "buf.ep_flag"));
            if (const char* n1 = getenv("FNX_EP_TWO_KERNELS")) e->ep_one_kernel = n1[0] != '1';
            if (const char* nd = getenv("FNX_NO_DP")) e->dp_mixers = nd[0] != '1';
            FNX_TRY(dalloc(e, &e->d_peer_x, (size_t) c.ep_size));
            FNX_TRY(dalloc(e, &e->d_peer_flag, (size_t) c.ep_size));
            FNX_TRY(dalloc(e, &e->d_xseq, 12));
        }
        FNX_TRY(dalloc(e, &e->best_i, d.MAXR, "buf.best_i"));
        FNX_TRY(dalloc(e, &e->best_v, d.MAXR, "buf.best_v"));
        FNX_TRY(dalloc(e, &e->cand_v, (size_t) d.MAXR * FNX_TOPK_N, "buf.cand_v"));
        FNX_TRY(dalloc(e, &e->cand_i, (size_t) d.MAXR * FNX_TOPK_N, "buf.cand_i"));
        FNX_TRY(dalloc(e, &e->result, 1 + 2 * FNX_MAX_ROWS, "buf.result"));
        FNX_TRY(dalloc(e, &e->d_tok, FNX_MAX_ROWS, "buf.tok"));
        FNX_TRY(dalloc(e, &e->d_parent, FNX_MAX_ROWS, "buf.parent"));
        FNX_TRY(dalloc(e, &e->d_depth, FNX_MAX_ROWS, "buf.depth"));
        FNX_TRY(dalloc(e, &e->d_path, FNX_MAX_ROWS, "buf.path"));
        FNX_TRY(dalloc(e, &e->d_mtok, FNX_MAX_ROWS, "buf.mtp_tok"));
        FNX_TRY(dalloc(e, &e->d_mpos, 1, "buf.mtp_pos"));
        FNX_TRY(dalloc(e, &e->d_mpos_base, FNX_MAX_ROWS, "buf.mtp_pos_base"));
        FNX_TRY(dalloc(e, &e->d_drafts, FNX_MAX_ROWS, "buf.draft"));
        FNX_TRY(dalloc(e, &e->d_step, c.n_seq, "seq.step"));
        FNX_TRY(dalloc(e, &e->d_lk, FNX_MAX_ROWS + 4, "buf.lookup"));
        FNX_TRY(dalloc(e, &e->d_lane_seq, FNX_MAX_ROWS, "buf.lane_seq"));
        FNX_TRY(dalloc(e, &e->d_lane_own, FNX_MAX_ROWS));
        FNX_TRY(dalloc(e, &e->d_lane_row0, FNX_MAX_ROWS + 1, "buf.lane_row0"));
        FNX_TRY(dalloc(e, &e->d_mlane_row0, FNX_MAX_ROWS + 1, "buf.mtp_lane_row0"));
        FNX_TRY(dalloc(e, &e->d_ident_row0, FNX_MAX_ROWS + 1, "buf.ident_row0"));
        FNX_TRY(dalloc(e, &e->d_keep, FNX_MAX_ROWS, "buf.lane_keep"));
        FNX_TRY(dalloc(e, &e->d_results, (size_t) FNX_MAX_ROWS * (1 + 2 * FNX_MAX_ROWS), "buf.lane_results"));
        FNX_TRY(dalloc(e, &e->d_mpos_seq, c.n_seq, "seq.mtp_pos"));
        FNX_TRY(dalloc(e, &e->d_ldrafts, (size_t) FNX_MAX_ROWS * FNX_MAX_ROWS, "buf.lane_drafts"));
        FNX_TRY(dalloc(e, &e->Rlast, (size_t) d.MAXR * d.H, "buf.Rlast"));
        FNX_TRY(dalloc(e, &e->d_pos, c.n_seq, "seq.pos"));
        FNX_TRY(dalloc(e, &e->d_cur, c.n_seq, "seq.cur"));
        FNX_TRY(dalloc(e, &e->d_ctx, (size_t) c.n_seq * e->cache_rows, "seq.ctx"));
        FNX_TRY(dalloc(e, &e->d_ctx_n, c.n_seq, "seq.ctx_n"));
        FNX_TRY(dalloc(e, &e->err, 1, "buf.err"));
        FNX_TRY(dalloc(e, &e->d_stats, 2, "buf.stats"));
        void* sc = nullptr;
        const size_t sb = fnx_attn_scratch_bytes(d.MAXR, d.nq, d.hd);
        FNX_TRY(dalloc(e, (uint8_t**) &sc, sb, "buf.attn_scratch"));
        e->att_scratch = sc;
        FNX_CUDA_OK(cudaHostAlloc((void**) &e->h_stage, sizeof(int) * 8 * FNX_MAX_ROWS, cudaHostAllocDefault));
        return FNX_OK;
    };
    rc = body();
    if (rc != FNX_OK) {
        fnx_engine_destroy(e);
        return rc;
    }
    *out = e;
    return FNX_OK;
}

extern "C" void fnx_engine_destroy(fnx_engine* e) {
    if (!e) return;
    if (e->st) cudaStreamSynchronize(e->st);
    for (auto& g : e->graphs) cudaGraphExecDestroy(g.second);
    for (void* q : e->ipc_opened) cudaIpcCloseMemHandle(q);
    if (e->comm && nccl() && nccl()->CommDestroy) nccl()->CommDestroy(e->comm);
    for (void* p : e->owned) cudaFree(p);
    if (e->d_bias_tok) cudaFree(e->d_bias_tok);
    if (e->d_bias_val) cudaFree(e->d_bias_val);
    if (e->h_stage) cudaFreeHost(e->h_stage);
    if (e->ev0) cudaEventDestroy(e->ev0);
    if (e->ev1) cudaEventDestroy(e->ev1);
    if (e->st) cudaStreamDestroy(e->st);
    delete e;
}

extern "C" int fnx_engine_init_synthetic(fnx_engine* e, uint64_t seed, float sigma) {
    FNX_REQUIRE(e, "fnx_engine_init_synthetic: null engine");
    const Dims d = dims(e->c);
    // staging: one chunk of f32 weights and its GGML blocks
    const size_t tw = (size_t) 32 << 20;
    float* tf = nullptr;
    uint8_t* tg = nullptr;
    FNX_CUDA_OK(cudaMalloc((void**) &tf, tw * sizeof(float)));
    FNX_CUDA_OK(cudaMalloc((void**) &tg, tw / 256 * IQ3S_BLOCK_BYTES));
    int rc = FNX_OK;
    auto body = [&]() -> int {
        for (int l = 0; l < e->c.n_layer; ++l) FNX_TRY(init_layer(e, e->layers[l], l, seed, sigma, tf, tg, tw));
        FNX_TRY(init_layer(e, e->mtp, 60, seed, sigma, tf, tg, tw));
        FNX_TRY(fill_const(e, e->mtp_hnorm, d.H, 1.0f));
        FNX_TRY(fill_const(e, e->mtp_enorm, d.H, 1.0f));
        FNX_TRY(fill_const(e, e->mtp_onorm, d.H, 1.0f));
        FNX_TRY(fill_const(e, e->out_norm, d.H, 1.0f));
        FNX_TRY(synth_iq3s(e, e->mtp_fc_hid, d.H, d.H, sigma, seed, (61u * 16 + 0) << 12, tf, tg, tw));
        FNX_TRY(synth_iq3s(e, e->mtp_fc_emb, d.H, d.H, sigma, seed, (61u * 16 + 1) << 12, tf, tg, tw));
        FNX_TRY(synth_iq3s(e, e->head, d.V, d.H, sigma, seed, (62u * 16) << 12, tf, tg, tw));
        if (e->mtp_head) {
            FNX_TRY(synth_iq3s(e, e->mtp_head, e->dvn, d.H, sigma, seed, (61u * 16 + 2) << 12, tf, tg, tw));
            k_fill_dvocab<<<(e->dvn + 255) / 256, 256, 0, e->st>>>(e->d_dvocab, e->dvn, d.V);
            FNX_LAUNCH_OK("draft vocabulary");
        }
        // the embedding table: N(0, 1) rounded to f16, in chunks of the staging buffer
        const size_t n = (size_t) d.V * d.H;
        uint32_t sub = 0;
        for (size_t o = 0; o < n; o += tw, ++sub) {
            const size_t m = n - o < tw ? n - o : tw;
            FNX_TRY(fnx_fill_normal(tf, m, 1.0f, seed, ((63u * 16) << 12) + sub, e->st));
            k_f32_to_f16<<<(unsigned) ((m + 255) / 256), 256, 0, e->st>>>(tf, e->embed + o, m);
            FNX_LAUNCH_OK("embed init");
        }
        FNX_CUDA_OK(cudaStreamSynchronize(e->st));
        return FNX_OK;
    };
    rc = body();
    cudaStreamSynchronize(e->st);
    cudaFree(tf);
    cudaFree(tg);
    return rc;
}

extern "C" size_t fnx_engine_device_bytes(const fnx_engine* e) { return e ? e->bytes : 0; }

extern "C" void* fnx_engine_tensor(fnx_engine* e, const char* name, size_t* bytes) {
    if (bytes) *bytes = 0;
    if (!e || !name) return nullptr;
    auto it = e->tensors.find(name);
    if (it == e->tensors.end()) return nullptr;
    if (bytes) *bytes = it->second.second;
    return it->second.first;
}

extern "C" int fnx_engine_reset(fnx_engine* e, int seq) {
    FNX_REQUIRE(e && seq >= 0 && seq < e->c.n_seq, "fnx_engine_reset: sequence %d", seq);
    const Dims d = dims(e->c);
    e->seqs[seq] = SeqState{};
    FNX_CUDA_OK(cudaMemsetAsync(e->d_pos + seq, 0, sizeof(int), e->st));
    FNX_CUDA_OK(cudaMemsetAsync(e->d_cur + seq, 0, sizeof(int), e->st));
    FNX_CUDA_OK(cudaMemsetAsync(e->d_ctx_n + seq, 0, sizeof(int), e->st));
    for (LayerW& L : e->layers)
        if (!L.attn) {
            FNX_CUDA_OK(cudaMemsetAsync(L.S_pool + (size_t) seq * e->NS * d.nv * d.hs * d.hs, 0, sizeof(float) * e->NS * d.nv * d.hs * d.hs, e->st));
            FNX_CUDA_OK(cudaMemsetAsync(L.hist_pool + (size_t) seq * e->NS * 3 * d.gdn_ch, 0, sizeof(float) * e->NS * 3 * d.gdn_ch, e->st));
        }
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    return FNX_OK;
}

extern "C" int fnx_engine_verify(fnx_engine* e, int seq, const int* h_tok, const int* h_parent, int T, int* h_result) {
    FNX_REQUIRE(e && h_tok && seq >= 0 && seq < e->c.n_seq, "fnx_engine_verify: bad arguments");
    FNX_REQUIRE(T >= 1 && T <= e->c.max_rows, "fnx_engine_verify: %d rows (1..%d)", T, e->c.max_rows);
    SeqState& s = e->seqs[seq];
    FNX_REQUIRE(s.pos + T <= e->c.max_ctx, "fnx_engine_verify: the window runs past the context of %d rows", e->c.max_ctx);
    for (int t = 0; t < T; ++t) {
        FNX_REQUIRE(h_tok[t] >= 0 && h_tok[t] < e->c.vocab, "fnx_engine_verify: token %d outside the vocabulary", h_tok[t]);
        if (h_parent) FNX_REQUIRE(h_parent[t] < t && h_parent[t] >= (t == 0 ? -1 : 0), "fnx_engine_verify: parent[%d] = %d is not an earlier row", t, h_parent[t]);
    }
    const bool tree = h_parent != nullptr;
    FNX_REQUIRE(!(tree && e->sampling_on), "fnx_engine_verify: the sampling rule is defined on chains (parent must be null)");
    FNX_REQUIRE(!(tree && e->rules_on && e->rules.last_n > 0), "fnx_engine_verify: penalty windows are defined on chains (parent must be null)");
    // the previous call's use of the staging buffer is over: every call that copies results back synchronises
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    // the device error word reports THIS window: whatever an earlier window left was returned with its result (or is
    // still readable through fnx_engine_error_bits until now)
    FNX_CUDA_OK(cudaMemsetAsync(e->err, 0, sizeof(unsigned), e->st));
    int* hs = e->h_stage;
    memcpy(hs, h_tok, sizeof(int) * T);
    FNX_CUDA_OK(cudaMemcpyAsync(e->d_tok, hs, sizeof(int) * T, cudaMemcpyHostToDevice, e->st));
    if (h_parent) {
        memcpy(hs + FNX_MAX_ROWS, h_parent, sizeof(int) * T);
        FNX_CUDA_OK(cudaMemcpyAsync(e->d_parent, hs + FNX_MAX_ROWS, sizeof(int) * T, cudaMemcpyHostToDevice, e->st));
    }
    if (e->sampling_on) {   // the window's Philox step is a host count: a window replayed or run twice draws the same uniforms
        hs[2 * FNX_MAX_ROWS] = (int) s.step++;
        FNX_CUDA_OK(cudaMemcpyAsync(e->d_step + seq, hs + 2 * FNX_MAX_ROWS, sizeof(int), cudaMemcpyHostToDevice, e->st));
    }
    const uint64_t key = ((uint64_t) 1 << 60) | ((uint64_t) seq << 20) | ((uint64_t) T << 1) | (tree ? 1 : 0);
    FNX_TRY(run_graph(e, key, [&]() { return enqueue_verify(e, seq, T, tree); }));
    s.last_T = T;
    e->last_seq = seq;
    e->lane_seqs.clear();
    if (h_result) {
        FNX_CUDA_OK(cudaMemcpyAsync(hs + 2 * FNX_MAX_ROWS, e->result, sizeof(int) * (1 + 2 * FNX_MAX_ROWS), cudaMemcpyDeviceToHost, e->st));
        FNX_CUDA_OK(cudaMemcpyAsync(hs + 5 * FNX_MAX_ROWS, e->err, sizeof(unsigned), cudaMemcpyDeviceToHost, e->st));
        FNX_CUDA_OK(cudaStreamSynchronize(e->st));
        FNX_CUDA_OK(cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1));
        memcpy(h_result, hs + 2 * FNX_MAX_ROWS, sizeof(int) * (1 + 2 * FNX_MAX_ROWS));
        const unsigned bits = (unsigned) hs[5 * FNX_MAX_ROWS];
        if (bits) return fail(FNX_E_STATE, "verify: device error bits 0x%x (1: a bounded wait gave up, 2: non-finite value, 16: non-finite logits)", bits);
    }
    return FNX_OK;
}

extern "C" int fnx_engine_set_sampling(fnx_engine* e, const fnx_sampling* s, uint64_t seed) {
    FNX_REQUIRE(e, "fnx_engine_set_sampling: null engine");
    FNX_REQUIRE(!s || s->temperature > 0.f, "fnx_engine_set_sampling: temperature %g (null selects greedy windows)", s ? (double) s->temperature : 0.0);
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    e->sampling_on = s != nullptr;
    if (s) e->sampling = *s;
    e->sample_seed = seed;
    FNX_CUDA_OK(cudaMemset(e->d_step, 0, sizeof(uint32_t) * e->c.n_seq));
    for (SeqState& q : e->seqs) q.step = 0;
    for (auto& g : e->graphs) cudaGraphExecDestroy(g.second);   // the rule is part of the captured windows
    e->graphs.clear();
    return FNX_OK;
}

extern "C" int fnx_engine_set_logit_rules(fnx_engine* e, const fnx_logit_rules* r) {
    FNX_REQUIRE(e, "fnx_engine_set_logit_rules: null engine");
    if (r) {
        FNX_REQUIRE(r->last_n >= 0 && r->last_n <= FNX_PENALTY_CAP, "fnx_engine_set_logit_rules: a penalty window of %d tokens (0..%d)", r->last_n, FNX_PENALTY_CAP);
        FNX_REQUIRE(r->last_n == 0 || (r->repeat > 0.f && std::isfinite(r->repeat) && std::isfinite(r->freq) && std::isfinite(r->present)),
                    "fnx_engine_set_logit_rules: penalties %g, %g, %g (repeat > 0, all finite)", (double) r->repeat, (double) r->freq, (double) r->present);
        FNX_REQUIRE(r->bias_n >= 0 && (r->bias_n == 0 || (r->bias_tok && r->bias_val)), "fnx_engine_set_logit_rules: a bias list of %d entries without its arrays", r->bias_n);
        for (int i = 0; i < r->bias_n; ++i)
            FNX_REQUIRE(r->bias_tok[i] >= 0 && r->bias_tok[i] < e->c.vocab && std::isfinite(r->bias_val[i]), "fnx_engine_set_logit_rules: bias entry %d (token %d)", i, r->bias_tok[i]);
    }
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    e->rules_on = r != nullptr && (r->last_n > 0 || r->bias_n > 0);
    if (e->rules_on) {
        e->rules = *r;
        if (r->bias_n > e->bias_cap) {   // the lists live on the device: the captured windows read them there
            if (e->d_bias_tok) cudaFree(e->d_bias_tok);
            if (e->d_bias_val) cudaFree(e->d_bias_val);
            e->d_bias_tok = nullptr;
            e->d_bias_val = nullptr;
            e->bias_cap = 0;
            FNX_CUDA_OK(cudaMalloc((void**) &e->d_bias_tok, sizeof(int) * (size_t) r->bias_n));
            FNX_CUDA_OK(cudaMalloc((void**) &e->d_bias_val, sizeof(float) * (size_t) r->bias_n));
            e->bias_cap = r->bias_n;
        }
        if (r->bias_n > 0) {
            FNX_CUDA_OK(cudaMemcpy(e->d_bias_tok, r->bias_tok, sizeof(int) * (size_t) r->bias_n, cudaMemcpyHostToDevice));
            FNX_CUDA_OK(cudaMemcpy(e->d_bias_val, r->bias_val, sizeof(float) * (size_t) r->bias_n, cudaMemcpyHostToDevice));
        }
        e->rules.bias_tok = nullptr;   // the caller's arrays are not kept
        e->rules.bias_val = nullptr;
    }
    for (auto& g : e->graphs) cudaGraphExecDestroy(g.second);   // the rules are part of the captured windows
    e->graphs.clear();
    return FNX_OK;
}

extern "C" int fnx_engine_lookup(fnx_engine* e, int seq, int lk, int d1, int root, int* h_out, int* h_n) {
    FNX_REQUIRE(e && h_out && h_n && seq >= 0 && seq < e->c.n_seq && lk >= 0 && lk <= FNX_MAX_ROWS, "fnx_engine_lookup: bad arguments");
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    int* hs = e->h_stage;
    int* out_n = e->d_lk + FNX_MAX_ROWS;
    const int* d1p = nullptr;
    if (d1 >= 0) {
        hs[0] = d1;
        FNX_CUDA_OK(cudaMemcpyAsync(e->d_lk + FNX_MAX_ROWS + 2, hs, sizeof(int), cudaMemcpyHostToDevice, e->st));
        d1p = e->d_lk + FNX_MAX_ROWS + 2;
    }
    // the context holds the committed tokens followed by the pending one (the next window's first row): both count;
    // a caller that will start the next window from another token says so (root >= 0)
    if (root >= 0) {
        FNX_REQUIRE(root < e->c.vocab, "fnx_engine_lookup: root token %d outside the vocabulary", root);
        hs[1] = root;
        FNX_CUDA_OK(cudaMemcpyAsync(e->d_ctx + (size_t) seq * e->cache_rows + e->seqs[seq].pos, hs + 1, sizeof(int), cudaMemcpyHostToDevice, e->st));
    }
    k_plus_one<<<1, 1, 0, e->st>>>(e->d_lk + FNX_MAX_ROWS + 3, e->d_ctx_n + seq);
    FNX_LAUNCH_OK("k_plus_one");
    FNX_TRY(fnx_lookup_draft(e->d_ctx + (size_t) seq * e->cache_rows, e->d_lk + FNX_MAX_ROWS + 3, lk, d1p, e->d_lk, out_n, e->st));
    FNX_CUDA_OK(cudaMemcpyAsync(hs + 8, e->d_lk, sizeof(int) * (FNX_MAX_ROWS + 2), cudaMemcpyDeviceToHost, e->st));
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    *h_n = hs[8 + FNX_MAX_ROWS];
    memcpy(h_out, hs + 8, sizeof(int) * (*h_n));
    return FNX_OK;
}

// Engine::prefill (engine/src/prefill.cu: the prompt pass): the prompt's first n - 1 tokens go through the model a chunk at a time,
// layer by layer, on the prompt-sized kernels - projections and experts on the tensor cores (fnx_dense_prompt, fnx_moe_prefill),
// DeltaNet as one scan with the state in registers (fnx_gdn_prompt), attention over twelve rows per block (fnx_attn_prompt), the
// router over all rows at once (fnx_router_rows) - and only caches, states and context are kept; the last token then goes through an ordinary one-row window,
// which leaves the engine exactly as after a verify + commit (logits, emitted token, the draft layer's source row).
extern "C" int fnx_engine_prompt(fnx_engine* e, int seq, const int* h_tok, int n) {
    FNX_REQUIRE(e && h_tok && seq >= 0 && seq < e->c.n_seq && n >= 1, "fnx_engine_prompt: bad arguments");
    FNX_REQUIRE(e->c.ep_size == 1, "fnx_engine_prompt: the prompt pass runs on one rank (expert-parallel ranks read prompts through windows)");
    SeqState& s = e->seqs[seq];
    FNX_REQUIRE(s.pos + n <= e->c.max_ctx, "fnx_engine_prompt: %d tokens run past the context of %d rows", n, e->c.max_ctx);
    for (int t = 0; t < n; ++t) FNX_REQUIRE(h_tok[t] >= 0 && h_tok[t] < e->c.vocab, "fnx_engine_prompt: token %d outside the vocabulary", h_tok[t]);
    const Dims d = dims(e->c);
    if (!e->pR) {   // the chunk: large enough that an expert's rows fill the 256-row tiles of the grouped product, within the context
        if (const char* pc = getenv("FNX_PROMPT_CHUNK")) e->prompt_chunk = atoi(pc) > 0 ? atoi(pc) : e->prompt_chunk;
        if (const char* pm = getenv("FNX_ATTN_PROMPT_MMA")) e->prompt_attn_mma_sync = atoi(pm) != 0;
        if (e->prompt_chunk > e->c.max_ctx) e->prompt_chunk = e->c.max_ctx;
    }
    const int CH = e->prompt_chunk, fast = n - 1;
    if (fast > 0 && !e->pR) {
        const int mixw = d.nq * d.hd > d.nv * d.hs ? d.nq * d.hd : d.nv * d.hs;
        FNX_TRY(dalloc(e, &e->pR, (size_t) CH * d.H));
        FNX_TRY(dalloc(e, &e->pproj, (size_t) CH * e->proj_ld));
        FNX_TRY(dalloc(e, &e->pmix, (size_t) CH * mixw));
        FNX_TRY(dalloc(e, &e->plogits, (size_t) CH * (d.E + 1)));
        FNX_TRY(dalloc(e, &e->ptopw, (size_t) CH * d.K));
        FNX_TRY(dalloc(e, &e->ptopi, (size_t) CH * d.K));
        FNX_TRY(dalloc(e, &e->d_ptok, (size_t) CH));
        uint8_t* q = nullptr;
        FNX_TRY(dalloc(e, &q, fnx_moe_prefill_scratch_bytes(CH, d.K, d.E, d.H, d.F)));
        e->p_moe_scratch = q;
        {   // the largest of the layers' input projections (rows x H) and output projections (H x mixer width)
            const int in_rows = d.attn_in > d.gdn_in ? d.attn_in : d.gdn_in;
            const size_t a = fnx_dense_prompt_scratch_bytes(CH, in_rows, d.H), b = fnx_dense_prompt_scratch_bytes(CH, d.H, mixw);
            FNX_TRY(dalloc(e, &q, a > b ? a : b));
        }
        e->p_dense_scratch = q;
        FNX_TRY(dalloc(e, &q, fnx_router_rows_scratch_bytes(CH, d.E, d.H)));
        e->p_router_scratch = q;
        FNX_TRY(dalloc(e, &q, fnx_gdn_prompt_scratch_bytes(CH, d.nk, d.nv, d.hs)));
        e->p_gdn_scratch = q;
        FNX_TRY(dalloc(e, &q, fnx_attn_prompt_scratch_bytes(CH, d.nq, d.hd)));
        e->p_attn_scratch = q;
    }
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    FNX_CUDA_OK(cudaMemsetAsync(e->err, 0, sizeof(unsigned), e->st));
    // FNX_PROMPT_PHASES=1: the device time of each kind of phase, summed over the prompt, to stderr (a tracing aid)
    const bool phases = getenv("FNX_PROMPT_PHASES") != nullptr || e->prompt_timing;
    if (phases)
        for (float& v : e->prompt_phase_ms) v = 0.f;
    enum { PH_INPROJ, PH_ATTN, PH_GDN, PH_OUTPROJ, PH_ROUTER, PH_MOE, PH_N };
    static const char* const ph_name[PH_N] = {"in-proj", "attention", "deltanet", "out-proj", "router", "experts"};
    std::vector<std::pair<int, std::pair<cudaEvent_t, cudaEvent_t>>> marks;
    auto mark = [&](int ph, bool begin) {
        if (!phases) return;
        cudaEvent_t ev;
        cudaEventCreate(&ev);
        cudaEventRecord(ev, e->st);
        if (begin) marks.push_back({ph, {ev, nullptr}});
        else marks.back().second.second = ev;
    };
    for (int c0 = 0; c0 < fast; c0 += CH) {
        const int nt = fast - c0 < CH ? fast - c0 : CH;
        FNX_CUDA_OK(cudaMemcpyAsync(e->d_ptok, h_tok + c0, sizeof(int) * nt, cudaMemcpyHostToDevice, e->st));
        FNX_TRY(fnx_embed_rows(e->embed, e->d_ptok, nt, d.H, e->pR, e->st));
        for (size_t l = 0; l < e->layers.size(); ++l) {
            const LayerW& L = e->layers[l];
            e->launches += 3 + (L.attn ? 3 : 3) + 3 + 2 + 7;   // this layer's kernels: projections 3 + 3, mixer 3, router 2, experts 7
            mark(PH_INPROJ, true);
            FNX_TRY(fnx_dense_prompt(L.w_in, L.in_rows, d.H, e->pR, nt, L.norm1, e->c.eps, e->pproj, e->proj_ld, 0, e->p_dense_scratch, e->err, e->st));
            mark(PH_INPROJ, false);
            mark(L.attn ? PH_ATTN : PH_GDN, true);
            int mixw_l;
            if (L.attn) {
                mixw_l = d.nq * d.hd;
                __half* kc = L.kc + (size_t) seq * e->cache_rows * d.kv_rows;
                __half* vc = L.vc + (size_t) seq * e->cache_rows * d.kv_rows;
                float* qg = e->pproj;
                float* k = qg + d.q_rows;
                float* v = k + d.kv_rows;
                FNX_TRY(fnx_attn_prep_append(qg, e->proj_ld, k, e->proj_ld, v, e->proj_ld, L.qn, L.kn, kc, vc, nt, d.nq, d.nkv, d.hd, d.nrot, e->d_pos + seq, nullptr,
                                             e->c.eps, e->c.rope_base, e->st));
                FNX_TRY(fnx_attn_prompt(qg, e->proj_ld, kc, vc, e->pmix, nt, d.nq, d.nkv, d.hd, e->d_pos + seq, e->p_attn_scratch, e->err, e->prompt_attn_mma_sync, e->st));
            } else {
                mixw_l = d.nv * d.hs;
                float* S = L.S_pool + (size_t) seq * e->NS * d.nv * d.hs * d.hs;
                float* hist = L.hist_pool + (size_t) seq * e->NS * 3 * d.gdn_ch;
                FNX_TRY(fnx_gdn_prompt(e->pproj, e->proj_ld, e->pproj + d.gdn_ch + d.nv * d.hs, e->proj_ld, hist, L.convw, L.dt, L.a, L.gnorm, S, s.cur, e->NS, e->pmix,
                                       d.nk, d.nv, d.hs, nt, e->c.eps, e->p_gdn_scratch, e->st));
            }
            mark(0, false);
            mark(PH_OUTPROJ, true);
            FNX_TRY(fnx_dense_prompt(L.w_out, d.H, mixw_l, e->pmix, nt, nullptr, e->c.eps, e->pR, d.H, 1, e->p_dense_scratch, e->err, e->st));
            mark(0, false);
            mark(PH_ROUTER, true);
            FNX_TRY(fnx_router_rows(L.wr, e->pR, L.norm2, e->c.eps, nt, d.E, d.H, d.K, e->plogits, e->ptopi, e->ptopw, e->p_router_scratch, e->err, e->st));
            mark(0, false);
            mark(PH_MOE, true);
            FNX_TRY(fnx_moe_prefill(L.wgu, e->gu_bytes, L.wdn, e->dn_bytes, L.wsh_gu, L.wsh_dn, 0, d.E, d.K, 0, d.E, 1, e->ptopi, e->ptopw, e->plogits, e->pR, L.norm2,
                                    e->c.eps, nt, d.H, d.F, e->pR, 1, e->p_moe_scratch, e->err, e->st));
            mark(0, false);
        }
        if (phases) {
            FNX_CUDA_OK(cudaStreamSynchronize(e->st));
            float sum[PH_N] = {0};
            for (auto& m : marks) {
                float ms = 0.f;
                cudaEventElapsedTime(&ms, m.second.first, m.second.second);
                sum[m.first] += ms;
                cudaEventDestroy(m.second.first);
                cudaEventDestroy(m.second.second);
            }
            marks.clear();
            for (int i = 0; i < PH_N; ++i) e->prompt_phase_ms[i] += sum[i];
            if (getenv("FNX_PROMPT_PHASES")) {
                fprintf(stderr, "prompt chunk at %d (%d rows):", s.pos, nt);
                for (int i = 0; i < PH_N; ++i) fprintf(stderr, " %s %.1f ms", ph_name[i], sum[i]);
                fprintf(stderr, "\n");
            }
        }
        k_prompt_context<<<(nt + 255) / 256, 256, 0, e->st>>>(e->d_ctx + (size_t) seq * e->cache_rows, e->d_ctx_n + seq, e->d_ptok, nt);
        FNX_LAUNCH_OK("prompt context");
        k_prompt_advance<<<1, 1, 0, e->st>>>(e->d_pos + seq, e->d_cur + seq, e->d_ctx_n + seq, nt, e->NS);
        FNX_LAUNCH_OK("prompt advance");
        e->launches += 3;   // embedding, context, advance
        FNX_CUDA_OK(cudaStreamSynchronize(e->st));   // the token copy's source and the chunk buffers are free again
        s.pos += nt;
        s.cur = (s.cur + nt) % e->NS;
    }
    s.kept = 0;
    s.last_T = 0;
    if (fast > 0) {   // what the chunks' kernels reported (the window below starts the word afresh)
        unsigned bits = 0;
        FNX_CUDA_OK(cudaMemcpy(&bits, e->err, sizeof bits, cudaMemcpyDeviceToHost));
        if (bits) return fail(FNX_E_STATE, "fnx_engine_prompt: device error bits 0x%x", bits);
    }
    // the last token: an ordinary window of one row, kept
    const int zero = 0;
    FNX_TRY(fnx_engine_verify(e, seq, h_tok + n - 1, nullptr, 1, nullptr));
    return fnx_engine_commit(e, seq, &zero, 1);
}

extern "C" int fnx_engine_prompt_timing(fnx_engine* e, int on, float* h_phase_ms6) {
    FNX_REQUIRE(e, "fnx_engine_prompt_timing: null engine");
    e->prompt_timing = on != 0;
    if (h_phase_ms6) memcpy(h_phase_ms6, e->prompt_phase_ms, sizeof e->prompt_phase_ms);
    return FNX_OK;
}

extern "C" int fnx_engine_commit(fnx_engine* e, int seq, const int* h_path, int n) {
    FNX_REQUIRE(e && h_path && seq >= 0 && seq < e->c.n_seq, "fnx_engine_commit: bad arguments");
    SeqState& s = e->seqs[seq];
    FNX_REQUIRE(s.last_T > 0, "fnx_engine_commit: no verified window to commit");
    FNX_REQUIRE(seq == e->last_seq, "fnx_engine_commit: sequence %d, but the window buffers hold sequence %d's window (commit before verifying another sequence)", seq,
                e->last_seq);
    FNX_REQUIRE(n >= 1 && n <= s.last_T && h_path[0] == 0, "fnx_engine_commit: %d rows of a window of %d (the first kept row is row 0)", n, s.last_T);
    for (int j = 1; j < n; ++j) FNX_REQUIRE(h_path[j] > h_path[j - 1] && h_path[j] < s.last_T, "fnx_engine_commit: path[%d] = %d is not increasing", j, h_path[j]);
    const Dims d = dims(e->c);
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    int* hs = e->h_stage;
    memcpy(hs, h_path, sizeof(int) * n);
    FNX_CUDA_OK(cudaMemcpyAsync(e->d_path, hs, sizeof(int) * n, cudaMemcpyHostToDevice, e->st));
    // device tables of the attention layers' caches for this sequence (built once per sequence)
    auto& tables = e->commit_tables;
    const int key = seq;
    if (!tables.count(key)) {
        std::vector<__half*> ks, vs;
        for (LayerW& L : e->layers)
            if (L.attn) {
                ks.push_back(L.kc + (size_t) seq * e->cache_rows * d.kv_rows);
                vs.push_back(L.vc + (size_t) seq * e->cache_rows * d.kv_rows);
            }
        __half **dk = nullptr, **dv = nullptr;
        FNX_TRY(dalloc(e, &dk, ks.size() + 1));
        FNX_TRY(dalloc(e, &dv, vs.size() + 1));
        FNX_CUDA_OK(cudaMemcpy(dk, ks.data(), sizeof(__half*) * ks.size(), cudaMemcpyHostToDevice));
        FNX_CUDA_OK(cudaMemcpy(dv, vs.data(), sizeof(__half*) * vs.size(), cudaMemcpyHostToDevice));
        tables[key] = {dk, dv};
    }
    int nattn = 0;
    for (LayerW& L : e->layers) nattn += L.attn;
    k_commit<<<nattn + 1, 256, 0, e->st>>>(tables[key].first, tables[key].second, nattn, d.kv_rows, e->d_path, e->d_tok, e->result + 1 + FNX_MAX_ROWS, n,
                                           e->d_pos + seq, e->d_cur + seq, e->NS, e->d_ctx + (size_t) seq * e->cache_rows, e->d_ctx_n + seq);
    FNX_LAUNCH_OK("commit");
    k_advance_pos<<<1, 1, 0, e->st>>>(e->d_pos + seq, n);
    FNX_LAUNCH_OK("commit (position)");
    s.kept = n;
    s.kept_pos0 = s.pos;
    s.cur = (s.cur + 1 + h_path[n - 1]) % e->NS;
    s.pos += n;
    s.last_T = 0;
    return FNX_OK;
}

extern "C" int fnx_engine_draft(fnx_engine* e, int seq, int k, int* h_drafts) {
    FNX_REQUIRE(e && h_drafts && seq >= 0 && seq < e->c.n_seq && k >= 1 && k < e->c.max_rows, "fnx_engine_draft: bad arguments");
    SeqState& s = e->seqs[seq];
    FNX_REQUIRE(s.kept >= 1, "fnx_engine_draft: nothing committed since the last draft");
    FNX_REQUIRE(seq == e->last_seq, "fnx_engine_draft: sequence %d, but the window buffers hold sequence %d's last window", seq, e->last_seq);
    const Dims d = dims(e->c);
    const int n = s.kept;
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    int* hs = e->h_stage;
    hs[0] = s.kept_pos0;
    FNX_CUDA_OK(cudaMemcpyAsync(e->d_mpos_base, hs, sizeof(int), cudaMemcpyHostToDevice, e->st));
    // The whole chain is one graph: the first call on the kept rows of the main model (gathered by path) with the tokens
    // the window emitted, then k - 1 single-row calls, each from the draft layer's own last row and the previous draft;
    // tokens and positions advance on the device, the k drafts come back in one copy.
    auto mtp_call = [&](int T, int* out) -> int {
        FNX_TRY(enqueue_mtp(e, seq, T, e->Rsrc));
        return fnx_argmax_mapped(e->logits, 1, e->dvn, e->d_dvocab, out, nullptr, e->err, e->st);
    };
    auto chain = [&]() -> int {
        // (the chain advances the position as it goes: it starts from a copy, so that running it again gives the same result)
        FNX_CUDA_OK(cudaMemcpyAsync(e->d_mpos, e->d_mpos_base, sizeof(int), cudaMemcpyDeviceToDevice, e->st));
        k_gather_rows<<<dim3((d.H + 255) / 256, n), 256, 0, e->st>>>(e->Rsrc, e->R, e->d_path, d.H);
        FNX_LAUNCH_OK("draft gather");
        FNX_CUDA_OK(cudaMemcpyAsync(e->d_mtok, e->result + 1 + FNX_MAX_ROWS, sizeof(int) * n, cudaMemcpyDeviceToDevice, e->st));
        FNX_TRY(mtp_call(n, e->d_drafts));
        for (int j = 1; j < k; ++j) {
            const int src_row = j == 1 ? n - 1 : 0;
            FNX_CUDA_OK(cudaMemcpyAsync(e->Rsrc, e->Rm + (size_t) src_row * d.H, sizeof(float) * d.H, cudaMemcpyDeviceToDevice, e->st));
            FNX_CUDA_OK(cudaMemcpyAsync(e->d_mtok, e->d_drafts + (j - 1), sizeof(int), cudaMemcpyDeviceToDevice, e->st));
            k_advance_pos<<<1, 1, 0, e->st>>>(e->d_mpos, j == 1 ? n : 1);
            FNX_LAUNCH_OK("draft position");
            FNX_TRY(mtp_call(1, e->d_drafts + j));
        }
        return FNX_OK;
    };
    FNX_TRY(run_graph(e, ((uint64_t) 3 << 60) | ((uint64_t) seq << 20) | ((uint64_t) k << 8) | (uint64_t) n, chain));
    FNX_CUDA_OK(cudaMemcpyAsync(hs + 8, e->d_drafts, sizeof(int) * k, cudaMemcpyDeviceToHost, e->st));
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    FNX_CUDA_OK(cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1));
    memcpy(h_drafts, hs + 8, sizeof(int) * k);
    s.kept = 0;
    return FNX_OK;
}

extern "C" float fnx_engine_last_ms(const fnx_engine* e) { return e ? e->last_ms : 0.f; }
extern "C" int fnx_engine_error_bits(fnx_engine* e, unsigned* h_bits) {
    FNX_REQUIRE(e && h_bits, "fnx_engine_error_bits: null pointer");
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    FNX_CUDA_OK(cudaMemcpy(h_bits, e->err, sizeof(unsigned), cudaMemcpyDeviceToHost));
    return FNX_OK;
}

extern "C" int fnx_engine_counters(fnx_engine* e, unsigned long long* h_out3) {
    FNX_REQUIRE(e && h_out3, "fnx_engine_counters: null pointer");
    unsigned long long st[2] = {0, 0};
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    FNX_CUDA_OK(cudaMemcpy(st, e->d_stats, sizeof st, cudaMemcpyDeviceToHost));
    h_out3[0] = e->launches;
    h_out3[1] = st[0];
    h_out3[2] = st[1];
    return FNX_OK;
}
extern "C" int fnx_engine_pos(const fnx_engine* e, int seq) { return e && seq >= 0 && seq < e->c.n_seq ? e->seqs[seq].pos : -1; }
extern "C" fnx_stream fnx_engine_stream(fnx_engine* e) { return e ? (fnx_stream) e->st : nullptr; }

extern "C" int fnx_engine_config(const fnx_engine* e, fnx_model_config* out) {
    FNX_REQUIRE(e && out, "fnx_engine_config: null argument");
    *out = e->c;
    return FNX_OK;
}

extern "C" int fnx_comm_unique_id(void* h_id128) {
    FNX_REQUIRE(h_id128, "fnx_comm_unique_id: null pointer");
    Nccl* n = nccl();
    if (!n) return fail(FNX_E_UNAVAILABLE, "NCCL (libnccl.so.2) could not be loaded");
    const int rc = n->GetUniqueId(h_id128);
    if (rc) return fail(FNX_E_CUDA, "ncclGetUniqueId: %s", n->GetErrorString ? n->GetErrorString(rc) : "error");
    return FNX_OK;
}

extern "C" int fnx_engine_comm_init(fnx_engine* e, const void* h_id128, int rank, int size) {
    FNX_REQUIRE(e && h_id128 && rank == e->c.ep_rank && size == e->c.ep_size, "fnx_engine_comm_init: rank %d of %d does not match the engine's shard", rank, size);
    Nccl* n = nccl();
    if (!n) return fail(FNX_E_UNAVAILABLE, "NCCL (libnccl.so.2) could not be loaded");
    NcclId id;
    memcpy(id.b, h_id128, 128);
    const int rc = n->CommInitRank(&e->comm, size, id, rank);
    if (rc) return fail(FNX_E_CUDA, "ncclCommInitRank: %s", n->GetErrorString ? n->GetErrorString(rc) : "error");
    return FNX_OK;
}

extern "C" int fnx_engine_ep_handles(fnx_engine* e, void* h_out128) {
    FNX_REQUIRE(e && h_out128 && e->xbuf && e->xflag, "fnx_engine_ep_handles: no expert-parallel engine");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h[2];
    FNX_CUDA_OK(cudaIpcGetMemHandle(&h[0], e->xbuf));
    FNX_CUDA_OK(cudaIpcGetMemHandle(&h[1], e->xflag));
    memcpy(h_out128, h, sizeof h);
    return FNX_OK;
}

extern "C" int fnx_engine_ep_open(fnx_engine* e, const void* h_all, int rank, int size) {
    FNX_REQUIRE(e && h_all && rank == e->c.ep_rank && size == e->c.ep_size && e->xbuf, "fnx_engine_ep_open: rank %d of %d does not match the engine's shard", rank, size);
    FNX_REQUIRE(!e->ep_peers, "fnx_engine_ep_open: already open");
    std::vector<float*> px(size);
    std::vector<unsigned*> pf(size);
    const cudaIpcMemHandle_t* h = (const cudaIpcMemHandle_t*) h_all;
    for (int r = 0; r < size; ++r) {
        if (r == rank) {
            px[r] = e->xbuf;
            pf[r] = e->xflag;
            continue;
        }
        void *a = nullptr, *b = nullptr;
        FNX_CUDA_OK(cudaIpcOpenMemHandle(&a, h[2 * r], cudaIpcMemLazyEnablePeerAccess));
        e->ipc_opened.push_back(a);
        FNX_CUDA_OK(cudaIpcOpenMemHandle(&b, h[2 * r + 1], cudaIpcMemLazyEnablePeerAccess));
        e->ipc_opened.push_back(b);
        px[r] = (float*) a;
        pf[r] = (unsigned*) b;
    }
    FNX_CUDA_OK(cudaMemcpy(e->d_peer_x, px.data(), sizeof(float*) * size, cudaMemcpyHostToDevice));
    FNX_CUDA_OK(cudaMemcpy(e->d_peer_flag, pf.data(), sizeof(unsigned*) * size, cudaMemcpyHostToDevice));
    e->ep_peers = true;
    for (auto& g : e->graphs) cudaGraphExecDestroy(g.second);   // windows captured with the NCCL path are captured again
    e->graphs.clear();
    return FNX_OK;
}

extern "C" int fnx_allreduce(fnx_engine* e, float* x, size_t count, fnx_stream st) {
    FNX_REQUIRE(e && x, "fnx_allreduce: null pointer");
    if (e->c.ep_size == 1) return FNX_OK;
    Nccl* n = nccl();
    if (!n || !e->comm) return fail(FNX_E_STATE, "fnx_allreduce: the communicator is not initialised (fnx_engine_comm_init)");
    // ncclFloat32 = 7, ncclSum = 0
    const int rc = n->AllReduce(x, x, count, 7, 0, e->comm, as_stream(st));
    if (rc) return fail(FNX_E_CUDA, "ncclAllReduce: %s", n->GetErrorString ? n->GetErrorString(rc) : "error");
    return FNX_OK;
}

// ------------------------------------------------------------------------------------------------ batched lanes: API
extern "C" int fnx_engine_verify_lanes(fnx_engine* e, int n_lanes, const int* h_seqs, const int* h_tok, int rows, int* h_results) {
    FNX_REQUIRE(n_lanes >= 1 && n_lanes <= FNX_MAX_ROWS, "fnx_engine_verify_lanes: %d lanes", n_lanes);
    int each[FNX_MAX_ROWS];
    for (int j = 0; j < n_lanes; ++j) each[j] = rows;
    return fnx_engine_verify_lanes_rows(e, n_lanes, h_seqs, each, h_tok, h_results);
}

extern "C" int fnx_engine_verify_lanes_rows(fnx_engine* e, int n_lanes, const int* h_seqs, const int* h_rows, const int* h_tok, int* h_results) {
    FNX_REQUIRE(e && h_seqs && h_rows && h_tok, "fnx_engine_verify_lanes: null pointer");
    FNX_REQUIRE(n_lanes >= 1 && n_lanes <= FNX_MAX_ROWS, "fnx_engine_verify_lanes: %d lanes", n_lanes);
    int T = 0, rows = 0;   // rows in all, the longest lane's
    for (int j = 0; j < n_lanes; ++j) {
        FNX_REQUIRE(h_rows[j] >= 1 && h_rows[j] <= FNX_LANE_ROWS, "fnx_engine_verify_lanes: lane %d has %d rows (1..%d)", j, h_rows[j], FNX_LANE_ROWS);
        FNX_REQUIRE(h_seqs[j] >= 0 && h_seqs[j] < e->c.n_seq, "fnx_engine_verify_lanes: sequence %d", h_seqs[j]);
        for (int i = 0; i < j; ++i) FNX_REQUIRE(h_seqs[i] != h_seqs[j], "fnx_engine_verify_lanes: sequence %d in two lanes", h_seqs[j]);
        FNX_REQUIRE(e->seqs[h_seqs[j]].pos + h_rows[j] <= e->c.max_ctx, "fnx_engine_verify_lanes: sequence %d runs past the context of %d rows", h_seqs[j], e->c.max_ctx);
        for (int t = 0; t < h_rows[j]; ++t)
            FNX_REQUIRE(h_tok[T + t] >= 0 && h_tok[T + t] < e->c.vocab, "fnx_engine_verify_lanes: token %d outside the vocabulary", h_tok[T + t]);
        T += h_rows[j];
        rows = h_rows[j] > rows ? h_rows[j] : rows;
    }
    FNX_REQUIRE(T <= e->c.max_rows, "fnx_engine_verify_lanes: %d rows in all (at most %d)", T, e->c.max_rows);
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    FNX_CUDA_OK(cudaMemsetAsync(e->err, 0, sizeof(unsigned), e->st));
    int* hs = e->h_stage;
    memcpy(hs, h_tok, sizeof(int) * T);
    FNX_CUDA_OK(cudaMemcpyAsync(e->d_tok, hs, sizeof(int) * T, cudaMemcpyHostToDevice, e->st));
    int* ht = hs + FNX_MAX_ROWS;
    for (int j = 0; j < n_lanes; ++j) ht[j] = h_seqs[j];
    ht[FNX_MAX_ROWS] = 0;
    for (int j = 0; j < n_lanes; ++j) ht[FNX_MAX_ROWS + j + 1] = ht[FNX_MAX_ROWS + j] + h_rows[j];
    FNX_CUDA_OK(cudaMemcpyAsync(e->d_lane_seq, ht, sizeof(int) * n_lanes, cudaMemcpyHostToDevice, e->st));
    {   // the table the mixers see on expert-parallel ranks: this rank's own sequences (sequence % ranks == rank)
        int* ho = hs + 5 * FNX_MAX_ROWS;
        for (int j = 0; j < n_lanes; ++j) ho[j] = h_seqs[j] % e->c.ep_size == e->c.ep_rank ? h_seqs[j] : -1;
        FNX_CUDA_OK(cudaMemcpyAsync(e->d_lane_own, ho, sizeof(int) * n_lanes, cudaMemcpyHostToDevice, e->st));
    }
    FNX_CUDA_OK(cudaMemcpyAsync(e->d_lane_row0, ht + FNX_MAX_ROWS, sizeof(int) * (n_lanes + 1), cudaMemcpyHostToDevice, e->st));
    if (e->sampling_on)
        for (int j = 0; j < n_lanes; ++j) {
            ht[3 * FNX_MAX_ROWS + j] = (int) e->seqs[h_seqs[j]].step++;
            FNX_CUDA_OK(cudaMemcpyAsync(e->d_step + h_seqs[j], ht + 3 * FNX_MAX_ROWS + j, sizeof(int), cudaMemcpyHostToDevice, e->st));
        }
    // one graph per layout (each lane's rows): the key is a hash of the counts under the lanes tag
    uint64_t hsh = 1469598103934665603ull;
    for (int j = 0; j < n_lanes; ++j) hsh = (hsh ^ (uint64_t) (h_rows[j] + 8 * j)) * 1099511628211ull;
    const uint64_t key = ((uint64_t) 4 << 60) | ((hsh ^ (uint64_t) n_lanes) & 0x0fffffffffffffffull);
    FNX_TRY(run_graph(e, key, [&]() { return enqueue_verify_lanes(e, n_lanes, rows, T); }));
    e->lane_seqs.assign(h_seqs, h_seqs + n_lanes);
    e->lane_rows.assign(h_rows, h_rows + n_lanes);
    e->last_seq = -1;
    for (int j = 0; j < n_lanes; ++j) e->seqs[h_seqs[j]].last_T = h_rows[j];
    if (h_results) {
        const size_t n = (size_t) n_lanes * (1 + 2 * FNX_MAX_ROWS);
        std::vector<int> tmp(n + 1);
        FNX_CUDA_OK(cudaMemcpyAsync(tmp.data(), e->d_results, sizeof(int) * n, cudaMemcpyDeviceToHost, e->st));
        FNX_CUDA_OK(cudaMemcpyAsync(tmp.data() + n, e->err, sizeof(unsigned), cudaMemcpyDeviceToHost, e->st));
        FNX_CUDA_OK(cudaStreamSynchronize(e->st));
        FNX_CUDA_OK(cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1));
        memcpy(h_results, tmp.data(), sizeof(int) * n);
        if (tmp[n]) return fail(FNX_E_STATE, "verify_lanes: device error bits 0x%x", (unsigned) tmp[n]);
    }
    return FNX_OK;
}

extern "C" int fnx_engine_commit_lanes(fnx_engine* e, int n_lanes, const int* h_seqs, const int* h_keep) {
    FNX_REQUIRE(e && h_seqs && h_keep, "fnx_engine_commit_lanes: null pointer");
    FNX_REQUIRE(n_lanes == (int) e->lane_seqs.size() && n_lanes >= 1, "fnx_engine_commit_lanes: %d lanes, the last lane window had %d", n_lanes, (int) e->lane_seqs.size());
    for (int j = 0; j < n_lanes; ++j) {
        FNX_REQUIRE(h_seqs[j] == e->lane_seqs[j], "fnx_engine_commit_lanes: lane %d is sequence %d in the window, %d here", j, e->lane_seqs[j], h_seqs[j]);
        FNX_REQUIRE(h_keep[j] >= 1 && h_keep[j] <= e->lane_rows[j], "fnx_engine_commit_lanes: lane %d keeps %d of %d rows", j, h_keep[j], e->lane_rows[j]);
    }
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    int* hs = e->h_stage;
    memcpy(hs, h_keep, sizeof(int) * n_lanes);
    FNX_CUDA_OK(cudaMemcpyAsync(e->d_keep, hs, sizeof(int) * n_lanes, cudaMemcpyHostToDevice, e->st));
    k_commit_lanes<<<1, 32, 0, e->st>>>(e->d_lane_seq, e->d_lane_row0, e->d_keep, e->d_tok, e->d_results, e->d_pos, e->d_cur, e->NS, e->d_ctx, (size_t) e->cache_rows,
                                        e->d_ctx_n, n_lanes);
    FNX_LAUNCH_OK("commit lanes");
    for (int j = 0; j < n_lanes; ++j) {
        SeqState& s = e->seqs[h_seqs[j]];
        s.kept = h_keep[j];
        s.kept_pos0 = s.pos;
        s.cur = (s.cur + h_keep[j]) % e->NS;
        s.pos += h_keep[j];
        s.last_T = 0;
    }
    return FNX_OK;
}

extern "C" int fnx_engine_draft_lanes(fnx_engine* e, int n_lanes, const int* h_seqs, int k, int* h_drafts) {
    FNX_REQUIRE(e && h_seqs && h_drafts && k >= 1 && k < e->c.max_rows, "fnx_engine_draft_lanes: bad arguments");
    FNX_REQUIRE(n_lanes == (int) e->lane_seqs.size() && n_lanes >= 1, "fnx_engine_draft_lanes: %d lanes, the last lane window had %d", n_lanes, (int) e->lane_seqs.size());
    const Dims d = dims(e->c);
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    int* hs = e->h_stage;
    int Tm = 0, maxn = 0;
    for (int j = 0; j < n_lanes; ++j) {
        FNX_REQUIRE(h_seqs[j] == e->lane_seqs[j], "fnx_engine_draft_lanes: lane %d is sequence %d in the window, %d here", j, e->lane_seqs[j], h_seqs[j]);
        const SeqState& s = e->seqs[h_seqs[j]];
        FNX_REQUIRE(s.kept >= 1, "fnx_engine_draft_lanes: sequence %d: nothing committed since the last draft", h_seqs[j]);
        hs[j] = Tm;
        Tm += s.kept;
        maxn = s.kept > maxn ? s.kept : maxn;
        hs[FNX_MAX_ROWS + 1 + j] = s.kept_pos0;
    }
    hs[n_lanes] = Tm;
    for (int j = 0; j <= n_lanes; ++j) hs[2 * FNX_MAX_ROWS + 2 + j] = j;
    FNX_CUDA_OK(cudaMemcpyAsync(e->d_mlane_row0, hs, sizeof(int) * (n_lanes + 1), cudaMemcpyHostToDevice, e->st));
    FNX_CUDA_OK(cudaMemcpyAsync(e->d_ident_row0, hs + 2 * FNX_MAX_ROWS + 2, sizeof(int) * (n_lanes + 1), cudaMemcpyHostToDevice, e->st));
    FNX_CUDA_OK(cudaMemcpyAsync(e->d_mpos_base, hs + FNX_MAX_ROWS + 1, sizeof(int) * n_lanes, cudaMemcpyHostToDevice, e->st));
    // one graph for the whole chain: the first call on every lane's kept rows, then k - 1 calls of one row per lane
    auto chain = [&]() -> int {
        // (the chain advances the lanes' positions as it goes: it starts from a copy, so that running it again gives the same result)
        k_mtp_set_pos_lanes<<<1, 32, 0, e->st>>>(e->d_mpos_seq, e->d_lane_seq, e->d_mpos_base, n_lanes);
        FNX_LAUNCH_OK("draft positions (lanes)");
        k_mtp_gather_lanes<<<dim3((d.H + 255) / 256, Tm), 256, 0, e->st>>>(e->Rsrc, e->R, e->d_mtok, e->d_results, e->d_lane_row0, e->d_mlane_row0, n_lanes, d.H);
        FNX_LAUNCH_OK("draft gather (lanes)");
        FNX_TRY(enqueue_mtp_lanes(e, n_lanes, Tm, maxn, e->d_mlane_row0, e->Rsrc));
        k_scatter_drafts<<<1, 32, 0, e->st>>>(e->d_ldrafts, e->best_i, n_lanes, k, 0);
        FNX_LAUNCH_OK("draft scatter");
        for (int j = 1; j < k; ++j) {
            // each lane's source row: its draft-layer last row (compact in Rlast), its token: the previous draft
            FNX_CUDA_OK(cudaMemcpyAsync(e->Rsrc, e->Rlast, sizeof(float) * (size_t) n_lanes * d.H, cudaMemcpyDeviceToDevice, e->st));
            FNX_CUDA_OK(cudaMemcpyAsync(e->d_mtok, e->best_i, sizeof(int) * n_lanes, cudaMemcpyDeviceToDevice, e->st));
            k_mtp_advance_lanes<<<1, 32, 0, e->st>>>(e->d_mpos_seq, e->d_lane_seq, e->d_mlane_row0, n_lanes, j == 1 ? 1 : 0);
            FNX_LAUNCH_OK("draft positions (lanes)");
            FNX_TRY(enqueue_mtp_lanes(e, n_lanes, n_lanes, 1, e->d_ident_row0, e->Rsrc));
            k_scatter_drafts<<<1, 32, 0, e->st>>>(e->d_ldrafts, e->best_i, n_lanes, k, j);
            FNX_LAUNCH_OK("draft scatter");
        }
        return FNX_OK;
    };
    // the graph's shape depends on the lanes' kept counts: key on all of them
    uint64_t key = ((uint64_t) 5 << 60) | ((uint64_t) k << 52) | ((uint64_t) n_lanes << 44);
    for (int j = 0; j < n_lanes; ++j) key = key * 1000003ull + (uint64_t) e->seqs[h_seqs[j]].kept;
    key |= (uint64_t) 5 << 60;
    FNX_TRY(run_graph(e, key, chain));
    std::vector<int> tmp((size_t) n_lanes * k);
    FNX_CUDA_OK(cudaMemcpyAsync(tmp.data(), e->d_ldrafts, sizeof(int) * tmp.size(), cudaMemcpyDeviceToHost, e->st));
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    FNX_CUDA_OK(cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1));
    memcpy(h_drafts, tmp.data(), sizeof(int) * tmp.size());
    for (int j = 0; j < n_lanes; ++j) e->seqs[h_seqs[j]].kept = 0;
    return FNX_OK;
}

// A synthetic context for throughput measurements: sequence `seq` is placed at position `pos` as if that many tokens had
// been read (its K/V rows and DeltaNet state keep whatever they hold: fill them through fnx_engine_tensor for a seeded
// stand-in).  Results after this call are a function of that memory, not of a token history.
extern "C" int fnx_engine_set_position(fnx_engine* e, int seq, int pos) {
    FNX_REQUIRE(e && seq >= 0 && seq < e->c.n_seq && pos >= 0 && pos + e->c.max_rows <= e->c.max_ctx, "fnx_engine_set_position: sequence %d at %d", seq, pos);
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    e->seqs[seq].pos = pos;
    FNX_CUDA_OK(cudaMemcpy(e->d_pos + seq, &pos, sizeof(int), cudaMemcpyHostToDevice));
    FNX_CUDA_OK(cudaMemcpy(e->d_ctx_n + seq, &pos, sizeof(int), cudaMemcpyHostToDevice));
    return FNX_OK;
}

// ------------------------------------------------------------------------------------------------ sequence-state cache
// Engine::save_state / load_state (engine/src/engine_common.cu:629-688): a committed sequence's recurrent states, conv histories,
// context tokens and (kv) cache rows, copied to host memory the caller owns, and put back later - into the same sequence (a
// rewind; without kv the engine must still hold the rows' K/V) or another one.  The image holds, after a header, the context
// tokens [0, pos] (the pending one included), then per layer in order: DeltaNet state and history of the current slot; with kv,
// an attention layer's K rows [0, pos) then V rows; the draft layer's cache last.
namespace fnxb {
struct StateHeader {
    uint32_t magic, kv;
    int32_t pos, n_layer, hidden, nv, hs, gdn_ch, kv_rows, has_mtp;
    uint32_t step, pad;
    uint64_t bytes;
};
constexpr uint32_t STATE_MAGIC = 0x53584e46u;   // "FNXS"
// the pieces of sequence `seq` at position pos with state slot cur, in image order: (device pointer, bytes)
static std::vector<std::pair<char*, size_t>> state_pieces(fnx_engine* e, int seq, int pos, int cur, bool kv) {
    const Dims d = dims(e->c);
    std::vector<std::pair<char*, size_t>> v;
    v.push_back({(char*) (e->d_ctx + (size_t) seq * e->cache_rows), sizeof(int) * ((size_t) pos + 1)});
    auto layer = [&](LayerW& L) {
        if (!L.attn) {
            const size_t ssz = (size_t) d.nv * d.hs * d.hs, hsz = (size_t) 3 * d.gdn_ch;
            v.push_back({(char*) (L.S_pool + ((size_t) seq * e->NS + cur) * ssz), ssz * sizeof(float)});
            v.push_back({(char*) (L.hist_pool + ((size_t) seq * e->NS + cur) * hsz), hsz * sizeof(float)});
        } else if (kv && pos > 0) {
            v.push_back({(char*) (L.kc + (size_t) seq * e->cache_rows * d.kv_rows), (size_t) pos * d.kv_rows * sizeof(__half)});
            v.push_back({(char*) (L.vc + (size_t) seq * e->cache_rows * d.kv_rows), (size_t) pos * d.kv_rows * sizeof(__half)});
        }
    };
    for (LayerW& L : e->layers) layer(L);
    layer(e->mtp);
    return v;
}
}  // namespace fnxb

extern "C" size_t fnx_engine_state_bytes(fnx_engine* e, int seq, int kv) {
    if (!e || seq < 0 || seq >= e->c.n_seq) return 0;
    size_t n = sizeof(StateHeader);
    for (const auto& p : state_pieces(e, seq, e->seqs[seq].pos, e->seqs[seq].cur, kv != 0)) n += (p.second + 15) & ~(size_t) 15;
    return n;
}

extern "C" int fnx_engine_save_state(fnx_engine* e, int seq, int kv, void* host, size_t bytes) {
    FNX_REQUIRE(e && host && seq >= 0 && seq < e->c.n_seq, "fnx_engine_save_state: bad arguments");
    SeqState& s = e->seqs[seq];
    FNX_REQUIRE(s.last_T == 0, "fnx_engine_save_state: a window of sequence %d is not committed", seq);
    const size_t need = fnx_engine_state_bytes(e, seq, kv);
    FNX_REQUIRE(bytes >= need, "fnx_engine_save_state: %zu bytes given, %zu needed", bytes, need);
    const Dims d = dims(e->c);
    StateHeader h{};
    h.magic = STATE_MAGIC; h.kv = kv != 0; h.pos = s.pos; h.n_layer = e->c.n_layer; h.hidden = d.H; h.nv = d.nv; h.hs = d.hs; h.gdn_ch = d.gdn_ch;
    h.kv_rows = d.kv_rows; h.has_mtp = 1; h.step = s.step; h.bytes = need;
    memcpy(host, &h, sizeof h);
    char* dst = (char*) host + sizeof h;
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    for (const auto& p : state_pieces(e, seq, s.pos, s.cur, kv != 0)) {
        FNX_CUDA_OK(cudaMemcpyAsync(dst, p.first, p.second, cudaMemcpyDeviceToHost, e->st));
        dst += (p.second + 15) & ~(size_t) 15;
    }
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    return FNX_OK;
}

extern "C" int fnx_engine_load_state(fnx_engine* e, int seq, const void* host, size_t bytes) {
    FNX_REQUIRE(e && host && seq >= 0 && seq < e->c.n_seq && bytes >= sizeof(StateHeader), "fnx_engine_load_state: bad arguments");
    SeqState& s = e->seqs[seq];
    FNX_REQUIRE(s.last_T == 0, "fnx_engine_load_state: a window of sequence %d is not committed", seq);
    StateHeader h;
    memcpy(&h, host, sizeof h);
    const Dims d = dims(e->c);
    FNX_REQUIRE(h.magic == STATE_MAGIC && h.n_layer == e->c.n_layer && h.hidden == d.H && h.nv == d.nv && h.hs == d.hs && h.gdn_ch == d.gdn_ch &&
                    h.kv_rows == d.kv_rows && h.bytes <= bytes,
                "fnx_engine_load_state: a state saved with another layout");
    FNX_REQUIRE(h.pos >= 0 && h.pos + 1 <= e->c.max_ctx, "fnx_engine_load_state: the state (%d rows) does not fit the context", h.pos);
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    const char* src = (const char*) host + sizeof h;
    if (!h.kv) {
        // the engine must still hold the rows' K/V: the sequence has to be a continuation of the saved one
        FNX_REQUIRE(s.pos >= h.pos, "fnx_engine_load_state: a checkpoint without K/V at row %d, the sequence holds %d rows", h.pos, s.pos);
        std::vector<int> have((size_t) h.pos);
        if (h.pos > 0) FNX_CUDA_OK(cudaMemcpy(have.data(), e->d_ctx + (size_t) seq * e->cache_rows, sizeof(int) * (size_t) h.pos, cudaMemcpyDeviceToHost));
        FNX_REQUIRE(h.pos == 0 || memcmp(have.data(), src, sizeof(int) * (size_t) h.pos) == 0,
                    "fnx_engine_load_state: a checkpoint of another sequence (the engine does not hold its K/V)");
    }
    // the state goes to slot 0, which becomes the current one
    const auto pieces = state_pieces(e, seq, h.pos, 0, h.kv != 0);
    size_t total = sizeof h;
    for (const auto& p : pieces) total += (p.second + 15) & ~(size_t) 15;
    FNX_REQUIRE(total == h.bytes, "fnx_engine_load_state: a state saved with another layout (%zu bytes against %llu)", total, (unsigned long long) h.bytes);
    for (const auto& p : pieces) {
        FNX_CUDA_OK(cudaMemcpyAsync(p.first, src, p.second, cudaMemcpyHostToDevice, e->st));
        src += (p.second + 15) & ~(size_t) 15;
    }
    const int zero = 0;
    FNX_CUDA_OK(cudaMemcpyAsync(e->d_pos + seq, &h.pos, sizeof(int), cudaMemcpyHostToDevice, e->st));
    FNX_CUDA_OK(cudaMemcpyAsync(e->d_ctx_n + seq, &h.pos, sizeof(int), cudaMemcpyHostToDevice, e->st));
    FNX_CUDA_OK(cudaMemcpyAsync(e->d_cur + seq, &zero, sizeof(int), cudaMemcpyHostToDevice, e->st));
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    s = SeqState{};
    s.pos = h.pos;
    s.cur = 0;
    s.step = h.step;
    return FNX_OK;
}

extern "C" int fnx_engine_set_wait_limit(fnx_engine* e, unsigned polls) {
    FNX_REQUIRE(e && polls >= 1, "fnx_engine_set_wait_limit: bad arguments");
    FNX_CUDA_OK(cudaStreamSynchronize(e->st));
    e->wait_limit = polls;
    for (auto& g : e->graphs) cudaGraphExecDestroy(g.second);   // the limit is a launch argument of the captured windows
    e->graphs.clear();
    e->graph_kernels.clear();
    return FNX_OK;
}

// Diagnostic: every peer of an expert-parallel engine is mapped to this rank's OWN landing buffer and flags.  The other
// ranks' flags then never arrive, so each window's first exchange runs out its bounded wait, raises FNX_ERR_TIMEOUT and
// returns with the context intact: the way to check, on one GPU and without a fault, that a missing peer cannot hang a rank.
extern "C" int fnx_engine_ep_open_loopback(fnx_engine* e) {
    FNX_REQUIRE(e && e->c.ep_size > 1 && e->xbuf && !e->ep_peers, "fnx_engine_ep_open_loopback: needs an expert-parallel engine whose exchange is not open");
    std::vector<float*> px(e->c.ep_size, e->xbuf);
    std::vector<unsigned*> pf(e->c.ep_size, e->xflag);
    FNX_CUDA_OK(cudaMemcpy(e->d_peer_x, px.data(), sizeof(float*) * px.size(), cudaMemcpyHostToDevice));
    FNX_CUDA_OK(cudaMemcpy(e->d_peer_flag, pf.data(), sizeof(unsigned*) * pf.size(), cudaMemcpyHostToDevice));
    e->ep_peers = true;
    for (auto& g : e->graphs) cudaGraphExecDestroy(g.second);
    e->graphs.clear();
    e->graph_kernels.clear();
    return FNX_OK;
}
