// Drafting and acceptance on the GPU: the 3-gram prompt-lookup drafter, greedy tree acceptance, and speculative
// sampling with Philox uniforms.
//
// The reference does all three on the host: lookup_drafts (engine/src/session.cpp:428-447), the greedy rule
// (:573) and the sampling rule (:575-612, with make_dist :41-75 and draw :77-84) fed by std::mt19937_64.  The rules
// are kept; the uniforms come from Philox4x32-10 addressed by (seed, sequence, step, slot), slots consumed in the
// reference's order, so that a CPU restatement given the same generator reproduces every decision.
#include "fnx_common.cuh"

namespace fnxb {

constexpr int LOOKUP_N = 3, LOOKUP_MIN = 3;   // engine/src/session.cpp:17-18

__global__ void __launch_bounds__(1024) k_lookup(const int* __restrict__ ctx, const int* __restrict__ np, int lk, const int* __restrict__ d1p,
                                                 int* __restrict__ out, int* __restrict__ out_n) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ int red[32];
    const int n = *np, tid = threadIdx.x;
    if (lk == 0 || n <= LOOKUP_N) {
        if (tid == 0) { out_n[0] = 0; out_n[1] = -1; }
        return;
    }
    const int n0 = n - LOOKUP_N;
    const int a = ctx[n0], b = ctx[n0 + 1], c = ctx[n0 + 2];
    int best = -1;
    for (int s = tid; s < n0; s += 1024)
        if (ctx[s] == a && ctx[s + 1] == b && ctx[s + 2] == c) best = s;   // s grows: the last hit is this thread's latest
    for (int o = 16; o; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if ((tid & 31) == 0) red[tid >> 5] = best;
    __syncthreads();
    if (tid != 0) return;
    for (int w = 0; w < 32; ++w) best = max(best, red[w]);
    int cnt = 0, match = -1;
    const int s = best, d1 = d1p ? *d1p : -1;
    if (s >= 0 && s + LOOKUP_N < n && (d1 < 0 || ctx[s + LOOKUP_N] == d1)) {
        int m = LOOKUP_N;
        while (m < lk && (m - LOOKUP_N) < s && ctx[s - 1 - (m - LOOKUP_N)] == ctx[n0 - 1 - (m - LOOKUP_N)]) ++m;
        const int k = min(lk, max(LOOKUP_MIN, m));
        const int end = min(n, s + LOOKUP_N + k);
        for (int i = s + LOOKUP_N; i < end; ++i) out[cnt++] = ctx[i];
        match = s;
    }
    out_n[0] = cnt;
    out_n[1] = match;
}

// result: [0] = n, [1 .. 1 + n) path, [1 + FNX_MAX_ROWS ..) emitted tokens
__device__ __forceinline__ void accept_greedy_walk(const int* __restrict__ tok, const int* __restrict__ parent, const int* __restrict__ best, int T,
                                                   int* __restrict__ result) {
    int cur = 0, n = 0;
    for (;;) {
        result[1 + n] = cur;
        result[1 + FNX_MAX_ROWS + n] = best[cur];
        ++n;
        int next = -1;
        for (int c = cur + 1; c < T; ++c)
            if ((parent ? parent[c] : c - 1) == cur && tok[c] == best[cur]) { next = c; break; }
        if (next < 0) break;
        cur = next;
    }
    result[0] = n;
}

__global__ void k_accept_greedy(const int* __restrict__ tok, const int* __restrict__ parent, const int* __restrict__ best, int T,
                                int* __restrict__ result) {
    pdl_wait();
    pdl_launch_dependents();
    if (threadIdx.x != 0) return;
    accept_greedy_walk(tok, parent, best, T, result);
}

// batched lanes: block j walks lane j's chain (rows [lane_row0[j], lane_row0[j + 1])) into result row j
__global__ void k_accept_greedy_lanes(const int* __restrict__ tok, const int* __restrict__ best, const int* __restrict__ lane_row0, int* __restrict__ result) {
    if (threadIdx.x != 0) return;
    const int lane = blockIdx.x, row0 = lane_row0[lane];
    accept_greedy_walk(tok + row0, nullptr, best + row0, lane_row0[lane + 1] - row0, result + (size_t) lane * (1 + 2 * FNX_MAX_ROWS));
}

struct DistS {
    int n;
    int ids[FNX_TOPK_N];
    double p[FNX_TOPK_N];
};

__device__ __forceinline__ double dist_prob(const int* ids, const double* p, int n, int id) {
    for (int i = 0; i < n; ++i)
        if (ids[i] == id) return p[i];
    return 0.0;
}

// A warp per row builds the row's distribution (make_dist): the exponentials in parallel, the sums in the
// reference's sequential order; then thread 0 walks the chain.
__device__ __forceinline__ void accept_sample_body(const float* __restrict__ cand_v, const int* __restrict__ cand_i, const int* __restrict__ tok, int T,
                                                   fnx_sampling sp, const int* __restrict__ q_ids, const double* __restrict__ q_p,
                                                   const int* __restrict__ q_n, uint64_t seed, uint32_t seq, uint32_t step, int* __restrict__ result,
                                                   uint8_t* smem) {
    DistS* dist = reinterpret_cast<DistS*>(smem);                                  // [T]
    double* ex = reinterpret_cast<double*>(smem + sizeof(DistS) * (size_t) T);     // [T][64] scratch
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int t = warp; t < T; t += 32) {
        const float* cv = cand_v + (size_t) t * FNX_TOPK_N;
        const int* ci = cand_i + (size_t) t * FNX_TOPK_N;
        double* e = ex + (size_t) t * FNX_TOPK_N;
        const int n = FNX_TOPK_N;
        const int k = (sp.top_k <= 0 || sp.top_k > n) ? n : sp.top_k;
        const double mx = cv[0];
        for (int i = lane; i < n; i += 32) e[i] = exp((double) cv[i] - mx);
        __syncwarp();
        if (lane == 0) {
            int keep = k;
            if (sp.top_p < 1.f) {
                double sum = 0.0;
                for (int i = 0; i < k; ++i) sum += e[i];
                double cum = 0.0;
                for (int i = 0; i < k; ++i) {
                    cum += e[i] / sum;
                    if (cum >= (double) sp.top_p) { keep = i + 1; break; }
                }
            }
            if (sp.min_p > 0.f) {
                const float thresh = cv[0] + logf(sp.min_p);
                for (int i = 1; i < keep; ++i)
                    if (cv[i] < thresh) { keep = i; break; }
            }
            dist[t].n = keep;
        }
        __syncwarp();
        const int keep = dist[t].n;
        const double inv_t = 1.0 / sp.temperature, smx = cv[0] * inv_t;
        for (int i = lane; i < keep; i += 32) {
            dist[t].ids[i] = ci[i];
            dist[t].p[i] = exp(cv[i] * inv_t - smx);
        }
        __syncwarp();
        if (lane == 0) {
            double sum = 0.0;
            for (int i = 0; i < keep; ++i) sum += dist[t].p[i];
            for (int i = 0; i < keep; ++i) dist[t].p[i] /= sum;
        }
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    uint32_t slot = 0;
    int n;
    double* p = ex;   // row scratch for the residual
    for (n = 0; n < T; ++n) {
        const DistS& d = dist[n];
        const double* pp = d.p;
        if (n + 1 < T) {
            const int dr = tok[n + 1];
            const int qn = q_n ? q_n[n] : 0;
            const int* qi = q_ids ? q_ids + (size_t) n * FNX_TOPK_N : nullptr;
            const double* qp = q_p ? q_p + (size_t) n * FNX_TOPK_N : nullptr;
            const bool fixed = qn == 0;
            const double u = philox_uniform(seed, seq, step, slot++);
            if (u * (fixed ? 1.0 : dist_prob(qi, qp, qn, dr)) < dist_prob(d.ids, d.p, d.n, dr)) {
                result[1 + n] = n;
                result[1 + FNX_MAX_ROWS + n] = dr;
                continue;
            }
            double rest = 0.0;
            for (int i = 0; i < d.n; ++i) {
                const double qv = fixed ? (d.ids[i] == dr ? 1.0 : 0.0) : dist_prob(qi, qp, qn, d.ids[i]);
                p[i] = d.p[i] - qv > 0.0 ? d.p[i] - qv : 0.0;
                rest += p[i];
            }
            if (rest > 1e-12) {
                for (int i = 0; i < d.n; ++i) p[i] /= rest;
                pp = p;
            }
        }
        const double u = philox_uniform(seed, seq, step, slot++);
        double cum = 0.0;
        int pick = d.ids[d.n - 1];
        for (int i = 0; i < d.n; ++i) {
            cum += pp[i];
            if (u < cum) { pick = d.ids[i]; break; }
        }
        result[1 + n] = n;
        result[1 + FNX_MAX_ROWS + n] = pick;
        ++n;
        break;
    }
    result[0] = n;
}

__global__ void __launch_bounds__(1024) k_accept_sample(const float* __restrict__ cand_v, const int* __restrict__ cand_i,
                                                        const int* __restrict__ tok, int T, fnx_sampling sp, const int* __restrict__ q_ids,
                                                        const double* __restrict__ q_p, const int* __restrict__ q_n, uint64_t seed,
                                                        uint32_t seq, const uint32_t* __restrict__ stepp, int* __restrict__ result) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) uint8_t smem[];
    accept_sample_body(cand_v, cand_i, tok, T, sp, q_ids, q_p, q_n, seed, seq, *stepp, result, smem);
}

// batched lanes: block j applies the rule to lane j's chain with sequence lane_seq[j]'s uniforms (drafts count as fixed)
__global__ void __launch_bounds__(1024) k_accept_sample_lanes(const float* __restrict__ cand_v, const int* __restrict__ cand_i,
                                                              const int* __restrict__ tok, fnx_sampling sp, uint64_t seed,
                                                              const int* __restrict__ lane_seq, const int* __restrict__ lane_row0,
                                                              const uint32_t* __restrict__ steps, int* __restrict__ result) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int lane = blockIdx.x, row0 = lane_row0[lane], seq = lane_seq[lane];
    accept_sample_body(cand_v + (size_t) row0 * FNX_TOPK_N, cand_i + (size_t) row0 * FNX_TOPK_N, tok + row0, lane_row0[lane + 1] - row0, sp, nullptr, nullptr, nullptr,
                       seed, (uint32_t) seq, steps[seq], result + (size_t) lane * (1 + 2 * FNX_MAX_ROWS), smem);
}

}  // namespace fnxb

using namespace fnxb;

extern "C" int fnx_lookup_draft(const int* ctx, const int* n, int lk, const int* d1, int* out, int* out_n, fnx_stream st) {
    FNX_REQUIRE(ctx && n && out && out_n && lk >= 0 && lk <= FNX_MAX_ROWS, "fnx_lookup_draft: bad arguments");
    {
        const cudaError_t le_ = launch_k(k_lookup, dim3(1), dim3(1024), 0, as_stream(st), ctx, n, lk, d1, out, out_n);
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "k_lookup: launch failed: %s", cudaGetErrorString(le_));
    }
    FNX_LAUNCH_OK("fnx_lookup_draft");
    return FNX_OK;
}

extern "C" int fnx_accept_greedy(const int* tok, const int* parent, const int* best, int T, int* result, fnx_stream st) {
    FNX_REQUIRE(tok && best && result && T >= 1 && T <= FNX_MAX_ROWS, "fnx_accept_greedy: bad arguments");
    {
        const cudaError_t le_ = launch_k(k_accept_greedy, dim3(1), dim3(32), 0, as_stream(st), tok, parent, best, T, result);
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "k_accept_greedy: launch failed: %s", cudaGetErrorString(le_));
    }
    FNX_LAUNCH_OK("fnx_accept_greedy");
    return FNX_OK;
}

extern "C" int fnx_accept_sample(const float* cand_v, const int* cand_i, const int* tok, int T, fnx_sampling s, const int* q_ids,
                                 const double* q_p, const int* q_n, uint64_t seed, uint32_t seq, const uint32_t* step, int* result,
                                 fnx_stream st) {
    FNX_REQUIRE(cand_v && cand_i && tok && step && result && T >= 1 && T <= FNX_MAX_ROWS, "fnx_accept_sample: bad arguments");
    FNX_REQUIRE(s.temperature > 0.f, "fnx_accept_sample: temperature %g (greedy windows use fnx_accept_greedy)", (double) s.temperature);
    const size_t smem = sizeof(DistS) * (size_t) T + sizeof(double) * FNX_TOPK_N * (size_t) T;
    if (int rc = set_smem_limit((const void*) k_accept_sample, 64 * 1024)) return rc;
    {
        const cudaError_t le_ = launch_k(k_accept_sample, dim3(1), dim3(1024), smem, as_stream(st), cand_v, cand_i, tok, T, s, q_ids, q_p, q_n, seed, seq, step, result);
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "k_accept_sample: launch failed: %s", cudaGetErrorString(le_));
    }
    FNX_LAUNCH_OK("fnx_accept_sample");
    return FNX_OK;
}

// ---- batched lanes: one result row of 1 + 2 FNX_MAX_ROWS ints per lane
extern "C" int fnx_accept_greedy_lanes(const int* tok, const int* best, const int* lane_row0, int n_lanes, int* result, fnx_stream st) {
    FNX_REQUIRE(tok && best && lane_row0 && result && n_lanes >= 1 && n_lanes <= FNX_MAX_ROWS, "fnx_accept_greedy_lanes: bad arguments");
    const cudaError_t le = launch_k(k_accept_greedy_lanes, dim3(n_lanes), dim3(32), 0, as_stream(st), tok, best, lane_row0, result);
    if (le != cudaSuccess) return fail(FNX_E_CUDA, "k_accept_greedy_lanes: launch failed: %s", cudaGetErrorString(le));
    FNX_LAUNCH_OK("fnx_accept_greedy_lanes");
    return FNX_OK;
}

extern "C" int fnx_accept_sample_lanes(const float* cand_v, const int* cand_i, const int* tok, fnx_sampling s, uint64_t seed, const int* lane_seq,
                                       const int* lane_row0, int n_lanes, int max_lane_rows, const uint32_t* steps, int* result, fnx_stream st) {
    FNX_REQUIRE(cand_v && cand_i && tok && lane_seq && lane_row0 && steps && result && n_lanes >= 1 && n_lanes <= FNX_MAX_ROWS && max_lane_rows >= 1 &&
                    max_lane_rows <= FNX_MAX_ROWS,
                "fnx_accept_sample_lanes: bad arguments");
    FNX_REQUIRE(s.temperature > 0.f, "fnx_accept_sample_lanes: temperature %g", (double) s.temperature);
    const size_t smem = sizeof(DistS) * (size_t) max_lane_rows + sizeof(double) * FNX_TOPK_N * (size_t) max_lane_rows;
    if (int rc = set_smem_limit((const void*) k_accept_sample_lanes, 64 * 1024)) return rc;
    const cudaError_t le = launch_k(k_accept_sample_lanes, dim3(n_lanes), dim3(1024), smem, as_stream(st), cand_v, cand_i, tok, s, seed, lane_seq, lane_row0, steps, result);
    if (le != cudaSuccess) return fail(FNX_E_CUDA, "k_accept_sample_lanes: launch failed: %s", cudaGetErrorString(le));
    FNX_LAUNCH_OK("fnx_accept_sample_lanes");
    return FNX_OK;
}
