// Routing of a window's rows from their router logits: top K per row, renormalised softmax weights, and the job list.
// One thread block does it (route_rows): the router kernel's last block (moe_route.cu), or every block of the gate|up
// kernel for itself (mmv_stage.cuh), which then needs no job list from memory.  The result is a function of the logits
// alone, so every block that computes it gets the same list.
#pragma once

#include "fnx_common.cuh"

namespace fnxb {

constexpr int RT_MAXE = 1024;

// float -> unsigned key with the same order (so that warp-wide integer maxima rank logits)
__device__ __forceinline__ unsigned rt_key(float v) {
    const unsigned u = __float_as_uint(v);
    return u & 0x80000000u ? ~u : u | 0x80000000u;
}

// Top K of one row's E logits by one warp: K rounds of (largest value, lowest index).  SL = slots per lane.
template <int SL>
__device__ __forceinline__ void rt_topk_row(const volatile float* l, int E, int K, int lane, int* topi_g, int* topi_s, float* topw_g) {
    unsigned key[SL];
#pragma unroll
    for (int j = 0; j < SL; ++j) key[j] = lane + 32 * j < E ? rt_key(l[lane + 32 * j]) : 0u;
    float top = 0.f, z = 0.f, mine = 0.f;
    for (int k = 0; k < K; ++k) {
        // the lane's largest key and its slot by a pairwise tree (depth log2 SL; among equals the lower slot)
        unsigned tk[SL];
        int tj[SL];
#pragma unroll
        for (int j = 0; j < SL; ++j) { tk[j] = key[j]; tj[j] = j; }
#pragma unroll
        for (int w = SL / 2; w >= 1; w >>= 1)
#pragma unroll
            for (int j = 0; j < w; ++j) {
                const bool hi = tk[j + w] > tk[j];   // slots j < j + w: keep j on a tie
                tk[j] = hi ? tk[j + w] : tk[j];
                tj[j] = hi ? tj[j + w] : tj[j];
            }
        const unsigned bk = tk[0];
        const int bj = tj[0];
        const unsigned wk = __reduce_max_sync(0xffffffffu, bk);
        const int bi = __reduce_min_sync(0xffffffffu, bk == wk ? lane + 32 * bj : 0x7fffffff);
        const unsigned u = wk & 0x80000000u ? wk & 0x7fffffffu : ~wk;
        const float bv = __uint_as_float(u);
        if (k == 0) top = bv;
        const float w = expf(bv - top);
        z += w;
        if (lane == k) mine = w;
        if (lane == 0) { topi_g[k] = bi; topi_s[k] = bi; }
#pragma unroll
        for (int j = 0; j < SL; ++j)
            if (lane + 32 * j == bi) key[j] = 0u;
    }
    if (lane < K) topw_g[lane] = mine / z;
}

// scratch of route_rows (shared memory)
struct RouteScratch {
    int topi[FNX_MAX_ROWS * 32];
    int cnt[RT_MAXE];
    int base[RT_MAXE];
    int wsum[32];
    int routed_total;
};

// Block-wide (NTH threads, all of them call it).  logits [T][E + 1] in global memory.  js: room for T * K + ceil(T / 4)
// jobs, zeroed by the callee.  topi_g / topw_g: where the picks go (global or shared; every block may pass its own or
// only one block the global arrays: pass null to keep them local).  Returns the number of jobs; sc.routed_total = the
// routed ones.  Jobs in ascending expert order (experts in [e_lo, e_hi)): an expert's rows in row order, 4 per job;
// then (add_shared) the shared expert's (w = E).  Ends with a block barrier.
template <int NTH>
__device__ __forceinline__ int route_rows(const float* logits, int T, int E, int K, int e_lo, int e_hi, int add_shared, RouteScratch& sc, fnx_job* js,
                                          int* topi_g, float* topw_g, float* topw_s, int tid) {
    const int warp = tid >> 5, lane = tid & 31;
    constexpr int NW = NTH / 32, EPT = RT_MAXE / NTH;
    for (int e = tid; e < RT_MAXE; e += NTH) sc.cnt[e] = 0;
    {
        const int cap = (T * K + (T + FNX_JOB_TOK - 1) / FNX_JOB_TOK) * (int) (sizeof(fnx_job) / 4);
        for (int w = tid; w < cap; w += NTH) reinterpret_cast<int*>(js)[w] = 0;
    }
    // top K per row: a warp per row, K rounds of (value, index) maximum, ties to the lower index
    for (int t = warp; t < T; t += NW) {
        const volatile float* l = logits + (size_t) t * (E + 1);
        int* tg = topi_g ? topi_g + t * K : sc.topi + t * K;
        float* wg = topw_g ? topw_g + t * K : topw_s + t * K;
        if (E <= 512) rt_topk_row<16>(l, E, K, lane, tg, sc.topi + t * K, wg);
        else rt_topk_row<RT_MAXE / 32>(l, E, K, lane, tg, sc.topi + t * K, wg);
        if (topw_g && topw_s && lane < K) topw_s[t * K + lane] = wg[lane];
    }
    __syncthreads();
    // how many rows picked each expert of this rank
    for (int i = tid; i < T * K; i += NTH) {
        const int e = sc.topi[i];
        if (e >= e_lo && e < e_hi) atomicAdd(&sc.cnt[e], 1);
    }
    __syncthreads();
    // thread `tid` owns experts [tid * EPT, (tid + 1) * EPT): a block-wide exclusive scan of their job counts gives each
    // expert's first job; then one thread per (row, pick) entry places itself
    int cnt_[EPT], mine = 0;
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const int e = tid * EPT + j;
        cnt_[j] = (sc.cnt[e] + FNX_JOB_TOK - 1) / FNX_JOB_TOK;
        mine += cnt_[j];
    }
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) sc.wsum[warp] = incl;
    __syncthreads();
    int base_ = incl - mine;
    for (int w = 0; w < warp; ++w) base_ += sc.wsum[w];
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        sc.base[tid * EPT + j] = base_;
        base_ += cnt_[j];
    }
    if (tid == NTH - 1) sc.routed_total = base_;
    __syncthreads();
    const int routed = sc.routed_total;
    for (int i = tid; i < T * K; i += NTH) {
        const int e = sc.topi[i];
        if (e < e_lo || e >= e_hi) continue;
        int rank = 0;   // entries of the same expert before this one (row order)
        for (int i2 = 0; i2 < i; ++i2) rank += sc.topi[i2] == e;
        fnx_job& jj = js[sc.base[e] + rank / FNX_JOB_TOK];
        jj.y[rank % FNX_JOB_TOK] = i / K;
        jj.out[rank % FNX_JOB_TOK] = i;
        if (rank % FNX_JOB_TOK == 0) {
            jj.w = e;
            jj.n = min(FNX_JOB_TOK, sc.cnt[e] - rank);
        }
    }
    if (add_shared)
        for (int t = tid; t < T; t += NTH) {
            fnx_job& j = js[routed + t / FNX_JOB_TOK];
            j.y[t % FNX_JOB_TOK] = t;
            j.out[t % FNX_JOB_TOK] = T * K + t;
            if (t % FNX_JOB_TOK == 0) {
                j.w = E;
                j.n = min(FNX_JOB_TOK, T - t);
            }
        }
    __syncthreads();
    return routed + (add_shared ? (T + FNX_JOB_TOK - 1) / FNX_JOB_TOK : 0);
}

}  // namespace fnxb
