// Routing pieces of the router kernels (moe_route.cu), the window form and the prompt form:
// order-preserving logit keys, the top-K of one row by one warp, and the block-wide job list builder.
// Semantics: k_topk + k_jobs (engine/src/kernels.cu:338-398) and k_router_route (engine/src/moe.cuh:382-411).
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
// topi_g / topw_g (global) may be null; topi_s / topw_s (shared) may be null.
template <int SL>
__device__ __forceinline__ void rt_topk_row(const volatile float* l, int E, int K, int lane, int* topi_g, int* topi_s, float* topw_g, float* topw_s) {
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
        if (lane == 0) {
            if (topi_g) topi_g[k] = bi;
            if (topi_s) topi_s[k] = bi;
        }
#pragma unroll
        for (int j = 0; j < SL; ++j)
            if (lane + 32 * j == bi) key[j] = 0u;
    }
    if (lane < K) {
        if (topw_g) topw_g[lane] = mine / z;
        if (topw_s) topw_s[lane] = mine / z;
    }
}

// Shared memory of the job list builder: s_topi [T][K] (filled by the caller), s_cnt and s_base [RT_MAXE], wsum [32],
// total [2], js = the job list (room for T K + ceil(T / 4) jobs).
struct RtJobSmem {
    int* s_topi;
    int* s_cnt;
    int* s_base;
    int* wsum;
    int* total;
    fnx_job* js;
};

// The job list of T rows' picks, by all NTH threads of the block (every thread calls; the function synchronises the
// block): jobs in ascending expert order, expert e's rows in row order, 4 per job; then (add_shared) the shared expert's.
// Thread `tid` owns experts [tid * EPT, (tid + 1) * EPT) below RT_MAXE: a block-wide exclusive scan of their job counts gives each
// expert's first job; then one thread per (row, pick) entry places itself.  Returns the number of jobs in total[0] and
// the routed ones in total[1] (valid after the call in every thread).
template <int NTH>
__device__ __forceinline__ void rt_build_jobs(const RtJobSmem& s, int tid, int T, int E, int K, int e_lo, int e_hi, int add_shared) {
    constexpr int EPT = (RT_MAXE + NTH - 1) / NTH, NW = NTH / 32;
    const int warp = tid >> 5, lane = tid & 31;
    for (int e = tid; e < RT_MAXE; e += NTH) s.s_cnt[e] = 0;
    {   // unused row slots of the jobs stay zero
        const int cap = (T * K + (T + FNX_JOB_TOK - 1) / FNX_JOB_TOK) * (int) (sizeof(fnx_job) / 4);
        for (int w = tid; w < cap; w += NTH) reinterpret_cast<int*>(s.js)[w] = 0;
    }
    __syncthreads();
    // how many rows picked each expert of this rank
    for (int i = tid; i < T * K; i += NTH) {
        const int e = s.s_topi[i];
        if (e >= e_lo && e < e_hi) atomicAdd(&s.s_cnt[e], 1);
    }
    __syncthreads();
    int cnt_[EPT], mine = 0;
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const int e = tid * EPT + j;
        cnt_[j] = e < RT_MAXE ? (s.s_cnt[e] + FNX_JOB_TOK - 1) / FNX_JOB_TOK : 0;
        mine += cnt_[j];
    }
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) s.wsum[warp] = incl;
    __syncthreads();
    int base_ = incl - mine;
    for (int w = 0; w < warp; ++w) base_ += s.wsum[w];
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        if (tid * EPT + j < RT_MAXE) s.s_base[tid * EPT + j] = base_;
        base_ += cnt_[j];
    }
    if (tid == NTH - 1) {
        s.total[1] = base_;
        s.total[0] = base_ + (add_shared ? (T + FNX_JOB_TOK - 1) / FNX_JOB_TOK : 0);
    }
    (void) NW;
    __syncthreads();
    const int routed_total = s.total[1];
    for (int i = tid; i < T * K; i += NTH) {
        const int e = s.s_topi[i];
        if (e < e_lo || e >= e_hi) continue;
        int rank = 0;   // entries of the same expert before this one (row order)
        for (int i2 = 0; i2 < i; ++i2) rank += s.s_topi[i2] == e;
        fnx_job& jj = s.js[s.s_base[e] + rank / FNX_JOB_TOK];
        jj.y[rank % FNX_JOB_TOK] = i / K;
        jj.out[rank % FNX_JOB_TOK] = i;
        if (rank % FNX_JOB_TOK == 0) {
            jj.w = e;
            jj.n = min(FNX_JOB_TOK, s.s_cnt[e] - rank);
        }
    }
    if (add_shared)
        for (int t = tid; t < T; t += NTH) {
            fnx_job& j = s.js[routed_total + t / FNX_JOB_TOK];
            j.y[t % FNX_JOB_TOK] = t;
            j.out[t % FNX_JOB_TOK] = T * K + t;
            if (t % FNX_JOB_TOK == 0) {
                j.w = E;
                j.n = min(FNX_JOB_TOK, T - t);
            }
        }
    __syncthreads();
}

}  // namespace fnxb
