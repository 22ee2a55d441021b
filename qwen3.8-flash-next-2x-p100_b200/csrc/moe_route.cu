// MoE routing and combine.
//
// fnx_router_route replaces router_route / k_router_route (engine/src/kernels.hpp:294-296, engine/src/moe.cuh:258-515)
// and its simple form route / k_topk + k_jobs (engine/src/kernels.cu:338-398): one launch computes the router logits
// (f32 weights, a warp per expert row, fixed summation order), and the last block to finish picks the top K per row,
// renormalises their softmax and lists the jobs.  fnx_moe_combine replaces k_combine (engine/src/kernels.cu:412-419).
#include <algorithm>

#include "fnx_common.cuh"

namespace fnxb {

constexpr int RT_WARPS = 8, RT_TOK = 8, RT_MAXE = 1024, RT_SPLIT = 2, RT_ROWS = RT_WARPS / RT_SPLIT;

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

// Grid: ceil((E + 1) / RT_ROWS) blocks of RT_WARPS warps; a block computes RT_ROWS logit rows, RT_SPLIT warps per row
// (each a contiguous share of the columns, summed in share order).
__global__ void __launch_bounds__(RT_WARPS * 32) k_router(const float* __restrict__ Wr, const float* __restrict__ x,
                                                          const float* __restrict__ norm_w, float eps, int T, int E, int H, int K,
                                                          int e_lo, int e_hi, int add_shared, float* __restrict__ logits,
                                                          int* __restrict__ topi, float* __restrict__ topw, fnx_job* __restrict__ jobs,
                                                          int* __restrict__ njobs, unsigned long long* __restrict__ stats, unsigned* __restrict__ err) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) float xs[];   // [RT_TOK][H]: x * norm_w (the row's 1 / rms is applied to the sums)
    __shared__ float rs[RT_TOK], ssw[RT_TOK][RT_WARPS], psum[RT_ROWS][RT_SPLIT][RT_TOK];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row = blockIdx.x * RT_ROWS + warp / RT_SPLIT, share = warp % RT_SPLIT;
    constexpr int NT = RT_WARPS * 32;
    const int HS = H / RT_SPLIT, c_lo = share * HS;   // this warp's columns
    // the warp's first weights are on their way before anything else (they depend on nothing)
    float4 w[8];
    if (row <= E) {
        const float* wr = Wr + (size_t) row * H + c_lo;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = lane * 4 + j * 128;
            w[j] = i < HS ? *reinterpret_cast<const float4*>(wr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    for (int t0 = 0; t0 < T; t0 += RT_TOK) {
        const int nt = min(RT_TOK, T - t0);
        __syncthreads();
        // stage the rows with 16-byte async copies, all in flight at once; then, from shared memory, each thread's
        // columns of every row: the sum of squares and the product with the norm weight
        for (int i = tid; i < nt * (H / 4); i += NT)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(xs + (size_t) i * 4)), "l"(x + (size_t) t0 * H + (size_t) i * 4) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
        float4 nw4[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = tid * 4 + j * NT * 4;
            nw4[j] = norm_w && c < H ? *reinterpret_cast<const float4*>(norm_w + c) : make_float4(1.f, 1.f, 1.f, 1.f);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = tid * 4 + j * NT * 4;
                if (c >= H) continue;
                float4 v = *reinterpret_cast<const float4*>(xs + (size_t) t * H + c);
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                v.x *= nw4[j].x; v.y *= nw4[j].y; v.z *= nw4[j].z; v.w *= nw4[j].w;
                *reinterpret_cast<float4*>(xs + (size_t) t * H + c) = v;
            }
            ss = warp_sum(ss);
            if (lane == 0) ssw[t][warp] = ss;
        }
        __syncthreads();
        if (tid < nt) {
            float ss = 0.f;
            for (int wq = 0; wq < RT_WARPS; ++wq) ss += ssw[tid][wq];
            rs[tid] = norm_w ? rsqrtf(ss / (float) H + eps) : 1.0f;
        }
        float acc[RT_TOK];
#pragma unroll
        for (int t = 0; t < RT_TOK; ++t) acc[t] = 0.f;
        if (row <= E) {
            const float* wr = Wr + (size_t) row * H + c_lo;
            for (int i0 = 0; i0 < HS; i0 += 1024) {   // 8 float4 of the weight row in flight per lane
                if (i0 > 0 || t0 > 0) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int i = i0 + lane * 4 + j * 128;
                        w[j] = i < HS ? *reinterpret_cast<const float4*>(wr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int i = i0 + lane * 4 + j * 128;
                    if (i >= HS) continue;
#pragma unroll
                    for (int t = 0; t < RT_TOK; ++t)
                        if (t < nt) {
                            const float4 v = *reinterpret_cast<const float4*>(xs + (size_t) t * H + c_lo + i);
                            acc[t] = fmaf(w[j].x, v.x, acc[t]);
                            acc[t] = fmaf(w[j].y, v.y, acc[t]);
                            acc[t] = fmaf(w[j].z, v.z, acc[t]);
                            acc[t] = fmaf(w[j].w, v.w, acc[t]);
                        }
                }
            }
#pragma unroll
            for (int t = 0; t < RT_TOK; ++t)
                if (t < nt) {
                    const float s = warp_sum(acc[t]);
                    if (lane == 0) psum[warp / RT_SPLIT][share][t] = s;
                }
        }
        __syncthreads();
        if (tid < RT_ROWS * RT_TOK) {
            const int r = tid / RT_TOK, t = tid % RT_TOK, grow = blockIdx.x * RT_ROWS + r;
            if (t < nt && grow <= E) {
                float s = 0.f;
#pragma unroll
                for (int q = 0; q < RT_SPLIT; ++q) s += psum[r][q][t];
                s *= rs[t];
                logits[(size_t) (t0 + t) * (E + 1) + grow] = s;
                if (!isfinite(s)) atomicOr(err, (unsigned) FNX_ERR_NONFINITE);
            }
        }
    }
    // ---- the last block to get here routes
    __shared__ bool last;
    __shared__ int s_topi[FNX_MAX_ROWS * 32];
    __shared__ int s_cnt[RT_MAXE];
    __threadfence();
    __syncthreads();
    if (tid == 0) last = atomicAdd(&njobs[1], 1) == (int) gridDim.x - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    for (int e = tid; e < RT_MAXE; e += NT) s_cnt[e] = 0;
    {   // the job list is built in the rows' shared memory (free by now): unused row slots stay zero
        const int cap = (T * K + (T + FNX_JOB_TOK - 1) / FNX_JOB_TOK) * (int) (sizeof(fnx_job) / 4);
        for (int w = tid; w < cap; w += NT) reinterpret_cast<int*>(xs)[w] = 0;
    }
    // top K per row: a warp per row, K rounds of (value, index) maximum, ties to the lower index
    for (int t = warp; t < T; t += RT_WARPS) {
        const volatile float* l = logits + (size_t) t * (E + 1);
        if (E <= 512) rt_topk_row<16>(l, E, K, lane, topi + t * K, s_topi + t * K, topw + t * K);
        else rt_topk_row<RT_MAXE / 32>(l, E, K, lane, topi + t * K, s_topi + t * K, topw + t * K);
    }
    __syncthreads();
    // how many rows picked each expert of this rank
    for (int i = tid; i < T * K; i += NT) {
        const int e = s_topi[i];
        if (e >= e_lo && e < e_hi) atomicAdd(&s_cnt[e], 1);
    }
    __syncthreads();
    // jobs in ascending expert order: expert e's rows in row order, 4 per job; then the shared expert's.
    // Thread `tid` owns experts [tid * EPT, (tid + 1) * EPT): a block-wide exclusive scan of their job counts gives
    // each expert's first job; then one thread per (row, pick) entry places itself, and the list is copied out.
    constexpr int NTH = RT_WARPS * 32, EPT = RT_MAXE / NTH;
    __shared__ int wsum_[RT_WARPS];
    __shared__ int routed_total;
    __shared__ int s_base[RT_MAXE];
    int cnt_[EPT], mine = 0;
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const int e = tid * EPT + j;
        cnt_[j] = (s_cnt[e] + FNX_JOB_TOK - 1) / FNX_JOB_TOK;
        mine += cnt_[j];
    }
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) wsum_[warp] = incl;
    __syncthreads();
    int base_ = incl - mine;
    for (int w = 0; w < warp; ++w) base_ += wsum_[w];
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        s_base[tid * EPT + j] = base_;
        base_ += cnt_[j];
    }
    if (tid == NTH - 1) {
        routed_total = base_;
        njobs[0] = base_ + (add_shared ? (T + FNX_JOB_TOK - 1) / FNX_JOB_TOK : 0);
        njobs[1] = 0;
        if (stats) {
            atomicAdd(&stats[0], (unsigned long long) base_);
            atomicAdd(&stats[1], 1ull);
        }
    }
    __syncthreads();
    fnx_job* js = reinterpret_cast<fnx_job*>(xs);
    const int total = routed_total + (add_shared ? (T + FNX_JOB_TOK - 1) / FNX_JOB_TOK : 0);
    for (int i = tid; i < T * K; i += NTH) {
        const int e = s_topi[i];
        if (e < e_lo || e >= e_hi) continue;
        int rank = 0;   // entries of the same expert before this one (row order)
        for (int i2 = 0; i2 < i; ++i2) rank += s_topi[i2] == e;
        fnx_job& jj = js[s_base[e] + rank / FNX_JOB_TOK];
        jj.y[rank % FNX_JOB_TOK] = i / K;
        jj.out[rank % FNX_JOB_TOK] = i;
        if (rank % FNX_JOB_TOK == 0) {
            jj.w = e;
            jj.n = min(FNX_JOB_TOK, s_cnt[e] - rank);
        }
    }
    if (add_shared)
        for (int t = tid; t < T; t += NTH) {
            fnx_job& j = js[routed_total + t / FNX_JOB_TOK];
            j.y[t % FNX_JOB_TOK] = t;
            j.out[t % FNX_JOB_TOK] = T * K + t;
            if (t % FNX_JOB_TOK == 0) {
                j.w = E;
                j.n = min(FNX_JOB_TOK, T - t);
            }
        }
    __syncthreads();
    constexpr int JW = sizeof(fnx_job) / 4;
    for (int w = tid; w < total * JW; w += NTH) reinterpret_cast<int*>(jobs)[w] = reinterpret_cast<const int*>(js)[w];
}

__global__ void k_combine(const float* __restrict__ part, const int* __restrict__ topi, const float* __restrict__ topw,
                          const float* __restrict__ logits, int T, int E, int H, int K, int e_lo, int e_hi, int add_shared,
                          float* __restrict__ out, int accumulate) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= H) return;
    // the picks' weights first (0 outside the expert range), then every addend's load at once
    float w[32], v[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        w[k] = 0.f;
        if (k < K) {
            const int e = topi[t * K + k];
            w[k] = e >= e_lo && e < e_hi ? topw[t * K + k] : 0.f;
        }
    }
#pragma unroll
    for (int k = 0; k < 32; ++k) v[k] = k < K && w[k] != 0.f ? part[((size_t) t * K + k) * H + i] : 0.f;
    const float shv = add_shared ? part[((size_t) T * K + t) * H + i] : 0.f;
    const float shl = add_shared ? logits[(size_t) t * (E + 1) + E] : 0.f;
    float* o = out + (size_t) t * H + i;
    const float prev = accumulate ? *o : 0.f;
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k)
        if (k < K) s = fmaf(w[k], v[k], s);
    if (add_shared) s += sigmoidf_(shl) * shv;
    *o = prev + s;
}

}  // namespace fnxb

using namespace fnxb;

extern "C" int fnx_router_route(const float* Wr, const float* x, const float* norm_w, float eps, int T, int E, int H, int K, int e_lo,
                                int e_hi, int add_shared, float* logits, int* topi, float* topw, fnx_job* jobs, int* njobs,
                                unsigned long long* stats, unsigned* err, fnx_stream st) {
    FNX_REQUIRE(Wr && x && logits && topi && topw && jobs && njobs && err, "fnx_router_route: null pointer");
    FNX_REQUIRE(T >= 1 && T <= FNX_MAX_ROWS, "fnx_router_route: %d rows (1..%d)", T, FNX_MAX_ROWS);
    FNX_REQUIRE(E >= K && E <= RT_MAXE && K >= 1 && K <= 32, "fnx_router_route: %d experts, top %d not supported", E, K);
    FNX_REQUIRE(H % 256 == 0 && H <= 4096, "fnx_router_route: hidden %d not supported", H);
    FNX_REQUIRE(0 <= e_lo && e_lo <= e_hi && e_hi <= E, "fnx_router_route: expert range [%d, %d) outside [0, %d)", e_lo, e_hi, E);
    const size_t jobs_cap = (size_t) T * K + (T + FNX_JOB_TOK - 1) / FNX_JOB_TOK;
    const size_t smem = std::max((size_t) RT_TOK * H * sizeof(float), jobs_cap * sizeof(fnx_job));
    static bool configured = false;
    if (!configured) {
        FNX_CUDA_OK(cudaFuncSetAttribute(k_router, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        configured = true;
    }
    const int blocks = (E + 1 + RT_ROWS - 1) / RT_ROWS;
    {
        const cudaError_t le_ = launch_k(k_router, dim3(blocks), dim3(RT_WARPS * 32), smem, as_stream(st), Wr, x, norm_w, eps, T, E, H, K, e_lo, e_hi, add_shared, logits, topi, topw, jobs,
                                                            njobs, stats, err);
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "k_router: launch failed: %s", cudaGetErrorString(le_));
    }
    FNX_LAUNCH_OK("fnx_router_route");
    return FNX_OK;
}

extern "C" int fnx_moe_combine(const float* part, const int* topi, const float* topw, const float* logits, int T, int E, int H, int K,
                               int e_lo, int e_hi, int add_shared, float* out, int accumulate, fnx_stream st) {
    FNX_REQUIRE(part && topi && topw && logits && out, "fnx_moe_combine: null pointer");
    FNX_REQUIRE(T >= 1 && T <= FNX_MAX_ROWS, "fnx_moe_combine: %d rows", T);
    {
        const cudaError_t le_ = launch_k(k_combine, dim3(dim3((H + 255) / 256, T)), dim3(256), 0, as_stream(st), part, topi, topw, logits, T, E, H, K, e_lo, e_hi, add_shared, out, accumulate);
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "k_combine: launch failed: %s", cudaGetErrorString(le_));
    }
    FNX_LAUNCH_OK("fnx_moe_combine");
    return FNX_OK;
}
