// MoE routing and combine.
//
// fnx_router_route replaces router_route / k_router_route (engine/src/kernels.hpp:294-296, engine/src/moe.cuh:258-515)
// and its simple form route / k_topk + k_jobs (engine/src/kernels.cu:338-398): one launch computes the router logits
// (f32 weights, a warp per expert row, fixed summation order), and the last block to finish picks the top K per row,
// renormalises their softmax and lists the jobs.  fnx_moe_combine replaces k_combine (engine/src/kernels.cu:412-419).
#include <algorithm>

#include "fnx_common.cuh"
#include <cstdlib>

#include "moe_route.cuh"
#include "mmv_core.cuh"

namespace fnxb {

constexpr int RT_WARPS = 8, RT_TOK = 8, RT_SPLIT = 2, RT_ROWS = RT_WARPS / RT_SPLIT;

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
    __shared__ int s_base[RT_MAXE];
    __shared__ int wsum_[32];
    __shared__ int total_[2];
    __threadfence();
    __syncthreads();
    if (tid == 0) last = atomicAdd(&njobs[1], 1) == (int) gridDim.x - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    // top K per row: a warp per row, K rounds of (value, index) maximum, ties to the lower index
    for (int t = warp; t < T; t += RT_WARPS) {
        const volatile float* l = logits + (size_t) t * (E + 1);
        if (E <= 512) rt_topk_row<16>(l, E, K, lane, topi + t * K, s_topi + t * K, topw + t * K, nullptr);
        else rt_topk_row<RT_MAXE / 32>(l, E, K, lane, topi + t * K, s_topi + t * K, topw + t * K, nullptr);
    }
    __syncthreads();
    // the job list is built in the rows' shared memory (free by now) and copied out
    RtJobSmem js;
    js.s_topi = s_topi; js.s_cnt = s_cnt; js.s_base = s_base; js.wsum = wsum_; js.total = total_;
    js.js = reinterpret_cast<fnx_job*>(xs);
    rt_build_jobs<NT>(js, tid, T, E, K, e_lo, e_hi, add_shared);
    const int total = total_[0];
    if (tid == 0) {
        njobs[0] = total;
        njobs[1] = 0;
        if (stats) {
            atomicAdd(&stats[0], (unsigned long long) total_[1]);
            atomicAdd(&stats[1], 1ull);
        }
    }
    constexpr int JW = sizeof(fnx_job) / 4;
    for (int w = tid; w < total * JW; w += NT) reinterpret_cast<int*>(jobs)[w] = reinterpret_cast<const int*>(js.js)[w];
}

// Routing for prompt-sized row counts: the logits of any number of rows, then the top K of every row by one warp each.
// A block stages eight window rows once (normed, as k_router does) and its sixteen warps walk the expert rows, four per warp at
// a time: a warp keeps a 512-column piece of its four weight rows in registers, so every 16-byte read of a staged row feeds
// sixteen multiply-adds, and carries its 4 x 8 sums in registers across the row's pieces; nothing in the walk is block-wide,
// so the warps hide one another's weight loads.  f32 throughout; the sums' order differs from k_router's, the values by rounding.
constexpr int RP_WARPS = 16, RP_RPW = 4, RP_TOK = 8;

__global__ void __launch_bounds__(RP_WARPS * 32) k_router_rows(const float* __restrict__ Wr, const float* __restrict__ x, const float* __restrict__ norm_w,
                                                               float eps, int T, int E, int H, float* __restrict__ logits, unsigned* __restrict__ err) {
    extern __shared__ __align__(16) float xs[];   // [RP_TOK][H]: x * norm_w (the row's 1 / rms is applied to the sums)
    __shared__ float rs[RP_TOK], ssw[RP_TOK][RP_WARPS];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int NT = RP_WARPS * 32;
    const int t0 = blockIdx.x * RP_TOK, nt = min(RP_TOK, T - t0);
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
        for (int wq = 0; wq < RP_WARPS; ++wq) ss += ssw[tid][wq];
        rs[tid] = norm_w ? rsqrtf(ss / (float) H + eps) : 1.0f;
    }
    __syncthreads();
    bool bad = false;
    for (int row0 = warp * RP_RPW; row0 <= E; row0 += RP_WARPS * RP_RPW) {
        float acc[RP_RPW][RP_TOK];
#pragma unroll
        for (int r = 0; r < RP_RPW; ++r)
#pragma unroll
            for (int t = 0; t < RP_TOK; ++t) acc[r][t] = 0.f;
        for (int i0 = 0; i0 < H; i0 += 512) {
            float4 w[RP_RPW][4];
#pragma unroll
            for (int r = 0; r < RP_RPW; ++r)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = i0 + lane * 4 + j * 128;
                    w[r][j] = row0 + r <= E && i < H ? *reinterpret_cast<const float4*>(Wr + (size_t) (row0 + r) * H + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = i0 + lane * 4 + j * 128;
                if (i >= H) continue;
#pragma unroll
                for (int t = 0; t < RP_TOK; ++t)
                    if (t < nt) {
                        const float4 v = *reinterpret_cast<const float4*>(xs + (size_t) t * H + i);
#pragma unroll
                        for (int r = 0; r < RP_RPW; ++r) {
                            acc[r][t] = fmaf(w[r][j].x, v.x, acc[r][t]);
                            acc[r][t] = fmaf(w[r][j].y, v.y, acc[r][t]);
                            acc[r][t] = fmaf(w[r][j].z, v.z, acc[r][t]);
                            acc[r][t] = fmaf(w[r][j].w, v.w, acc[r][t]);
                        }
                    }
            }
        }
#pragma unroll
        for (int r = 0; r < RP_RPW; ++r)
#pragma unroll
            for (int t = 0; t < RP_TOK; ++t)
                if (t < nt && row0 + r <= E) {
                    const float s = warp_sum(acc[r][t]) * rs[t];
                    if (lane == 0) {
                        logits[(size_t) (t0 + t) * (E + 1) + row0 + r] = s;
                        bad |= !isfinite(s);
                    }
                }
    }
    if (bad) atomicOr(err, (unsigned) FNX_ERR_NONFINITE);
}

// one warp per row: the top K of its E logits and their renormalised softmax weights
__global__ void __launch_bounds__(256) k_topk_rows(const float* __restrict__ logits, int T, int E, int K, int* __restrict__ topi, float* __restrict__ topw) {
    const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    const volatile float* l = logits + (size_t) t * (E + 1);
    if (E <= 512) rt_topk_row<16>(l, E, K, lane, topi + (size_t) t * K, nullptr, topw + (size_t) t * K, nullptr);
    else rt_topk_row<RT_MAXE / 32>(l, E, K, lane, topi + (size_t) t * K, nullptr, topw + (size_t) t * K, nullptr);
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
    // the addends are summed as 2^-32 fixed-point integers: the sum does not depend on their order, so a row's result does not
    // depend on how its picks are split over kernels or expert-parallel ranks
    unsigned long long s = 0ull;
#pragma unroll
    for (int k = 0; k < 32; ++k)
        if (k < K && w[k] != 0.f) s += fix_from_float(w[k] * v[k]);
    if (add_shared) s += fix_from_float(sigmoidf_(shl) * shv);
    *o = prev + fix_to_float(s);
}

// k_combine that also leaves the new rows' image for the next dense product (fnx_dense_image): one warp per (256-column block,
// row), the lane's 8 columns of every addend in flight at once; the sums and the residual update are k_combine's, the image
// cells are those the dense kernel's own quantisation (quant_finish) makes of the same values, so the product's bits do not
// change.  The blocks of an image's last live row also clear the rows of its last group that hold nothing.
__global__ void __launch_bounds__(32) k_combine_image(const float* __restrict__ part, const int* __restrict__ topi, const float* __restrict__ topw,
                                                      const float* __restrict__ logits, int T, int E, int H, int K, float* __restrict__ out,
                                                      uint8_t* __restrict__ img_out, const float* __restrict__ img_norm_w, size_t img_stride) {
    pdl_wait();
    pdl_launch_dependents();
    const int blk = blockIdx.x, t = blockIdx.y, lane = threadIdx.x, KB = H / 256;
    const size_t col = (size_t) blk * 256 + lane * 8;
    float w[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) w[k] = k < K ? topw[t * K + k] : 0.f;
    const float shl = logits[(size_t) t * (E + 1) + E];
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
    quant_fetch(q[0], img_norm_w, lane, v[0], nw[0]);   // the old values and the norm weights
    unsigned long long s[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i] = 0ull;
    // the addends in two halves of up to 16 picks, all of a half's loads in flight at once
#pragma unroll
    for (int k0 = 0; k0 < 32; k0 += 16) {
        if (k0 >= K) break;
        float4 a[16][2];
#pragma unroll
        for (int k = 0; k < 16; ++k)
            if (k0 + k < K) {
                const float4* src = reinterpret_cast<const float4*>(part + ((size_t) t * K + k0 + k) * H + col);
                a[k][0] = src[0];
                a[k][1] = src[1];
            }
#pragma unroll
        for (int k = 0; k < 16; ++k)
            if (k0 + k < K) {
                const float wk = w[k0 + k];
                const float e8[8] = {a[k][0].x, a[k][0].y, a[k][0].z, a[k][0].w, a[k][1].x, a[k][1].y, a[k][1].z, a[k][1].w};
#pragma unroll
                for (int i = 0; i < 8; ++i) s[i] += fix_from_float(wk * e8[i]);
            }
    }
    {
        const float4* src = reinterpret_cast<const float4*>(part + ((size_t) T * K + t) * H + col);
        const float4 a0 = src[0], a1 = src[1];
        const float g = sigmoidf_(shl);
        const float e8[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i] += fix_from_float(g * e8[i]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) v[0][i] += fix_to_float(s[i]);
    float* dst = out + (size_t) t * H + col;
    *reinterpret_cast<float4*>(dst) = make_float4(v[0][0], v[0][1], v[0][2], v[0][3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(v[0][4], v[0][5], v[0][6], v[0][7]);
    // the image of the row's group of FNX_DENSE_ROWS
    const int t0 = t - t % FNX_DENSE_ROWS, nt = min((int) FNX_DENSE_ROWS, T - t0), NG = (nt + 3) / 4;
    uint2* cells = reinterpret_cast<uint2*>(img_out + (size_t) (t0 / FNX_DENSE_ROWS) * img_stride);
    float* scales = reinterpret_cast<float*>(cells + (size_t) NG * (H / 32) * 32);
    float* rs = scales + (size_t) NG * KB * 8;
    quant_finish(q, v, nw, H, img_norm_w, cells, scales, rs, lane);
    if (t == t0 + nt - 1)
        for (int td = nt; td < 4 * NG; ++td) {
            const int ng = td >> 2, n = td & 3;
            for (int i = lane; i < 64; i += 32) {   // (sub-block of the column block, level, q)
                const int sbG = blk * 8 + (i >> 3), lvl = (i >> 2) & 1, qq = i & 3;
                cells[((size_t) (ng * (H / 32) + sbG) * 8 + n + 4 * lvl) * 4 + qq] = make_uint2(0u, 0u);
            }
            if (lane < 2) scales[(size_t) (ng * KB + blk) * 8 + n + 4 * lane] = 0.f;
            if (lane == 2) rs[td * 16 + blk] = 0.f;
        }
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
    if (int rc = set_smem_limit((const void*) k_router, 160 * 1024)) return rc;
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

extern "C" int fnx_moe_combine_image(const float* part, const int* topi, const float* topw, const float* logits, int T, int E, int H, int K, float* R,
                                     void* img_out, const float* img_norm_w, fnx_stream st) {
    FNX_REQUIRE(part && topi && topw && logits && R && img_out && img_norm_w, "fnx_moe_combine_image: null pointer");
    FNX_REQUIRE(T >= 1 && T <= FNX_MAX_ROWS && K >= 1 && K <= 32, "fnx_moe_combine_image: %d rows, top %d", T, K);
    FNX_REQUIRE(H == 256 || H == 512 || H == 1024 || H == 2048 || H == 4096, "fnx_moe_combine_image: hidden %d", H);
    FNX_REQUIRE(((uintptr_t) img_out & 15) == 0 && ((uintptr_t) R & 15) == 0 && ((uintptr_t) part & 15) == 0, "fnx_moe_combine_image: 16-byte alignment");
    {
        const cudaError_t le_ = launch_k(k_combine_image, dim3(H / 256, T), dim3(32), 0, as_stream(st), part, topi, topw, logits, T, E, H, K, R, (uint8_t*) img_out,
                                         img_norm_w, fnx_dense_image_bytes(H));
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "k_combine_image: launch failed: %s", cudaGetErrorString(le_));
    }
    FNX_LAUNCH_OK("fnx_moe_combine_image");
    return FNX_OK;
}

// ---- the router over a prompt's rows as a tensor-core product (gemm_tma.cu): the normed rows and the f32 weights are split
// into f16 high and low parts (weights times 256 first, so that their low parts stay clear of f16's subnormals); three
// products (high x high, high x low, low x high) restore the f32 operands (the tensor core's truncating f32 accumulation leaves
// the logits good to a few 1e-5).  The shared expert's gate row is a plain dot.
__global__ void __launch_bounds__(256) k_router_split_x(const float* __restrict__ x, const float* __restrict__ norm_w, const float* __restrict__ w_gate, int H,
                                                        float eps, __half* __restrict__ xh, __half* __restrict__ xl, float* __restrict__ logits, int ldl, int E) {
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* xr = x + (size_t) t * H;
    __shared__ float ws[8], s_r;
    float ss = 0.f;
    for (int i = tid * 4; i < H; i += 1024) {
        const float4 v = *reinterpret_cast<const float4*>(xr + i);
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) ws[tid >> 5] = ss;
    __syncthreads();
    if (tid == 0) {
        float a = 0.f;
        for (int w = 0; w < 8; ++w) a += ws[w];
        s_r = norm_w ? rsqrtf(a / (float) H + eps) : 1.0f;
    }
    __syncthreads();
    const float r = s_r;
    float dot = 0.f;
    for (int i = tid * 4; i < H; i += 1024) {
        float4 v = *reinterpret_cast<const float4*>(xr + i);
        if (norm_w) {
            const float4 w = *reinterpret_cast<const float4*>(norm_w + i);
            v.x *= w.x * r; v.y *= w.y * r; v.z *= w.z * r; v.w *= w.w * r;
        }
        const float4 g = *reinterpret_cast<const float4*>(w_gate + i);
        dot = fmaf(v.x, g.x, fmaf(v.y, g.y, fmaf(v.z, g.z, fmaf(v.w, g.w, dot))));
        const float e[4] = {v.x, v.y, v.z, v.w};
        __half h[4], l[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            h[k] = __float2half_rn(e[k]);
            l[k] = __float2half_rn(e[k] - __half2float(h[k]));
        }
        *reinterpret_cast<uint2*>(xh + (size_t) t * H + i) = make_uint2((uint32_t) __half_as_ushort(h[0]) | ((uint32_t) __half_as_ushort(h[1]) << 16),
                                                                        (uint32_t) __half_as_ushort(h[2]) | ((uint32_t) __half_as_ushort(h[3]) << 16));
        *reinterpret_cast<uint2*>(xl + (size_t) t * H + i) = make_uint2((uint32_t) __half_as_ushort(l[0]) | ((uint32_t) __half_as_ushort(l[1]) << 16),
                                                                        (uint32_t) __half_as_ushort(l[2]) | ((uint32_t) __half_as_ushort(l[3]) << 16));
    }
    dot = warp_sum(dot);
    __syncthreads();
    if ((tid & 31) == 0) ws[tid >> 5] = dot;
    __syncthreads();
    if (tid == 0) {
        float a = 0.f;
        for (int w = 0; w < 8; ++w) a += ws[w];
        logits[(size_t) t * ldl + E] = a;
    }
}

__global__ void k_router_split_w(const float* __restrict__ w, size_t n, __half* __restrict__ wh, __half* __restrict__ wl) {
    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = w[i] * 256.0f;
    const __half h = __float2half_rn(v);
    wh[i] = h;
    wl[i] = __float2half_rn(v - __half2float(h));
}

namespace fnxb {
int gemm_tma_launch(const __half* w, const __half* wl, const __half* x, const __half* xl, float* y, int ldy, int T, int rows, int K, int accumulate, float scale,
                    unsigned* err, cudaStream_t st);
static size_t rr_align(size_t v) { return (v + 255) & ~(size_t) 255; }
}  // namespace fnxb

extern "C" size_t fnx_router_rows_scratch_bytes(int T, int E, int H) {
    return 2 * rr_align((size_t) T * H * sizeof(__half)) + 2 * rr_align((size_t) E * H * sizeof(__half));
}

extern "C" int fnx_router_rows(const float* Wr, const float* x, const float* norm_w, float eps, int T, int E, int H, int K, float* logits, int* topi,
                               float* topw, void* scratch, unsigned* err, fnx_stream st) {
    FNX_REQUIRE(Wr && x && logits && topi && topw && err, "fnx_router_rows: null pointer");
    FNX_REQUIRE(T >= 1, "fnx_router_rows: %d rows", T);
    FNX_REQUIRE(E >= K && E <= RT_MAXE && K >= 1 && K <= 32, "fnx_router_rows: %d experts, top %d not supported", E, K);
    FNX_REQUIRE(H % 256 == 0 && H <= 4096, "fnx_router_rows: hidden %d not supported", H);
    static const bool gemm_off = []() { const char* e = getenv("FNX_PROMPT_GEMM"); return e && atoi(e) == 0; }();
    if (scratch && T >= 1024 && !gemm_off) {
        uint8_t* b = (uint8_t*) scratch;
        __half* xh = (__half*) b; b += rr_align((size_t) T * H * sizeof(__half));
        __half* xl = (__half*) b; b += rr_align((size_t) T * H * sizeof(__half));
        __half* wh = (__half*) b; b += rr_align((size_t) E * H * sizeof(__half));
        __half* wl = (__half*) b;
        k_router_split_x<<<T, 256, 0, as_stream(st)>>>(x, norm_w, Wr + (size_t) E * H, H, eps, xh, xl, logits, E + 1, E);
        FNX_LAUNCH_OK("k_router_split_x");
        const size_t n = (size_t) E * H;
        k_router_split_w<<<(unsigned) ((n + 255) / 256), 256, 0, as_stream(st)>>>(Wr, n, wh, wl);
        FNX_LAUNCH_OK("k_router_split_w");
        if (int rc = gemm_tma_launch(wh, wl, xh, xl, logits, E + 1, T, E, H, 0, 1.0f / 256.0f, err, as_stream(st))) return rc;
    } else {
        const size_t smem = (size_t) RP_TOK * H * sizeof(float);
        if (int rc = set_smem_limit((const void*) k_router_rows, 160 * 1024)) return rc;
        k_router_rows<<<(T + RP_TOK - 1) / RP_TOK, RP_WARPS * 32, smem, as_stream(st)>>>(Wr, x, norm_w, eps, T, E, H, logits, err);
        FNX_LAUNCH_OK("k_router_rows");
    }
    k_topk_rows<<<(T + 7) / 8, 256, 0, as_stream(st)>>>(logits, T, E, K, topi, topw);
    FNX_LAUNCH_OK("k_topk_rows");
    return FNX_OK;
}
