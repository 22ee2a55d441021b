// The verify window as ONE persistent kernel: a cooperative grid of one block per SM walks every phase of every
// layer (input projection, mixer, output projection, router, routed experts gate|up, down, combine) and the head,
// with a bounded grid barrier between phases.
//
// Why: a window moves ~70 MB per layer, about 11 us at HBM speed, while a separately launched kernel costs several
// microseconds before its first byte arrives (launch, table set-up, cold pipeline) - measured: a 44 MB streaming
// kernel alone takes 13 us on B200.  The reference replays ~10 launches per layer from a CUDA graph
// (engine/src/engine.cu:1760-1848 under engine_common.cu:994-1018); at B200 speeds those launch boundaries cost more
// than the data.  Here
//   - the codebook table and the barriers are set up once per window;
//   - a block that has finished a phase stages the first steps of its NEXT phase's weights (bulk async copies)
//     before it waits at the grid barrier, so the HBM pipe keeps running across phases;
//   - activations are normalised and quantised once per phase by the last block to finish the producing phase
//     (an atomic arrival counter), and every block fetches that 17-66 KB image with one bulk copy;
//   - routing (top-K, job list) is done once, by the last block to finish the router's logits.
// Every wait (grid barrier, mbarrier) is bounded and raises FNX_ERR_TIMEOUT instead of hanging.
//
// Phase bodies restate the stand-alone kernels (iq3s_mmv.cu, moe_route.cu, attn.cu, gdn.cu, head.cu, spec.cu), which
// remain the path for windows of more than 8 rows and for expert-parallel ranks, and the reference citations given
// there apply here too.
#include <cooperative_groups.h>

#include "mmv_core.cuh"
#include "step.cuh"

namespace fnxb {

constexpr int NST = 3;                    // weight steps in flight
constexpr int XQ_BYTES = 65536 + 1024;    // the largest activation image: 8 rows x 4096 columns
constexpr int PART_BYTES = 8192;
constexpr int MISC_BYTES = 2048;
constexpr int NWARP = STEP_THREADS / 32;

struct Smem {
    uint8_t* table;
    uint8_t* ring;
    uint8_t* xq;       // activation image (cells then scales); scratch for the non-matrix phases
    float* part;
    float* misc;
    uint64_t* bars;    // [NST] ring, [NST] image
    StepParams* P;
};

size_t step_smem_bytes() { return (size_t) CORE_TABLE_BYTES + NST * CORE_STEP_BYTES + XQ_BYTES + PART_BYTES + MISC_BYTES + 64 + sizeof(StepParams) + 64; }

struct Flow {
    unsigned issued = 0, consumed = 0;   // ring ordinals (block-uniform)
    unsigned ximg = 0;                   // image copies so far
    unsigned epoch = 0;                  // grid barriers passed
    bool dead = false;                   // a wait gave up: stop waiting, finish quickly
    unsigned long long* prof = nullptr;  // block 0, thread 0: tagged %globaltimer stamps
    int nstamp = 0;
};

// stamp `id` (block 0's thread 0 only; the tag rides in the top byte)
__device__ __forceinline__ void stamp(Flow& f, int id) {
    if (f.prof && f.nstamp < 4000) {
        unsigned long long t_;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_));
        f.prof[1 + f.nstamp++] = ((unsigned long long) id << 56) | (t_ & 0x00ffffffffffffffull);
    }
}

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void bar_named(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

// every block arrives; nobody leaves before all have (or the poll limit runs out)
__device__ void grid_barrier(const Smem& sm, Flow& f, int tid) {
    __syncthreads();
    ++f.epoch;
    stamp(f, 2);
    if (tid == 0) {
        __threadfence();
        atomicAdd(&sm.P->sync[0], 1u);
        const unsigned target = f.epoch * gridDim.x;
        if (!f.dead) {
            unsigned it = 0;
            while (ld_acquire(&sm.P->sync[0]) < target) {
                if (++it > 20000000u) {
                    atomicOr(sm.P->err, (unsigned) FNX_ERR_TIMEOUT);
                    sm.misc[500] = 1.f;
                    break;
                }
            }
        }
        __threadfence();
    }
    stamp(f, 3);
    __syncthreads();
    if (sm.misc[500] != 0.f) f.dead = true;
}

// true (in every thread) in the block that arrives last at counter `which`: it then sees every block's writes
__device__ bool last_block(const Smem& sm, Flow& f, int which, int tid) {
    stamp(f, 20);
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned old = atomicAdd(&sm.P->sync[which], 1u);
        sm.misc[501] = ((old + 1u) % gridDim.x) == 0u ? 1.f : 0.f;
    }
    __syncthreads();
    const bool l = sm.misc[501] != 0.f;
    if (l) __threadfence();
    stamp(f, l ? 22 : 21);
    return l;
}

__device__ __forceinline__ bool wait_bar(uint64_t* bar, unsigned parity, Flow& f, const Smem& sm) {
    if (f.dead) return false;
    if (mbar_wait_bounded(bar, parity, 8000000u)) return true;
    atomicOr(sm.P->err, (unsigned) FNX_ERR_TIMEOUT);
    return false;
}

// ------------------------------------------------------------------------------------------------ activation images
// Built by ONE block (all its threads) into global memory: rows [0, T) of K columns.
// mode 0: x (f32 rows, stride ldx), optionally RMS-normed with norm_w (the codes are those of x * w; the row's 1 / rms
//         goes into the block scales); xnorm (optional): the f32 normalised rows as well (the router's input).
// mode 1: the DeltaNet output: o * rsqrt(mean_head(o^2) + eps) * gnorm * sigmoid(z)   (k_gdn_out_norm,
//         engine/src/kernels.cu:495-505), K = nv * hs columns; sq holds each head's four partial square sums.
__device__ void build_image(const Smem& sm, int tid, int T, int K, int mode, const float* x, int ldx, const float* norm_w, float eps,
                            float* xnorm, const float* sq, const float* z, int ldz, const float* gnorm, int hs) {
    const int warp = tid >> 5, lane = tid & 31, KB = K / 256;
    const int CB = KB < 4 ? KB : 4, nchunk = KB / CB;
    uint2* xq = reinterpret_cast<uint2*>(sm.P->ximg);
    float* xs = reinterpret_cast<float*>(sm.P->ximg + img_cells(T, K) * sizeof(uint2));
    float* rs = sm.misc;   // [T][nchunk <= 4] square sums, then [T] factors at +64
    const bool norm = mode == 0 && norm_w != nullptr;
    // rows past T in the last group: zero cells and scales
    const int Tpad = (T + 3) / 4 * 4;
    for (int task = warp; task < Tpad * nchunk; task += NWARP) {
        const int t = task / nchunk, ck = task % nchunk, ng = t >> 2, n = t & 3;
        const bool live = t < T;
        float v[4][8];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (j < CB) {
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
                if (live) {
                    const float* xr = x + (size_t) t * ldx + (ck * CB + j) * 256 + lane * 8;
                    a = *reinterpret_cast<const float4*>(xr);
                    b = *reinterpret_cast<const float4*>(xr + 4);
                }
                v[j][0] = a.x; v[j][1] = a.y; v[j][2] = a.z; v[j][3] = a.w;
                v[j][4] = b.x; v[j][5] = b.y; v[j][6] = b.z; v[j][7] = b.w;
            }
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (j < CB) {
                const int blk = ck * CB + j, col = blk * 256 + lane * 8;
                if (norm) {
                    const float4 w0 = *reinterpret_cast<const float4*>(norm_w + col), w1 = *reinterpret_cast<const float4*>(norm_w + col + 4);
                    const float w8[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        ss = fmaf(v[j][i], v[j][i], ss);
                        v[j][i] *= w8[i];
                    }
                } else if (mode == 1 && live) {
                    const int head = col / hs, hc = col % hs;
                    const float* s4 = sq + ((size_t) t * (K / hs) + head) * 4;
                    const float ms = ((s4[0] + s4[1]) + (s4[2] + s4[3])) / (float) hs;
                    const float r = rsqrtf(ms + eps);
                    const float* zr = z + (size_t) t * ldz + col;
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[j][i] = v[j][i] * r * gnorm[hc + i] / (1.0f + expf(-zr[i]));
                }
                float am = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) am = fmaxf(am, fabsf(v[j][i]));
                am = warp_max(am);
                uint2 c1, c2;
                float d;
                core_quant_cell(v[j], am, c1, c2, d);
                const int sbG = blk * 8 + (lane >> 2), q = lane & 3;
                uint2* cell = xq + ((size_t) (ng * (K / 32) + sbG) * 8 + n) * 4 + q;
                cell[0] = c1;
                cell[16] = c2;
                if (lane == 0) {
                    float* s = xs + (size_t) (ng * KB + blk) * 8;
                    s[n] = d;
                    s[n + 4] = d * (1.0f / 256.0f);
                }
            }
        if (norm) {
            ss = warp_sum(ss);
            if (lane == 0) rs[t * 4 + ck] = ss;
        }
    }
    __syncthreads();
    if (norm) {
        if (tid < T) {
            float ss = 0.f;
            for (int c = 0; c < nchunk; ++c) ss += rs[tid * 4 + c];
            rs[64 + tid] = rsqrtf(ss / (float) K + eps);
        }
        __syncthreads();
        for (int i = tid; i < T * KB; i += STEP_THREADS) {
            const int t = i / KB, blk = i % KB;
            float* s = xs + (size_t) ((t >> 2) * KB + blk) * 8;
            s[t & 3] *= rs[64 + t];
            s[(t & 3) + 4] *= rs[64 + t];
        }
        if (xnorm)
            for (int i = tid * 4; i < T * K; i += STEP_THREADS * 4) {
                const int t = i / K, c = i % K;
                const float4 a = *reinterpret_cast<const float4*>(x + (size_t) t * ldx + c), w = *reinterpret_cast<const float4*>(norm_w + c);
                const float r = rs[64 + t];
                *reinterpret_cast<float4*>(xnorm + (size_t) t * K + c) = make_float4(a.x * w.x * r, a.y * w.y * r, a.z * w.z * r, a.w * w.w * r);
            }
    }
    __threadfence();
    __syncthreads();
}

// the image into shared memory: one bulk copy, waited for by everyone
__device__ void fetch_image(const Smem& sm, Flow& f, int tid, int T, int K) {
    const unsigned bytes = (unsigned) img_bytes(T, K);
    uint64_t* bar = &sm.bars[NST + (f.ximg % NST)];
    if (tid == 0) {
        fence_proxy_async();
        mbar_expect_tx(bar, bytes);
        bulk_g2s(sm.xq, sm.P->ximg, bytes, bar);
    }
    wait_bar(bar, (f.ximg / NST) & 1u, f, sm);
    ++f.ximg;
}

// ------------------------------------------------------------------------------------------------ matrix phases
enum { M_DENSE = 0, M_GATEUP = 1, M_DOWN = 2 };

struct MatWork {
    const uint8_t* W;        // dense matrix, or the experts' base
    size_t expert_stride;
    const uint8_t* Wsh;
    int E;
    const fnx_job* jobs;
    int njobs;               // 1 for a dense matrix
    int rows, K;             // output rows per job (gate|up: F)
    const float* h;          // down: the f32 rows to quantise per job
    float* out;
    int ldo, accumulate, T;
};

__device__ __forceinline__ int mat_spj(int mode, int rows, int K) {
    const int TPS = CORE_ITEMS / (K / 256);
    return mode == M_GATEUP ? rows / (8 * TPS) : rows / (16 * TPS);
}
__device__ __forceinline__ void mat_range(int mode, const MatWork& w, int& s0, int& s1) {
    const long long total = (long long) w.njobs * mat_spj(mode, w.rows, w.K);
    s0 = (int) (total * blockIdx.x / gridDim.x);
    s1 = (int) (total * (blockIdx.x + 1) / gridDim.x);
}
__device__ __forceinline__ const uint8_t* mat_weights(const MatWork& w, int j) {
    if (!w.jobs) return w.W;
    const int e = w.jobs[j].w;
    return e >= w.E ? w.Wsh : w.W + (size_t) e * w.expert_stride;
}
// thread 0: stage the weights of this block's step s
__device__ void mat_issue(const Smem& sm, Flow& f, int mode, const MatWork& w, int s) {
    const int KB = w.K / 256, spj = mat_spj(mode, w.rows, w.K), j = s / spj, ls = s % spj;
    const uint8_t* W = mat_weights(w, j);
    const unsigned st = f.issued % NST;
    uint8_t* dst = sm.ring + (size_t) st * CORE_STEP_BYTES;
    fence_proxy_async();
    mbar_expect_tx(&sm.bars[st], CORE_STEP_BYTES);
    if (mode == M_GATEUP) {
        const size_t half = CORE_STEP_BYTES / 2;
        bulk_g2s(dst, W + (size_t) ls * half, (unsigned) half, &sm.bars[st]);
        bulk_g2s(dst + half, W + (size_t) (w.rows / 16) * KB * TILE_BYTES + (size_t) ls * half, (unsigned) half, &sm.bars[st]);
    } else {
        bulk_g2s(dst, W + (size_t) ls * CORE_STEP_BYTES, CORE_STEP_BYTES, &sm.bars[st]);
    }
    ++f.issued;
}
// before the barrier that precedes the phase: its first steps on their way.  Returns how many were issued.
__device__ int mat_preissue(const Smem& sm, Flow& f, int tid, int mode, const MatWork& w) {
    int s0, s1;
    mat_range(mode, w, s0, s1);
    const int n = min(NST, s1 - s0);
    if (tid == 0)
        for (int i = 0; i < n; ++i) mat_issue(sm, f, mode, w, s0 + i);
    return n > 0 ? n : 0;
}

// per-job quantisation of the down projection's inputs (rows of F values) into the shared image region
__device__ void quant_job_rows(const Smem& sm, int tid, const float* h, int ldh, const int* rows, int ntok, int K) {
    const int warp = tid >> 5, lane = tid & 31, KB = K / 256;
    uint2* xq = reinterpret_cast<uint2*>(sm.xq);
    float* xs = reinterpret_cast<float*>(sm.xq + img_cells(4, K) * sizeof(uint2));
    for (int task = warp; task < 4 * KB; task += NWARP) {
        const int t = task / KB, blk = task % KB;
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (t < ntok) {
            const float* xr = h + (size_t) rows[t] * ldh + blk * 256 + lane * 8;
            const float4 a = *reinterpret_cast<const float4*>(xr), b = *reinterpret_cast<const float4*>(xr + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
        float am = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) am = fmaxf(am, fabsf(v[i]));
        am = warp_max(am);
        uint2 c1, c2;
        float d;
        core_quant_cell(v, am, c1, c2, d);
        uint2* cell = xq + ((size_t) (blk * 8 + (lane >> 2)) * 8 + t) * 4 + (lane & 3);
        cell[0] = c1;
        cell[16] = c2;
        if (lane == 0) {
            xs[blk * 8 + t] = d;
            xs[blk * 8 + t + 4] = d * (1.0f / 256.0f);
        }
    }
    __syncthreads();
}

// One matrix phase of this block: steps [s0, s1) of the job list.  `pre` steps were issued before the barrier.
template <int NG, int MODE>
__device__ void mat_phase(const Smem& sm, Flow& f, int tid, const MatWork& w, int pre, bool have_image) {
    const int warp = tid >> 5, lane = tid & 31;
    const int KB = w.K / 256, TPS = CORE_ITEMS / KB, spj = mat_spj(MODE, w.rows, w.K);
    constexpr int PB = NG == 1 ? 2 : 1;   // partial-sum buffers
    int s0, s1;
    mat_range(MODE, w, s0, s1);
    const int n = s1 - s0;
    int next = pre;   // next step (relative) to issue
    if (tid == 0)
        while (next < n && next < NST) mat_issue(sm, f, MODE, w, s0 + next), ++next;
    next = min(n, max(pre, NST));
    stamp(f, 10);
    if (MODE != M_DOWN && have_image && n > 0) fetch_image(sm, f, tid, w.T, w.K);
    stamp(f, 11);
    const uint2* xq = reinterpret_cast<const uint2*>(sm.xq);
    const float* xs = reinterpret_cast<const float*>(sm.xq + img_cells(MODE == M_DOWN ? 4 : w.T, w.K) * sizeof(uint2));
    LaneX<NG> lx;
    if (MODE == M_DENSE) lx = lane_x_dense<NG>(xq, xs, w.K, w.T, lane);
    int cur_job = -1, ntok = w.T;
    int orow[4 * NG];
#pragma unroll
    for (int i = 0; i < 4 * NG; ++i) orow[i] = i;
    for (int i = 0; i < n; ++i) {
        const int s = s0 + i, j = s / spj, ls = s % spj;
        if (MODE != M_DENSE && j != cur_job) {
            cur_job = j;
            const fnx_job jb = w.jobs[j];
            ntok = min(jb.n, 4);
            int yrow[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                yrow[k] = jb.y[k];
                orow[k] = jb.out[k];
            }
            if (MODE == M_GATEUP) {
                if constexpr (NG == 1) lx = lane_x_job(xq, xs, w.K, yrow, ntok, lane);
            } else {
                __syncthreads();   // the previous job's cells are no longer read
                quant_job_rows(sm, tid, w.h, w.K, orow, ntok, w.K);
                lx = lane_x_dense<NG>(xq, xs, w.K, ntok, lane);
            }
        }
        const unsigned st = f.consumed % NST;
        const bool ok = wait_bar(&sm.bars[st], (f.consumed / NST) & 1u, f, sm);
        ++f.consumed;
        stamp(f, 12);
        const uint8_t* stage = sm.ring + (size_t) st * CORE_STEP_BYTES;
        float* part = sm.part + (size_t) (PB == 2 ? (i & 1) : 0) * CORE_ITEMS * 16 * 4 * NG;
        if (ok) {
            const int it = warp, blk = it % KB;
            float acc[NG][4];
#pragma unroll
            for (int ng = 0; ng < NG; ++ng)
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[ng][k] = 0.f;
            core_item<NG>(smem_u32(stage + (size_t) it * TILE_BYTES), smem_u32(sm.table), lx, blk, lane, acc);
            const int g = lane >> 2, q = lane & 3;
#pragma unroll
            for (int ng = 0; ng < NG; ++ng) {
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[ng][k] += __shfl_xor_sync(0xffffffffu, acc[ng][k], 2);
                if (q < 2) {
                    float* pr = part + ((size_t) it * 16 + g) * (4 * NG) + ng * 4 + 2 * q;
                    *reinterpret_cast<float2*>(pr) = make_float2(acc[ng][0], acc[ng][1]);
                    *reinterpret_cast<float2*>(pr + 8 * 4 * NG) = make_float2(acc[ng][2], acc[ng][3]);
                }
            }
        }
        __syncthreads();
        stamp(f, 13);
        if (tid == 0 && next < n) mat_issue(sm, f, MODE, w, s0 + next);
        if (next < n) ++next;
        if (ok) {
            if (MODE == M_GATEUP) {
                const int HPS = TPS / 2;
                for (int o = tid; o < HPS * 16 * ntok; o += STEP_THREADS) {
                    const int tok = o / (HPS * 16), rr = o % (HPS * 16), tl = rr / 16, r = rr % 16;
                    float gs = 0.f, us = 0.f;
                    for (int b = 0; b < KB; ++b) {
                        gs += part[((size_t) (tl * KB + b) * 16 + r) * (4 * NG) + tok];
                        us += part[((size_t) (8 + tl * KB + b) * 16 + r) * (4 * NG) + tok];
                    }
                    w.out[(size_t) orow[tok] * w.ldo + (size_t) ls * HPS * 16 + rr] = siluf_(gs) * us;
                }
            } else {
                for (int o = tid; o < TPS * 16 * ntok; o += STEP_THREADS) {
                    const int tok = o / (TPS * 16), rr = o % (TPS * 16), tl = rr / 16, r = rr % 16;
                    float sum = 0.f;
                    for (int b = 0; b < KB; ++b) sum += part[((size_t) (tl * KB + b) * 16 + r) * (4 * NG) + tok];
                    float* dst = w.out + (size_t) orow[tok] * w.ldo + (size_t) ls * TPS * 16 + rr;
                    *dst = w.accumulate ? *dst + sum : sum;
                }
            }
        }
        if (PB == 1) __syncthreads();
        stamp(f, 14);
    }
}

// ------------------------------------------------------------------------------------------------ embedding
__device__ void embed_phase(const Smem& sm, int tid) {
    const StepParams& P = *sm.P;
    if (blockIdx.x == 0 && tid < P.T) {
        int d = 0;
        for (int a = P.tree ? P.parent[tid] : tid - 1; a >= 0; a = P.tree ? P.parent[a] : a - 1) ++d;
        P.depth[tid] = d;
    }
    const int per = P.T * P.H;
    for (int i = blockIdx.x * STEP_THREADS + tid; i < per; i += gridDim.x * STEP_THREADS) {
        const int t = i / P.H, c = i % P.H;
        P.R[i] = __half2float(P.embed[(size_t) P.tok[t] * P.H + c]);
    }
}

// ------------------------------------------------------------------------------------------------ router
// logits = Wr . xnorm (k_router_route, engine/src/moe.cuh:258-515): row r of the E + 1 on warp r / gridDim of block r % gridDim
__device__ void router_phase(const Smem& sm, Flow& f, int tid, const StepLayer& L) {
    const StepParams& P = *sm.P;
    const int warp = tid >> 5, lane = tid & 31, H = P.H, T = P.T;
    float* xs = reinterpret_cast<float*>(sm.xq);   // [T][H] f32
    const int nrows = (P.E + 1 + gridDim.x - 1 - blockIdx.x) / gridDim.x;   // rows blockIdx, blockIdx + grid, ...
    if (nrows > 0) {
        const unsigned bytes = (unsigned) (T * H * sizeof(float));
        uint64_t* bar = &sm.bars[NST + (f.ximg % NST)];
        if (tid == 0) {
            fence_proxy_async();
            mbar_expect_tx(bar, bytes);
            bulk_g2s(xs, P.xnorm, bytes, bar);
        }
        const bool ok = wait_bar(bar, (f.ximg / NST) & 1u, f, sm);
        ++f.ximg;
        if (ok && warp < nrows) {
            const int row = blockIdx.x + warp * gridDim.x;
            const float* wr = L.wr + (size_t) row * H;
            float acc[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) acc[t] = 0.f;
            for (int i0 = 0; i0 < H; i0 += 1024) {
                float4 w[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int i = i0 + lane * 4 + j * 128;
                    w[j] = i < H ? *reinterpret_cast<const float4*>(wr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int i = i0 + lane * 4 + j * 128;
                    if (i >= H) continue;
#pragma unroll
                    for (int t = 0; t < 8; ++t)
                        if (t < T) {
                            const float4 v = *reinterpret_cast<const float4*>(xs + (size_t) t * H + i);
                            acc[t] = fmaf(w[j].x, v.x, acc[t]);
                            acc[t] = fmaf(w[j].y, v.y, acc[t]);
                            acc[t] = fmaf(w[j].z, v.z, acc[t]);
                            acc[t] = fmaf(w[j].w, v.w, acc[t]);
                        }
                }
            }
#pragma unroll
            for (int t = 0; t < 8; ++t)
                if (t < T) {
                    const float s = warp_sum(acc[t]);
                    if (lane == 0) {
                        P.rlogits[(size_t) t * (P.E + 1) + row] = s;
                        if (!isfinite(s)) atomicOr(P.err, (unsigned) FNX_ERR_NONFINITE);
                    }
                }
        }
    }
}

// top-K, renormalised softmax and the job list, by one block (k_topk / k_jobs, engine/src/kernels.cu:338-398)
__device__ void route_finalize(const Smem& sm, int tid) {
    const StepParams& P = *sm.P;
    const int warp = tid >> 5, lane = tid & 31, E = P.E, K = P.K, T = P.T;
    int* s_topi = reinterpret_cast<int*>(sm.xq);   // [T][K]
    for (int t = warp; t < T; t += NWARP) {
        const float* l = P.rlogits + (size_t) t * (E + 1);
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = lane + 32 * j < E ? l[lane + 32 * j] : -INFINITY;
        float top = 0.f, z = 0.f, mine = 0.f;
        for (int k = 0; k < K; ++k) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (v[j] > bv) { bv = v[j]; bi = lane + 32 * j; }
#pragma unroll
            for (int o = 16; o; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (k == 0) top = bv;
            const float w = expf(bv - top);
            z += w;
            if (lane == k) mine = w;
            if (lane == 0) { P.topi[t * K + k] = bi; s_topi[t * K + k] = bi; }
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (lane + 32 * j == bi) v[j] = -INFINITY;
        }
        if (lane < K) P.topw[t * K + lane] = mine / z;
    }
    __syncthreads();
    // jobs in ascending expert order, rows in row order, 4 per job; then the shared expert's
    constexpr int EPT = 1024 / STEP_THREADS;
    int* wsum = reinterpret_cast<int*>(sm.misc) + 128;
    int cnt[EPT], mine = 0;
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const int e = tid * EPT + j;
        int c = 0;
        if (e < E)
            for (int i = 0; i < T * K; ++i) c += s_topi[i] == e;
        cnt[j] = (c + FNX_JOB_TOK - 1) / FNX_JOB_TOK;
        mine += cnt[j];
    }
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    int base = incl - mine;
    for (int w = 0; w < warp; ++w) base += wsum[w];
    if (tid == STEP_THREADS - 1) {
        const int s = base + mine;
        wsum[NWARP] = s;
        P.njobs[0] = s + (T + FNX_JOB_TOK - 1) / FNX_JOB_TOK;
        if (P.stats) {
            atomicAdd(&P.stats[0], (unsigned long long) s);
            atomicAdd(&P.stats[1], 1ull);
        }
    }
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const int e = tid * EPT + j;
        if (cnt[j]) {
            int nn = 0;
            fnx_job* jb = P.jobs + base;
            for (int i = 0; i < T * K; ++i)
                if (s_topi[i] == e) {
                    fnx_job& jj = jb[nn / FNX_JOB_TOK];
                    jj.w = e;
                    jj.y[nn % FNX_JOB_TOK] = i / K;
                    jj.out[nn % FNX_JOB_TOK] = i;
                    jj.n = nn % FNX_JOB_TOK + 1;
                    ++nn;
                }
            base += cnt[j];
        }
    }
    __syncthreads();
    const int routed = wsum[NWARP];
    for (int t = tid; t < T; t += STEP_THREADS) {
        fnx_job& j = P.jobs[routed + t / FNX_JOB_TOK];
        j.w = E;
        j.y[t % FNX_JOB_TOK] = t;
        j.out[t % FNX_JOB_TOK] = T * K + t;
        if (t % FNX_JOB_TOK == FNX_JOB_TOK - 1 || t == T - 1) j.n = t % FNX_JOB_TOK + 1;
    }
    __threadfence();
    __syncthreads();
}

// R[t] += sum_k topw * part[t K + k] + sigmoid(logit[t][E]) * part[T K + t]   (k_combine, engine/src/kernels.cu:412-419)
__device__ void combine_phase(const Smem& sm, int tid) {
    const StepParams& P = *sm.P;
    const int per = P.T * P.H;
    for (int i = blockIdx.x * STEP_THREADS + tid; i < per; i += gridDim.x * STEP_THREADS) {
        const int t = i / P.H, c = i % P.H;
        float w[32], v[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) w[k] = k < P.K ? P.topw[t * P.K + k] : 0.f;
#pragma unroll
        for (int k = 0; k < 32; ++k) v[k] = k < P.K ? P.part[((size_t) t * P.K + k) * P.H + c] : 0.f;
        const float shv = P.part[((size_t) P.T * P.K + t) * P.H + c], shl = P.rlogits[(size_t) t * (P.E + 1) + P.E];
        const float prev = P.R[i];
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < 32; ++k)
            if (k < P.K) s = fmaf(w[k], v[k], s);
        s += sigmoidf_(shl) * shv;
        P.R[i] = prev + s;
    }
}

// ------------------------------------------------------------------------------------------------ gated DeltaNet
// One (value head, column quarter) item on 128 threads: gdn.cu's kernel without its cluster; the head's square sums
// go to global memory and the gated norm is applied when the output projection's image is built.
constexpr int G_HS = 128, G_Q = 4, G_QC = 32, G_THREADS = 128;

__device__ void gdn_item(const Smem& sm, int tid, const StepLayer& L, int item) {
    const StepParams& P = *sm.P;
    const int T = P.T, nk = P.nk, nv = P.nv, NS = P.NS, stride = P.proj_ld;
    const int lv = item / G_Q, qq = item % G_Q, kh = lv % nk, warp = tid >> 5, lane = tid & 31;
    const int ch = (2 * nk + nv) * G_HS, cur = *P.cur;
    const size_t hsz = (size_t) 3 * ch, ssz = (size_t) nv * G_HS * G_HS;
    const float* qkvz = P.proj;
    const float* ab = P.proj + ch + nv * G_HS;
    const int* parent = P.tree ? P.parent : nullptr;
    float* smf = reinterpret_cast<float*>(sm.xq);
    float* xq = smf;
    float* xk = xq + (size_t) T * G_HS;
    float* vs = xk + (size_t) T * G_HS;
    float* gates = vs + (size_t) T * G_QC;
    float* kred = gates + 2 * T;
    float* ared = kred + 2 * 4 * G_QC;
    float* red = ared + (size_t) T * 4 * G_QC;
    float* xin = red + 8 * T;
    int* anc = reinterpret_cast<int*>(xin + (size_t) (T + 3) * (2 * G_HS + G_QC));
    const float* hin = L.hist + (size_t) cur * hsz;
    if (tid < T) {
        const float* abt = ab + (size_t) tid * stride;
        const float x = abt[lv] + L.dt[lv];
        gates[2 * tid] = expf((x > 20.0f ? x : log1pf(expf(x))) * L.a[lv]);
        gates[2 * tid + 1] = 1.0f / (1.0f + expf(-abt[nv + lv]));
    }
    constexpr int NC = 2 * G_HS + G_QC;
    auto chan = [&](int e) {
        return e < G_HS ? kh * G_HS + e : e < 2 * G_HS ? nk * G_HS + kh * G_HS + (e - G_HS) : 2 * nk * G_HS + lv * G_HS + qq * G_QC + (e - 2 * G_HS);
    };
    for (int i0 = tid; i0 < (T + 3) * NC; i0 += 4 * G_THREADS) {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = i0 + j * G_THREADS;
            v[j] = 0.f;
            if (i < (T + 3) * NC) {
                const int r = i / NC, c = chan(i % NC);
                v[j] = r < 3 ? hin[(size_t) r * ch + c] : qkvz[(size_t) (r - 3) * stride + c];
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = i0 + j * G_THREADS;
            if (i < (T + 3) * NC) xin[i] = v[j];
        }
    }
    if (tid < T) {
        int a = tid;
        for (int k = 1; k <= 3; ++k) {
            if (a >= 0) a = parent ? parent[a] : a - 1;
            else --a;
            anc[tid * 3 + k - 1] = 3 + a;
        }
    }
    bar_named(1, G_THREADS);
    for (int e = tid; e < NC; e += G_THREADS) {
        const int part = e < G_HS ? 0 : e < 2 * G_HS ? 1 : 2, i = part < 2 ? e - part * G_HS : e - 2 * G_HS;
        const int c = chan(e);
        const float4 cw = *reinterpret_cast<const float4*>(L.convw + c * 4);
        const bool writes = part == 2 || (lv < nk && qq == 0);
        for (int t = 0; t < T; ++t) {
            const float x3 = xin[anc[t * 3 + 2] * NC + e], x2 = xin[anc[t * 3 + 1] * NC + e], x1 = xin[anc[t * 3] * NC + e];
            const float x0 = xin[(3 + t) * NC + e];
            const float x = cw.x * x3 + cw.y * x2 + cw.z * x1 + cw.w * x0;
            const float v = x / (1.0f + expf(-x));
            if (part == 0) xq[t * G_HS + i] = v;
            else if (part == 1) xk[t * G_HS + i] = v;
            else vs[t * G_QC + i] = v;
            if (writes) {
                float* hout = L.hist + (size_t) ((cur + 1 + t) % NS) * hsz;
                hout[c] = x2;
                hout[ch + c] = x1;
                hout[2 * ch + c] = x0;
            }
        }
    }
    bar_named(1, G_THREADS);
    for (int t = 0; t < T; ++t) {
        const float qv = xq[t * G_HS + tid], kv = xk[t * G_HS + tid];
        const float sq = warp_sum(qv * qv), sk = warp_sum(kv * kv);
        if (lane == 0) { red[warp * 2 * T + t] = sq; red[warp * 2 * T + T + t] = sk; }
    }
    bar_named(1, G_THREADS);
    for (int t = 0; t < T; ++t) {
        float sq = 0.f, sk = 0.f;
        for (int w = 0; w < 4; ++w) { sq += red[w * 2 * T + t]; sk += red[w * 2 * T + T + t]; }
        xq[t * G_HS + tid] *= rsqrtf(sq + 1e-6f);
        xk[t * G_HS + tid] *= rsqrtf(sk + 1e-6f);
    }
    bar_named(1, G_THREADS);
    const int part = warp, col = qq * G_QC + lane;
    const size_t soff = (size_t) lv * G_HS * G_HS + (size_t) part * 32 * G_HS + col;
    float s[32];
    int have = -2;
    const float scale = rsqrtf((float) G_HS);
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        const int par = parent ? parent[t] : t - 1;
        if (par != have) {
            const float* src = L.S + (size_t) (par < 0 ? cur : (cur + 1 + par) % NS) * ssz + soff;
#pragma unroll
            for (int r = 0; r < 32; ++r) s[r] = src[(size_t) r * G_HS];
        }
        const float gv = gates[2 * t], bv = gates[2 * t + 1];
        const float* kt = xk + t * G_HS + part * 32;
        const float* qt = xq + t * G_HS + part * 32;
        float kvd = 0.f;
#pragma unroll
        for (int r = 0; r < 32; ++r) kvd = fmaf(s[r], kt[r], kvd);
        float* kr = kred + (t & 1) * 4 * G_QC;
        kr[part * G_QC + lane] = kvd;
        bar_named(1, G_THREADS);
        const float kvs = (kr[lane] + kr[G_QC + lane]) + (kr[2 * G_QC + lane] + kr[3 * G_QC + lane]);
        const float delta = (vs[t * G_QC + lane] - gv * kvs) * bv;
        float at = 0.f;
        float* dst = L.S + (size_t) ((cur + 1 + t) % NS) * ssz + soff;
#pragma unroll
        for (int r = 0; r < 32; ++r) {
            s[r] = fmaf(kt[r], delta, gv * s[r]);
            at = fmaf(s[r], qt[r], at);
            dst[(size_t) r * G_HS] = s[r];
        }
        ared[(t * 4 + part) * G_QC + lane] = at;
        have = t;
    }
    bar_named(1, G_THREADS);
    for (int t = warp; t < T; t += 4) {
        const float o = ((ared[(t * 4 + 0) * G_QC + lane] + ared[(t * 4 + 1) * G_QC + lane]) +
                         (ared[(t * 4 + 2) * G_QC + lane] + ared[(t * 4 + 3) * G_QC + lane])) * scale;
        P.gdn_o[(size_t) t * nv * G_HS + lv * G_HS + col] = o;
        const float sq = warp_sum(o * o);
        if (lane == 0) P.gdn_sq[((size_t) t * nv + lv) * 4 + qq] = sq;
    }
    bar_named(1, G_THREADS);   // the scratch is free for the block's next item
}

// ------------------------------------------------------------------------------------------------ attention
constexpr int A_CH = 32, A_ROWS = 5, A_THREADS = 256, A_MAXQ = 8;

// norm + rotary + append for item (head h of nq + 2 nkv, row t): 256 threads (attn.cu k_attn_prep_append)
__device__ void attn_prep_item(const Smem& sm, int tid, const StepLayer& L, int item, float* scratch) {
    const StepParams& P = *sm.P;
    const int nq = P.nq, nkv = P.nkv, hd = P.hd, nrot = P.nrot, heads = nq + 2 * nkv;
    const int t = item / heads, h = item % heads, i = tid, ld = P.proj_ld;
    const int pos0 = *P.pos0, pos = pos0 + P.depth[t];
    float* qg = P.proj;
    float* k = P.proj + nq * 2 * hd;
    const float* v = k + nkv * hd;
    float* xrow = scratch;         // hd floats
    float* red = scratch + hd;     // 8
    const size_t crow = (size_t) (pos0 + t) * nkv * hd;
    if (h >= nq + nkv) {
        const int kvh = h - nq - nkv;
        L.vc[crow + (size_t) kvh * hd + i] = __float2half_rn(v[(size_t) t * ld + (size_t) kvh * hd + i]);
        return;
    }
    float* x = h < nq ? qg + (size_t) t * ld + (size_t) h * 2 * hd : k + (size_t) t * ld + (size_t) (h - nq) * hd;
    const float* w = h < nq ? L.qn : L.kn;
    const float val = x[i];
    float ss = warp_sum(val * val);
    if ((i & 31) == 0) red[i >> 5] = ss;
    bar_named(2, A_THREADS);
    ss = 0.f;
    for (int j = 0; j < hd / 32; ++j) ss += red[j];
    xrow[i] = val * rsqrtf(ss / (float) hd + P.eps) * w[i];
    bar_named(2, A_THREADS);
    float y = xrow[i];
    if (i < nrot) {
        const int pr = i < nrot / 2 ? i : i - nrot / 2;
        const float fe = (float) pow((double) P.rope_base, -2.0 * (double) pr / (double) nrot);
        float sn, cs;
        sincosf((float) pos * fe, &sn, &cs);
        const float x0 = xrow[pr], x1 = xrow[pr + nrot / 2];
        y = i < nrot / 2 ? x0 * cs - x1 * sn : x0 * sn + x1 * cs;
    }
    x[i] = y;
    if (h >= nq) L.kc[crow + (size_t) (h - nq) * hd + i] = __float2half_rn(y);
    bar_named(2, A_THREADS);
}

// split-K attention partial for item (split s of S, KV head, row group): 256 threads, scratch = the weight ring
__device__ void attn_part_item(const Smem& sm, int tid, const StepLayer& L, int s, int S, int kvh, int r0) {
    const StepParams& P = *sm.P;
    const int T = P.T, nq = P.nq, nkv = P.nkv, hd = P.hd, ldq = P.proj_ld;
    const int nr = min(A_ROWS, T - r0), qpk = nq / nkv, NQ = nr * qpk;
    const int warp = tid >> 5, lane = tid & 31;
    const int pos0 = *P.pos0, ctx = pos0 + T;
    const int KS = hd + 8;
    const float* qg = P.proj;
    const int* parent = P.tree ? P.parent : nullptr;
    float* qs = reinterpret_cast<float*>(sm.ring);
    __half* Ks = reinterpret_cast<__half*>(qs + A_ROWS * A_MAXQ * hd);
    __half* Vs = Ks + A_CH * KS;
    float* es = reinterpret_cast<float*>(Vs + A_CH * hd);
    float* fs = es + A_ROWS * A_MAXQ * A_CH;
    float* ms = fs + A_ROWS * A_MAXQ;
    float* zs = ms + A_ROWS * A_MAXQ;
    unsigned* see = reinterpret_cast<unsigned*>(zs + A_ROWS * A_MAXQ);
    const int nch = (ctx + A_CH - 1) / A_CH;
    const int c0 = (int) ((long long) nch * s / S), c1 = (int) ((long long) nch * (s + 1) / S);
    if (c0 >= c1) {
        if (tid < NQ) {
            const int r = tid / qpk, hh = tid % qpk;
            P.att_mz[((size_t) (r0 + r) * nq + kvh * qpk + hh) * S + s] = AttPartialS{-INFINITY, 0.f};
        }
        return;
    }
    for (int i0 = tid; i0 < NQ * hd / 4; i0 += 8 * A_THREADS) {
        float4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = i0 + j * A_THREADS;
            if (i < NQ * hd / 4) {
                const int qi = i / (hd / 4), d4 = i % (hd / 4), r = qi / qpk, hh = qi % qpk;
                v[j] = *reinterpret_cast<const float4*>(qg + (size_t) (r0 + r) * ldq + (size_t) (kvh * qpk + hh) * 2 * hd + d4 * 4);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = i0 + j * A_THREADS;
            if (i < NQ * hd / 4) reinterpret_cast<float4*>(qs)[i] = v[j];
        }
    }
    if (tid < NQ) { ms[tid] = -INFINITY; zs[tid] = 0.f; }
    if (tid < nr) {
        unsigned m = 0;
        for (int a = r0 + tid; a >= 0; a = parent ? parent[a] : a - 1) m |= 1u << a;
        see[tid] = m;
    }
    float acc[A_ROWS * A_MAXQ];
#pragma unroll
    for (int i = 0; i < A_ROWS * A_MAXQ; ++i) acc[i] = 0.f;
    const float scale = rsqrtf((float) hd);
    for (int c = c0; c < c1; ++c) {
        const int p0 = c * A_CH, np = min(A_CH, ctx - p0);
        bar_named(2, A_THREADS);
        {
            constexpr int NL = A_CH * 256 / 8 / A_THREADS;
            uint4 kv4[NL], vv4[NL];
#pragma unroll
            for (int j = 0; j < NL; ++j) {
                const int i = tid + j * A_THREADS, pp = i / (hd / 8), d8 = i % (hd / 8);
                kv4[j] = vv4[j] = make_uint4(0, 0, 0, 0);
                if (pp < np) {
                    const size_t g = ((size_t) (p0 + pp) * nkv + kvh) * hd + d8 * 8;
                    kv4[j] = *reinterpret_cast<const uint4*>(L.kc + g);
                    vv4[j] = *reinterpret_cast<const uint4*>(L.vc + g);
                }
            }
#pragma unroll
            for (int j = 0; j < NL; ++j) {
                const int i = tid + j * A_THREADS, pp = i / (hd / 8), d8 = i % (hd / 8);
                *reinterpret_cast<uint4*>(Ks + pp * KS + d8 * 8) = kv4[j];
                *reinterpret_cast<uint4*>(Vs + pp * hd + d8 * 8) = vv4[j];
            }
        }
        bar_named(2, A_THREADS);
        for (int qi = warp; qi < NQ; qi += A_THREADS / 32) {
            const float* q = qs + qi * hd;
            const __half* kr = Ks + lane * KS;
            float sacc = 0.f;
            for (int d = 0; d < hd; d += 8) {
                const uint4 kk = *reinterpret_cast<const uint4*>(kr + d);
                const float4 q0 = *reinterpret_cast<const float4*>(q + d), q1 = *reinterpret_cast<const float4*>(q + d + 4);
                const float2 k0 = __half22float2(*reinterpret_cast<const __half2*>(&kk.x));
                const float2 k1 = __half22float2(*reinterpret_cast<const __half2*>(&kk.y));
                const float2 k2 = __half22float2(*reinterpret_cast<const __half2*>(&kk.z));
                const float2 k3 = __half22float2(*reinterpret_cast<const __half2*>(&kk.w));
                sacc = fmaf(q0.x, k0.x, sacc); sacc = fmaf(q0.y, k0.y, sacc);
                sacc = fmaf(q0.z, k1.x, sacc); sacc = fmaf(q0.w, k1.y, sacc);
                sacc = fmaf(q1.x, k2.x, sacc); sacc = fmaf(q1.y, k2.y, sacc);
                sacc = fmaf(q1.z, k3.x, sacc); sacc = fmaf(q1.w, k3.y, sacc);
            }
            const int p = p0 + lane, r = qi / qpk;
            const bool vis = lane < np && (p < pos0 || ((see[r] >> (p - pos0)) & 1u));
            const float sv = vis ? sacc * scale : -INFINITY;
            const float mo = ms[qi], mn = fmaxf(mo, warp_max(sv));
            const float w = sv == -INFINITY ? 0.f : expf(sv - mn);
            const float fsc = mo == -INFINITY ? 0.f : expf(mo - mn);
            const float zn = zs[qi] * fsc + warp_sum(w);
            es[qi * A_CH + lane] = w;
            __syncwarp();
            if (lane == 0) { ms[qi] = mn; zs[qi] = zn; fs[qi] = fsc; }
        }
        bar_named(2, A_THREADS);
        {
            const int d = tid;
#pragma unroll
            for (int qi = 0; qi < A_ROWS * A_MAXQ; ++qi)
                if (qi < NQ) acc[qi] *= fs[qi];
            for (int pp = 0; pp < A_CH; pp += 4) {
                const float v0 = __half2float(Vs[pp * hd + d]), v1 = __half2float(Vs[(pp + 1) * hd + d]);
                const float v2 = __half2float(Vs[(pp + 2) * hd + d]), v3 = __half2float(Vs[(pp + 3) * hd + d]);
#pragma unroll
                for (int qi = 0; qi < A_ROWS * A_MAXQ; ++qi)
                    if (qi < NQ) {
                        const float4 e4 = *reinterpret_cast<const float4*>(es + qi * A_CH + pp);
                        acc[qi] = fmaf(e4.x, v0, acc[qi]);
                        acc[qi] = fmaf(e4.y, v1, acc[qi]);
                        acc[qi] = fmaf(e4.z, v2, acc[qi]);
                        acc[qi] = fmaf(e4.w, v3, acc[qi]);
                    }
            }
        }
    }
    bar_named(2, A_THREADS);
#pragma unroll
    for (int qi = 0; qi < A_ROWS * A_MAXQ; ++qi)
        if (qi < NQ) {
            const int r = qi / qpk, hh = qi % qpk;
            const size_t slot = ((size_t) (r0 + r) * nq + kvh * qpk + hh) * S + s;
            P.att_acc[slot * hd + tid] = acc[qi];
        }
    if (tid < NQ) {
        const int r = tid / qpk, hh = tid % qpk;
        P.att_mz[((size_t) (r0 + r) * nq + kvh * qpk + hh) * S + s] = AttPartialS{ms[tid], zs[tid]};
    }
    bar_named(2, A_THREADS);
}

// merge of the splits of item (head, row) + the sigmoid gate -> mix: 256 threads
__device__ void attn_merge_item(const Smem& sm, int tid, int item, int S, float* scratch) {
    const StepParams& P = *sm.P;
    const int nq = P.nq, hd = P.hd, t = item / nq, h = item % nq, i = tid;
    float* sm_m = scratch;
    float* sm_w = scratch + 256;
    float* sm_z = scratch + 512;
    const size_t base = ((size_t) t * nq + h) * S;
    AttPartialS p = AttPartialS{-INFINITY, 0.f};
    if (i < S) p = P.att_mz[base + i];
    sm_m[i] = i < S ? p.m : -INFINITY;
    bar_named(2, A_THREADS);
    float mx = -INFINITY;
    for (int s = 0; s < S; ++s) mx = fmaxf(mx, sm_m[s]);
    sm_w[i] = i < S && p.m != -INFINITY ? expf(p.m - mx) : 0.f;
    sm_z[i] = i < S && p.m != -INFINITY ? expf(p.m - mx) * p.z : 0.f;
    bar_named(2, A_THREADS);
    float z = 0.f;
    for (int s = 0; s < S; ++s) z += sm_z[s];
    float acc = 0.f;
    for (int s0 = 0; s0 < S; s0 += 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = s0 + j < S && sm_w[s0 + j] != 0.f ? P.att_acc[(base + s0 + j) * hd + i] : 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc = fmaf(s0 + j < S ? sm_w[s0 + j] : 0.f, v[j], acc);
    }
    const float gate = P.proj[(size_t) t * P.proj_ld + (size_t) h * 2 * hd + hd + i];
    P.mix[((size_t) t * nq + h) * hd + i] = acc / z * sigmoidf_(gate);
    bar_named(2, A_THREADS);
}

// ------------------------------------------------------------------------------------------------ head tail
__device__ __forceinline__ uint32_t fkey_(float v) {
    const uint32_t b = __float_as_uint(v);
    return b & 0x80000000u ? ~b : b | 0x80000000u;
}
// argmax of row t (k_argmax, engine/src/kernels.cu:1056-1083): value first, the lower index on ties
__device__ void argmax_row(const Smem& sm, int tid, int t) {
    const StepParams& P = *sm.P;
    const float* l = P.logits + (size_t) t * P.V;
    unsigned long long* red = reinterpret_cast<unsigned long long*>(sm.misc + 256);
    unsigned long long best = 0;
    bool bad = false;
    const int V4 = P.V / 4;
    for (int i0 = tid; i0 < V4; i0 += 4 * STEP_THREADS) {
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            v[j] = i0 + STEP_THREADS * j < V4 ? reinterpret_cast<const float4*>(l)[i0 + STEP_THREADS * j] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = i0 + STEP_THREADS * j;
            if (i >= V4) continue;
            const float e[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                bad |= !isfinite(e[c]);
                const unsigned long long k = ((unsigned long long) fkey_(e[c]) << 32) | (uint32_t) ~(4 * i + c);
                best = k > best ? k : best;
            }
        }
    }
    for (int i = 4 * V4 + tid; i < P.V; i += STEP_THREADS) {
        const float v = l[i];
        bad |= !isfinite(v);
        const unsigned long long k = ((unsigned long long) fkey_(v) << 32) | (uint32_t) ~i;
        best = k > best ? k : best;
    }
    for (int o = 16; o; o >>= 1) {
        const unsigned long long ok = __shfl_xor_sync(0xffffffffu, best, o);
        best = ok > best ? ok : best;
    }
    if ((tid & 31) == 0) red[tid >> 5] = best;
    if (bad) atomicOr(P.err, (unsigned) FNX_ERR_LOGITS);
    __syncthreads();
    if (tid < 32) {
        best = tid < NWARP ? red[tid] : 0ull;
        for (int o = 16; o; o >>= 1) {
            const unsigned long long ok = __shfl_xor_sync(0xffffffffu, best, o);
            best = ok > best ? ok : best;
        }
        if (tid == 0) {
            P.best_i[t] = (int) ~(uint32_t) best;
            const uint32_t kk = (uint32_t) (best >> 32);
            P.best_v[t] = __uint_as_float(kk & 0x80000000u ? kk & 0x7fffffffu : ~kk);
        }
    }
    __syncthreads();
}

// greedy acceptance over the tree (engine/src/session.cpp:573): one thread
__device__ void accept_greedy_one(const StepParams& P) {
    const int* parent = P.tree ? P.parent : nullptr;
    int cur = 0, n = 0;
    for (;;) {
        P.result[1 + n] = cur;
        P.result[1 + FNX_MAX_ROWS + n] = P.best_i[cur];
        ++n;
        int next = -1;
        for (int c = cur + 1; c < P.T; ++c)
            if ((parent ? parent[c] : c - 1) == cur && P.tok[c] == P.best_i[cur]) { next = c; break; }
        if (next < 0) break;
        cur = next;
    }
    P.result[0] = n;
}

// ------------------------------------------------------------------------------------------------ the kernel
#define STAMP() stamp(f, 1)

template <int NG>
__global__ void __launch_bounds__(STEP_THREADS, 1) k_verify_step(const StepParams* __restrict__ gp) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int tid = threadIdx.x;
    Smem sm;
    {
        uint8_t* b = smem_raw;
        sm.table = b; b += CORE_TABLE_BYTES;
        sm.ring = b; b += NST * CORE_STEP_BYTES;
        sm.xq = b; b += XQ_BYTES;
        sm.part = reinterpret_cast<float*>(b); b += PART_BYTES;
        sm.misc = reinterpret_cast<float*>(b); b += MISC_BYTES;
        sm.bars = reinterpret_cast<uint64_t*>(b); b += 64;
        sm.P = reinterpret_cast<StepParams*>(b);
    }
    for (int i = tid; i < (int) (sizeof(StepParams) / 4); i += STEP_THREADS) reinterpret_cast<uint32_t*>(sm.P)[i] = reinterpret_cast<const uint32_t*>(gp)[i];
    core_fill_table(sm.table, tid, STEP_THREADS);
    if (tid == 0) {
        for (int i = 0; i < 2 * NST; ++i) mbar_init(&sm.bars[i], 1);
        fence_barrier_init();
        sm.misc[500] = 0.f;
    }
    __syncthreads();
    const StepParams& P = *sm.P;
    Flow f;
    if (P.prof && blockIdx.x == 0 && tid == 0) f.prof = P.prof;
    const int T = P.T, H = P.H;
    const int warpgroup_gdn = tid < G_THREADS, warpgroup_att = tid < A_THREADS;
    STAMP();

    auto dense_work = [&](const uint8_t* W, int rows, int K, float* out, int ldo, int accumulate) {
        MatWork w{};
        w.W = W; w.njobs = 1; w.rows = rows; w.K = K; w.out = out; w.ldo = ldo; w.accumulate = accumulate; w.T = T;
        return w;
    };

    // ---- tokens -> residual rows; the first layer's input image
    embed_phase(sm, tid);
    if (last_block(sm, f, 1, tid)) build_image(sm, tid, T, H, 0, P.R, H, P.layers[0].norm1, P.eps, nullptr, nullptr, nullptr, 0, nullptr, 0);
    int pre = 0;
    {
        const MatWork w = dense_work(P.layers[0].w_in, P.layers[0].in_rows, H, P.proj, P.proj_ld, 0);
        pre = mat_preissue(sm, f, tid, M_DENSE, w);
    }
    grid_barrier(sm, f, tid);
    STAMP();

    for (int l = 0; l < P.n_layer; ++l) {
        const StepLayer& L = P.layers[l];
        // ---- input projection
        {
            const MatWork w = dense_work(L.w_in, L.in_rows, H, P.proj, P.proj_ld, 0);
            mat_phase<NG, M_DENSE>(sm, f, tid, w, pre, true);
        }
        grid_barrier(sm, f, tid);
        STAMP();
        const int mixK = L.attn ? P.nq * P.hd : P.nv * P.hs;
        const MatWork wout = dense_work(L.w_out, H, mixK, P.R, H, 1);
        if (L.attn) {
            const int heads = P.nq + 2 * P.nkv;
            for (int item = blockIdx.x; item < T * heads; item += gridDim.x)
                if (warpgroup_att) attn_prep_item(sm, tid, L, item, reinterpret_cast<float*>(sm.xq));
            grid_barrier(sm, f, tid);
            const int S = gridDim.x / P.nkv > 0 ? gridDim.x / P.nkv : 1, groups = (T + A_ROWS - 1) / A_ROWS;
            for (int item = blockIdx.x; item < S * P.nkv * groups; item += gridDim.x)
                if (warpgroup_att) attn_part_item(sm, tid, L, item % S, S, (item / S) % P.nkv, (item / (S * P.nkv)) * A_ROWS);
            grid_barrier(sm, f, tid);
            for (int item = blockIdx.x; item < T * P.nq; item += gridDim.x)
                if (warpgroup_att) attn_merge_item(sm, tid, item, S, reinterpret_cast<float*>(sm.xq));
            if (last_block(sm, f, 2, tid)) build_image(sm, tid, T, mixK, 0, P.mix, mixK, nullptr, P.eps, nullptr, nullptr, nullptr, 0, nullptr, 0);
        } else {
            for (int item = blockIdx.x; item < P.nv * G_Q; item += gridDim.x)
                if (warpgroup_gdn) gdn_item(sm, tid, L, item);
            if (last_block(sm, f, 2, tid))
                build_image(sm, tid, T, mixK, 1, P.gdn_o, mixK, nullptr, P.eps, nullptr, P.gdn_sq, P.proj + (2 * P.nk + P.nv) * P.hs, P.proj_ld, L.gnorm, P.hs);
        }
        pre = mat_preissue(sm, f, tid, M_DENSE, wout);
        grid_barrier(sm, f, tid);
        STAMP();
        // ---- output projection into the residual; then the FFN's input image and the router's f32 rows
        mat_phase<NG, M_DENSE>(sm, f, tid, wout, pre, true);
        if (last_block(sm, f, 3, tid)) build_image(sm, tid, T, H, 0, P.R, H, L.norm2, P.eps, P.xnorm, nullptr, nullptr, 0, nullptr, 0);
        grid_barrier(sm, f, tid);
        STAMP();
        // ---- router logits; the last block routes
        router_phase(sm, f, tid, L);
        if (last_block(sm, f, 4, tid)) route_finalize(sm, tid);
        grid_barrier(sm, f, tid);
        STAMP();
        // ---- routed + shared experts: gate|up + SwiGLU, then down
        MatWork wg{};
        wg.W = L.wgu; wg.expert_stride = P.gu_bytes; wg.Wsh = L.wsh_gu; wg.E = P.E; wg.jobs = P.jobs; wg.njobs = *P.njobs;
        wg.rows = P.F; wg.K = H; wg.out = P.hbuf; wg.ldo = P.F; wg.T = T;
        mat_phase<1, M_GATEUP>(sm, f, tid, wg, 0, true);
        MatWork wd{};
        wd.W = L.wdn; wd.expert_stride = P.dn_bytes; wd.Wsh = L.wsh_dn; wd.E = P.E; wd.jobs = P.jobs; wd.njobs = wg.njobs;
        wd.rows = H; wd.K = P.F; wd.h = P.hbuf; wd.out = P.part; wd.ldo = H; wd.T = T;
        pre = mat_preissue(sm, f, tid, M_DOWN, wd);
        grid_barrier(sm, f, tid);
        STAMP();
        mat_phase<1, M_DOWN>(sm, f, tid, wd, pre, false);
        grid_barrier(sm, f, tid);
        STAMP();
        // ---- combine into the residual; the next matrix phase's image and first steps
        combine_phase(sm, tid);
        const bool more = l + 1 < P.n_layer;
        if (last_block(sm, f, 5, tid)) build_image(sm, tid, T, H, 0, P.R, H, more ? P.layers[l + 1].norm1 : P.out_norm, P.eps, nullptr, nullptr, nullptr, 0, nullptr, 0);
        {
            const MatWork w = more ? dense_work(P.layers[l + 1].w_in, P.layers[l + 1].in_rows, H, P.proj, P.proj_ld, 0) : dense_work(P.head, P.V, H, P.logits, P.V, 0);
            pre = mat_preissue(sm, f, tid, M_DENSE, w);
        }
        grid_barrier(sm, f, tid);
        STAMP();
    }
    // ---- head, argmax, acceptance
    {
        const MatWork w = dense_work(P.head, P.V, H, P.logits, P.V, 0);
        mat_phase<NG, M_DENSE>(sm, f, tid, w, pre, true);
    }
    grid_barrier(sm, f, tid);
    STAMP();
    for (int t = blockIdx.x; t < T; t += gridDim.x) argmax_row(sm, tid, t);
    if (last_block(sm, f, 6, tid) && tid == 0) accept_greedy_one(P);
    STAMP();
    if (f.prof) f.prof[0] = (unsigned long long) f.nstamp;
}

int step_launch(const StepParams* dev_params, int T, unsigned* sync_words, cudaStream_t st) {
    if (T < 1 || T > 8) return fail(FNX_E_ARG, "step kernel: %d rows (1..8)", T);
    static bool configured = false;
    const size_t smem = step_smem_bytes();
    if (!configured) {
        FNX_CUDA_OK(cudaFuncSetAttribute(k_verify_step<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
        FNX_CUDA_OK(cudaFuncSetAttribute(k_verify_step<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
        configured = true;
    }
    FNX_CUDA_OK(cudaMemsetAsync(sync_words, 0, sizeof(unsigned) * STEP_SYNC_WORDS, st));
    void* args[1] = {(void*) &dev_params};
    const void* fn = T <= 4 ? (const void*) k_verify_step<1> : (const void*) k_verify_step<2>;
    FNX_CUDA_OK(cudaLaunchCooperativeKernel(fn, dim3(sm_count()), dim3(STEP_THREADS), args, smem, st));
    return FNX_OK;
}

}  // namespace fnxb
