// Gated DeltaNet core for a verify window, one launch.
//
// Replaces gdn_core / k_gdn_core (engine/src/kernels.hpp:97-99, engine/src/gdn_core.cuh:20-225; unfused statement
// engine/src/kernels.cu:422-506): conv4 + SiLU over the q|k|v channels, L2 norms of q and k, the gates, the delta
// rule on the fp32 state, the gated RMS norm of the output.  Differences by design:
//   - rows form a tree (parent[t]); row t starts from its parent's state and conv history, not from row t - 1's;
//   - the state after every row, and the history keeping it would leave, go to ring slot (*cur + 1 + t) % NS
//     instead of the snap / hsnap buffers, so that a commit is a change of *cur and copies nothing
//     (engine/src/engine_common.cu:710-754 copies the kept snapshot back);
//   - the four blocks that share a value head form a thread-block cluster and add up the head's square sums
//     through distributed shared memory, where the reference uses a global scratch buffer and atomic counters.
#include <cooperative_groups.h>

#include "fnx_common.cuh"

namespace cg = cooperative_groups;

namespace fnxb {

constexpr int GDN_HS = 128, GDN_Q = 4, GDN_QC = GDN_HS / GDN_Q, GDN_THREADS = 128;

// One block of the (value head, column quarter) grid: the cluster's four blocks share a value head.
__device__ __forceinline__ void gdn_body(const float* __restrict__ qkvz, int stride, const float* __restrict__ ab, int ldab, float* __restrict__ hist_pool,
                                         const float* __restrict__ convw, const float* __restrict__ dt, const float* __restrict__ a_,
                                         const float* __restrict__ nw, float* __restrict__ S_pool, int cur, int NS, const int* __restrict__ parent,
                                         float* __restrict__ y, int nk, int nv, int T, float eps, float* sm, bool last_only = false) {
    // (last_only: a prompt's window, every row of which is kept: only the last row's state and history are written)
    cg::cluster_group cluster = cg::this_cluster();
    const int lv = blockIdx.x / GDN_Q, qq = blockIdx.x % GDN_Q, kh = lv % nk, tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int ch = (2 * nk + nv) * GDN_HS;
    const size_t hsz = (size_t) 3 * ch, ssz = (size_t) nv * GDN_HS * GDN_HS;
    float* xq = sm;                              // [T][HS] q after conv, silu, norm
    float* xk = xq + (size_t) T * GDN_HS;        // [T][HS]
    float* vs = xk + (size_t) T * GDN_HS;        // [T][QC]
    float* gates = vs + (size_t) T * GDN_QC;     // [T][2]
    float* kred = gates + 2 * T;                 // [2][4][QC]
    float* ared = kred + 2 * 4 * GDN_QC;         // [T][4][QC]
    float* osum = ared + (size_t) T * 4 * GDN_QC;   // [T] this block's square sums (read by the cluster)
    float* red = osum + T;                       // [4][2 T]
    float* xin = red + 8 * T;                    // [T + 3][2 HS + QC] conv inputs
    int* anc = reinterpret_cast<int*>(xin + (size_t) (T + 3) * (2 * GDN_HS + GDN_QC));   // [T][3]
    const float* hin = hist_pool + (size_t) cur * hsz;
    // the starting state of the warp's key rows is on its way before anything else: row 0's parent is the root
    const int part = warp, col = qq * GDN_QC + lane;
    const size_t soff = (size_t) lv * GDN_HS * GDN_HS + (size_t) part * 32 * GDN_HS + col;
    float s[32];
    {
        const float* src = S_pool + (size_t) cur * ssz + soff;
#pragma unroll
        for (int r = 0; r < 32; ++r) s[r] = src[(size_t) r * GDN_HS];
    }
    if (tid < T) {
        const float* abt = ab + (size_t) tid * ldab;
        const float x = abt[lv] + dt[lv];
        gates[2 * tid] = expf((x > 20.0f ? x : log1pf(expf(x))) * a_[lv]);
        gates[2 * tid + 1] = 1.0f / (1.0f + expf(-abt[nv + lv]));
    }
    // ---- the conv inputs this block needs, staged with every load in flight at once: rows 0..2 = the starting
    // history (oldest first), row 3 + t = window row t; columns = the head's q (HS), k (HS), this block's v (QC)
    constexpr int NC = 2 * GDN_HS + GDN_QC;
    auto chan = [&](int e) {
        return e < GDN_HS ? kh * GDN_HS + e : e < 2 * GDN_HS ? nk * GDN_HS + kh * GDN_HS + (e - GDN_HS) : 2 * nk * GDN_HS + lv * GDN_HS + qq * GDN_QC + (e - 2 * GDN_HS);
    };
    constexpr int SB = 20;   // loads in flight per thread: a 5-row window's conv inputs in one round
    // the conv weights of this thread's channels ride along
    float4 cw3[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const int e = tid + k * GDN_THREADS;
        cw3[k] = e < NC ? *reinterpret_cast<const float4*>(convw + chan(e) * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int i0 = tid; i0 < (T + 3) * NC; i0 += SB * GDN_THREADS) {
        float v[SB];
#pragma unroll
        for (int j = 0; j < SB; ++j) {
            const int i = i0 + j * GDN_THREADS;
            v[j] = 0.f;
            if (i < (T + 3) * NC) {
                const int r = i / NC, c = chan(i % NC);
                v[j] = r < 3 ? hin[(size_t) r * ch + c] : qkvz[(size_t) (r - 3) * stride + c];
            }
        }
#pragma unroll
        for (int j = 0; j < SB; ++j) {
            const int i = i0 + j * GDN_THREADS;
            if (i < (T + 3) * NC) xin[i] = v[j];
        }
    }
    // the three rows before each window row on its path, as rows of xin (past the root: the history)
    if (tid < T) {
        int a = tid;
        for (int k = 1; k <= 3; ++k) {
            if (a >= 0) a = parent ? parent[a] : a - 1;
            else --a;                      // a = -1 - (rows past the root)
            anc[tid * 3 + k - 1] = a >= 0 ? 3 + a : 3 + a;   // -1 -> row 2 (newest history), -2 -> row 1, -3 -> row 0
        }
    }
    __syncthreads();
#pragma unroll
    for (int k3 = 0; k3 < 3; ++k3) {
        const int e = tid + k3 * GDN_THREADS;
        if (e >= NC) continue;
        const int part = e < GDN_HS ? 0 : e < 2 * GDN_HS ? 1 : 2, i = part < 2 ? e - part * GDN_HS : e - 2 * GDN_HS;
        const int c = chan(e);
        const float4 cw = cw3[k3];
        const float w0 = cw.x, w1 = cw.y, w2 = cw.z, w3 = cw.w;
        const bool writes = part == 2 || (lv < nk && qq == 0);   // one block per channel writes its history
        for (int t = 0; t < T; ++t) {
            const float x3 = xin[anc[t * 3 + 2] * NC + e], x2 = xin[anc[t * 3 + 1] * NC + e], x1 = xin[anc[t * 3] * NC + e];
            const float x0 = xin[(3 + t) * NC + e];
            const float x = w0 * x3 + w1 * x2 + w2 * x1 + w3 * x0;
            const float v = x / (1.0f + expf(-x));
            if (part == 0) xq[t * GDN_HS + i] = v;
            else if (part == 1) xk[t * GDN_HS + i] = v;
            else vs[t * GDN_QC + i] = v;
            if (writes && (!last_only || t == T - 1)) {
                float* hout = hist_pool + (size_t) ((cur + 1 + t) % NS) * hsz;
                hout[c] = x2;
                hout[ch + c] = x1;
                hout[2 * ch + c] = x0;
            }
        }
    }
    __syncthreads();
    // ---- L2 norms of q and k per row: thread = element (HS == GDN_THREADS)
    for (int t = 0; t < T; ++t) {
        const float qv = xq[t * GDN_HS + tid], kv = xk[t * GDN_HS + tid];
        const float sq = warp_sum(qv * qv), sk = warp_sum(kv * kv);
        if (lane == 0) { red[warp * 2 * T + t] = sq; red[warp * 2 * T + T + t] = sk; }
    }
    __syncthreads();
    for (int t = 0; t < T; ++t) {
        float sq = 0.f, sk = 0.f;
        for (int w = 0; w < 4; ++w) { sq += red[w * 2 * T + t]; sk += red[w * 2 * T + T + t]; }
        xq[t * GDN_HS + tid] *= rsqrtf(sq + 1e-6f);
        xk[t * GDN_HS + tid] *= rsqrtf(sk + 1e-6f);
    }
    __syncthreads();
    // ---- the delta rule: warp `part` holds key rows [32 part, +32) of the block's QC value columns, lane = column
    int have = -1;   // the row whose result the registers hold (-1: the starting state)
    const float scale = rsqrtf((float) GDN_HS);
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        const int par = parent ? parent[t] : t - 1;
        if (par != have) {
            const float* src = S_pool + (size_t) (par < 0 ? cur : (cur + 1 + par) % NS) * ssz + soff;
#pragma unroll
            for (int r = 0; r < 32; ++r) s[r] = src[(size_t) r * GDN_HS];
        }
        const float gv = gates[2 * t], bv = gates[2 * t + 1];
        const float* kt = xk + t * GDN_HS + part * 32;
        const float* qt = xq + t * GDN_HS + part * 32;
        float kvd = 0.f;
#pragma unroll
        for (int r = 0; r < 32; ++r) kvd = fmaf(s[r], kt[r], kvd);
        float* kr = kred + (t & 1) * 4 * GDN_QC;
        kr[part * GDN_QC + lane] = kvd;
        __syncthreads();
        const float kvs = (kr[lane] + kr[GDN_QC + lane]) + (kr[2 * GDN_QC + lane] + kr[3 * GDN_QC + lane]);
        const float delta = (vs[t * GDN_QC + lane] - gv * kvs) * bv;
        float at = 0.f;
        float* dst = S_pool + (size_t) ((cur + 1 + t) % NS) * ssz + soff;
        const bool keep = !last_only || t == T - 1;
#pragma unroll
        for (int r = 0; r < 32; ++r) {
            s[r] = fmaf(kt[r], delta, gv * s[r]);
            at = fmaf(s[r], qt[r], at);
            if (keep) dst[(size_t) r * GDN_HS] = s[r];
        }
        ared[(t * 4 + part) * GDN_QC + lane] = at;
        have = t;
    }
    __syncthreads();
    // ---- this block's outputs and their square sums per row
    float ov[FNX_MAX_ROWS / 4];   // warp w keeps rows w, w + 4, ... of column `lane`
    for (int t = warp, j = 0; t < T; t += 4, ++j) {
        const float o = ((ared[(t * 4 + 0) * GDN_QC + lane] + ared[(t * 4 + 1) * GDN_QC + lane]) +
                         (ared[(t * 4 + 2) * GDN_QC + lane] + ared[(t * 4 + 3) * GDN_QC + lane])) * scale;
        ov[j] = o;
        const float sq = warp_sum(o * o);
        if (lane == 0) osum[t] = sq;
    }
    // the gate inputs z, fetched while the cluster gathers (they do not depend on it)
    float zv[FNX_MAX_ROWS / 4];
    for (int t = warp, j = 0; t < T; t += 4, ++j) zv[j] = qkvz[(size_t) t * stride + ch + lv * GDN_HS + col];
    const float nwv = nw[col];
    cluster.sync();
    // every block's T square sums into this block's shared memory, one remote read per thread
    float* msum = red;   // [T] (red is free by now)
    for (int i = tid; i < T * GDN_Q; i += GDN_THREADS) kred[i] = cluster.map_shared_rank(osum, i % GDN_Q)[i / GDN_Q];
    __syncthreads();
    if (tid < T) msum[tid] = ((kred[tid * GDN_Q] + kred[tid * GDN_Q + 1]) + (kred[tid * GDN_Q + 2] + kred[tid * GDN_Q + 3])) / (float) GDN_HS;
    __syncthreads();
    for (int t = warp, j = 0; t < T; t += 4, ++j)
        y[(size_t) t * nv * GDN_HS + lv * GDN_HS + col] = ov[j] * rsqrtf(msum[t] + eps) * nwv / (1.0f + expf(-zv[j]));
    cluster.sync();   // no block may leave while a neighbour still reads its shared memory
}

__global__ void __cluster_dims__(GDN_Q, 1, 1) __launch_bounds__(GDN_THREADS)
    k_gdn_core(const float* __restrict__ qkvz, int stride, const float* __restrict__ ab, int ldab, float* __restrict__ hist_pool,
               const float* __restrict__ convw, const float* __restrict__ dt, const float* __restrict__ a_,
               const float* __restrict__ nw, float* __restrict__ S_pool, const int* __restrict__ curp, int NS,
               const int* __restrict__ parent, float* __restrict__ y, int nk, int nv, int T, float eps, int cur_off, int last_only) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) float sm[];
    gdn_body(qkvz, stride, ab, ldab, hist_pool, convw, dt, a_, nw, S_pool, (*curp + cur_off) % NS, NS, parent, y, nk, nv, T, eps, sm, last_only != 0);
}

// Batched lanes: blockIdx.y = lane j, the rows [lane_row0[j], lane_row0[j + 1]) of sequence lane_seq[j], a chain from
// that sequence's state slot cur[seq] in its own rings (hist_pool + seq * hist_stride, S_pool + seq * s_stride)
// (gdn_core_segs, engine/src/kernels.cu:2112-2156).  Every block of a cluster has the same lane, so all of them take
// the same path.
__global__ void __cluster_dims__(GDN_Q, 1, 1) __launch_bounds__(GDN_THREADS)
    k_gdn_core_lanes(const float* __restrict__ qkvz, int stride, const float* __restrict__ ab, int ldab, float* __restrict__ hist_pool, size_t hist_stride,
                     const float* __restrict__ convw, const float* __restrict__ dt, const float* __restrict__ a_, const float* __restrict__ nw,
                     float* __restrict__ S_pool, size_t s_stride, const int* __restrict__ cur, int NS, const int* __restrict__ lane_seq,
                     const int* __restrict__ lane_row0, float* __restrict__ y, int nk, int nv, float eps) {
    extern __shared__ __align__(16) float sm[];
    const int lane = blockIdx.y, row0 = lane_row0[lane], T = lane_row0[lane + 1] - row0, seq = lane_seq[lane];
    if (T <= 0 || seq < 0) return;   // (a negative sequence: another rank's lane)
    gdn_body(qkvz + (size_t) row0 * stride, stride, ab + (size_t) row0 * ldab, ldab, hist_pool + seq * hist_stride, convw, dt, a_, nw, S_pool + seq * s_stride,
             cur[seq], NS, nullptr, y + (size_t) row0 * nv * GDN_HS, nk, nv, T, eps, sm);
}

// ------------------------------------------------------------------------------------------------ prompts
// A prompt's rows are a chain of which every row is kept, so the work splits by what depends on what (gdn_prompt,
// engine/src/kernels.cu:2158): conv + SiLU, the q / k norms and the gates of every row at once (k_gdn_pre); the delta rule, the
// only sequential part, with the state in registers from the first row to the last and the rows' q, k, v streamed through
// shared memory (k_gdn_scan); the gated RMS norm of every row at once (k_gdn_post).  Only the last row's state and the last
// three rows' conv inputs are written back.
constexpr int GDP_THREADS = 256;

// block = one row; thread = channels tid, tid + 256, ...  xq / xk [T][nk][HS], xv [T][nv][HS], gates [T][nv][2]
__global__ void __launch_bounds__(GDP_THREADS) k_gdn_pre(const float* __restrict__ qkvz, int stride, const float* __restrict__ ab, int ldab,
                                                         const float* __restrict__ hin, float* __restrict__ hout, const float* __restrict__ convw,
                                                         const float* __restrict__ dt, const float* __restrict__ a_, float* __restrict__ xq,
                                                         float* __restrict__ xk, float* __restrict__ xv, float* __restrict__ gates, int nk, int nv, int T) {
    __shared__ float red[GDP_THREADS / 32];
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ch = (2 * nk + nv) * GDN_HS;
    // row t - k of the chain: a row of this call, or the history the call starts from (rows 0..2, oldest first)
    auto xrow = [&](int r, int c) { return r >= 0 ? qkvz[(size_t) r * stride + c] : hin[(size_t) (3 + r) * ch + c]; };
    for (int c0 = 0; c0 < ch; c0 += GDP_THREADS) {
        const int c = c0 + tid;
        const float4 cw = *reinterpret_cast<const float4*>(convw + (size_t) c * 4);
        const float x3 = xrow(t - 3, c), x2 = xrow(t - 2, c), x1 = xrow(t - 1, c), x0 = xrow(t, c);
        const float x = cw.x * x3 + cw.y * x2 + cw.z * x1 + cw.w * x0;
        float v = x / (1.0f + expf(-x));
        if (t == T - 1) {   // the history the next call starts from
            hout[c] = x2;
            hout[ch + c] = x1;
            hout[2 * ch + c] = x0;
        }
        if (c < 2 * nk * GDN_HS) {
            // q and k heads: the L2 norm over the head's 128 channels = four warps of this pass (two heads per pass)
            const float sq = warp_sum(v * v);
            __syncthreads();
            if (lane == 0) red[warp] = sq;
            __syncthreads();
            const int w0 = warp & ~3;
            float ssum = 0.f;
            for (int w = 0; w < 4; ++w) ssum += red[w0 + w];
            v *= rsqrtf(ssum + 1e-6f);
            if (c < nk * GDN_HS) xq[(size_t) t * nk * GDN_HS + c] = v;
            else xk[(size_t) t * nk * GDN_HS + (c - nk * GDN_HS)] = v;
        } else {
            xv[(size_t) t * nv * GDN_HS + (c - 2 * nk * GDN_HS)] = v;
        }
    }
    if (tid < nv) {
        const float* abt = ab + (size_t) t * ldab;
        const float x = abt[tid] + dt[tid];
        gates[((size_t) t * nv + tid) * 2] = expf((x > 20.0f ? x : log1pf(expf(x))) * a_[tid]);
        gates[((size_t) t * nv + tid) * 2 + 1] = 1.0f / (1.0f + expf(-abt[nv + tid]));
    }
}

// block = (value head, column quarter) as in the window kernel: warp `part` holds key rows [32 part, +32) of the block's 32 value
// columns, lane = column.  Rows stream through two shared-memory tiles of GDS_ROWS rows.
// two f32 in a 64-bit register and the packed multiply-add on them (fma.rn.f32x2: each half rounded as the scalar fmaf is, so the
// scan's products are those of its scalar form, at half the arithmetic instructions: the scan is bound by instruction issue, with
// one warp per scheduler)
__device__ __forceinline__ uint64_t f2_pack(float x, float y) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
    return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t r, float& x, float& y) { asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(r)); }
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

constexpr int GDS_ROWS = 16;
__global__ void __launch_bounds__(GDN_THREADS) k_gdn_scan(const float* __restrict__ xq, const float* __restrict__ xk, const float* __restrict__ xv,
                                                          const float* __restrict__ gates, const float* __restrict__ S_in, float* __restrict__ S_out,
                                                          float* __restrict__ o, int nk, int nv, int T) {
    constexpr int ROWF = 2 * GDN_HS + GDN_QC + 2;   // floats of a staged row: k, q, the block's v, the two gates
    __shared__ __align__(16) float tile[2][GDS_ROWS][ROWF + 2];
    __shared__ float kred[2][4][GDN_QC], ared[GDS_ROWS][4][GDN_QC];
    const int lv = blockIdx.x / GDN_Q, qq = blockIdx.x % GDN_Q, kh = lv % nk, tid = threadIdx.x;
    const int part = tid >> 5, lane = tid & 31, col = qq * GDN_QC + lane;
    const size_t soff = (size_t) lv * GDN_HS * GDN_HS + (size_t) part * 32 * GDN_HS + col;
    uint64_t s[16];   // the thread's 32 state values, in pairs (rows 2 i, 2 i + 1)
#pragma unroll
    for (int r = 0; r < 32; r += 2) s[r / 2] = f2_pack(S_in[soff + (size_t) r * GDN_HS], S_in[soff + (size_t) (r + 1) * GDN_HS]);
    auto stage = [&](int buf, int t0) {
        const int nr = min(GDS_ROWS, T - t0);
        for (int i = tid; i < nr * (ROWF / 2); i += GDN_THREADS) {   // 8-byte pieces
            const int r = i / (ROWF / 2), e = (i % (ROWF / 2)) * 2, t = t0 + r;
            const float* src;
            if (e < GDN_HS) src = xk + ((size_t) t * nk + kh) * GDN_HS + e;
            else if (e < 2 * GDN_HS) src = xq + ((size_t) t * nk + kh) * GDN_HS + (e - GDN_HS);
            else if (e < 2 * GDN_HS + GDN_QC) src = xv + ((size_t) t * nv + lv) * GDN_HS + qq * GDN_QC + (e - 2 * GDN_HS);
            else src = gates + ((size_t) t * nv + lv) * 2;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(&tile[buf][r][e])), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const float scale = rsqrtf((float) GDN_HS);
    stage(0, 0);
    int buf = 0;
    for (int t0 = 0; t0 < T; t0 += GDS_ROWS, buf ^= 1) {
        const int nr = min(GDS_ROWS, T - t0);
        if (t0 + GDS_ROWS < T) {
            stage(buf ^ 1, t0 + GDS_ROWS);   // (its last readers passed the barrier that ended the previous tile)
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
#pragma unroll 1
        for (int r0 = 0; r0 < nr; ++r0) {
            const float* row = tile[buf][r0];
            const float* kt = row + part * 32;
            const float* qt = row + GDN_HS + part * 32;
            const float gv = row[2 * GDN_HS + GDN_QC], bv = row[2 * GDN_HS + GDN_QC + 1];
            // (the row's k and q for this warp's 32 key rows: eight 16-byte broadcast reads each, as pairs)
            uint64_t kp[16], qp[16];
#pragma unroll
            for (int r = 0; r < 32; r += 4) {
                const ulonglong2 a = *reinterpret_cast<const ulonglong2*>(kt + r), b = *reinterpret_cast<const ulonglong2*>(qt + r);
                kp[r / 2] = a.x; kp[r / 2 + 1] = a.y;
                qp[r / 2] = b.x; qp[r / 2 + 1] = b.y;
            }
            // eight running sums in four pairs (row r of the 32 goes to sum r % 8): four independent chains of packed products
            uint64_t kacc[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) kacc[i] = f2_pack(0.f, 0.f);
#pragma unroll
            for (int r = 0; r < 16; r += 4)
#pragma unroll
                for (int i = 0; i < 4; ++i) kacc[i] = f2_fma(s[r + i], kp[r + i], kacc[i]);
            float k0, k1, k2, k3, k4, k5, k6, k7;
            f2_unpack(kacc[0], k0, k1);
            f2_unpack(kacc[1], k2, k3);
            f2_unpack(kacc[2], k4, k5);
            f2_unpack(kacc[3], k6, k7);
            float* kr = &kred[r0 & 1][0][0];
            kr[part * GDN_QC + lane] = ((k0 + k1) + (k2 + k3)) + ((k4 + k5) + (k6 + k7));
            __syncthreads();
            const float kvs = (kr[lane] + kr[GDN_QC + lane]) + (kr[2 * GDN_QC + lane] + kr[3 * GDN_QC + lane]);
            const float delta = (row[2 * GDN_HS + lane] - gv * kvs) * bv;
            const uint64_t d2 = f2_pack(delta, delta), g2 = f2_pack(gv, gv);
            uint64_t aacc[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) aacc[i] = f2_pack(0.f, 0.f);
#pragma unroll
            for (int r = 0; r < 16; r += 4)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    s[r + i] = f2_fma(kp[r + i], d2, f2_mul(g2, s[r + i]));
                    aacc[i] = f2_fma(s[r + i], qp[r + i], aacc[i]);
                }
            float a0, a1, a2, a3, a4, a5, a6, a7;
            f2_unpack(aacc[0], a0, a1);
            f2_unpack(aacc[1], a2, a3);
            f2_unpack(aacc[2], a4, a5);
            f2_unpack(aacc[3], a6, a7);
            ared[r0][part][lane] = ((a0 + a1) + (a2 + a3)) + ((a4 + a5) + (a6 + a7));
        }
        __syncthreads();   // the tile's sums are complete; its buffer may be refilled two tiles on
        for (int i = tid; i < nr * GDN_QC; i += GDN_THREADS) {
            const int r0 = i / GDN_QC, c = i % GDN_QC;
            o[((size_t) (t0 + r0) * nv + lv) * GDN_HS + qq * GDN_QC + c] = ((ared[r0][0][c] + ared[r0][1][c]) + (ared[r0][2][c] + ared[r0][3][c])) * scale;
        }
    }
#pragma unroll
    for (int r = 0; r < 32; r += 2) {
        float x, y;
        f2_unpack(s[r / 2], x, y);
        S_out[soff + (size_t) r * GDN_HS] = x;
        S_out[soff + (size_t) (r + 1) * GDN_HS] = y;
    }
}

// block = one row, warp = a quarter (32 columns) of a value head at a time: y = o * rsqrt(mean(o^2) + eps) * nw * sigmoid(z)
__global__ void __launch_bounds__(GDP_THREADS) k_gdn_post(const float* __restrict__ o, const float* __restrict__ qkvz, int stride, const float* __restrict__ nw,
                                                          float* __restrict__ y, int nk, int nv, float eps) {
    __shared__ float red[GDP_THREADS / 32];
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ch = (2 * nk + nv) * GDN_HS;
    for (int c0 = 0; c0 < nv * GDN_HS; c0 += GDP_THREADS) {
        const int c = c0 + tid, col = c % GDN_HS;
        const float ov = o[(size_t) t * nv * GDN_HS + c];
        const float zv = qkvz[(size_t) t * stride + ch + c];
        const float sq = warp_sum(ov * ov);
        __syncthreads();
        if (lane == 0) red[warp] = sq;
        __syncthreads();
        const int w0 = warp & ~3;
        const float ms = ((red[w0] + red[w0 + 1]) + (red[w0 + 2] + red[w0 + 3])) / (float) GDN_HS;
        y[(size_t) t * nv * GDN_HS + c] = ov * rsqrtf(ms + eps) * nw[col] / (1.0f + expf(-zv));
    }
}

static size_t gdn_smem_bytes(int T) {
    return sizeof(float) * ((size_t) 2 * T * GDN_HS + (size_t) T * GDN_QC + 2 * T + 2 * 4 * GDN_QC + (size_t) T * 4 * GDN_QC + T + 8 * T +
                            (size_t) (T + 3) * (2 * GDN_HS + GDN_QC) + 3 * T);
}

}  // namespace fnxb

using namespace fnxb;

extern "C" int fnx_gdn_core(const float* qkvz, int ldx, const float* ab, int ldab, float* hist_pool, const float* convw, const float* dt, const float* a,
                            const float* nw, float* S_pool, const int* cur, int NS, const int* parent, float* y, int nk, int nv, int hs,
                            int T, float eps, fnx_stream st) {
    FNX_REQUIRE(qkvz && ab && hist_pool && convw && dt && a && nw && S_pool && cur && y, "fnx_gdn_core: null pointer");
    FNX_REQUIRE(hs == GDN_HS, "fnx_gdn_core: head dim %d (this build: %d)", hs, GDN_HS);
    FNX_REQUIRE(T >= 1 && T <= FNX_MAX_ROWS && NS >= T + 1, "fnx_gdn_core: %d rows need at least %d state slots, have %d", T, T + 1, NS);
    FNX_REQUIRE(nk >= 1 && nv >= nk && nv % nk == 0, "fnx_gdn_core: %d key heads, %d value heads", nk, nv);
    const size_t smem = gdn_smem_bytes(T);
    if (int rc = set_smem_limit((const void*) k_gdn_core, 96 * 1024)) return rc;
    {
        const cudaError_t le_ = launch_k(k_gdn_core, dim3(nv * GDN_Q), dim3(GDN_THREADS), smem, as_stream(st), qkvz, ldx, ab, ldab, hist_pool, convw, dt, a, nw, S_pool, cur, NS, parent, y, nk, nv, T, eps, 0, 0);
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "k_gdn_core: launch failed: %s", cudaGetErrorString(le_));
    }
    FNX_LAUNCH_OK("fnx_gdn_core");
    return FNX_OK;
}

extern "C" size_t fnx_gdn_prompt_scratch_bytes(int T, int nk, int nv, int hs) {
    return sizeof(float) * ((size_t) T * (2 * nk + 2 * nv) * hs + (size_t) T * nv * 2 + (size_t) 3 * (2 * nk + nv) * hs) + 1024;
}

extern "C" int fnx_gdn_prompt(const float* qkvz, int ldx, const float* ab, int ldab, float* hist_pool, const float* convw, const float* dt, const float* a,
                              const float* nw, float* S_pool, int cur_host, int NS, float* y, int nk, int nv, int hs, int T, float eps, void* scratch,
                              fnx_stream st) {
    FNX_REQUIRE(qkvz && ab && hist_pool && convw && dt && a && nw && S_pool && y && scratch, "fnx_gdn_prompt: null pointer");
    FNX_REQUIRE(hs == GDN_HS, "fnx_gdn_prompt: head dim %d (this build: %d)", hs, GDN_HS);
    FNX_REQUIRE(T >= 1 && NS >= 2 && cur_host >= 0 && cur_host < NS, "fnx_gdn_prompt: %d rows, slot %d of %d", T, cur_host, NS);
    FNX_REQUIRE(nk >= 1 && nv >= nk && nv % nk == 0 && nv <= GDP_THREADS && ((2 * nk + nv) * GDN_HS) % GDP_THREADS == 0, "fnx_gdn_prompt: %d key heads, %d value heads", nk, nv);
    const int ch = (2 * nk + nv) * GDN_HS, out_slot = (cur_host + T) % NS;
    const size_t hsz = (size_t) 3 * ch, ssz = (size_t) nv * GDN_HS * GDN_HS;
    float* xq = (float*) scratch;
    float* xk = xq + (size_t) T * nk * GDN_HS;
    float* xv = xk + (size_t) T * nk * GDN_HS;
    float* o = xv + (size_t) T * nv * GDN_HS;
    float* gates = o + (size_t) T * nv * GDN_HS;
    cudaStream_t s = as_stream(st);
    // the history the call starts from is read from a copy: the slot it leaves its own in may be the same one
    float* hin = gates + (size_t) T * nv * 2;
    FNX_CUDA_OK(cudaMemcpyAsync(hin, hist_pool + (size_t) cur_host * hsz, hsz * sizeof(float), cudaMemcpyDeviceToDevice, s));
    k_gdn_pre<<<T, GDP_THREADS, 0, s>>>(qkvz, ldx, ab, ldab, hin, hist_pool + (size_t) out_slot * hsz, convw, dt, a, xq, xk, xv, gates, nk,
                                         nv, T);
    FNX_LAUNCH_OK("k_gdn_pre");
    k_gdn_scan<<<nv * GDN_Q, GDN_THREADS, 0, s>>>(xq, xk, xv, gates, S_pool + (size_t) cur_host * ssz, S_pool + (size_t) out_slot * ssz, o, nk, nv, T);
    FNX_LAUNCH_OK("k_gdn_scan");
    k_gdn_post<<<T, GDP_THREADS, 0, s>>>(o, qkvz, ldx, nw, y, nk, nv, eps);
    FNX_LAUNCH_OK("k_gdn_post");
    return FNX_OK;
}

extern "C" int fnx_gdn_core_lanes(const float* qkvz, int ldx, const float* ab, int ldab, float* hist_pool, size_t hist_seq_stride, const float* convw,
                                  const float* dt, const float* a, const float* nw, float* S_pool, size_t s_seq_stride, const int* cur, int NS,
                                  const int* lane_seq, const int* lane_row0, int n_lanes, int max_lane_rows, float* y, int nk, int nv, int hs, float eps,
                                  fnx_stream st) {
    FNX_REQUIRE(qkvz && ab && hist_pool && convw && dt && a && nw && S_pool && cur && lane_seq && lane_row0 && y, "fnx_gdn_core_lanes: null pointer");
    FNX_REQUIRE(hs == GDN_HS, "fnx_gdn_core_lanes: head dim %d (this build: %d)", hs, GDN_HS);
    FNX_REQUIRE(n_lanes >= 1 && n_lanes <= FNX_MAX_ROWS && max_lane_rows >= 1 && NS >= max_lane_rows + 1, "fnx_gdn_core_lanes: %d lanes of up to %d rows, %d state slots",
                n_lanes, max_lane_rows, NS);
    FNX_REQUIRE(nk >= 1 && nv >= nk && nv % nk == 0, "fnx_gdn_core_lanes: %d key heads, %d value heads", nk, nv);
    if (int rc = set_smem_limit((const void*) k_gdn_core_lanes, 96 * 1024)) return rc;
    const cudaError_t le = launch_k(k_gdn_core_lanes, dim3(nv * GDN_Q, n_lanes), dim3(GDN_THREADS), gdn_smem_bytes(max_lane_rows), as_stream(st), qkvz, ldx, ab, ldab,
                                    hist_pool, hist_seq_stride, convw, dt, a, nw, S_pool, s_seq_stride, cur, NS, lane_seq, lane_row0, y, nk, nv, eps);
    if (le != cudaSuccess) return fail(FNX_E_CUDA, "k_gdn_core_lanes: launch failed: %s", cudaGetErrorString(le));
    FNX_LAUNCH_OK("fnx_gdn_core_lanes");
    return FNX_OK;
}
