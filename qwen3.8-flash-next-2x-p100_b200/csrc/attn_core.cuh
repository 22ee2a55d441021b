// Device bodies of the gated-attention kernels (attn.cu), shared by their single-sequence, batched-lane and prompt forms:
// per-head norm + rotary + KV append, the tree-masked split-K partial, and the merge of the splits.
// Reference: attn_prep_append / norm_rope (engine/src/kernels.cu:1880-1910, 513-530), k_attn_part / k_attn_combine
// (engine/src/kernels.cu:558-667, 786-803).
#pragma once

#include "fnx_common.cuh"

namespace fnxb {

struct SyncBlock {
    __device__ __forceinline__ void operator()() const { __syncthreads(); }
};
// a named barrier of n threads (n a multiple of 32), for a group of warps inside a larger block
struct SyncNamed {
    int id, n;
    __device__ __forceinline__ void operator()() const { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
};

// ------------------------------------------------------------------------------------------------ prep + append
// One (head h of nq + 2 nkv, row t) item by hd threads (i = the thread's element); xrow: hd floats, red: 32 floats of
// shared memory; sync() is a barrier of the item's threads.
template <typename Sync>
__device__ __forceinline__ void attn_prep_body(float* qg, int ldq, float* k, int ldk, const float* v, int ldv, const float* qn, const float* kn,
                                               __half* kc, __half* vc, int nq, int nkv, int hd, int nrot, int pos0, const int* depth, float eps,
                                               float rope_base, int t, int h, int i, float* xrow, float* red, Sync sync) {
    const int pos = pos0 + (depth ? depth[t] : t);
    const size_t crow = (size_t) (pos0 + t) * nkv * hd;
    if (h >= nq + nkv) {   // a V head: store only
        const int kvh = h - nq - nkv;
        vc[crow + (size_t) kvh * hd + i] = __float2half_rn(v[(size_t) t * ldv + (size_t) kvh * hd + i]);
        return;
    }
    float* x = h < nq ? qg + (size_t) t * ldq + (size_t) h * 2 * hd : k + (size_t) t * ldk + (size_t) (h - nq) * hd;
    const float* w = h < nq ? qn : kn;
    const float val = x[i];
    float ss = warp_sum(val * val);
    if ((i & 31) == 0) red[i >> 5] = ss;
    sync();
    ss = 0.f;
    for (int j = 0; j < hd / 32; ++j) ss += red[j];
    xrow[i] = val * rsqrtf(ss / (float) hd + eps) * w[i];
    sync();
    float y = xrow[i];
    if (i < nrot) {
        const int pr = i < nrot / 2 ? i : i - nrot / 2;
        // the unit frequency through double: the correctly rounded f32 of base^(-2 i / nrot) (engine/src/rope.hpp:33-35)
        const float fe = (float) pow((double) rope_base, -2.0 * (double) pr / (double) nrot);
        float sn, cs;
        sincosf((float) pos * fe, &sn, &cs);
        const float x0 = xrow[pr], x1 = xrow[pr + nrot / 2];
        y = i < nrot / 2 ? x0 * cs - x1 * sn : x0 * sn + x1 * cs;
    }
    x[i] = y;
    if (h >= nq) kc[crow + (size_t) (h - nq) * hd + i] = __float2half_rn(y);
}

// ------------------------------------------------------------------------------------------------ attention
constexpr int ATT_SC = 64;        // positions per step
constexpr int ATT_ROWS = 5;       // window rows one block serves
constexpr int ATT_THREADS = 256;
constexpr int ATT_MAXQ = 8;       // q heads per KV head
constexpr int ATT_MQ = 48;        // the block's ATT_ROWS * ATT_MAXQ queries, padded to three 16-row MMA tiles
constexpr int ATT_HD = 256;
constexpr int ATT_QS = ATT_HD + 8;    // row strides (halves) of the Q, K, V tiles: 8 rows of a ldmatrix land in 8 bank groups
constexpr int ATT_SS = ATT_SC + 4;    // score rows (floats)
constexpr int ATT_PS = ATT_SC + 8;    // probability rows (halves)

// shared memory of a block that serves `rows` window rows (mq = their queries padded to 16-row MMA tiles; qlo: the queries' low
// halves are kept too)
constexpr size_t attn_part_smem_of(int rows, int mq, bool qlo) {
    return (size_t) ((qlo ? 2 : 1) * mq + 4 * ATT_SC) * ATT_QS * sizeof(__half) + (size_t) mq * ATT_SS * sizeof(float) +
           (size_t) mq * ATT_PS * sizeof(__half) + 3 * mq * sizeof(float) + rows * sizeof(unsigned);
}
constexpr size_t attn_part_smem() { return attn_part_smem_of(ATT_ROWS, ATT_MQ, true); }
// the prompt form: twelve rows per block (96 queries), f16 queries, rows a chain of any length
constexpr int ATP_ROWS = 12, ATP_MQ = 96;
constexpr size_t attn_prompt_smem() { return attn_part_smem_of(ATP_ROWS, ATP_MQ, false); }

struct AttPartial {   // one (row, head, split)
    float m, z;
};

__device__ __forceinline__ void ldsm_x4(uint32_t a, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t a, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}

// One block: KV head kvh, split s of S (every S-th 64-position chunk of [0, ctx)), window rows [r0, r0 + ATT_ROWS):
// their (up to 40) queries against the share, on the tensor cores (mma.sync m16n8k16, f16 x f16 -> f32):
//   scores  = Q K^T with Q = Qhi + Qlo, two f16 halves of the f32 queries, so that only K's own f16 rounding remains;
//   weights = exp(score - running max), rounded to f16 (their sum is taken over the rounded values);
//   sums   += weights V, accumulated in f32 registers across the steps of 64 positions.
// scratch: acc [T][nq][S][hd] floats, then mz [T][nq][S]
// (tid: the thread among the item's ATT_THREADS; smem: attn_part_smem() bytes, 16-byte aligned; sync(): their barrier)
// ROWS / MQ: window rows per block and their queries padded to 16-row tiles.  QLO: scores from both f16 halves of the queries
// (the window path); without it from the rounded queries alone (the prompt pass, whose activations are f16 anyway).  CHAIN: the
// rows are a chain of any length (row r sees every position up to its own), no ancestor bitmaps.
template <int ROWS, int MQ, bool QLO, bool CHAIN, typename Sync>
__device__ __forceinline__ void attn_part_body_t(const float* qg, int ldq, const __half* kc, const __half* vc, float* acc_out, AttPartial* mz_out, int T,
                                                 int nq, int nkv, int pos0, const int* parent, int s, int S, int kvh, int r0, int tid, uint8_t* smem,
                                                 Sync sync) {
    constexpr int ATT_MQ = MQ, ATT_ROWS = ROWS, MT = MQ / 16;   // (shadow the window form's constants)
    const int nr = min(ATT_ROWS, T - r0), qpk = nq / nkv, NQ = nr * qpk;
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, q = lane & 3;
    const int ctx = CHAIN ? pos0 + r0 + nr : pos0 + T;      // a chain's rows see nothing past the block's last row
    __half* Qh = reinterpret_cast<__half*>(smem);           // [ATT_MQ][ATT_QS]
    __half* Ql = Qh + ATT_MQ * ATT_QS;
    __half* Ks = Qh + (QLO ? 2 : 1) * ATT_MQ * ATT_QS;      // two buffers of [K: ATT_SC][ATT_QS], [V: ATT_SC][ATT_QS]
    __half* Vs = Ks + ATT_SC * ATT_QS;
    constexpr int KVB = 2 * ATT_SC * ATT_QS;                // halves per buffer: the next step's rows land while this step is used
    float* Sf = reinterpret_cast<float*>(Ks + 2 * KVB);     // [ATT_MQ][ATT_SS]
    __half* Pp = reinterpret_cast<__half*>(Sf + ATT_MQ * ATT_SS); // [ATT_MQ][ATT_PS]
    float* ms = reinterpret_cast<float*>(Pp + ATT_MQ * ATT_PS);   // running max, sum, rescale per query
    float* zs = ms + ATT_MQ;
    float* fs = zs + ATT_MQ;
    unsigned* see = reinterpret_cast<unsigned*>(fs + ATT_MQ);     // per local row: window rows it sees
    // Split s takes the 64-position chunks s, s + S, s + 2 S, ... in order.  Chunks are cut at absolute positions, so what a
    // row's partial of split s sums, and in which order, depends on the row's own position only - not on the window it
    // arrived in: a row verified alone and the same row verified among drafts give the same bits.
    const int pa = s * ATT_SC;
    if (pa >= ctx) {   // a block with no positions leaves only empty partials: the merge skips them without reading their sums
        if (tid < NQ) {
            const int r = tid / qpk, hh = tid % qpk;
            mz_out[((size_t) (r0 + r) * nq + kvh * qpk + hh) * S + s] = AttPartial{-INFINITY, 0.f};
        }
        return;
    }
    // the first step's K and V rows are on their way while the queries are split
    auto fetch_kv = [&](int buf, int p0, int np) {
#pragma unroll
        for (int j = 0; j < ATT_SC * (ATT_HD / 8) / ATT_THREADS; ++j) {
            const int i = tid + j * ATT_THREADS, pp = i / (ATT_HD / 8), d8 = i % (ATT_HD / 8);
            __half* kd = Ks + buf * KVB + pp * ATT_QS + d8 * 8;
            __half* vd = Vs + buf * KVB + pp * ATT_QS + d8 * 8;
            if (pp < np) {
                const size_t go = ((size_t) (p0 + pp) * nkv + kvh) * ATT_HD + d8 * 8;
                cp_async16(kd, kc + go);
                cp_async16(vd, vc + go);
            } else {
                *reinterpret_cast<uint4*>(kd) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vd) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch_kv(0, pa, min(ATT_SC, ctx - pa));
    // the queries as f16 pairs (hi, lo); rows past NQ are zero
    for (int i0 = tid; i0 < ATT_MQ * (ATT_HD / 4); i0 += 6 * ATT_THREADS) {
        float4 v[6];
#pragma unroll
        for (int j = 0; j < 6; ++j) {
            const int i = i0 + j * ATT_THREADS, qi = i / (ATT_HD / 4), d4 = i % (ATT_HD / 4);
            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < ATT_MQ * (ATT_HD / 4) && qi < NQ) {
                const int r = qi / qpk, hh = qi % qpk;
                v[j] = *reinterpret_cast<const float4*>(qg + (size_t) (r0 + r) * ldq + (size_t) (kvh * qpk + hh) * 2 * ATT_HD + d4 * 4);
            }
        }
#pragma unroll
        for (int j = 0; j < 6; ++j) {
            const int i = i0 + j * ATT_THREADS, qi = i / (ATT_HD / 4), d4 = i % (ATT_HD / 4);
            if (i >= ATT_MQ * (ATT_HD / 4)) continue;
            const float x[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
            __half h[4], l[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                h[k] = __float2half_rn(x[k]);
                l[k] = __float2half_rn(x[k] - __half2float(h[k]));
            }
            *reinterpret_cast<uint2*>(Qh + qi * ATT_QS + d4 * 4) = make_uint2((uint32_t) __half_as_ushort(h[0]) | ((uint32_t) __half_as_ushort(h[1]) << 16),
                                                                                (uint32_t) __half_as_ushort(h[2]) | ((uint32_t) __half_as_ushort(h[3]) << 16));
            if (QLO)
                *reinterpret_cast<uint2*>(Ql + qi * ATT_QS + d4 * 4) = make_uint2((uint32_t) __half_as_ushort(l[0]) | ((uint32_t) __half_as_ushort(l[1]) << 16),
                                                                                (uint32_t) __half_as_ushort(l[2]) | ((uint32_t) __half_as_ushort(l[3]) << 16));
        }
    }
    if (tid < ATT_MQ) { ms[tid] = -INFINITY; zs[tid] = 0.f; fs[tid] = 0.f; }
    if (!CHAIN && tid < nr) {
        unsigned m = 0;
        for (int a = r0 + tid; a >= 0; a = parent ? parent[a] : a - 1) m |= 1u << a;
        see[tid] = m;
    }
    float acc[MT][4][4];   // [query tile][8-dim tile of the warp's 32 dims][c]
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[m][n][k] = 0.f;
    const float scale = rsqrtf((float) ATT_HD);
    // the window row of each of the lane's score rows (query m * 16 + g + 8 * hrow), once: -1 = no such query
    int qrow[MT][2];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            const int qi = m * 16 + g + 8 * hrow;
            qrow[m][hrow] = qi < NQ ? qi / qpk : -1;
        }
    const uint32_t qh_s = smem_u32(Qh), ql_s = smem_u32(Ql), ks0_s = smem_u32(Ks), vs0_s = smem_u32(Vs), pp_s = smem_u32(Pp);
    // ldmatrix lane addresses: A tiles (16 rows x 16 columns), B tiles of K (8 positions x 32 dims), of V (16 positions x 16 dims, transposed)
    const uint32_t a_off = (uint32_t) ((lane & 15) * ATT_QS + (lane >> 4) * 8) * 2u;
    const uint32_t bk_off = (uint32_t) ((warp * 8 + (lane & 7)) * ATT_QS + (lane >> 3) * 8) * 2u;
    const uint32_t bv_off = (uint32_t) (((lane & 7) + ((lane >> 3) & 1) * 8) * ATT_QS + warp * 32 + (lane >> 4) * 8) * 2u;
    const uint32_t ap_off = (uint32_t) ((lane & 15) * ATT_PS + (lane >> 4) * 8) * 2u;
    int buf = 0;
    for (int p0 = pa; p0 < ctx; p0 += S * ATT_SC, buf ^= 1) {
        const int np = min(ATT_SC, ctx - p0);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        sync();   // this step's rows have landed, and every thread is done with the previous step: its buffer is free
        {
            const int pn = p0 + S * ATT_SC;
            if (pn < ctx) fetch_kv(buf ^ 1, pn, min(ATT_SC, ctx - pn));
        }
        const uint32_t ks_s = ks0_s + (uint32_t) (buf * KVB * 2), vs_s = vs0_s + (uint32_t) (buf * KVB * 2);
        // ---- scores: warp w = positions [8 w, 8 w + 8) of the step, all 48 query rows
        {
            float c[MT][4];
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int k = 0; k < 4; ++k) c[m][k] = 0.f;
#pragma unroll 2
            for (int k0 = 0; k0 < ATT_HD; k0 += 32) {
                // every fragment of the 32 dims first, then the products: the loads' latency is paid once per 32 dims, not once
                // per product (the asm statements keep their order)
                uint32_t b0, b1, b2, b3;   // (b0, b1): dims k0 .. k0 + 15, (b2, b3): k0 + 16 .. k0 + 31
                ldsm_x4(ks_s + bk_off + k0 * 2, b0, b1, b2, b3);
                uint32_t ah[MT][2][4], al[QLO ? MT : 1][2][4];
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const uint32_t ao = a_off + (uint32_t) (m * 16 * ATT_QS + k0) * 2u;
                    ldsm_x4(qh_s + ao, ah[m][0][0], ah[m][0][1], ah[m][0][2], ah[m][0][3]);
                    ldsm_x4(qh_s + ao + 32, ah[m][1][0], ah[m][1][1], ah[m][1][2], ah[m][1][3]);
                    if (QLO) {
                        ldsm_x4(ql_s + ao, al[m][0][0], al[m][0][1], al[m][0][2], al[m][0][3]);
                        ldsm_x4(ql_s + ao + 32, al[m][1][0], al[m][1][1], al[m][1][2], al[m][1][3]);
                    }
                }
#pragma unroll
                for (int m = 0; m < MT; ++m) mma_f16(c[m], ah[m][0][0], ah[m][0][1], ah[m][0][2], ah[m][0][3], b0, b1);
                if (QLO) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) mma_f16(c[m], al[QLO ? m : 0][0][0], al[QLO ? m : 0][0][1], al[QLO ? m : 0][0][2], al[QLO ? m : 0][0][3], b0, b1);
                }
#pragma unroll
                for (int m = 0; m < MT; ++m) mma_f16(c[m], ah[m][1][0], ah[m][1][1], ah[m][1][2], ah[m][1][3], b2, b3);
                if (QLO) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) mma_f16(c[m], al[QLO ? m : 0][1][0], al[QLO ? m : 0][1][1], al[QLO ? m : 0][1][2], al[QLO ? m : 0][1][3], b2, b3);
                }
            }
            // scaled and masked into the score tile: row = query, column = position of the step
            // a step that lies wholly before the window's first row is visible to every row: no masks to work out
            const bool open_step = np == ATT_SC && p0 + ATT_SC <= pos0 + (CHAIN ? r0 : 0);
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const int qi = m * 16 + g + 8 * hrow, qr = qrow[m][hrow];
                    float2 o;
                    float* ov = &o.x;
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const int col = warp * 8 + 2 * q + k, p = p0 + col;
                        bool vis = qr >= 0;
                        if (!open_step) {
                            vis = vis && col < np;
                            if (CHAIN) vis = vis && p <= pos0 + r0 + qr;
                            else if (vis && p >= pos0) vis = (see[qr] >> (p - pos0)) & 1u;
                        }
                        ov[k] = vis ? c[m][2 * hrow + k] * scale : -INFINITY;
                    }
                    *reinterpret_cast<float2*>(Sf + qi * ATT_SS + warp * 8 + 2 * q) = o;
                }
        }
        sync();
        // ---- weights: warp w = queries w, w + 8, ..., four at a time: eight lanes per query, eight positions per lane
        {
            constexpr int RW = ATT_MQ / (ATT_THREADS / 32);
            auto ex = [](float x) { return CHAIN ? __expf(x) : expf(x); };   // (the prompt form takes the hardware exponential)
#pragma unroll
            for (int j0 = 0; j0 < RW; j0 += 4) {
                const int j = j0 + (lane >> 3), l8 = lane & 7;
                const bool act = j < RW;
                const int qi = warp + (ATT_THREADS / 32) * (act ? j : 0);
                const float4 x0 = *reinterpret_cast<const float4*>(Sf + qi * ATT_SS + 8 * l8), x1 = *reinterpret_cast<const float4*>(Sf + qi * ATT_SS + 8 * l8 + 4);
                const float v[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                float mx = fmaxf(fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3])), fmaxf(fmaxf(v[4], v[5]), fmaxf(v[6], v[7])));
#pragma unroll
                for (int o = 4; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                const float mo = ms[qi], mn = fmaxf(mo, mx);
                __half h[8];
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    h[i] = __float2half_rn(v[i] == -INFINITY ? 0.f : ex(v[i] - mn));
                    sum += __half2float(h[i]);
                }
#pragma unroll
                for (int o = 4; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                const float f = mo == -INFINITY ? 0.f : ex(mo - mn);
                const float zn = zs[qi] * f + sum;
                __syncwarp();   // every lane has read the query's running values
                if (act) {
                    uint4 pk;
                    pk.x = (uint32_t) __half_as_ushort(h[0]) | ((uint32_t) __half_as_ushort(h[1]) << 16);
                    pk.y = (uint32_t) __half_as_ushort(h[2]) | ((uint32_t) __half_as_ushort(h[3]) << 16);
                    pk.z = (uint32_t) __half_as_ushort(h[4]) | ((uint32_t) __half_as_ushort(h[5]) << 16);
                    pk.w = (uint32_t) __half_as_ushort(h[6]) | ((uint32_t) __half_as_ushort(h[7]) << 16);
                    *reinterpret_cast<uint4*>(Pp + qi * ATT_PS + 8 * l8) = pk;
                    if (l8 == 0) { ms[qi] = mn; zs[qi] = zn; fs[qi] = f; }
                }
            }
        }
        sync();
        // ---- sums: warp w = dims [32 w, 32 w + 32), all 48 query rows
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float fa = fs[m * 16 + g], fb = fs[m * 16 + g + 8];
            // (deep into a long context the running maxima rarely move: a tile whose factors are all 1 is left alone)
            if (__all_sync(0xffffffffu, fa == 1.0f && fb == 1.0f)) continue;
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                acc[m][n][0] *= fa; acc[m][n][1] *= fa;
                acc[m][n][2] *= fb; acc[m][n][3] *= fb;
            }
        }
#pragma unroll
        for (int k0 = 0; k0 < ATT_SC; k0 += 16) {
            uint32_t a[MT][4], bv[2][4];
#pragma unroll
            for (int m = 0; m < MT; ++m) ldsm_x4(pp_s + ap_off + (uint32_t) (m * 16 * ATT_PS + k0) * 2u, a[m][0], a[m][1], a[m][2], a[m][3]);
#pragma unroll
            for (int n2 = 0; n2 < 2; ++n2)   // (b0, b1): dims 16 n2 .. + 7, (b2, b3): + 8 .. + 15
                ldsm_x4_t(vs_s + bv_off + (uint32_t) (k0 * ATT_QS + n2 * 16) * 2u, bv[n2][0], bv[n2][1], bv[n2][2], bv[n2][3]);
#pragma unroll
            for (int n2 = 0; n2 < 2; ++n2) {
#pragma unroll
                for (int m = 0; m < MT; ++m) mma_f16(acc[m][2 * n2], a[m][0], a[m][1], a[m][2], a[m][3], bv[n2][0], bv[n2][1]);
#pragma unroll
                for (int m = 0; m < MT; ++m) mma_f16(acc[m][2 * n2 + 1], a[m][0], a[m][1], a[m][2], a[m][3], bv[n2][2], bv[n2][3]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            const int qi = m * 16 + g + 8 * hrow;
            if (qi < NQ) {
                const int r = qi / qpk, hh = qi % qpk;
                const size_t slot = ((size_t) (r0 + r) * nq + kvh * qpk + hh) * S + s;
#pragma unroll
                for (int n = 0; n < 4; ++n)
                    *reinterpret_cast<float2*>(acc_out + slot * ATT_HD + warp * 32 + n * 8 + 2 * q) = make_float2(acc[m][n][2 * hrow], acc[m][n][2 * hrow + 1]);
            }
        }
    if (tid < NQ) {
        const int r = tid / qpk, hh = tid % qpk;
        mz_out[((size_t) (r0 + r) * nq + kvh * qpk + hh) * S + s] = AttPartial{ms[tid], zs[tid]};
    }
}

// the window form: five rows per block, queries in two f16 halves, tree masks
template <typename Sync>
__device__ __forceinline__ void attn_part_body(const float* qg, int ldq, const __half* kc, const __half* vc, float* acc_out, AttPartial* mz_out, int T,
                                               int nq, int nkv, int pos0, const int* parent, int s, int S, int kvh, int r0, int tid, uint8_t* smem,
                                               Sync sync) {
    attn_part_body_t<ATT_ROWS, ATT_MQ, true, false>(qg, ldq, kc, vc, acc_out, mz_out, T, nq, nkv, pos0, parent, s, S, kvh, r0, tid, smem, sync);
}

// merge the splits of (row, head): out = sum_s exp(m_s - m) acc_s / sum_s exp(m_s - m) z_s * sigmoid(gate)
constexpr int ATC_G = 4;   // groups of hd threads that share the splits of one (row, head)

// By PG * ATT_THREADS threads (PG = 4: one thread group per role; PG = 2: a thread group plays roles g and g + 2);
// sm: (3 + ATC_G) * 256 floats of shared memory; sync(): the barrier of those threads.
template <int PG, typename Sync>
__device__ __forceinline__ void attn_combine_body(const float* acc_in, const AttPartial* mz_in, const float* qg, int ldq, float* out, int nq, int hd, int S,
                                                  int h, int t, int tid, float* sm, Sync sync) {
    float* sm_m = sm;
    float* sm_w = sm + 256;
    float* sm_z = sm + 512;
    float (*sm_p)[ATT_THREADS] = reinterpret_cast<float (*)[ATT_THREADS]>(sm + 768);
    const int i = tid % ATT_THREADS, g = tid / ATT_THREADS;
    const size_t base = ((size_t) t * nq + h) * S;
    AttPartial p = AttPartial{-INFINITY, 0.f};
    if (g == 0) {
        if (i < S) p = mz_in[base + i];
        sm_m[i] = i < S ? p.m : -INFINITY;
    }
    sync();
    // block maximum of m (S <= 256)
    float mx = -INFINITY;
    for (int s = 0; s < S; ++s) mx = fmaxf(mx, sm_m[s]);
    if (g == 0) {
        const float w = i < S && p.m != -INFINITY ? expf(p.m - mx) : 0.f;
        sm_w[i] = w;
        sm_z[i] = w * p.z;
    }
    sync();
    // group g adds the live splits g, g + G, ... in order (8 loads in flight); group 0 then adds the groups in order
    for (int gg = g; gg < ATC_G; gg += PG) {
        float acc = 0.f;
        for (int s0 = gg; s0 < S; s0 += 8 * ATC_G) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int sp = s0 + j * ATC_G;
                v[j] = sp < S && sm_w[sp] != 0.f ? acc_in[(base + sp) * hd + i] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int sp = s0 + j * ATC_G;
                acc = fmaf(sp < S ? sm_w[sp] : 0.f, v[j], acc);
            }
        }
        sm_p[gg][i] = acc;
    }
    sync();
    if (g != 0) return;
    float z = 0.f;
    for (int s = 0; s < S; ++s) z += sm_z[s];        // fixed order: deterministic
    float tot = sm_p[0][i];
#pragma unroll
    for (int k = 1; k < ATC_G; ++k) tot += sm_p[k][i];
    const float gate = qg[(size_t) t * ldq + (size_t) h * 2 * hd + hd + i];
    out[((size_t) t * nq + h) * hd + i] = tot / z * sigmoidf_(gate);
}


}  // namespace fnxb
