// Gated attention for a verify window: per-head norm + rotary + KV append, then tree-masked split-K attention.
//
// fnx_attn_prep_append replaces attn_prep_append / k_attn_prep_append (engine/src/kernels.hpp:259,
// engine/src/kernels.cu:1880-1910; norm_rope :513-530).  fnx_attn replaces attn / k_attn_part + k_attn_local +
// k_attn_combine (engine/src/kernels.hpp:238, engine/src/kernels.cu:558-667, 786-803): the same online-softmax
// split over positions, except that one block serves every row of the window for its share of the positions (the
// K and V rows are read once per window, not once per row), the cache is not split across cards by position, and
// a row may see only the window rows on its path to the root (the reference's windows are chains).
#include "fnx_common.cuh"

namespace fnxb {

// ------------------------------------------------------------------------------------------------ prep + append
__global__ void k_attn_prep_append(float* __restrict__ qg, int ldq, float* __restrict__ k, int ldk, const float* __restrict__ v, int ldv,
                                   const float* __restrict__ qn, const float* __restrict__ kn, __half* __restrict__ kc,
                                   __half* __restrict__ vc, int nq, int nkv, int hd, int nrot, const int* __restrict__ pos0p,
                                   const int* __restrict__ depth, float eps, float rope_base) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float xrow[];   // hd floats
    __shared__ float red[32];
    const int t = blockIdx.y, h = blockIdx.x, i = threadIdx.x, pos0 = *pos0p;
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
    __syncthreads();
    ss = 0.f;
    for (int j = 0; j < hd / 32; ++j) ss += red[j];
    xrow[i] = val * rsqrtf(ss / (float) hd + eps) * w[i];
    __syncthreads();
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
constexpr int ATT_CH = 32;        // positions per chunk
constexpr int ATT_ROWS = 5;       // window rows one block serves
constexpr int ATT_THREADS = 256;
constexpr int ATT_MAXQ = 8;       // q heads per KV head

struct AttPartial {   // one (row, head, split)
    float m, z;
};

// scratch: acc [T][nq][S][hd] floats, then mz [T][nq][S]
__global__ void __launch_bounds__(ATT_THREADS) k_attn_part(const float* __restrict__ qg, int ldq, const __half* __restrict__ kc,
                                                           const __half* __restrict__ vc, float* __restrict__ acc_out,
                                                           AttPartial* __restrict__ mz_out, int T, int nq, int nkv, int hd,
                                                           const int* __restrict__ pos0p, const int* __restrict__ parent) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) uint8_t smem[];
    const int s = blockIdx.x, S = gridDim.x, kvh = blockIdx.y, r0 = blockIdx.z * ATT_ROWS;
    const int nr = min(ATT_ROWS, T - r0), qpk = nq / nkv, NQ = nr * qpk;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pos0 = *pos0p, ctx = pos0 + T;
    const int KS = hd + 8;   // padded K row (halves): 16-byte reads by 8 lanes land in 8 different bank groups
    float* qs = reinterpret_cast<float*>(smem);                        // [ATT_ROWS * ATT_MAXQ][hd]
    __half* Ks = reinterpret_cast<__half*>(qs + ATT_ROWS * ATT_MAXQ * hd);   // [ATT_CH][KS]
    __half* Vs = Ks + ATT_CH * KS;                                     // [ATT_CH][hd]
    float* es = reinterpret_cast<float*>(Vs + ATT_CH * hd);            // [NQ max][ATT_CH]
    float* fs = es + ATT_ROWS * ATT_MAXQ * ATT_CH;                     // rescale per query
    float* ms = fs + ATT_ROWS * ATT_MAXQ;                              // running max
    float* zs = ms + ATT_ROWS * ATT_MAXQ;                              // running sum
    unsigned* see = reinterpret_cast<unsigned*>(zs + ATT_ROWS * ATT_MAXQ);   // per local row: window rows it sees
    {   // a block with no positions leaves only empty partials: the merge skips them without reading their sums
        const int nch0 = (ctx + ATT_CH - 1) / ATT_CH;
        if ((int) ((long long) nch0 * s / S) >= (int) ((long long) nch0 * (s + 1) / S)) {
            if (tid < NQ) {
                const int r = tid / qpk, hh = tid % qpk;
                mz_out[((size_t) (r0 + r) * nq + kvh * qpk + hh) * S + s] = AttPartial{-INFINITY, 0.f};
            }
            return;
        }
    }
    // the queries: 16 bytes per thread per load, 8 loads in flight
    for (int i0 = tid; i0 < NQ * hd / 4; i0 += 8 * ATT_THREADS) {
        float4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = i0 + j * ATT_THREADS;
            if (i < NQ * hd / 4) {
                const int qi = i / (hd / 4), d4 = i % (hd / 4), r = qi / qpk, hh = qi % qpk;
                v[j] = *reinterpret_cast<const float4*>(qg + (size_t) (r0 + r) * ldq + (size_t) (kvh * qpk + hh) * 2 * hd + d4 * 4);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = i0 + j * ATT_THREADS;
            if (i < NQ * hd / 4) reinterpret_cast<float4*>(qs)[i] = v[j];
        }
    }
    if (tid < NQ) { ms[tid] = -INFINITY; zs[tid] = 0.f; }
    if (tid < nr) {
        unsigned m = 0;
        for (int a = r0 + tid; a >= 0; a = parent ? parent[a] : a - 1) m |= 1u << a;
        see[tid] = m;
    }
    float acc[ATT_ROWS * ATT_MAXQ];
#pragma unroll
    for (int i = 0; i < ATT_ROWS * ATT_MAXQ; ++i) acc[i] = 0.f;
    // this block's chunks: a contiguous share of the ceil(ctx / 32) chunks
    const int nch = (ctx + ATT_CH - 1) / ATT_CH;
    const int c0 = (int) ((long long) nch * s / S), c1 = (int) ((long long) nch * (s + 1) / S);
    const float scale = rsqrtf((float) hd);
    for (int c = c0; c < c1; ++c) {
        const int p0 = c * ATT_CH, np = min(ATT_CH, ctx - p0);
        __syncthreads();
        // K and V rows of the chunk, 16 bytes per thread per step
        {
            constexpr int NL = ATT_CH * 256 / 8 / ATT_THREADS;   // 4 K and 4 V loads per thread, all in flight (hd == 256)
            uint4 kv4[NL], vv4[NL];
#pragma unroll
            for (int j = 0; j < NL; ++j) {
                const int i = tid + j * ATT_THREADS, pp = i / (hd / 8), d8 = i % (hd / 8);
                kv4[j] = vv4[j] = make_uint4(0, 0, 0, 0);
                if (pp < np) {
                    const size_t g = ((size_t) (p0 + pp) * nkv + kvh) * hd + d8 * 8;
                    kv4[j] = *reinterpret_cast<const uint4*>(kc + g);
                    vv4[j] = *reinterpret_cast<const uint4*>(vc + g);
                }
            }
#pragma unroll
            for (int j = 0; j < NL; ++j) {
                const int i = tid + j * ATT_THREADS, pp = i / (hd / 8), d8 = i % (hd / 8);
                *reinterpret_cast<uint4*>(Ks + pp * KS + d8 * 8) = kv4[j];
                *reinterpret_cast<uint4*>(Vs + pp * hd + d8 * 8) = vv4[j];
            }
        }
        __syncthreads();
        // scores: warp w takes queries w, w + 8, ... together (one read of the K row feeds all of them); lane = position
        {
            constexpr int NWQ = ATT_THREADS / 32, QPW = (ATT_ROWS * ATT_MAXQ + NWQ - 1) / NWQ;
            const __half* kr = Ks + lane * KS;
            float sacc[QPW];
#pragma unroll
            for (int j = 0; j < QPW; ++j) sacc[j] = 0.f;
            for (int d = 0; d < hd; d += 8) {
                const uint4 kk = *reinterpret_cast<const uint4*>(kr + d);
                const float2 k0 = __half22float2(*reinterpret_cast<const __half2*>(&kk.x));
                const float2 k1 = __half22float2(*reinterpret_cast<const __half2*>(&kk.y));
                const float2 k2 = __half22float2(*reinterpret_cast<const __half2*>(&kk.z));
                const float2 k3 = __half22float2(*reinterpret_cast<const __half2*>(&kk.w));
#pragma unroll
                for (int j = 0; j < QPW; ++j) {
                    const int qi = warp + j * NWQ;
                    if (qi < NQ) {
                        const float* q = qs + qi * hd + d;
                        const float4 q0 = *reinterpret_cast<const float4*>(q), q1 = *reinterpret_cast<const float4*>(q + 4);
                        float a = sacc[j];
                        a = fmaf(q0.x, k0.x, a); a = fmaf(q0.y, k0.y, a);
                        a = fmaf(q0.z, k1.x, a); a = fmaf(q0.w, k1.y, a);
                        a = fmaf(q1.x, k2.x, a); a = fmaf(q1.y, k2.y, a);
                        a = fmaf(q1.z, k3.x, a); a = fmaf(q1.w, k3.y, a);
                        sacc[j] = a;
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < QPW; ++j) {
                const int qi = warp + j * NWQ;
                if (qi >= NQ) continue;
                const int p = p0 + lane, r = qi / qpk;
                const bool vis = lane < np && (p < pos0 || ((see[r] >> (p - pos0)) & 1u));
                const float sv = vis ? sacc[j] * scale : -INFINITY;
                const float mo = ms[qi], mn = fmaxf(mo, warp_max(sv));
                const float w = sv == -INFINITY ? 0.f : expf(sv - mn);
                const float f = mo == -INFINITY ? 0.f : expf(mo - mn);
                const float zn = zs[qi] * f + warp_sum(w);
                es[qi * ATT_CH + lane] = w;
                __syncwarp();
                if (lane == 0) { ms[qi] = mn; zs[qi] = zn; fs[qi] = f; }
            }
        }
        __syncthreads();
        // values: thread = dimension (hd == ATT_THREADS), all queries
        for (int d = tid; d < hd; d += ATT_THREADS) {
#pragma unroll
            for (int qi = 0; qi < ATT_ROWS * ATT_MAXQ; ++qi)
                if (qi < NQ) acc[qi] *= fs[qi];
            for (int pp = 0; pp < ATT_CH; pp += 4) {
                const float v0 = __half2float(Vs[pp * hd + d]), v1 = __half2float(Vs[(pp + 1) * hd + d]);
                const float v2 = __half2float(Vs[(pp + 2) * hd + d]), v3 = __half2float(Vs[(pp + 3) * hd + d]);
#pragma unroll
                for (int qi = 0; qi < ATT_ROWS * ATT_MAXQ; ++qi)
                    if (qi < NQ) {
                        const float4 e4 = *reinterpret_cast<const float4*>(es + qi * ATT_CH + pp);
                        acc[qi] = fmaf(e4.x, v0, acc[qi]);
                        acc[qi] = fmaf(e4.y, v1, acc[qi]);
                        acc[qi] = fmaf(e4.z, v2, acc[qi]);
                        acc[qi] = fmaf(e4.w, v3, acc[qi]);
                    }
            }
        }
    }
    __syncthreads();
    if (tid < hd) {
#pragma unroll
        for (int qi = 0; qi < ATT_ROWS * ATT_MAXQ; ++qi)
            if (qi < NQ) {
                const int r = qi / qpk, hh = qi % qpk;
                const size_t slot = ((size_t) (r0 + r) * nq + kvh * qpk + hh) * S + s;
                acc_out[slot * hd + tid] = acc[qi];
            }
    }
    if (tid < NQ) {
        const int r = tid / qpk, hh = tid % qpk;
        mz_out[((size_t) (r0 + r) * nq + kvh * qpk + hh) * S + s] = AttPartial{ms[tid], zs[tid]};
    }
}

// merge the splits of (row, head): out = sum_s exp(m_s - m) acc_s / sum_s exp(m_s - m) z_s * sigmoid(gate)
constexpr int ATC_G = 4;   // groups of hd threads that share the splits of one (row, head)

__global__ void __launch_bounds__(ATT_THREADS * ATC_G) k_attn_combine(const float* __restrict__ acc_in, const AttPartial* __restrict__ mz_in,
                                                                      const float* __restrict__ qg, int ldq, float* __restrict__ out, int nq, int hd,
                                                                      int S) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float sm_m[256], sm_w[256], sm_z[256], sm_p[ATC_G][ATT_THREADS];
    const int h = blockIdx.x, t = blockIdx.y, i = threadIdx.x % ATT_THREADS, g = threadIdx.x / ATT_THREADS;
    const size_t base = ((size_t) t * nq + h) * S;
    AttPartial p = AttPartial{-INFINITY, 0.f};
    if (g == 0) {
        if (i < S) p = mz_in[base + i];
        sm_m[i] = i < S ? p.m : -INFINITY;
    }
    __syncthreads();
    // block maximum of m (S <= 256)
    float mx = -INFINITY;
    for (int s = 0; s < S; ++s) mx = fmaxf(mx, sm_m[s]);
    if (g == 0) {
        const float w = i < S && p.m != -INFINITY ? expf(p.m - mx) : 0.f;
        sm_w[i] = w;
        sm_z[i] = w * p.z;
    }
    __syncthreads();
    // group g adds the live splits g, g + G, ... in order (8 loads in flight); group 0 then adds the groups in order
    float acc = 0.f;
    for (int s0 = g; s0 < S; s0 += 8 * ATC_G) {
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
    sm_p[g][i] = acc;
    __syncthreads();
    if (g != 0) return;
    float z = 0.f;
    for (int s = 0; s < S; ++s) z += sm_z[s];        // fixed order: deterministic
    float tot = sm_p[0][i];
#pragma unroll
    for (int k = 1; k < ATC_G; ++k) tot += sm_p[k][i];
    const float gate = qg[(size_t) t * ldq + (size_t) h * 2 * hd + hd + i];
    out[((size_t) t * nq + h) * hd + i] = tot / z * sigmoidf_(gate);
}

static int attn_splits(int nkv) {
    const int s = sm_count() / (nkv > 0 ? nkv : 1);
    return s < 1 ? 1 : s;
}

}  // namespace fnxb

using namespace fnxb;

extern "C" int fnx_attn_prep_append(float* qg, int ldq, float* k, int ldk, const float* v, int ldv, const float* q_norm, const float* k_norm,
                                    void* kc, void* vc, int T, int nq, int nkv, int hd, int nrot, const int* pos0, const int* depth, float eps,
                                    float rope_base, fnx_stream st) {
    FNX_REQUIRE(qg && k && v && q_norm && k_norm && kc && vc && pos0, "fnx_attn_prep_append: null pointer");
    FNX_REQUIRE(T >= 1 && T <= FNX_MAX_ROWS, "fnx_attn_prep_append: %d rows", T);
    FNX_REQUIRE(hd % 32 == 0 && hd <= 1024 && nrot <= hd && nrot % 2 == 0, "fnx_attn_prep_append: head dim %d, rotary %d", hd, nrot);
    {
        const cudaError_t le_ = launch_k(k_attn_prep_append, dim3(dim3(nq + 2 * nkv, T)), dim3(hd), hd * sizeof(float), as_stream(st), qg, ldq, k, ldk, v, ldv, q_norm, k_norm, (__half*) kc, (__half*) vc,
                                                                                        nq, nkv, hd, nrot, pos0, depth, eps, rope_base);
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "k_attn_prep_append: launch failed: %s", cudaGetErrorString(le_));
    }
    FNX_LAUNCH_OK("fnx_attn_prep_append");
    return FNX_OK;
}

extern "C" size_t fnx_attn_scratch_bytes(int T, int nq, int hd) {
    const size_t S = (size_t) sm_count();   // an upper bound of the splits for any KV-head count
    return (size_t) T * nq * S * ((size_t) hd * sizeof(float) + sizeof(AttPartial));
}

extern "C" int fnx_attn(const float* qg, int ldq, const void* kc, const void* vc, float* out, int T, int nq, int nkv, int hd, const int* pos0,
                        const int* parent, void* scratch, fnx_stream st) {
    FNX_REQUIRE(qg && kc && vc && out && pos0 && scratch, "fnx_attn: null pointer");
    FNX_REQUIRE(T >= 1 && T <= FNX_MAX_ROWS, "fnx_attn: %d rows", T);
    FNX_REQUIRE(hd == ATT_THREADS, "fnx_attn: head dim %d (this build: %d)", hd, ATT_THREADS);
    FNX_REQUIRE(nkv >= 1 && nq % nkv == 0 && nq / nkv <= ATT_MAXQ, "fnx_attn: %d q heads over %d KV heads", nq, nkv);
    const int S = attn_splits(nkv);
    FNX_REQUIRE(S <= 256, "fnx_attn: %d splits", S);
    float* acc = (float*) scratch;
    AttPartial* mz = (AttPartial*) (acc + (size_t) T * nq * S * hd);
    const size_t smem = (size_t) ATT_ROWS * ATT_MAXQ * hd * sizeof(float) + (size_t) ATT_CH * (hd + 8) * sizeof(__half) +
                        (size_t) ATT_CH * hd * sizeof(__half) + (size_t) ATT_ROWS * ATT_MAXQ * (ATT_CH + 3) * sizeof(float) +
                        ATT_ROWS * sizeof(unsigned);
    static bool configured = false;
    if (!configured) {
        FNX_CUDA_OK(cudaFuncSetAttribute(k_attn_part, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
        configured = true;
    }
    {
        const cudaError_t le_ = launch_k(k_attn_part, dim3(dim3(S, nkv, (T + ATT_ROWS - 1) / ATT_ROWS)), dim3(ATT_THREADS), smem, as_stream(st), qg, ldq, (const __half*) kc, (const __half*) vc,
                                                                                                   acc, mz, T, nq, nkv, hd, pos0, parent);
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "k_attn_part: launch failed: %s", cudaGetErrorString(le_));
    }
    FNX_LAUNCH_OK("fnx_attn (partials)");
    {
        const cudaError_t le_ = launch_k(k_attn_combine, dim3(dim3(nq, T)), dim3(hd * ATC_G), 0, as_stream(st), acc, mz, qg, ldq, out, nq, hd, S);
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "k_attn_combine: launch failed: %s", cudaGetErrorString(le_));
    }
    FNX_LAUNCH_OK("fnx_attn (combine)");
    return FNX_OK;
}

// ---- allocation-free variant: the split partials live in a file-scope device array -------------------------------------------------

namespace fnxb {

constexpr int ATT_STATIC_SLOTS = FNX_ATTN_STATIC_MAX_SLOTS;   // (row, head, split) partials
constexpr int ATT_STATIC_HD = ATT_THREADS;
constexpr size_t ATT_STATIC_BYTES = (size_t) ATT_STATIC_SLOTS * (ATT_STATIC_HD * sizeof(float) + sizeof(AttPartial));
static __device__ __align__(256) unsigned char g_attn_static_scratch[ATT_STATIC_BYTES];

constexpr int ATT_STATIC_MAX_DEV = 64;
static void* g_attn_static_ptr[ATT_STATIC_MAX_DEV];   // per device: the array's address, resolved once

static int attn_static_resolve(void** out) {
    int dev = -1;
    FNX_CUDA_OK(cudaGetDevice(&dev));
    FNX_REQUIRE(dev >= 0 && dev < ATT_STATIC_MAX_DEV, "fnx_attn_static: device %d", dev);
    if (!g_attn_static_ptr[dev]) {
        void* p = nullptr;
        const cudaError_t rc = cudaGetSymbolAddress((void**) &p, g_attn_static_scratch);
        if (rc != cudaSuccess || !p) return fail(FNX_E_CUDA, "fnx_attn_static: cudaGetSymbolAddress: %s", cudaGetErrorString(rc));
        FNX_CUDA_OK(cudaFuncSetAttribute(k_attn_part, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
        g_attn_static_ptr[dev] = p;
    }
    *out = g_attn_static_ptr[dev];
    return FNX_OK;
}

}  // namespace fnxb

extern "C" int fnx_attn_static_setup(void) {
    void* p = nullptr;
    return attn_static_resolve(&p);
}

extern "C" int fnx_attn_static(const float* qg, int ldq, const void* kc, const void* vc, float* out, int T, int nq, int nkv, int hd, const int* pos0,
                               const int* parent, fnx_stream st) {
    FNX_REQUIRE(qg && kc && vc && out && pos0, "fnx_attn_static: null pointer");
    FNX_REQUIRE(T >= 1 && T <= FNX_MAX_ROWS, "fnx_attn_static: %d rows", T);
    FNX_REQUIRE(hd == ATT_THREADS, "fnx_attn_static: head dim %d (this build: %d)", hd, ATT_THREADS);
    FNX_REQUIRE(nkv >= 1 && nq % nkv == 0 && nq / nkv <= ATT_MAXQ, "fnx_attn_static: %d q heads over %d KV heads", nq, nkv);
    const int S = attn_splits(nkv);
    FNX_REQUIRE(S <= 256, "fnx_attn_static: %d splits", S);
    const long long slots = (long long) T * nq * S;
    FNX_REQUIRE(slots <= ATT_STATIC_SLOTS,
                "fnx_attn_static: %d rows x %d heads x %d splits = %lld partials exceed the built-in scratch of %d; use fnx_attn with caller scratch",
                T, nq, S, slots, ATT_STATIC_SLOTS);
    void* scratch = nullptr;
    if (const int rc = attn_static_resolve(&scratch)) return rc;
    float* acc = (float*) scratch;
    AttPartial* mz = (AttPartial*) (acc + (size_t) slots * hd);
    const size_t smem = (size_t) ATT_ROWS * ATT_MAXQ * hd * sizeof(float) + (size_t) ATT_CH * (hd + 8) * sizeof(__half) +
                        (size_t) ATT_CH * hd * sizeof(__half) + (size_t) ATT_ROWS * ATT_MAXQ * (ATT_CH + 3) * sizeof(float) +
                        ATT_ROWS * sizeof(unsigned);
    cudaError_t le = launch_k(k_attn_part, dim3(S, nkv, (T + ATT_ROWS - 1) / ATT_ROWS), dim3(ATT_THREADS), smem, as_stream(st), qg, ldq,
                              (const __half*) kc, (const __half*) vc, acc, mz, T, nq, nkv, hd, pos0, parent);
    if (le != cudaSuccess) return fail(FNX_E_CUDA, "k_attn_part: launch failed: %s", cudaGetErrorString(le));
    FNX_LAUNCH_OK("fnx_attn_static (partials)");
    le = launch_k(k_attn_combine, dim3(nq, T), dim3(hd * ATC_G), 0, as_stream(st), acc, mz, qg, ldq, out, nq, hd, S);
    if (le != cudaSuccess) return fail(FNX_E_CUDA, "k_attn_combine: launch failed: %s", cudaGetErrorString(le));
    FNX_LAUNCH_OK("fnx_attn_static (combine)");
    return FNX_OK;
}
