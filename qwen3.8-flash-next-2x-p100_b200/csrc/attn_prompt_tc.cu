// Prompt attention on the 5th-generation tensor cores: the chunk's query rows against the sequence's K/V cache, causal,
// for models whose KV head serves eight query heads of 256 dims (the benchmark's shape).  The counterpart of the reference's
// attn_prompt (engine/src/kernels.hpp:252); same arithmetic as the mma.sync form it stands in for (fnx_attn_prompt's other
// path): f16 queries, f32 scores, an online softmax over steps of 64 positions with f16 weights, f32 sums, the sigmoid gate.
//
// One block = 16 chunk rows x the 8 query heads of one KV head = 128 score rows (tensor-memory lanes), so a K/V tile is
// fetched once for 128 rows.  Per step of 64 positions:
//   S = Q K^T        16 x tcgen05.mma M128 N64 K16   (Q, K in shared memory, K-major core matrices; S in tensor memory)
//   softmax          one thread per row: tcgen05.ld of its 64 scores, running max / sum, weights rounded to f16 into shared
//                    memory (the A operand of the next product); the row of O is rescaled in tensor memory only when some
//                    row of the warp moved its maximum
//   O += P V         4 x tcgen05.mma M128 N256 K16   (V as it lies in the cache: dims contiguous = an MN-major B operand)
// K and V tiles are double-buffered (16-byte async copies by four loader warps run one step ahead).  Every wait is bounded.
#include <cuda_fp16.h>

#include "fnx_common.cuh"

namespace fnxb {

constexpr int TA_M = 128;          // score rows per block: 16 positions x 8 heads
constexpr int TA_POS = 16;
constexpr int TA_QPK = 8;
constexpr int TA_N = 64;           // positions per step
constexpr int TA_HD = 256;
constexpr int TA_THREADS = 256;    // warps 0-3: one thread per row; warps 4-7: loaders, and the thread that issues the products
// Core matrices (8 rows x 16 bytes).  Q: 128 bytes apart along K (dense).  K and P: 144 bytes apart, V's 8-dim groups 1040
// bytes apart: a quarter warp's 16-byte pieces (4 positions x 8 dim groups: 128-byte runs of the cache) then fall into eight
// different 16-byte bank groups.
constexpr int TA_LBO_Q = 128;
constexpr int TA_SBO_Q = (TA_HD / 8) * TA_LBO_Q;  // between 8-row groups of Q
constexpr int TA_LBO = 144;                       // K and P: between core matrices along K (dims, positions)
constexpr int TA_SBO_K = (TA_HD / 8) * TA_LBO;    // between 8-position groups of K
constexpr int TA_SBO_P = (TA_N / 8) * TA_LBO;     // between 8-row groups of P
constexpr int TA_V_LBO = 128;                     // V, MN-major: between 8-position groups
constexpr int TA_V_SBO = (TA_N / 8) * TA_V_LBO + 16;   // ... between 8-dim groups
constexpr int TA_Q_BYTES = (TA_M / 8) * TA_SBO_Q, TA_K_BYTES = (TA_N / 8) * TA_SBO_K, TA_V_BYTES = (TA_HD / 8) * TA_V_SBO, TA_P_BYTES = (TA_M / 8) * TA_SBO_P;
constexpr int TA_SMEM = TA_Q_BYTES + 2 * TA_K_BYTES + 2 * TA_V_BYTES + TA_P_BYTES + 64;
static_assert(TA_SMEM <= 227 * 1024, "the tiles fit one block's shared memory");
constexpr int TA_TMEM_COLS = 512;  // S: columns [0, 64); O: [64, 320)
constexpr unsigned TA_WAIT = 20000000u;

__device__ __forceinline__ uint64_t ta_desc(uint32_t saddr, int lbo, int sbo) {
    // shared-memory matrix descriptor: start address, leading and stride byte offsets in 16-byte units, version 1, no swizzle
    return (uint64_t) ((saddr & 0x3FFFFu) >> 4) | ((uint64_t) (lbo >> 4) << 16) | ((uint64_t) (sbo >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ void ta_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void ta_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void ta_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void ta_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])),
        "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])),
        "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])),
        "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
        "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ void ta_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void ta_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void ta_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// grid (16-row tiles of the chunk, latest first; KV heads)
__global__ void __launch_bounds__(TA_THREADS, 1) k_attn_prompt_tc(const float* __restrict__ qg, int ldq, const __half* __restrict__ kc,
                                                                 const __half* __restrict__ vc, float* __restrict__ out, int T, int nq, int nkv,
                                                                 const int* __restrict__ pos0p, unsigned* __restrict__ err) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* Qs = smem;
    uint8_t* Ks = Qs + TA_Q_BYTES;                 // two buffers
    uint8_t* Vs = Ks + 2 * TA_K_BYTES;             // two buffers
    uint8_t* Ps = Vs + 2 * TA_V_BYTES;
    uint64_t* bar_s = reinterpret_cast<uint64_t*>(Ps + TA_P_BYTES);
    uint64_t* bar_o = bar_s + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_o + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = (int) gridDim.x - 1 - (int) blockIdx.x, kvh = blockIdx.y;
    const int t0 = tile * TA_POS, nr = min(TA_POS, T - t0), pos0 = *pos0p;
    const int ctx = pos0 + t0 + nr;                // the tile's rows see positions [0, ctx): a chain's rows see nothing past themselves
    const int nsteps = (ctx + TA_N - 1) / TA_N;
    if (tid == 0) {
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        fence_barrier_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TA_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // K and V rows of one step into buffer b: one 16-byte piece = 8 dims of one position = one core-matrix row
    auto fetch_kv = [&](int b, int p0) {
        const int np = min(TA_N, ctx - p0), lt = tid - TA_THREADS / 2;
        uint8_t* kd = Ks + b * TA_K_BYTES;
        uint8_t* vd = Vs + b * TA_V_BYTES;
#pragma unroll 4
        for (int j = 0; j < TA_N * (TA_HD / 8) / (TA_THREADS / 2); ++j) {
            // a quarter warp takes 4 positions x 8 pieces of 8 dims: four full 128-byte lines of the cache
            const int i = lt + j * (TA_THREADS / 2), rest = i >> 5, n = (rest & 15) * 4 + (i & 3), d8 = (rest >> 4) * 8 + ((i >> 2) & 7);
            const uint32_t ko = (uint32_t) ((n >> 3) * TA_SBO_K + d8 * TA_LBO + (n & 7) * 16);
            const uint32_t vo = (uint32_t) (d8 * TA_V_SBO + (n >> 3) * TA_V_LBO + (n & 7) * 16);
            if (n < np) {
                const size_t go = ((size_t) (p0 + n) * nkv + kvh) * TA_HD + d8 * 8;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(kd + ko)), "l"(kc + go) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(vd + vo)), "l"(vc + go) : "memory");
            } else {
                *reinterpret_cast<uint4*>(kd + ko) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vd + vo) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (warp >= 4) fetch_kv(0, 0);
    // the queries as f16: row r = head (r / 16), chunk row t0 + r % 16; rows past the chunk's end are zero
    for (int i = tid; i < TA_M * (TA_HD / 8); i += TA_THREADS) {
        const int r = i % TA_M, d8 = i / TA_M, hh = r >> 4, pi = r & 15;
        uint4 pk = make_uint4(0, 0, 0, 0);
        if (pi < nr) {
            const float* src = qg + (size_t) (t0 + pi) * ldq + (size_t) (kvh * TA_QPK + hh) * 2 * TA_HD + d8 * 8;
            const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
            const __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(a.z, a.w), h2 = __floats2half2_rn(b.x, b.y), h3 = __floats2half2_rn(b.z, b.w);
            pk = make_uint4(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1), *reinterpret_cast<const uint32_t*>(&h2),
                            *reinterpret_cast<const uint32_t*>(&h3));
        }
        *reinterpret_cast<uint4*>(Qs + (r >> 3) * TA_SBO_Q + d8 * TA_LBO_Q + (r & 7) * 16) = pk;
    }
    ta_fence_before();
    __syncthreads();
    ta_fence_after();
    const uint32_t tmem = *tmem_slot, tm_s = tmem, tm_o = tmem + TA_N;
    // f32 accumulate, f16 x f16, M = 128; S: both operands K-major, N = 64; O: B (V) MN-major, N = 256
    constexpr uint32_t IDESC_S = (1u << 4) | ((uint32_t) (TA_N >> 3) << 17) | ((uint32_t) (TA_M >> 4) << 24);
    constexpr uint32_t IDESC_O = (1u << 4) | (1u << 16) | ((uint32_t) (TA_HD >> 3) << 17) | ((uint32_t) (TA_M >> 4) << 24);
    const uint32_t q_s = smem_u32(Qs), k_s = smem_u32(Ks), v_s = smem_u32(Vs), p_s = smem_u32(Ps);
    const int r = tid & (TA_M - 1), pi = min(r & 15, nr - 1);   // (warps 0-3) the thread's row and its chunk row (a row past the end: the last one's mask)
    const int my_pos = pos0 + t0 + pi;
    const uint32_t lane_base = (uint32_t) (32 * (warp & 3)) << 16;
    float m_run = -INFINITY, z_run = 0.f;
    bool ok = true;
    for (int j = 0; j < nsteps; ++j) {
        const int b = j & 1, p0 = j * TA_N;
        if (warp >= 4) {
            asm volatile("cp.async.wait_group 0;" ::: "memory");   // this step's rows have landed
        }
        fence_proxy_async();   // the tiles were written through the generic proxy; the tensor core reads them through the async one
        if (__syncthreads_or(!ok)) {
            ok = false;
            break;
        }
        if (tid == TA_THREADS / 2) {
            ta_fence_after();
#pragma unroll
            for (int k16 = 0; k16 < TA_HD / 16; ++k16)
                ta_mma(tm_s, ta_desc(q_s + k16 * 2 * TA_LBO_Q, TA_LBO_Q, TA_SBO_Q), ta_desc(k_s + b * TA_K_BYTES + k16 * 2 * TA_LBO, TA_LBO, TA_SBO_K), IDESC_S,
                       k16 != 0);
            ta_commit(bar_s);
        }
        if (warp >= 4) {
            __syncwarp();
            if (j + 1 < nsteps) {
                // the other buffer held the last step's V: free once its product has finished
                if (j >= 1) ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_o, (unsigned) ((j - 1) & 1), TA_WAIT));
                if (ok) fetch_kv(b ^ 1, p0 + TA_N);
            }
        } else {
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_s, (unsigned) (j & 1), TA_WAIT));
            ta_fence_after();
            float f = 1.f;
            if (ok) {
                float s[TA_N];
                {
                    float a[32], c[32];
                    ta_ld32(tm_s + lane_base, a);
                    ta_ld32(tm_s + lane_base + 32, c);
#pragma unroll
                    for (int i = 0; i < 32; ++i) { s[i] = a[i]; s[32 + i] = c[i]; }
                }
                // scaled and masked: a step wholly before the tile's first row is visible to every row
                const bool open_step = p0 + TA_N <= pos0 + t0 + 1;
                float mx = -INFINITY;
#pragma unroll
                for (int i = 0; i < TA_N; ++i) {
                    const bool vis = open_step || p0 + i <= my_pos;
                    s[i] = vis ? s[i] * 0.0625f : -INFINITY;   // 1 / sqrt(256)
                    mx = fmaxf(mx, s[i]);
                }
                const float mn = fmaxf(m_run, mx);
                float sum = 0.f;
                uint32_t pk[TA_N / 2];
#pragma unroll
                for (int i = 0; i < TA_N; i += 2) {
                    const __half2 h = __floats2half2_rn(s[i] == -INFINITY ? 0.f : __expf(s[i] - mn), s[i + 1] == -INFINITY ? 0.f : __expf(s[i + 1] - mn));
                    const float2 back = __half22float2(h);
                    sum += back.x;
                    sum += back.y;
                    pk[i / 2] = *reinterpret_cast<const uint32_t*>(&h);
                }
                f = m_run == -INFINITY ? 0.f : __expf(m_run - mn);
                z_run = z_run * f + sum;
                m_run = mn;
                // the last step's product has read P and written O
                if (j >= 1) {
                    ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_o, (unsigned) ((j - 1) & 1), TA_WAIT));
                    ta_fence_after();
                }
                if (ok) {
#pragma unroll
                    for (int c8 = 0; c8 < TA_N / 8; ++c8)
                        *reinterpret_cast<uint4*>(Ps + (r >> 3) * TA_SBO_P + c8 * TA_LBO + (r & 7) * 16) =
                            make_uint4(pk[c8 * 4], pk[c8 * 4 + 1], pk[c8 * 4 + 2], pk[c8 * 4 + 3]);
                    // (deep into a long context the running maxima rarely move: a warp whose factors are all 1 leaves O alone)
                    if (j >= 1 && __any_sync(0xffffffffu, f != 1.0f)) {
#pragma unroll 1
                        for (int c32 = 0; c32 < TA_HD / 32; ++c32) {
                            float o[32];
                            ta_ld32(tm_o + lane_base + c32 * 32, o);
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] *= f;
                            ta_st32(tm_o + lane_base + c32 * 32, o);
                        }
                        ta_wait_st();
                    }
                }
            }
            ta_fence_before();
        }
        fence_proxy_async();   // P went through the generic proxy
        if (__syncthreads_or(!ok)) {
            ok = false;
            break;
        }
        if (tid == TA_THREADS / 2) {
            ta_fence_after();
#pragma unroll
            for (int k16 = 0; k16 < TA_N / 16; ++k16)
                ta_mma(tm_o, ta_desc(p_s + k16 * 2 * TA_LBO, TA_LBO, TA_SBO_P), ta_desc(v_s + b * TA_V_BYTES + k16 * 2 * TA_V_LBO, TA_V_LBO, TA_V_SBO), IDESC_O,
                       (j | k16) != 0);
            ta_commit(bar_o);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (ok && warp < 4) ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_o, (unsigned) ((nsteps - 1) & 1), TA_WAIT));
    ok = __syncthreads_and(ok) != 0;
    ta_fence_after();
    if (!ok && tid == 0 && err) atomicOr(err, (unsigned) FNX_ERR_TIMEOUT);
    if (ok && warp < 4) {
        // out = O / z * sigmoid(gate): the thread's row, 32 dims at a time (the tensor-memory loads are warp-wide: rows past the
        // chunk's end take part in them and write nothing)
        const bool live = (r & 15) < nr;
        const int hh = r >> 4, t = t0 + min(r & 15, nr - 1), h = kvh * TA_QPK + hh;
        const float* gate = qg + (size_t) t * ldq + (size_t) h * 2 * TA_HD + TA_HD;
        float* o_row = out + ((size_t) t * nq + h) * TA_HD;
        const float iz = 1.0f / z_run;
#pragma unroll 1
        for (int c32 = 0; c32 < TA_HD / 32; ++c32) {
            float o[32];
            ta_ld32(tm_o + lane_base + c32 * 32, o);
            if (live) {
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const float4 g = *reinterpret_cast<const float4*>(gate + c32 * 32 + i);
                    *reinterpret_cast<float4*>(o_row + c32 * 32 + i) =
                        make_float4(o[i] * iz * sigmoidf_(g.x), o[i + 1] * iz * sigmoidf_(g.y), o[i + 2] * iz * sigmoidf_(g.z), o[i + 3] * iz * sigmoidf_(g.w));
                }
            }
        }
    }
    ta_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TA_TMEM_COLS) : "memory");
}

bool attn_prompt_tc_fits(int nq, int nkv, int hd) { return hd == TA_HD && nkv >= 1 && nq == nkv * TA_QPK; }

int attn_prompt_tc_launch(const float* qg, int ldq, const __half* kc, const __half* vc, float* out, int T, int nq, int nkv, const int* pos0, unsigned* err,
                          cudaStream_t st) {
    if (int rc = set_smem_limit((const void*) k_attn_prompt_tc, TA_SMEM)) return rc;
    k_attn_prompt_tc<<<dim3((T + TA_POS - 1) / TA_POS, nkv), TA_THREADS, TA_SMEM, st>>>(qg, ldq, kc, vc, out, T, nq, nkv, pos0, err);
    FNX_LAUNCH_OK("fnx_attn_prompt (tensor-core form)");
    return FNX_OK;
}

}  // namespace fnxb
