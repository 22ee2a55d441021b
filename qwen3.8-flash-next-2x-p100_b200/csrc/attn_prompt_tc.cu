// Prompt attention on the 5th-generation tensor cores: the chunk's query rows against the sequence's K/V cache, causal,
// for models whose KV head serves eight query heads of 256 dims (the benchmark's shape).  The counterpart of the reference's
// attn_prompt (engine/src/kernels.hpp:252); same arithmetic as the mma.sync form it stands in for (fnx_attn_prompt's other
// path): f16 queries, f32 scores, an online softmax over steps of 64 positions with f16 weights, f32 sums, the sigmoid gate.
//
// One block = 16 chunk rows x the 8 query heads of one KV head = 128 score rows (tensor-memory lanes), so a K/V tile is
// fetched once for 128 rows.  Per step of 64 positions:
//   S = Q K^T        16 x tcgen05.mma M128 N64 K16   (Q, K in shared memory, K-major core matrices; S in tensor memory)
//   softmax          two threads per row: tcgen05.ld of their 32 scores each, running max / sum, weights rounded to f16 into
//                    shared memory (the A operand of the next product); the row of O is rescaled in tensor memory only when
//                    some row of the warp moved its maximum
//   O += P V         4 x tcgen05.mma M128 N256 K16   (V as it lies in the cache: dims contiguous = an MN-major B operand)
// K and V tiles are double-buffered and arrive as tensor copies (cp.async.bulk.tensor, 64 dims x 64 positions a box, 128-byte
// swizzle: the layout the products' shared-memory descriptors name), issued one step ahead by a loader thread; only a step that
// the context ends in is fetched by 16-byte async copies (the loader warps), so that nothing past the context is ever read.
// The 16-byte copies alone fed a block 3.3 TB/s over all SMs, the tensor copies 6.5 (loads only, measured).  Every wait is bounded.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>

#include "fnx_common.cuh"

namespace fnxb {

constexpr int TA_M = 128;          // score rows per block: 16 positions x 8 heads
constexpr int TA_POS = 16;
constexpr int TA_QPK = 8;
constexpr int TA_N = 64;           // positions per step
constexpr int TA_HD = 256;
constexpr int TA_SOFT = 256;       // warps 0-7: two threads per score row (a half of the step's positions each); thread 0 issues the products
constexpr int TA_THREADS = 512;    // warps 8-15: the loaders of the next step's K and V rows
// Q and P: core matrices (8 rows x 16 bytes), no swizzle.  Q: 128 bytes apart along K (dense).  P: 144 bytes apart, so that a
// quarter warp's 16-byte stores fall into eight different bank groups.
constexpr int TA_LBO_Q = 128;
constexpr int TA_SBO_Q = (TA_HD / 8) * TA_LBO_Q;  // between 8-row groups of Q
constexpr int TA_LBO = 144;                       // P: between core matrices along K (positions)
constexpr int TA_SBO_P = (TA_N / 8) * TA_LBO;     // between 8-row groups of P
// K and V: four boxes of 64 dims per buffer, each 64 positions x 128 bytes with the 128-byte swizzle (the 16-byte piece c of
// position n lies at piece c ^ (n % 8) of its row)
constexpr int TA_BOX_BYTES = TA_N * 128;          // 8 KB
constexpr int TA_SW_SBO = 8 * 128;                // between 8-position groups
constexpr int TA_Q_BYTES = (TA_M / 8) * TA_SBO_Q, TA_K_BYTES = (TA_HD / 64) * TA_BOX_BYTES, TA_V_BYTES = TA_K_BYTES, TA_P_BYTES = (TA_M / 8) * TA_SBO_P;
constexpr int TA_TAIL = 64 + 4 * TA_M * 4;        // barriers, the halves' exchange
constexpr int TA_SMEM = 1024 + 2 * TA_K_BYTES + 2 * TA_V_BYTES + TA_Q_BYTES + TA_P_BYTES + TA_TAIL;   // (1024: the swizzled tiles start on a 1024-byte boundary)
static_assert(TA_SMEM <= 227 * 1024, "the tiles fit one block's shared memory");
constexpr int TA_TMEM_COLS = 512;  // S: columns [0, 64); O: [64, 320)
constexpr unsigned TA_WAIT = 20000000u;

__device__ __forceinline__ uint64_t ta_desc(uint32_t saddr, int lbo, int sbo) {
    // shared-memory matrix descriptor: start address, leading and stride byte offsets in 16-byte units, version 1, no swizzle
    return (uint64_t) ((saddr & 0x3FFFFu) >> 4) | ((uint64_t) (lbo >> 4) << 16) | ((uint64_t) (sbo >> 4) << 32) | (1ull << 46);
}
// the same for a 128-byte-swizzled tile (layout type 2); K-major: the leading offset is not used; MN-major: it is the
// distance between the 64-element swizzle atoms along MN
__device__ __forceinline__ uint64_t ta_desc_sw(uint32_t saddr, int lbo, int sbo) {
    return (uint64_t) ((saddr & 0x3FFFFu) >> 4) | ((uint64_t) (lbo >> 4) << 16) | ((uint64_t) (sbo >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// one box of a rank-3 tensor map into shared memory, completion counted in bytes on `bar`
__device__ __forceinline__ void ta_tma_3d(uint32_t dst_s, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst_s), "l"(map),
                 "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
                 : "memory");
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
__device__ __forceinline__ float ta_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void ta_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void ta_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void ta_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// grid (16-row tiles of the chunk, latest first; KV heads).  Thread tid: score row tid % 128 (tensor-memory lane), column half
// tid / 128 (the step's positions [32 half, 32 half + 32); the output's dims [128 half, 128 half + 128)): the two threads of a
// row agree on the step's maximum through shared memory and keep half of the row's sum each.
__global__ void __launch_bounds__(TA_THREADS, 1) k_attn_prompt_tc(const float* __restrict__ qg, int ldq, const __half* __restrict__ kc,
                                                                 const __half* __restrict__ vc, float* __restrict__ out, int T, int nq, int nkv,
                                                                 const int* __restrict__ pos0p, unsigned* __restrict__ err, int use_tma,
                                                                 const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* Ks = smem;                            // two buffers
    uint8_t* Vs = Ks + 2 * TA_K_BYTES;             // two buffers
    uint8_t* Qs = Vs + 2 * TA_V_BYTES;
    uint8_t* Ps = Qs + TA_Q_BYTES;
    uint64_t* bar_s = reinterpret_cast<uint64_t*>(Ps + TA_P_BYTES);
    uint64_t* bar_o = bar_s + 1;
    uint64_t* bar_ld = bar_o + 1;                  // two: a buffer's boxes have landed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_ld + 2);
    float* xch = reinterpret_cast<float*>(Ps + TA_P_BYTES + 64);   // [2 step parities][2 halves][128 rows]: the halves' maxima (and, at the end, sums)
    const int tid = threadIdx.x, warp = tid >> 5;
    const int tile = (int) gridDim.x - 1 - (int) blockIdx.x, kvh = blockIdx.y;
    const int t0 = tile * TA_POS, nr = min(TA_POS, T - t0), pos0 = *pos0p;
    const int ctx = pos0 + t0 + nr;                // the tile's rows see positions [0, ctx): a chain's rows see nothing past themselves
    const int nsteps = (ctx + TA_N - 1) / TA_N;
    if (tid == 0) {
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        mbar_init(bar_ld, 1);
        mbar_init(bar_ld + 1, 1);
        fence_barrier_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TA_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // K and V rows of one step into buffer b.  A whole step: eight boxes by one thread.  The step the context ends in: 16-byte
    // pieces by the loader warps, placed where the swizzle puts them, the rows past the context zero.
    auto fetch_kv = [&](int b, int p0) {
        const int np = min(TA_N, ctx - p0);
        uint8_t* kd = Ks + b * TA_K_BYTES;
        uint8_t* vd = Vs + b * TA_V_BYTES;
        if (np == TA_N && use_tma) {
            if (tid == TA_SOFT) {
                mbar_expect_tx(bar_ld + b, 2 * TA_K_BYTES);
#pragma unroll
                for (int c = 0; c < TA_HD / 64; ++c) {
                    ta_tma_3d(smem_u32(kd + c * TA_BOX_BYTES), &map_k, c * 64, kvh, p0, bar_ld + b);
                    ta_tma_3d(smem_u32(vd + c * TA_BOX_BYTES), &map_v, c * 64, kvh, p0, bar_ld + b);
                }
            }
            return;
        }
#pragma unroll
        for (int j = 0; j < TA_N * (TA_HD / 8) / (TA_THREADS - TA_SOFT); ++j) {
            // a quarter warp takes 4 positions x 8 pieces of 8 dims: four full 128-byte lines of the cache
            const int i = (tid - TA_SOFT) + j * (TA_THREADS - TA_SOFT), rest = i >> 5, n = (rest & 15) * 4 + (i & 3), d8 = (rest >> 4) * 8 + ((i >> 2) & 7);
            const uint32_t off = (uint32_t) ((d8 >> 3) * TA_BOX_BYTES + n * 128 + (((d8 & 7) ^ (n & 7)) * 16));
            if (n < np) {
                const size_t go = ((size_t) (p0 + n) * nkv + kvh) * TA_HD + d8 * 8;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(kd + off)), "l"(kc + go) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(vd + off)), "l"(vc + go) : "memory");
            } else {
                *reinterpret_cast<uint4*>(kd + off) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vd + off) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const bool loader = tid >= TA_SOFT;
    __syncthreads();   // the barriers are initialised before the first tensor copy names one
    if (loader) fetch_kv(0, 0);
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
    const int r = tid & (TA_M - 1), half = (tid >> 7) & 1, pi = min(r & 15, nr - 1);   // the thread's row, its half, its chunk row (a row past the end: the last one's mask)
    const int my_pos = pos0 + t0 + pi;
    const uint32_t lane_base = (uint32_t) (32 * (warp & 3)) << 16;
    const unsigned pair_bar = 1u + (unsigned) (warp & 3);   // the named barrier of the row group's two warps
    // scores in the base-2 domain: exp(x - m) = exp2(x log2 e - m log2 e)
    const float scale2 = 0.0625f * 1.4426950408889634f;   // 1 / sqrt(256) x log2 e
    float m_run = -INFINITY, z_half = 0.f;
    bool ok = true;
    for (int j = 0; j < nsteps; ++j) {
        const int b = j & 1, p0 = j * TA_N;
        // this step's rows have landed: the boxes of a whole step on its buffer's barrier, the pieces of the context's last step
        // with their threads' copy groups
        if (use_tma && p0 + TA_N <= ctx) ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_ld + b, (unsigned) ((j >> 1) & 1), TA_WAIT));
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        fence_proxy_async();   // what went through the generic proxy (pieces, P, Q) before the tensor core reads it through the async one
        if (__syncthreads_or(!ok)) {
            ok = false;
            break;
        }
        if (tid == 0) {
            ta_fence_after();
#pragma unroll
            for (int k16 = 0; k16 < TA_HD / 16; ++k16)
                ta_mma(tm_s, ta_desc(q_s + k16 * 2 * TA_LBO_Q, TA_LBO_Q, TA_SBO_Q),
                       ta_desc_sw(k_s + b * TA_K_BYTES + (k16 >> 2) * TA_BOX_BYTES + (k16 & 3) * 32, 16, TA_SW_SBO), IDESC_S, k16 != 0);
            ta_commit(bar_s);
        }
        __syncwarp();
        // the last step's product has read P and its V buffer and written O: the next step's rows may land, P and O may change
        if (j >= 1) ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_o, (unsigned) ((j - 1) & 1), TA_WAIT));
        if (loader) {
            if (ok && j + 1 < nsteps) fetch_kv(b ^ 1, p0 + TA_N);
        } else {
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_s, (unsigned) (j & 1), TA_WAIT));
        ta_fence_after();
        float s[32];
        float mx = -INFINITY;
        if (ok) {
            ta_ld32(tm_s + lane_base + 32 * half, s);
            // scaled and masked: a step wholly before the tile's first row is visible to every row
            const bool open_step = p0 + TA_N <= pos0 + t0 + 1;
            const int c0 = p0 + 32 * half;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const bool vis = open_step || c0 + i <= my_pos;
                s[i] = vis ? s[i] * scale2 : -INFINITY;
                mx = fmaxf(mx, s[i]);
            }
        }
        float* x = xch + (j & 1) * 2 * TA_M;
        x[half * TA_M + r] = mx;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");   // (every thread takes it, whatever its waits saw)
        if (ok) {
            const float mn = fmaxf(m_run, fmaxf(mx, x[(half ^ 1) * TA_M + r]));
            float sum = 0.f;
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                const __half2 h = __floats2half2_rn(s[i] == -INFINITY ? 0.f : ta_ex2(s[i] - mn), s[i + 1] == -INFINITY ? 0.f : ta_ex2(s[i + 1] - mn));
                const float2 back = __half22float2(h);
                sum += back.x;
                sum += back.y;
                pk[i / 2] = *reinterpret_cast<const uint32_t*>(&h);
            }
            const float f = m_run == -INFINITY ? 0.f : ta_ex2(m_run - mn);
            z_half = z_half * f + sum;
            m_run = mn;
#pragma unroll
            for (int c8 = 0; c8 < 4; ++c8)
                *reinterpret_cast<uint4*>(Ps + (r >> 3) * TA_SBO_P + (4 * half + c8) * TA_LBO + (r & 7) * 16) =
                    make_uint4(pk[c8 * 4], pk[c8 * 4 + 1], pk[c8 * 4 + 2], pk[c8 * 4 + 3]);
            // (deep into a long context the running maxima rarely move: a warp whose factors are all 1 leaves O alone)
            if (j >= 1 && __any_sync(0xffffffffu, f != 1.0f)) {
#pragma unroll 1
                for (int c32 = 0; c32 < TA_HD / 64; ++c32) {
                    float o[32];
                    ta_ld32(tm_o + lane_base + 128 * half + c32 * 32, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= f;
                    ta_st32(tm_o + lane_base + 128 * half + c32 * 32, o);
                }
                ta_wait_st();
            }
        }
        ta_fence_before();
        }   // (the score threads)
        fence_proxy_async();   // P went through the generic proxy
        if (__syncthreads_or(!ok)) {
            ok = false;
            break;
        }
        if (tid == 0) {
            ta_fence_after();
#pragma unroll
            for (int k16 = 0; k16 < TA_N / 16; ++k16)
                ta_mma(tm_o, ta_desc(p_s + k16 * 2 * TA_LBO, TA_LBO, TA_SBO_P), ta_desc_sw(v_s + b * TA_V_BYTES + k16 * 2 * TA_SW_SBO, TA_BOX_BYTES, TA_SW_SBO),
                       IDESC_O, (j | k16) != 0);
            ta_commit(bar_o);
        }
        __syncwarp();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_o, (unsigned) ((nsteps - 1) & 1), TA_WAIT));
    if (!loader) xch[half * TA_M + r] = z_half;
    ok = __syncthreads_and(ok) != 0;
    ta_fence_after();
    if (!ok && tid == 0 && err) atomicOr(err, (unsigned) FNX_ERR_TIMEOUT);
    if (ok && !loader) {
        // out = O / z * sigmoid(gate): the thread's row and half of its dims, 32 at a time (the tensor-memory loads are warp-wide:
        // rows past the chunk's end take part in them and write nothing)
        const bool live = (r & 15) < nr;
        const int hh = r >> 4, t = t0 + min(r & 15, nr - 1), h = kvh * TA_QPK + hh;
        const float* gate = qg + (size_t) t * ldq + (size_t) h * 2 * TA_HD + TA_HD + 128 * half;
        float* o_row = out + ((size_t) t * nq + h) * TA_HD + 128 * half;
        const float iz = 1.0f / (xch[r] + xch[TA_M + r]);
#pragma unroll 1
        for (int c32 = 0; c32 < TA_HD / 64; ++c32) {
            float o[32];
            ta_ld32(tm_o + lane_base + 128 * half + c32 * 32, o);
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

// the caches as rank-3 tensors (dims, KV heads, positions) for the tensor copies: boxes of 64 dims x 1 head x 64 positions,
// 128-byte swizzle.  The position extent is nominal: the kernel asks only for whole steps below the context's end.
static int attn_prompt_tc_map(CUtensorMap* map, const __half* base, int nkv) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                 CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        FNX_CUDA_OK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) return fail(FNX_E_UNAVAILABLE, "fnx_attn_prompt: the driver has no cuTensorMapEncodeTiled");
        encode = (EncodeFn) fn;
    }
    const cuuint64_t dims[3] = {(cuuint64_t) TA_HD, (cuuint64_t) nkv, (cuuint64_t) 1 << 24};
    const cuuint64_t strides[2] = {(cuuint64_t) TA_HD * 2, (cuuint64_t) nkv * TA_HD * 2};
    const cuuint32_t box[3] = {64, 1, (cuuint32_t) TA_N}, estr[3] = {1, 1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, (void*) base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(FNX_E_CUDA, "fnx_attn_prompt: cuTensorMapEncodeTiled failed (%d)", (int) rc);
    return FNX_OK;
}

int attn_prompt_tc_launch(const float* qg, int ldq, const __half* kc, const __half* vc, float* out, int T, int nq, int nkv, const int* pos0, unsigned* err,
                          cudaStream_t st) {
    if (int rc = set_smem_limit((const void*) k_attn_prompt_tc, TA_SMEM)) return rc;
    // FNX_ATTN_PROMPT_NO_TMA=1: every step's tiles by 16-byte async copies (the comparison form)
    static const int use_tma = []() { const char* v = getenv("FNX_ATTN_PROMPT_NO_TMA"); return v && atoi(v) ? 0 : 1; }();
    CUtensorMap map_k, map_v;
    memset(&map_k, 0, sizeof map_k);
    memset(&map_v, 0, sizeof map_v);
    if (use_tma) {
        FNX_TRY(attn_prompt_tc_map(&map_k, kc, nkv));
        FNX_TRY(attn_prompt_tc_map(&map_v, vc, nkv));
    }
    k_attn_prompt_tc<<<dim3((T + TA_POS - 1) / TA_POS, nkv), TA_THREADS, TA_SMEM, st>>>(qg, ldq, kc, vc, out, T, nq, nkv, pos0, err, use_tma, map_k, map_v);
    FNX_LAUNCH_OK("fnx_attn_prompt (tensor-core form)");
    return FNX_OK;
}

}  // namespace fnxb
