// The verify window as ONE persistent kernel: a cooperative grid of one 512-thread block per SM walks every phase of
// every layer (input projection, mixer, output projection, router, routed experts gate|up, down) and the head, with a
// bounded grid barrier between phases.  It replaces the reference's per-window graph of ~10 launches per layer
// (Engine::enqueue, engine/src/engine.cu:1760-1848; ffn_half :1569-1757; replayed by engine_common.cu:994-1018) for
// windows of up to 8 rows; the launch-per-operator path (engine.cu) remains for wider windows.
//
// Why one kernel: a 5-row window moves ~70 MB per layer, about 11 us at HBM speed, while a separately launched kernel
// pays several microseconds before its first byte arrives (launch, codebook table, cold pipeline).  Here
//   - the 64 KB codebook table, the warps' rings of bulk copies and their barriers are set up once per window;
//   - the matrix phases are the per-warp streaming stage of mmv_stage.cuh (the stand-alone kernel's own body);
//   - a block that has finished a phase whose successor's weights are known stages that phase's first tile blocks
//     BEFORE it waits at the grid barrier, so the HBM pipe keeps running across phases;
//   - the expert block has no combine phase: the down projection adds weight x value into 2^-32 fixed-point sums with
//     integer atomics (order-free, hence deterministic), and the next projection's row fetch folds them into the
//     residual;
//   - every block routes for itself from the logits (top-K and the job list are identical everywhere), so no block
//     waits for a designated router;
//   - expert-parallel ranks exchange the fixed-point sums slice by slice over NVLink peer memory (plain peer stores
//     and one release flag per slice) inside the same kernel.
// Every wait (grid barrier, mbarrier, peer flag) is bounded and raises FNX_ERR_TIMEOUT instead of hanging.
#include <cooperative_groups.h>

#include "attn_core.cuh"
#include "mmv_stage.cuh"
#include "moe_route.cuh"
#include "window.cuh"

namespace fnxb {

constexpr int WIN_R = 2;                                              // ring slots per warp
constexpr int WIN_RING_BYTES = MMV_WARPS * WIN_R * TILE_BYTES;        // 56,320
constexpr int WIN_BAR_BYTES = MMV_WARPS * WIN_R * 8;                  // 256
constexpr int WIN_IMG_BYTES = 2 * (128 * 32 * 8 + 16 * 8 * 4) + 512;    // two row groups x 4096 columns + block sums: 67,072
constexpr int WIN_PIECE_BYTES = MMV_WARPS * 2 * PIECE_BYTES;
constexpr int WIN_MAX_TOPK = 12;
constexpr int WIN_JOBS_MAX = WIN_MAX_ROWS * WIN_MAX_TOPK + 2;
constexpr int WIN_MISC_FLOATS = 320;                                  // row factors, router partial sums, pair weights
constexpr int WIN_MISC_ROWF = 0, WIN_MISC_PSUM = 16, WIN_MISC_PAIRW = 160;
constexpr int WIN_SCRATCH_BYTES = WIN_RING_BYTES + WIN_IMG_BYTES + WIN_PIECE_BYTES;   // contiguous: ring | image | pieces
constexpr int WIN_ROUTER_SPLIT = 4;                                   // warps per logit row
static_assert(WIN_MISC_PAIRW + WIN_MAX_ROWS * WIN_MAX_TOPK + WIN_MAX_ROWS <= WIN_MISC_FLOATS, "pair weights overflow the scratch floats");
static_assert(WIN_SCRATCH_BYTES >= (int) attn_part_smem(), "the attention partial's tiles must fit the scratch region");

// bytes of the three-group activation image of K columns (cells, scales, block sums) that the gate|up phase reads
__host__ __device__ constexpr int win_img3_bytes(int K) { return 3 * (K / 32) * 32 * 8 + 3 * (K / 256) * 8 * 4 + 12 * 16 * 4; }


// Post-fetch transform of a dense phase's rows, chosen at run time (the dense phase is one piece of code)
enum { POST_NONE = 0, POST_FOLD = 1, POST_GDN = 2 };

// The block's running state, in shared memory: nothing but a loop counter lives in registers across phases, so the
// phases' inner loops get the whole register file (local-memory spills would go to L2: with 227 KB of shared memory
// the L1 that caches them is a few KB).
struct Blk {
    unsigned epoch;          // grid barriers passed
    int dead;                // a wait gave up: no wait waits again
    int nstamp;
    int njobs;
    int post;                // POST_*
    int xok;
    unsigned xseq;
    int pad;
    const float* gnorm;      // POST_GDN: the layer's gated-norm weights
    MmvParams mp;            // the matrix phase in progress, or the next one once its first tile blocks are on their way
    WarpRing ring[MMV_WARPS];
};

// the block's shared memory: compile-time offsets from its base, so any function rebuilds the carve for free
struct Ctx {
    const WinParams* P;      // the kernel's parameter block (constant bank)
    Blk* B;
    StageSmem S;             // the fixed carve: table, slots, barriers, pieces, jobs; images set per phase
    uint8_t* img;
    uint8_t* scratch;        // [ring | image | pieces] as one region for the phases that stream no tiles
    float* misc;
    int* s_topi;
    int tid;
};

extern __shared__ __align__(128) uint8_t win_smem[];

// Thread and block indices read through volatile asm: the compiler may not hoist them (and everything derived from
// them: lane addresses, unit ranges) out of the phase loop, where they would stay alive across every phase and push
// the phases' inner loops into local-memory spills.
__device__ __forceinline__ int opaque_tid() {
    int t;
    asm volatile("mov.u32 %0, %%tid.x;" : "=r"(t));
    return t;
}
__device__ __forceinline__ int opaque_bid() {
    int t;
    asm volatile("mov.u32 %0, %%ctaid.x;" : "=r"(t));
    return t;
}
__device__ __forceinline__ int opaque_nblk() {
    int t;
    asm volatile("mov.u32 %0, %%nctaid.x;" : "=r"(t));
    return t;
}

__device__ __forceinline__ Ctx make_ctx(const WinParams& P) {
    Ctx c;
    uint8_t* b = win_smem;
    c.S.table_s = smem_u32(b); b += CORE_TABLE_BYTES;
    c.S.bars = reinterpret_cast<uint64_t*>(b); b += WIN_BAR_BYTES;
    c.S.bar_stride = WIN_R;
    c.scratch = b;
    c.S.slots = b; b += WIN_RING_BYTES;
    c.img = b; b += WIN_IMG_BYTES;
    c.S.pieces = reinterpret_cast<PieceSlot*>(b); b += WIN_PIECE_BYTES;
    c.S.jobs_s = reinterpret_cast<fnx_job*>(b); b += WIN_JOBS_MAX * sizeof(fnx_job);
    c.misc = reinterpret_cast<float*>(b); b += WIN_MISC_FLOATS * sizeof(float);
    c.s_topi = reinterpret_cast<int*>(b); b += WIN_MAX_ROWS * WIN_MAX_TOPK * sizeof(int);
    c.B = reinterpret_cast<Blk*>(b);
    c.P = &P;
    c.S.cells = nullptr; c.S.scales = nullptr; c.S.rs = nullptr;
    c.tid = opaque_tid();
    return c;
}

// tagged %globaltimer stamp of block 0 (thread 0), when a buffer is registered
__device__ __forceinline__ void w_stamp(const Ctx& c, int id) {
    if (blockIdx.x == 0 && threadIdx.x == 0 && c.P->prof) {
        const int n = c.B->nstamp;
        if (n < WIN_PROF_WORDS - 2) {
            unsigned long long t_;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_));
            c.P->prof[1 + n] = ((unsigned long long) id << 56) | (t_ & 0x00ffffffffffffffull);
            c.B->nstamp = n + 1;
        }
    }
}

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ bool is_dead(const Ctx& c) { return *reinterpret_cast<volatile int*>(&c.B->dead) != 0; }

// every block arrives; nobody leaves before all have (or the poll limit runs out: then nothing waits again)
__device__ __forceinline__ void grid_barrier(const Ctx& c) {
    __syncthreads();
    w_stamp(c, 101);
    if (threadIdx.x == 0) {
        const unsigned epoch = ++c.B->epoch;
        __threadfence();
        atomicAdd(&c.P->sync[0], 1u);
        const unsigned target = epoch * gridDim.x;
        if (!c.B->dead) {
            unsigned it = 0;
            while (ld_acquire_gpu(&c.P->sync[0]) < target) {
                if (++it > 20000000u) {
                    atomicOr(c.P->err, (unsigned) FNX_ERR_TIMEOUT);
                    c.B->dead = 1;
                    break;
                }
            }
        }
        __threadfence();
    }
    __syncthreads();
    w_stamp(c, 102);
}

// the warp's ring between phases: lane 0 holds the issue cursor, every lane the same read position
__device__ __forceinline__ WarpRing ring_load(const Ctx& c) { return c.B->ring[c.tid >> 5]; }
__device__ __forceinline__ void ring_save(const Ctx& c, const WarpRing& r) {
    if ((c.tid & 31) == 0) c.B->ring[c.tid >> 5] = r;
}

__device__ __forceinline__ StageSmem stage_images(const Ctx& c, int slots, int NG, int K, int offset = 0) {
    StageSmem S = c.S;
    S.cells = reinterpret_cast<uint2*>(c.img + offset);
    S.scales = reinterpret_cast<float*>(S.cells + (size_t) slots * NG * (K / 32) * 32);
    S.rs = S.scales + (size_t) slots * NG * (K / 256) * 8;
    return S;
}

// ------------------------------------------------------------------------------------------------ row transforms
// A fetched block (row t, block blk, 8 values per lane) of a dense phase's input:
//   POST_FOLD  the residual: + the expert block's fixed-point sums;
//   POST_GDN   the DeltaNet output: o * rsqrt(mean_head(o^2) + eps) * gnorm * sigmoid(z)  (k_gdn_out_norm,
//              engine/src/kernels.cu:495-505) from each head's four partial square sums and the gate rows z.
struct PostAny {
    const Ctx* c;
    __device__ __forceinline__ void operator()(int t, int blk, int lane, float (&v)[8]) const {
        const int mode = c->B->post;
        const WinParams& P = *c->P;
        if (mode == POST_FOLD) {
            const ulonglong2* a = reinterpret_cast<const ulonglong2*>(P.racc + (size_t) t * P.H + blk * 256 + lane * 8);
            const ulonglong2 a0 = a[0], a1 = a[1], a2 = a[2], a3 = a[3];
            v[0] += fix_to_float(a0.x); v[1] += fix_to_float(a0.y);
            v[2] += fix_to_float(a1.x); v[3] += fix_to_float(a1.y);
            v[4] += fix_to_float(a2.x); v[5] += fix_to_float(a2.y);
            v[6] += fix_to_float(a3.x); v[7] += fix_to_float(a3.y);
        } else if (mode == POST_GDN) {
            const int hs = P.hs, nv = P.nv;
            const int col = blk * 256 + lane * 8, head = col / hs, hc = col % hs;
            const float4 s4 = *reinterpret_cast<const float4*>(P.gdn_sq + ((size_t) t * nv + head) * 4);
            const float ms = ((s4.x + s4.y) + (s4.z + s4.w)) / (float) hs;
            const float r = rsqrtf(ms + P.eps);
            const float* zr = P.proj + (2 * P.nk + nv) * hs + (size_t) t * P.proj_ld + col;
            const float* gn = c->B->gnorm + hc;
            const float4 z0 = *reinterpret_cast<const float4*>(zr), z1 = *reinterpret_cast<const float4*>(zr + 4);
            const float4 g0 = *reinterpret_cast<const float4*>(gn), g1 = *reinterpret_cast<const float4*>(gn + 4);
            const float zz[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w}, gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = v[i] * r * gg[i] / (1.0f + expf(-zz[i]));
        }
    }
};

// ------------------------------------------------------------------------------------------------ dense phases
// thread 0: the parameters of a dense phase into shared memory
__device__ __forceinline__ void dense_set(const Ctx& c, const uint8_t* W, int rows, int K, const float* x, int ldx, int T, const float* norm_w, float* out,
                                          int ldo, int accumulate, int post, const float* gnorm) {
    MmvParams& p = c.B->mp;
    p = MmvParams{};
    p.W = W; p.T = T; p.x = x; p.ldx = ldx; p.norm_w = norm_w; p.eps = c.P->eps;
    p.out = out; p.ldo = ldo; p.rows = rows; p.K = K; p.accumulate = accumulate; p.R = WIN_R; p.err = c.P->err;
    c.B->post = post;
    c.B->gnorm = gnorm;
}

// the first tile blocks of the dense phase in B->mp on their way (before the barrier that precedes the phase)
__device__ __forceinline__ void dense_preissue(const Ctx& c) {
    const MmvParams& p = c.B->mp;
    MatDesc m{};
    m.W = p.W; m.rows = p.rows; m.K = p.K;
    const int upj = p.rows / 16;
    const int u0 = (int) ((unsigned) upj * blockIdx.x / gridDim.x), u1 = (int) ((unsigned) upj * (blockIdx.x + 1) / gridDim.x);
    if (u0 < u1 && !is_dead(c)) {
        WarpRing ring = ring_load(c);
        mat_preissue<MAT_DENSE>(m, u0, u1, ring, c.tid >> 5, MMV_WARPS, c.tid & 31, WIN_R);
        ring_save(c, ring);
    }
}

// the dense phase in B->mp
template <int NG>
__device__ __forceinline__ void dense_phase(const Ctx& c) {
    const MmvParams& p = c.B->mp;
    const StageSmem S = stage_images(c, 1, NG, p.K);
    WarpRing ring = ring_load(c);
    if (is_dead(c)) {
        ring.pre = 0;
        ring_save(c, ring);
        return;
    }
    StageRegs h;
    const PostAny post{&c};
    stage_begin<NG, MAT_DENSE>(p, h, c.tid, post);
    w_stamp(c, 21);
    stage_run<NG, MAT_DENSE>(p, S, ring, h, c.tid, opaque_bid(), opaque_nblk(), post, [&]() { w_stamp(c, 22); });
    ring_save(c, ring);
    __syncthreads();
}

// ------------------------------------------------------------------------------------------------ embedding, fold
// rows of the f16 table -> f32 rows; the rows' depths; the fixed-point sums cleared
__device__ __forceinline__ void embed_phase(const Ctx& c, float* dst) {
    const WinParams& P = *c.P;
    if (blockIdx.x == 0 && c.tid < P.T) {
        int d = 0;
        for (int a = P.tree ? P.parent[c.tid] : c.tid - 1; a >= 0; a = P.tree ? P.parent[a] : a - 1) ++d;
        P.depth[c.tid] = d;
    }
    const int per = P.T * P.H;
    for (int i = blockIdx.x * WIN_THREADS + c.tid; i < per; i += gridDim.x * WIN_THREADS) {
        const int t = i / P.H, col = i % P.H;
        dst[i] = __half2float(P.embed[(size_t) P.tok[t] * P.H + col]);
        P.racc[i] = 0ull;
    }
}

// R += the fixed-point sums, which are cleared: this block's slice (no other block touches it in this phase)
__device__ __forceinline__ void fold_update(const Ctx& c) {
    const WinParams& P = *c.P;
    const int n = P.T * P.H;
    const int i0 = (int) ((long long) n * blockIdx.x / gridDim.x), i1 = (int) ((long long) n * (blockIdx.x + 1) / gridDim.x);
    for (int i = i0 + c.tid; i < i1; i += WIN_THREADS) {
        const unsigned long long a = P.racc[i];
        P.R[i] += fix_to_float(a);
        P.racc[i] = 0ull;
    }
}

// ------------------------------------------------------------------------------------------------ gated DeltaNet
// One (value head, column quarter) item on 128 threads: gdn.cu's kernel (gdn_core / k_gdn_core,
// engine/src/gdn_core.cuh:20-225) without its cluster: the head's four partial square sums go to global memory and the
// gated norm is applied by the output projection's row fetch (PostGdnNorm).
constexpr int G_HS = 128, G_Q = 4, G_QC = 32, G_THREADS = 128;

__device__ __forceinline__ void gdn_item(const Ctx& c, const WinLayer& L, int item, int cur) {
    const WinParams& P = *c.P;
    const int tid = c.tid;
    const int T = P.T, nk = P.nk, nv = P.nv, NS = P.NS, stride = P.proj_ld;
    const int lv = item / G_Q, qq = item % G_Q, kh = lv % nk, warp = tid >> 5, lane = tid & 31;
    const int ch = (2 * nk + nv) * G_HS;
    const size_t hsz = (size_t) 3 * ch, ssz = (size_t) nv * G_HS * G_HS;
    const float* qkvz = P.proj;
    const float* ab = P.proj + ch + nv * G_HS;
    const int* parent = P.tree ? P.parent : nullptr;
    const SyncNamed sync{1, G_THREADS};
    float* smf = reinterpret_cast<float*>(c.img);
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
    // the starting state of the warp's key rows is on its way before anything else: row 0's parent is the root
    const int part = warp, col = qq * G_QC + lane;
    const size_t soff = (size_t) lv * G_HS * G_HS + (size_t) part * 32 * G_HS + col;
    float s[32];
    {
        const float* src = L.S + (size_t) cur * ssz + soff;
#pragma unroll
        for (int r = 0; r < 32; ++r) s[r] = src[(size_t) r * G_HS];
    }
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
    constexpr int SB = 20;   // loads in flight per thread: a 5-row window's conv inputs in one round
    float4 cw3[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const int e = tid + k * G_THREADS;
        cw3[k] = e < NC ? *reinterpret_cast<const float4*>(L.convw + chan(e) * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int i0 = tid; i0 < (T + 3) * NC; i0 += SB * G_THREADS) {
        float v[SB];
#pragma unroll
        for (int j = 0; j < SB; ++j) {
            const int i = i0 + j * G_THREADS;
            v[j] = 0.f;
            if (i < (T + 3) * NC) {
                const int r = i / NC, cc = chan(i % NC);
                v[j] = r < 3 ? hin[(size_t) r * ch + cc] : qkvz[(size_t) (r - 3) * stride + cc];
            }
        }
#pragma unroll
        for (int j = 0; j < SB; ++j) {
            const int i = i0 + j * G_THREADS;
            if (i < (T + 3) * NC) xin[i] = v[j];
        }
    }
    // the three rows before each window row on its path, as rows of xin (past the root: the history)
    if (tid < T) {
        int a = tid;
        for (int k = 1; k <= 3; ++k) {
            if (a >= 0) a = parent ? parent[a] : a - 1;
            else --a;                      // a = -1 - (rows past the root)
            anc[tid * 3 + k - 1] = 3 + a;  // -1 -> row 2 (newest history), -2 -> row 1, -3 -> row 0
        }
    }
    sync();
#pragma unroll
    for (int k3 = 0; k3 < 3; ++k3) {
        const int e = tid + k3 * G_THREADS;
        if (e >= NC) continue;
        const int pt = e < G_HS ? 0 : e < 2 * G_HS ? 1 : 2, i = pt < 2 ? e - pt * G_HS : e - 2 * G_HS;
        const int cc = chan(e);
        const float4 cw = cw3[k3];
        const bool writes = pt == 2 || (lv < nk && qq == 0);   // one block per channel writes its history
        for (int t = 0; t < T; ++t) {
            const float x3 = xin[anc[t * 3 + 2] * NC + e], x2 = xin[anc[t * 3 + 1] * NC + e], x1 = xin[anc[t * 3] * NC + e];
            const float x0 = xin[(3 + t) * NC + e];
            const float x = cw.x * x3 + cw.y * x2 + cw.z * x1 + cw.w * x0;
            const float v = x / (1.0f + expf(-x));
            if (pt == 0) xq[t * G_HS + i] = v;
            else if (pt == 1) xk[t * G_HS + i] = v;
            else vs[t * G_QC + i] = v;
            if (writes) {
                float* hout = L.hist + (size_t) ((cur + 1 + t) % NS) * hsz;
                hout[cc] = x2;
                hout[ch + cc] = x1;
                hout[2 * ch + cc] = x0;
            }
        }
    }
    sync();
    for (int t = 0; t < T; ++t) {
        const float qv = xq[t * G_HS + tid], kv = xk[t * G_HS + tid];
        const float sq = warp_sum(qv * qv), sk = warp_sum(kv * kv);
        if (lane == 0) { red[warp * 2 * T + t] = sq; red[warp * 2 * T + T + t] = sk; }
    }
    sync();
    for (int t = 0; t < T; ++t) {
        float sq = 0.f, sk = 0.f;
        for (int w = 0; w < 4; ++w) { sq += red[w * 2 * T + t]; sk += red[w * 2 * T + T + t]; }
        xq[t * G_HS + tid] *= rsqrtf(sq + 1e-6f);
        xk[t * G_HS + tid] *= rsqrtf(sk + 1e-6f);
    }
    sync();
    int have = -1;   // the row whose result the registers hold (-1: the starting state)
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
        sync();
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
    sync();
    for (int t = warp; t < T; t += 4) {
        const float o = ((ared[(t * 4 + 0) * G_QC + lane] + ared[(t * 4 + 1) * G_QC + lane]) +
                         (ared[(t * 4 + 2) * G_QC + lane] + ared[(t * 4 + 3) * G_QC + lane])) * scale;
        P.gdn_o[(size_t) t * nv * G_HS + lv * G_HS + col] = o;
        const float sq = warp_sum(o * o);
        if (lane == 0) P.gdn_sq[((size_t) t * nv + lv) * 4 + qq] = sq;
    }
    sync();   // the scratch is free for the block's next item
}

// ------------------------------------------------------------------------------------------------ router
// Logits of this block's rows: row r of the E + 1 on WIN_ROUTER_SPLIT warps (each a quarter of the columns, summed in
// share order), f32 throughout as k_router (moe_route.cu; k_router_route, engine/src/moe.cuh:258-515).  Meanwhile every
// block quantises the window's normalised rows into the image the gate|up phase reads (three row groups; rows past
// T hold zeros).  xs: [T][H] f32 in the ring region.
__device__ __forceinline__ void router_phase(const Ctx& c, const WinLayer& L) {
    const WinParams& P = *c.P;
    const int tid = c.tid, warp = tid >> 5, lane = tid & 31, H = P.H, T = P.T, KB = H / 256;
    float* xs = reinterpret_cast<float*>(c.scratch);
    const StageSmem S = stage_images(c, 1, 3, H, WIN_IMG_BYTES - win_img3_bytes(H));
    float* rowf = c.misc + WIN_MISC_ROWF;   // [T] 1 / rms
    float* psum = c.misc + WIN_MISC_PSUM;   // [warp][8]
    constexpr int RPB = MMV_WARPS / WIN_ROUTER_SPLIT;   // rows per block
    const int nrow = P.E + 1;
    const int per = (nrow + (int) gridDim.x - 1) / (int) gridDim.x;   // rows per block, rounded up
    const int passes = (per + RPB - 1) / RPB;
    // the rows into shared memory, all copies in flight at once
    for (int i = tid; i < T * (H / 4); i += WIN_THREADS)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(xs + (size_t) i * 4)), "l"(P.R + (size_t) i * 4) : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
    // the image of the normalised rows (the same tasks and arithmetic as the stand-alone kernel's own quantiser)
    for (int id0 = warp; id0 < T * KB; id0 += MMV_WARPS * QUANT_BATCH) {
        QuantTask q[QUANT_BATCH];
        float v[QUANT_BATCH][8], w[QUANT_BATCH][8];
#pragma unroll
        for (int j = 0; j < QUANT_BATCH; ++j) {
            const int id = id0 + j * MMV_WARPS;
            q[j].src = nullptr;
            q[j].t = q[j].blk = 0;
            if (id < T * KB) {
                q[j].t = id % T;
                q[j].blk = id / T;
                q[j].src = P.R + (size_t) q[j].t * H + q[j].blk * 256;
            }
            quant_fetch(q[j], L.norm2, lane, v[j], w[j]);
        }
        quant_finish(q, v, w, H, L.norm2, S.cells, S.scales, S.rs, lane);
    }
    {
        constexpr int NROW = 12, TPR = WIN_THREADS / 16;
        const int t = tid / TPR;
        if (t < NROW && t >= T) quant_zero_row(t, H, S.cells, S.scales, S.rs, tid % TPR, TPR);
    }
    w_stamp(c, 50);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    w_stamp(c, 51);
    if (tid < T) rowf[tid] = quant_row_factor(S.rs, tid, H, P.eps);
    const int HS = H / WIN_ROUTER_SPLIT;
    for (int ps = 0; ps < passes; ++ps) {
        const int row = (int) blockIdx.x * per + ps * RPB + warp / WIN_ROUTER_SPLIT, share = warp % WIN_ROUTER_SPLIT;
        const bool live = row < nrow && row < ((int) blockIdx.x + 1) * per;
        float acc[WIN_MAX_ROWS];
#pragma unroll
        for (int t = 0; t < WIN_MAX_ROWS; ++t) acc[t] = 0.f;
        if (live) {
            const float* wr = L.wr + (size_t) row * H + share * HS;
            const float* nw = L.norm2 + share * HS;
            for (int i0 = 0; i0 < HS; i0 += 512) {
                float4 w[4], n4[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = i0 + lane * 4 + j * 128;
                    w[j] = i < HS ? *reinterpret_cast<const float4*>(wr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                    n4[j] = i < HS ? *reinterpret_cast<const float4*>(nw + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = i0 + lane * 4 + j * 128;
                    if (i >= HS) continue;
#pragma unroll
                    for (int t = 0; t < WIN_MAX_ROWS; ++t)
                        if (t < T) {
                            const float4 v = *reinterpret_cast<const float4*>(xs + (size_t) t * H + share * HS + i);
                            acc[t] = fmaf(w[j].x, v.x * n4[j].x, acc[t]);
                            acc[t] = fmaf(w[j].y, v.y * n4[j].y, acc[t]);
                            acc[t] = fmaf(w[j].z, v.z * n4[j].z, acc[t]);
                            acc[t] = fmaf(w[j].w, v.w * n4[j].w, acc[t]);
                        }
                }
            }
        }
#pragma unroll
        for (int t = 0; t < WIN_MAX_ROWS; ++t)
            if (t < T) {
                const float s = warp_sum(acc[t]);
                if (lane == 0) psum[(warp / WIN_ROUTER_SPLIT * WIN_ROUTER_SPLIT + share) * 8 + t] = s;
            }
        __syncthreads();
        if (tid < RPB * 8) {
            const int r = tid / 8, t = tid % 8, grow = (int) blockIdx.x * per + ps * RPB + r;
            if (t < T && grow < nrow && grow < ((int) blockIdx.x + 1) * per) {
                float s = 0.f;
#pragma unroll
                for (int q = 0; q < WIN_ROUTER_SPLIT; ++q) s += psum[(r * WIN_ROUTER_SPLIT + q) * 8 + t];
                s *= rowf[t];
                P.rlogits[(size_t) t * nrow + grow] = s;
                if (!isfinite(s)) atomicOr(P.err, (unsigned) FNX_ERR_NONFINITE);
            }
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------------ routed experts
// lane pointers of one job over the window image (three row groups; row WIN_ZROW and up hold zeros)
__device__ __forceinline__ void lane_x_window(const StageSmem& S, int K, float eps, const fnx_job& jb, int ntok, int zrow, int lane, LaneX<1>& lx) {
    const int g = lane >> 2, q = lane & 3, KB = K / 256;
    {
        const int row = (g & 3) < ntok ? jb.y[g & 3] : zrow;
        lx.b[0] = smem_u32(S.cells + ((size_t) (row >> 2) * (K / 32) * 8 + (row & 3) + 4 * (g >> 2)) * 4 + q);
    }
    const int c0 = 2 * q, c1 = 2 * q + 1;
    {
        const int row = (c0 & 3) < ntok ? jb.y[c0 & 3] : zrow;
        lx.s0[0] = smem_u32(S.scales + (size_t) (row >> 2) * KB * 8 + (row & 3) + 4 * (c0 >> 2));
        lx.r0[0] = quant_row_factor(S.rs, row, K, eps);
    }
    {
        const int row = (c1 & 3) < ntok ? jb.y[c1 & 3] : zrow;
        lx.s1[0] = smem_u32(S.scales + (size_t) (row >> 2) * KB * 8 + (row & 3) + 4 * (c1 >> 2));
        lx.r1[0] = quant_row_factor(S.rs, row, K, eps);
    }
}

// Every block: top-K of the rows from the logits, the job list (identical in every block), the pairs' weights; block 0
// publishes them.  Returns the number of jobs.
__device__ __forceinline__ int route_local(const Ctx& c, bool add_shared) {
    const WinParams& P = *c.P;
    const int tid = c.tid, warp = tid >> 5, lane = tid & 31, T = P.T, K = P.K, E = P.E;
    const bool pub = blockIdx.x == 0;
    float* pairw = c.misc + WIN_MISC_PAIRW;          // [T K + T]
    float* topw_s = pairw;
    for (int t = warp; t < T; t += MMV_WARPS) {
        const volatile float* l = P.rlogits + (size_t) t * (E + 1);
        if (E <= 512) rt_topk_row<16>(l, E, K, lane, pub ? P.topi + t * K : nullptr, c.s_topi + t * K, pub ? P.topw + t * K : nullptr, topw_s + t * K);
        else rt_topk_row<RT_MAXE / 32>(l, E, K, lane, pub ? P.topi + t * K : nullptr, c.s_topi + t * K, pub ? P.topw + t * K : nullptr, topw_s + t * K);
        if (lane == 0) pairw[T * K + t] = sigmoidf_(l[E]);
    }
    __syncthreads();
    w_stamp(c, 60);
    RtJobSmem js;
    js.s_topi = c.s_topi;
    js.s_cnt = reinterpret_cast<int*>(c.S.pieces);          // the pieces are free until the tile products start
    js.s_base = js.s_cnt + RT_MAXE;
    js.wsum = js.s_base + RT_MAXE;
    js.total = js.wsum + 32;
    js.js = c.S.jobs_s;
    rt_build_jobs<WIN_THREADS>(js, tid, T, E, K, P.e_lo, P.e_hi, add_shared ? 1 : 0);
    const int total = js.total[0], routed = js.total[1];
    __syncthreads();
    if (pub) {
        constexpr int JW = sizeof(fnx_job) / 4;
        for (int w = tid; w < total * JW; w += WIN_THREADS) reinterpret_cast<int*>(P.jobs)[w] = reinterpret_cast<const int*>(c.S.jobs_s)[w];
        if (tid == 0) {
            P.njobs[0] = total;
            if (P.stats) {
                atomicAdd(&P.stats[0], (unsigned long long) routed);
                atomicAdd(&P.stats[1], 1ull);
            }
        }
    }
    return total;
}

__device__ __forceinline__ MatDesc expert_desc(const Ctx& c, const uint8_t* W, size_t stride, const uint8_t* Wsh, int rows, int K, float* out, int ldo) {
    const WinParams& P = *c.P;
    MatDesc m{};
    m.W = W; m.expert_stride = stride; m.e_base = P.e_base; m.Wsh = Wsh; m.E = P.E; m.jobs = c.S.jobs_s;
    m.rows = rows; m.K = K; m.out = out; m.ldo = ldo;
    return m;
}

// gate|up + SwiGLU of this block's share of the jobs, from the window image
__device__ __forceinline__ void gateup_phase(const Ctx& c, const WinLayer& L, int njobs) {
    const WinParams& P = *c.P;
    const int tid = c.tid, warp = tid >> 5, lane = tid & 31;
    const StageSmem S = stage_images(c, 1, 3, P.H, WIN_IMG_BYTES - win_img3_bytes(P.H));
    const MatDesc m = expert_desc(c, L.wgu, P.gu_bytes, L.wsh_gu, P.F, P.H, P.hbuf, P.F);
    const int upj = P.F / 16;
    const unsigned total = (unsigned) njobs * upj;
    const int u0 = (int) (total * blockIdx.x / gridDim.x), u1 = (int) (total * (blockIdx.x + 1) / gridDim.x);
    bool ok = !is_dead(c);
    WarpRing ring = ring_load(c);
    if (u0 < u1 && ok) {
        auto lane_x = [&](int j, LaneX<1>& lx, int& ntok, int (&orow)[4]) {
            const fnx_job& jb = S.jobs_s[j];
            ntok = min(jb.n, 4);
#pragma unroll
            for (int i = 0; i < 4; ++i) orow[i] = jb.out[i];
            lane_x_window(S, P.H, P.eps, jb, ntok, P.T, lane, lx);
        };
        ok = mat_items<1, MAT_GATEUP>(m, u0, u1, S.table_s, ring, S.pieces, warp, MMV_WARPS, lane, lane_x);
        if (!ok) {
            atomicOr(P.err, (unsigned) FNX_ERR_TIMEOUT);
            c.B->dead = 1;
        }
    }
    ring_save(c, ring);
    __syncthreads();
    w_stamp(c, 30);
    if (u0 < u1 && ok) mat_combine<1, MAT_GATEUP>(m, S.pieces, warp, MMV_WARPS, lane);
    __syncthreads();
    w_stamp(c, 31);
}

// down projection of this block's share of the jobs; weight x value goes to the fixed-point sums
__device__ __forceinline__ MmvParams down_params(const Ctx& c, const WinLayer& L, int njobs_max) {
    const WinParams& P = *c.P;
    MmvParams p{};
    p.W = L.wdn; p.expert_stride = P.dn_bytes; p.e_base = P.e_base; p.Wsh = L.wsh_dn; p.E = P.E;
    p.jobs = P.jobs; p.njobs = P.njobs; p.njobs_max = njobs_max;
    p.x = P.hbuf; p.ldx = P.F; p.out = nullptr; p.ldo = P.H; p.rows = P.H; p.K = P.F; p.R = WIN_R; p.err = P.err;
    p.pairw = c.misc + WIN_MISC_PAIRW; p.racc = P.racc; p.TK = P.T * P.K; p.Ktop = P.K;
    return p;
}

__device__ __forceinline__ void down_phase(const Ctx& c, const WinLayer& L) {
    const WinParams& P = *c.P;
    const int njobs_max = P.T * P.K + (P.T + FNX_JOB_TOK - 1) / FNX_JOB_TOK;
    if (c.tid == 0) c.B->mp = down_params(c, L, njobs_max);
    __syncthreads();
    const MmvParams& p = c.B->mp;
    const StageSmem S = stage_images(c, mmv_jmax<MAT_DOWN>(), 1, P.F);
    if (is_dead(c)) return;
    WarpRing ring = ring_load(c);
    StageRegs h;
    stage_begin<1, MAT_DOWN>(p, h, c.tid, RowPlain());
    stage_run<1, MAT_DOWN>(p, S, ring, h, c.tid, opaque_bid(), opaque_nblk(), RowPlain(), [&]() { w_stamp(c, 40); });
    ring_save(c, ring);
    __syncthreads();
}

// ------------------------------------------------------------------------------------------------ expert-parallel sum
// After the barrier that follows the down phase: this block's slice of the rank's fixed-point sums goes to every
// peer's landing plane (plain peer stores, then one release flag per peer and slice); the block then waits (bounded)
// for the peers' flags of its own slice and adds their planes.  Integer sums: every rank ends with the same bits.
__device__ __forceinline__ void ep_exchange(const Ctx& c, unsigned seq) {
    const WinParams& P = *c.P;
    const int tid = c.tid, R = P.ep_size, me = P.ep_rank;
    const int n = P.T * P.H / 2;   // in 16-byte pairs
    const int i0 = (int) ((long long) n * blockIdx.x / gridDim.x), i1 = (int) ((long long) n * (blockIdx.x + 1) / gridDim.x);
    const int slot = (int) (seq & 1u);
    const size_t plane = (size_t) P.maxr * P.H;
    const ulonglong2* mine = reinterpret_cast<const ulonglong2*>(P.racc);
    for (int r = 0; r < R; ++r) {
        if (r == me) continue;
        ulonglong2* dst = reinterpret_cast<ulonglong2*>(P.peers.x[r] + ((size_t) slot * R + me) * plane);
        for (int i = i0 + tid; i < i1; i += WIN_THREADS) dst[i] = mine[i];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < R && tid != me) {
        unsigned* f = P.peers.flag[tid] + ((size_t) slot * R + me) * gridDim.x + blockIdx.x;
        const unsigned v = seq + 1u;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(v) : "memory");
    }
    if (tid == 0) {
        bool all = false;
        const unsigned* fl = P.peers.flag[me] + (size_t) slot * R * gridDim.x + blockIdx.x;
        for (unsigned it = 0; it < 4000000u && !all && !c.B->dead; ++it) {
            all = true;
            for (int r = 0; r < R; ++r) {
                if (r == me) continue;
                unsigned v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(fl + (size_t) r * gridDim.x) : "memory");
                all = all && v == seq + 1u;
            }
        }
        if (!all) {
            atomicOr(P.err, (unsigned) FNX_ERR_TIMEOUT);
            c.B->dead = 1;
        }
        c.B->xok = all ? 1 : 0;
    }
    __syncthreads();
    if (c.B->xok) {
        ulonglong2* acc = reinterpret_cast<ulonglong2*>(P.racc);
        for (int i = i0 + tid; i < i1; i += WIN_THREADS) {
            ulonglong2 s = acc[i];
            for (int r = 0; r < R; ++r) {
                if (r == me) continue;
                const ulonglong2 v = __ldcv(reinterpret_cast<const ulonglong2*>(P.peers.x[me] + ((size_t) slot * R + r) * plane) + i);
                s.x += v.x;
                s.y += v.y;
            }
            acc[i] = s;
        }
    }
}

// ------------------------------------------------------------------------------------------------ the kernel
// The window is a sequence of phases with a grid barrier after each; one loop interprets it, so the code of a phase
// exists once whatever the number of places it runs (input and output projections, the draft layer's two, the head).
enum { K_EMBED = 0, K_MTP_HID, K_MTP_EMB, K_INPROJ, K_GDN, K_ATTN_PREP, K_ATTN_PART, K_ATTN_MERGE, K_OUTPROJ, K_ROUTER, K_GATEUP, K_DOWN, K_EP, K_FOLD, K_HEAD,
       K_END };

__device__ __forceinline__ bool phase_is_dense(int k) { return k == K_MTP_HID || k == K_MTP_EMB || k == K_INPROJ || k == K_OUTPROJ || k == K_HEAD; }

// the phase that follows phase k of layer l
__device__ __forceinline__ void phase_next(const WinParams& P, int& l, int& k) {
    switch (k) {
        case K_EMBED: k = P.mtp ? K_MTP_HID : K_INPROJ; break;
        case K_MTP_HID: k = K_MTP_EMB; break;
        case K_MTP_EMB: k = K_INPROJ; break;
        case K_INPROJ: k = P.layers[l].attn ? K_ATTN_PREP : K_GDN; break;
        case K_GDN: k = K_OUTPROJ; break;
        case K_ATTN_PREP: k = K_ATTN_PART; break;
        case K_ATTN_PART: k = K_ATTN_MERGE; break;
        case K_ATTN_MERGE: k = K_OUTPROJ; break;
        case K_OUTPROJ: k = K_ROUTER; break;
        case K_ROUTER: k = K_GATEUP; break;
        case K_GATEUP: k = K_DOWN; break;
        case K_DOWN:
            if (P.ep_size > 1) {
                k = K_EP;
                break;
            }
            // fall through
        case K_EP:
            ++l;
            k = l < P.n_layer ? K_INPROJ : K_FOLD;
            break;
        case K_FOLD: k = K_HEAD; break;
        default: k = K_END; break;
    }
}

// thread 0: the parameters of dense phase k of layer l
__device__ __forceinline__ void phase_dense_set(const Ctx& c, int l, int k) {
    const WinParams& P = *c.P;
    const int T = P.T, H = P.H;
    if (k == K_MTP_HID) dense_set(c, P.fc_hid, H, H, P.src, H, T, P.hnorm, P.R, H, 0, POST_NONE, nullptr);
    else if (k == K_MTP_EMB) dense_set(c, P.fc_emb, H, H, P.emb, H, T, P.enorm, P.R, H, 1, POST_NONE, nullptr);
    else if (k == K_INPROJ) {
        const WinLayer& L = P.layers[l];
        dense_set(c, L.w_in, L.in_rows, H, P.R, H, T, L.norm1, P.proj, P.proj_ld, 0, POST_FOLD, nullptr);
    } else if (k == K_OUTPROJ) {
        const WinLayer& L = P.layers[l];
        const int mixK = L.attn ? P.nq * P.hd : P.nv * P.hs;
        dense_set(c, L.w_out, H, mixK, L.attn ? P.mix : P.gdn_o, mixK, T, nullptr, P.R, H, 1, L.attn ? POST_NONE : POST_GDN, L.gnorm);
    } else {
        const int hr = P.head_row0;
        dense_set(c, P.head, P.V, H, P.R + (size_t) hr * H, H, T - hr, P.out_norm, P.logits + (size_t) hr * P.V, P.V, 0, POST_NONE, nullptr);
    }
}

template <int NG>
__global__ void __launch_bounds__(WIN_THREADS, 1) k_window(const __grid_constant__ WinParams P) {
    {
        const Ctx c = make_ctx(P);
        const int tid = c.tid, warp = tid >> 5, lane = tid & 31;
        core_fill_table(win_smem, tid, WIN_THREADS);
        if (lane == 0) {
            for (int i = 0; i < WIN_R; ++i) mbar_init(&c.S.bars[warp * WIN_R + i], 1);
            fence_barrier_init();
            WarpRing ring;
            ring.parity = 0;
            ring.ahead = ring.ab = ring.al = ring.aj = 0;
            ring.aw = ring.asrc = nullptr;
            stage_ring(ring, c.S, WIN_R, warp);
            c.B->ring[warp] = ring;
        }
        if (tid == 0) {
            c.B->epoch = 0;
            c.B->dead = 0;
            c.B->nstamp = 0;
            c.B->njobs = 0;
            c.B->post = POST_NONE;
            c.B->xok = 0;
        }
    }
    __syncthreads();
    {
        const Ctx c = make_ctx(P);
        if (c.tid == 0) c.B->xseq = P.ep_size > 1 ? *P.xseq : 0u;
        w_stamp(c, 100);
    }

    int l = 0, k = K_EMBED;
#pragma unroll 1
    while (k != K_END) {
        const Ctx c = make_ctx(P);   // a fresh carve per phase (see opaque_tid)
        const int tid = c.tid;
        switch (k) {
            case K_EMBED:   // tokens -> residual rows (the draft layer: -> embedding rows, its input projections follow)
                embed_phase(c, P.mtp ? P.emb : P.R);
                break;
            case K_MTP_HID:
            case K_MTP_EMB:
            case K_INPROJ:   // rmsnorm(R + the previous expert block's sums) -> the mixer's inputs
            case K_OUTPROJ:  // the mixer's output -> += R
            case K_HEAD:
                dense_phase<NG>(c);
                if (P.dbg && k == K_INPROJ) {
                    w_stamp(c, 25);
                    dense_phase<NG>(c);
                }
                break;
            case K_GDN: {
                fold_update(c);
                const WinLayer& L = P.layers[l];
                const int cur = *P.cur;
                for (int item = blockIdx.x; item < P.nv * G_Q; item += gridDim.x)
                    if (tid < G_THREADS) gdn_item(c, L, item, cur);
                break;
            }
            case K_ATTN_PREP: {   // per-head norm + rotary + append: two items at a time, one per half of the block
                fold_update(c);
                const WinLayer& L = P.layers[l];
                const int pos0 = *P.pos0, T = P.T;
                const int heads = P.nq + 2 * P.nkv, half = tid / ATT_THREADS, i = tid % ATT_THREADS;
                float* xrow = reinterpret_cast<float*>(c.img) + half * 512;
                const SyncNamed sync{2 + half, ATT_THREADS};
                float* kk = P.proj + P.nq * 2 * P.hd;
                for (int item = (int) blockIdx.x * 2 + half; item < T * heads; item += (int) gridDim.x * 2) {
                    const int t = item / heads, hh = item % heads;
                    attn_prep_body(P.proj, P.proj_ld, kk, P.proj_ld, kk + P.nkv * P.hd, P.proj_ld, L.qn, L.kn, L.kc, L.vc, P.nq, P.nkv, P.hd, P.nrot, pos0,
                                   P.depth, P.eps, P.rope_base, t, hh, i, xrow, xrow + 256, sync);
                    sync();
                }
                break;
            }
            case K_ATTN_PART: {
                const WinLayer& L = P.layers[l];
                const int pos0 = *P.pos0, T = P.T;
                const int S = (int) gridDim.x / P.nkv > 0 ? (int) gridDim.x / P.nkv : 1, groups = (T + ATT_ROWS - 1) / ATT_ROWS;
                AttPartial* mz = reinterpret_cast<AttPartial*>(P.att_mz);
                for (int item = blockIdx.x; item < S * P.nkv * groups; item += gridDim.x) {
                    if (tid < ATT_THREADS) {
                        const SyncNamed sync{2, ATT_THREADS};
                        attn_part_body(P.proj, P.proj_ld, L.kc, L.vc, P.att_acc, mz, T, P.nq, P.nkv, pos0, P.tree ? P.parent : nullptr, item % S, S,
                                       (item / S) % P.nkv, (item / (S * P.nkv)) * ATT_ROWS, tid, c.scratch, sync);
                        sync();
                    }
                }
                break;
            }
            case K_ATTN_MERGE: {
                const int S = (int) gridDim.x / P.nkv > 0 ? (int) gridDim.x / P.nkv : 1;
                const AttPartial* mz = reinterpret_cast<const AttPartial*>(P.att_mz);
                for (int item = blockIdx.x; item < P.T * P.nq; item += gridDim.x) {
                    attn_combine_body<WIN_THREADS / ATT_THREADS>(P.att_acc, mz, P.proj, P.proj_ld, P.mix, P.nq, P.hd, S, item % P.nq, item / P.nq, tid,
                                                                 reinterpret_cast<float*>(c.img), SyncBlock());
                    __syncthreads();
                }
                break;
            }
            case K_ROUTER:   // router logits; the expert block's activation image
                router_phase(c, P.layers[l]);
                if (P.dbg) {
                    __syncthreads();
                    w_stamp(c, 55);
                    router_phase(c, P.layers[l]);
                }
                break;
            case K_GATEUP: {   // routing (every block for itself), gate|up + SwiGLU
                const int njobs = route_local(c, P.ep_size == 1 || l % P.ep_size == P.ep_rank);
                w_stamp(c, 61);
                gateup_phase(c, P.layers[l], njobs);
                break;
            }
            case K_DOWN:   // down projection into the fixed-point sums
                down_phase(c, P.layers[l]);
                break;
            case K_EP:
                ep_exchange(c, c.B->xseq);
                __syncthreads();
                if (tid == 0) ++c.B->xseq;
                break;
            case K_FOLD:   // the residual takes the last sums in
                fold_update(c);
                break;
            default: break;
        }
        // the next phase; if it is a matrix product whose weights depend on nothing, its first tile blocks leave now
        const int done = k;
        phase_next(P, l, k);
        __syncthreads();
        if (phase_is_dense(k)) {
            if (tid == 0) phase_dense_set(c, l, k);
            __syncthreads();
            dense_preissue(c);
        }
        if (k != K_END) grid_barrier(c);
        w_stamp(c, 110 + done);
    }
    const Ctx c = make_ctx(P);
    if (P.ep_size > 1 && blockIdx.x == 0 && c.tid == 0) *P.xseq = c.B->xseq;
    if (blockIdx.x == 0 && c.tid == 0 && P.prof) P.prof[0] = (unsigned long long) c.B->nstamp;
}

size_t win_smem_bytes() {
    return (size_t) CORE_TABLE_BYTES + WIN_BAR_BYTES + WIN_SCRATCH_BYTES + WIN_JOBS_MAX * sizeof(fnx_job) + WIN_MISC_FLOATS * sizeof(float) +
           WIN_MAX_ROWS * WIN_MAX_TOPK * sizeof(int) + (sizeof(Blk) + 15) / 16 * 16;
}

int win_setup() {
    const size_t smem = win_smem_bytes();
    FNX_REQUIRE(smem <= 227 * 1024, "window kernel: %zu bytes of shared memory", smem);
    if (int rc = set_smem_limit((const void*) k_window<1>, (int) smem)) return rc;
    return set_smem_limit((const void*) k_window<2>, (int) smem);
}

int win_launch(const WinParams& params, unsigned* sync_words, cudaStream_t st) {
    const int T = params.T;
    if (T < 1 || T > WIN_MAX_ROWS) return fail(FNX_E_ARG, "window kernel: %d rows (1..%d)", T, WIN_MAX_ROWS);
    if (params.n_layer < 1 || params.n_layer > WIN_MAX_LAYERS) return fail(FNX_E_ARG, "window kernel: %d layers (1..%d)", params.n_layer, WIN_MAX_LAYERS);
    if (int rc = win_setup()) return rc;
    FNX_CUDA_OK(cudaMemsetAsync(sync_words, 0, sizeof(unsigned) * WIN_SYNC_WORDS, st));
    void* args[1] = {(void*) &params};
    const void* fn = T <= 4 ? (const void*) k_window<1> : (const void*) k_window<2>;
    FNX_CUDA_OK(cudaLaunchCooperativeKernel(fn, dim3(sm_count()), dim3(WIN_THREADS), args, win_smem_bytes(), st));
    return FNX_OK;
}

}  // namespace fnxb
