// Head-side kernels: per-row argmax, the sampler's 64 candidates, embedding rows, RMS norm rows.
//
// fnx_argmax replaces argmax / k_argmax (engine/src/kernels.hpp:433, engine/src/kernels.cu:1056-1083): the same
// total order, value first and the lower index on ties.  fnx_top_tokens replaces top_tokens / k_topk_rows
// (engine/src/kernels.hpp:445, engine/src/topk.cuh:17-155) without penalties or logit bias: a radix select over the
// 64-bit key (ordered logit bits, ~index), which has no ties, then a rank sort of the 64 survivors.
#include "fnx_common.cuh"

namespace fnxb {

// float -> uint32 with the same order
__device__ __forceinline__ uint32_t fkey(float v) {
    const uint32_t b = __float_as_uint(v);
    return b & 0x80000000u ? ~b : b | 0x80000000u;
}
__device__ __forceinline__ float fkey_inv(uint32_t k) { return __uint_as_float(k & 0x80000000u ? k & 0x7fffffffu : ~k); }
__device__ __forceinline__ unsigned long long key64(float v, int i) { return ((unsigned long long) fkey(v) << 32) | (uint32_t) ~i; }

// Rows are scanned by ARGMAX_NB blocks each; the blocks of a row meet in a per-row slot of device memory (largest key by
// atomicMax, an arrival counter) and the last one to arrive writes the result and clears the slot for the next call.
// The slots are shared by every call on the device: calls must not overlap in time (the engine's are stream-ordered).
constexpr int ARGMAX_NB = 16, ARGMAX_ROWS = 1024;
__device__ unsigned long long g_argmax_key[ARGMAX_ROWS];
__device__ unsigned g_argmax_cnt[ARGMAX_ROWS];

__global__ void __launch_bounds__(1024) k_argmax(const float* __restrict__ logits, int V, const int* __restrict__ map, int* __restrict__ best_i,
                                                 float* __restrict__ best_v, unsigned* __restrict__ err) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ unsigned long long red[32];
    const int t = blockIdx.x, tid = threadIdx.x, nb = gridDim.y;
    const float* l = logits + (size_t) t * V;
    unsigned long long best = 0;
    bool bad = false;
    // this block's slice, in float4 units where the row allows; four float4 per thread in flight
    const int V4 = (((uintptr_t) l & 15) == 0) ? V / 4 : 0;
    const int a4 = (int) ((long long) V4 * blockIdx.y / nb), b4 = (int) ((long long) V4 * (blockIdx.y + 1) / nb);
    for (int i0 = a4 + tid; i0 < b4; i0 += 4096) {
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = i0 + 1024 * j < b4 ? reinterpret_cast<const float4*>(l)[i0 + 1024 * j] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = i0 + 1024 * j;
            if (i >= b4) continue;
            const float e[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                bad |= !isfinite(e[c]);
                const unsigned long long k = key64(e[c], 4 * i + c);
                best = k > best ? k : best;
            }
        }
    }
    if (blockIdx.y == nb - 1)   // what float4 units do not cover
        for (int i = 4 * V4 + tid; i < V; i += 1024) {
            const float v = l[i];
            bad |= !isfinite(v);
            const unsigned long long k = key64(v, i);
            best = k > best ? k : best;
        }
    for (int o = 16; o; o >>= 1) {
        const unsigned long long ok = __shfl_xor_sync(0xffffffffu, best, o);
        best = ok > best ? ok : best;
    }
    if ((tid & 31) == 0) red[tid >> 5] = best;
    if (bad) atomicOr(err, (unsigned) FNX_ERR_LOGITS);
    __syncthreads();
    if (tid < 32) {
        best = red[tid];
        for (int o = 16; o; o >>= 1) {
            const unsigned long long ok = __shfl_xor_sync(0xffffffffu, best, o);
            best = ok > best ? ok : best;
        }
        if (tid == 0) {
            if (nb > 1) {
                atomicMax(&g_argmax_key[t], best);
                __threadfence();
                if (atomicAdd(&g_argmax_cnt[t], 1u) != (unsigned) nb - 1) return;
                __threadfence();
                best = atomicExch(&g_argmax_key[t], 0ull);
                g_argmax_cnt[t] = 0;
            }
            const int row = (int) ~(uint32_t) best;
            best_i[t] = map ? map[row] : row;
            if (best_v) best_v[t] = fkey_inv((uint32_t) (best >> 32));
        }
    }
}

__global__ void __launch_bounds__(1024) k_top_tokens(const float* __restrict__ logits, int V, float* __restrict__ out_v, int* __restrict__ out_i) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ unsigned hist[256];
    __shared__ unsigned long long prefix_s, sel[FNX_TOPK_N];
    __shared__ unsigned need_s, nsel;
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* l = logits + (size_t) t * V;
    if (tid == 0) { prefix_s = 0; need_s = FNX_TOPK_N; nsel = 0; }
    __syncthreads();
    // 8 passes of 8 bits from the top: after pass p the first 8 (p + 1) bits of the 64th largest key are known
    for (int pass = 0; pass < 8; ++pass) {
        const int shift = 56 - 8 * pass;
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const unsigned long long prefix = prefix_s;
        const unsigned long long mask = pass == 0 ? 0ull : ~0ull << (shift + 8);
        for (int i = tid; i < V; i += 1024) {
            const unsigned long long k = key64(l[i], i);
            if ((k & mask) == prefix) atomicAdd(&hist[(unsigned) (k >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            unsigned need = need_s, b = 255;
            for (;; --b) {
                if (hist[b] >= need) break;
                need -= hist[b];
                if (b == 0) break;
            }
            need_s = need;
            prefix_s = prefix | ((unsigned long long) b << shift);
        }
        __syncthreads();
    }
    const unsigned long long thr = prefix_s;   // the 64th largest key (keys are distinct)
    for (int i = tid; i < V; i += 1024) {
        const unsigned long long k = key64(l[i], i);
        if (k >= thr) {
            const unsigned at = atomicAdd(&nsel, 1u);
            if (at < FNX_TOPK_N) sel[at] = k;
        }
    }
    __syncthreads();
    const unsigned n = min(nsel, (unsigned) FNX_TOPK_N);
    if (tid < (int) n) {
        const unsigned long long k = sel[tid];
        unsigned rank = 0;
        for (unsigned j = 0; j < n; ++j) rank += sel[j] > k;
        out_v[t * FNX_TOPK_N + rank] = fkey_inv((uint32_t) (k >> 32));
        out_i[t * FNX_TOPK_N + rank] = (int) ~(uint32_t) k;
    }
}

__global__ void k_embed_rows(const __half* __restrict__ table, const int* __restrict__ tok, int H, float* __restrict__ R) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < H) R[(size_t) t * H + i] = __half2float(table[(size_t) tok[t] * H + i]);
}

__global__ void __launch_bounds__(256) k_rmsnorm(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y, int n, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float red[8];
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* xr = x + (size_t) r * n;
    float ss = 0.f;
    for (int i = tid; i < n; i += 256) ss += xr[i] * xr[i];
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    ss = 0.f;
    for (int j = 0; j < 8; ++j) ss += red[j];
    const float sc = rsqrtf(ss / (float) n + eps);
    for (int i = tid; i < n; i += 256) y[(size_t) r * n + i] = xr[i] * sc * w[i];
}

}  // namespace fnxb

using namespace fnxb;

extern "C" int fnx_argmax_mapped(const float* logits, int T, int V, const int* map, int* best_i, float* best_v, unsigned* err, fnx_stream st) {
    FNX_REQUIRE(logits && best_i && err && T >= 1 && V >= 1, "fnx_argmax: bad arguments");
    {
        const cudaError_t le_ = launch_k(k_argmax, dim3(T, T <= ARGMAX_ROWS && V >= 65536 ? ARGMAX_NB : 1), dim3(1024), 0, as_stream(st), logits, V, map, best_i, best_v, err);
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "k_argmax: launch failed: %s", cudaGetErrorString(le_));
    }
    FNX_LAUNCH_OK("fnx_argmax");
    return FNX_OK;
}

extern "C" int fnx_argmax(const float* logits, int T, int V, int* best_i, float* best_v, unsigned* err, fnx_stream st) {
    return fnx_argmax_mapped(logits, T, V, nullptr, best_i, best_v, err, st);
}

extern "C" int fnx_top_tokens(const float* logits, int T, int V, float* out_v, int* out_i, fnx_stream st) {
    FNX_REQUIRE(logits && out_v && out_i && T >= 1 && V >= FNX_TOPK_N, "fnx_top_tokens: bad arguments (vocabulary of at least %d)", FNX_TOPK_N);
    {
        const cudaError_t le_ = launch_k(k_top_tokens, dim3(T), dim3(1024), 0, as_stream(st), logits, V, out_v, out_i);
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "k_top_tokens: launch failed: %s", cudaGetErrorString(le_));
    }
    FNX_LAUNCH_OK("fnx_top_tokens");
    return FNX_OK;
}

// ---- the sampler's logit changes (the first half of k_topk_rows, engine/src/topk.cuh:30-45): per window row, the request's
// logit_bias added, then llama.cpp's penalties stage over the row's penalty window: each token of the window once, `repeat`
// multiplying a non-positive logit and dividing a positive one, then frequency x count and presence taken off.
// Row j's window is the last `last_n` tokens of (the sequence's kept tokens, then window rows 0..j): the tokens before the
// one row j's logits choose.  One block per row; the window is staged in shared memory and each thread settles the tokens
// whose first place in the window is its own.
constexpr int ADJ_THREADS = 256;

__global__ void __launch_bounds__(ADJ_THREADS) k_logit_adjust(float* __restrict__ logits, int V, const int* __restrict__ ctx, const int* __restrict__ ctx_n,
                                                             const int* __restrict__ tok, int last_n, float repeat, float freq, float present,
                                                             const int* __restrict__ bias_tok, const float* __restrict__ bias_val, int bias_n) {
    extern __shared__ int win[];
    pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    float* L = logits + (size_t) row * V;
    for (int i = tid; i < bias_n; i += ADJ_THREADS) {   // each token once in the list
        const int t = bias_tok[i];
        if (t >= 0 && t < V) L[t] += bias_val[i];
    }
    if (last_n <= 0) return;
    const int n = *ctx_n, len = n + row + 1, start = len > last_n ? len - last_n : 0, w = len - start;
    for (int i = tid; i < w; i += ADJ_THREADS) {
        const int at = start + i;
        win[i] = at < n ? ctx[at] : tok[at - n];
    }
    __syncthreads();   // the window staged, and a token in both lists has its bias in before its penalty
    for (int i = tid; i < w; i += ADJ_THREADS) {
        const int t = win[i];
        if (t < 0 || t >= V) continue;
        bool first = true;
        for (int j = 0; j < i && first; ++j) first = win[j] != t;
        if (!first) continue;
        int cnt = 1;
        for (int j = i + 1; j < w; ++j) cnt += win[j] == t;
        float l = L[t];
        l = l <= 0.f ? l * repeat : l / repeat;
        L[t] = __fsub_rn(__fsub_rn(l, __fmul_rn((float) cnt, freq)), present);   // each step rounded, as written (no fused multiply-add)
    }
}

extern "C" int fnx_logit_adjust(float* logits, int T, int V, const int* ctx, const int* ctx_n, const int* tok, int last_n, float repeat, float freq,
                                float present, const int* bias_tok, const float* bias_val, int bias_n, fnx_stream st) {
    FNX_REQUIRE(logits && T >= 1 && T <= FNX_MAX_ROWS && V >= 1, "fnx_logit_adjust: bad arguments");
    FNX_REQUIRE(last_n >= 0 && last_n <= FNX_PENALTY_CAP, "fnx_logit_adjust: a penalty window of %d tokens (0..%d)", last_n, FNX_PENALTY_CAP);
    FNX_REQUIRE(last_n == 0 || (ctx && ctx_n && tok), "fnx_logit_adjust: penalties need the context and the window's tokens");
    FNX_REQUIRE(last_n == 0 || repeat > 0.f, "fnx_logit_adjust: repeat penalty %g (> 0)", (double) repeat);
    FNX_REQUIRE(bias_n >= 0 && (bias_n == 0 || (bias_tok && bias_val)), "fnx_logit_adjust: a bias list of %d entries without its arrays", bias_n);
    {
        const cudaError_t le_ = launch_k(k_logit_adjust, dim3(T), dim3(ADJ_THREADS), sizeof(int) * (size_t) (last_n > 0 ? last_n : 1), as_stream(st), logits, V, ctx,
                                         ctx_n, tok, last_n, repeat, freq, present, bias_tok, bias_val, bias_n);
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "k_logit_adjust: launch failed: %s", cudaGetErrorString(le_));
    }
    FNX_LAUNCH_OK("fnx_logit_adjust");
    return FNX_OK;
}

extern "C" int fnx_embed_rows(const void* table_f16, const int* tok, int T, int H, float* R, fnx_stream st) {
    FNX_REQUIRE(table_f16 && tok && R && T >= 1, "fnx_embed_rows: bad arguments");
    {
        const cudaError_t le_ = launch_k(k_embed_rows, dim3(dim3((H + 255) / 256, T)), dim3(256), 0, as_stream(st), (const __half*) table_f16, tok, H, R);
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "k_embed_rows: launch failed: %s", cudaGetErrorString(le_));
    }
    FNX_LAUNCH_OK("fnx_embed_rows");
    return FNX_OK;
}

// The draft layer's input rows (the step of mtp_enqueue that no other layer has, engine/src/engine.cu:2103-2113):
// R[t] = fc_hid . rmsnorm(h[t]) * hnorm  +  fc_emb . rmsnorm(table[tok[t]]) * enorm.  The embedding rows pass through emb.
extern "C" int fnx_mtp_input(const void* fc_hid, const void* fc_emb, const void* table_f16, const float* hnorm, const float* enorm, float eps,
                             const float* h, int ldh, const int* tok, int T, int H, float* emb, float* R, unsigned* err, fnx_stream st) {
    FNX_REQUIRE(fc_hid && fc_emb && table_f16 && hnorm && enorm && h && tok && emb && R, "fnx_mtp_input: null pointer");
    FNX_REQUIRE(T >= 1 && ldh >= H, "fnx_mtp_input: %d rows, row stride %d for %d columns", T, ldh, H);
    FNX_TRY(fnx_embed_rows(table_f16, tok, T, H, emb, st));
    const int per = fnx_dense_rows(H);
    for (int t0 = 0; t0 < T; t0 += per) {
        const int nt = T - t0 < per ? T - t0 : per;
        FNX_TRY(fnx_dense(fc_hid, H, H, h + (size_t) t0 * ldh, ldh, nt, hnorm, eps, R + (size_t) t0 * H, H, 0, err, st));
    }
    for (int t0 = 0; t0 < T; t0 += per) {
        const int nt = T - t0 < per ? T - t0 : per;
        FNX_TRY(fnx_dense(fc_emb, H, H, emb + (size_t) t0 * H, H, nt, enorm, eps, R + (size_t) t0 * H, H, 1, err, st));
    }
    return FNX_OK;
}

extern "C" int fnx_rmsnorm(const float* x, const float* w, float* y, int rows, int n, float eps, fnx_stream st) {
    FNX_REQUIRE(x && w && y && rows >= 1 && n >= 1, "fnx_rmsnorm: bad arguments");
    {
        const cudaError_t le_ = launch_k(k_rmsnorm, dim3(rows), dim3(256), 0, as_stream(st), x, w, y, n, eps);
        if (le_ != cudaSuccess) return fail(FNX_E_CUDA, "k_rmsnorm: launch failed: %s", cudaGetErrorString(le_));
    }
    FNX_LAUNCH_OK("fnx_rmsnorm");
    return FNX_OK;
}
