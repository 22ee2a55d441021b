// Gated attention for a verify window: per-head norm + rotary + KV append, then tree-masked split-K attention.
//
// fnx_attn_prep_append replaces attn_prep_append / k_attn_prep_append (engine/src/kernels.hpp:259,
// engine/src/kernels.cu:1880-1910; norm_rope :513-530).  fnx_attn replaces attn / k_attn_part + k_attn_local +
// k_attn_combine (engine/src/kernels.hpp:238, engine/src/kernels.cu:558-667, 786-803): the same online-softmax
// split over positions, except that one block serves every row of the window for its share of the positions (the
// K and V rows are read once per window, not once per row), the cache is not split across cards by position, and
// a row may see only the window rows on its path to the root (the reference's windows are chains).
#include "attn_core.cuh"

namespace fnxb {


__global__ void k_attn_prep_append(float* __restrict__ qg, int ldq, float* __restrict__ k, int ldk, const float* __restrict__ v, int ldv,
                                   const float* __restrict__ qn, const float* __restrict__ kn, __half* __restrict__ kc,
                                   __half* __restrict__ vc, int nq, int nkv, int hd, int nrot, const int* __restrict__ pos0p,
                                   const int* __restrict__ depth, float eps, float rope_base) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float xrow[];   // hd floats
    __shared__ float red[32];
    attn_prep_body(qg, ldq, k, ldk, v, ldv, qn, kn, kc, vc, nq, nkv, hd, nrot, *pos0p, depth, eps, rope_base, (int) blockIdx.y, (int) blockIdx.x,
                   (int) threadIdx.x, xrow, red, SyncBlock());
}

// grid (splits, KV heads, row groups of ATT_ROWS); scratch: acc [T][nq][S][hd] floats, then mz [T][nq][S]
__global__ void __launch_bounds__(ATT_THREADS) k_attn_part(const float* __restrict__ qg, int ldq, const __half* __restrict__ kc,
                                                           const __half* __restrict__ vc, float* __restrict__ acc_out,
                                                           AttPartial* __restrict__ mz_out, int T, int nq, int nkv, int hd,
                                                           const int* __restrict__ pos0p, const int* __restrict__ parent) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) uint8_t smem[];
    attn_part_body(qg, ldq, kc, vc, acc_out, mz_out, T, nq, nkv, *pos0p, parent, (int) blockIdx.x, (int) gridDim.x, (int) blockIdx.y,
                   (int) blockIdx.z * ATT_ROWS, (int) threadIdx.x, smem, SyncBlock());
}

__global__ void __launch_bounds__(ATT_THREADS * ATC_G) k_attn_combine(const float* __restrict__ acc_in, const AttPartial* __restrict__ mz_in,
                                                                      const float* __restrict__ qg, int ldq, float* __restrict__ out, int nq, int hd,
                                                                      int S) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float sm[(3 + ATC_G) * 256];
    attn_combine_body<ATC_G>(acc_in, mz_in, qg, ldq, out, nq, hd, S, (int) blockIdx.x, (int) blockIdx.y, (int) threadIdx.x, sm, SyncBlock());
}

// ---- batched lanes: the rows of several sequences in one window.  Lane j holds the consecutive rows
// [lane_row0[j], lane_row0[j + 1]) of sequence lane_seq[j]: a chain that starts at that sequence's position pos[seq] and
// reads / appends that sequence's caches (kc_base + seq * seq_stride halves).  The bodies are the single-sequence ones
// with their pointers moved to the lane's rows (GdnLanes / enqueue_rows, engine/src/kernels.hpp:103-110,
// engine/src/engine.cu:1936).
__global__ void k_attn_prep_append_lanes(float* __restrict__ qg, int ldq, float* __restrict__ k, int ldk, const float* __restrict__ v, int ldv,
                                         const float* __restrict__ qn, const float* __restrict__ kn, __half* __restrict__ kc_base,
                                         __half* __restrict__ vc_base, size_t seq_stride, int nq, int nkv, int hd, int nrot,
                                         const int* __restrict__ pos, const int* __restrict__ lane_seq, const int* __restrict__ lane_row0, float eps,
                                         float rope_base) {
    extern __shared__ float xrow[];   // hd floats
    __shared__ float red[32];
    const int lane = blockIdx.z, t = blockIdx.y, row0 = lane_row0[lane];
    if (t >= lane_row0[lane + 1] - row0) return;
    const int seq = lane_seq[lane];
    if (seq < 0) return;   // another rank's lane
    attn_prep_body(qg + (size_t) row0 * ldq, ldq, k + (size_t) row0 * ldk, ldk, v + (size_t) row0 * ldv, ldv, qn, kn, kc_base + seq * seq_stride,
                   vc_base + seq * seq_stride, nq, nkv, hd, nrot, pos[seq], nullptr, eps, rope_base, t, (int) blockIdx.x, (int) threadIdx.x, xrow, red,
                   SyncBlock());
}

// grid (splits, KV heads, lanes); a lane has at most ATT_ROWS rows
__global__ void __launch_bounds__(ATT_THREADS) k_attn_part_lanes(const float* __restrict__ qg, int ldq, const __half* __restrict__ kc_base,
                                                                 const __half* __restrict__ vc_base, size_t seq_stride, float* __restrict__ acc_out,
                                                                 AttPartial* __restrict__ mz_out, int nq, int nkv, const int* __restrict__ pos,
                                                                 const int* __restrict__ lane_seq, const int* __restrict__ lane_row0) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int lane = blockIdx.z, row0 = lane_row0[lane], T = lane_row0[lane + 1] - row0, seq = lane_seq[lane], S = gridDim.x;
    if (T <= 0 || seq < 0) return;   // (a negative sequence: another rank's lane)
    attn_part_body(qg + (size_t) row0 * ldq, ldq, kc_base + seq * seq_stride, vc_base + seq * seq_stride, acc_out + (size_t) row0 * nq * S * ATT_HD,
                   mz_out + (size_t) row0 * nq * S, T, nq, nkv, pos[seq], nullptr, (int) blockIdx.x, S, (int) blockIdx.y, 0, (int) threadIdx.x, smem, SyncBlock());
}

// the prompt form: grid (1, KV heads, groups of ATP_ROWS rows); every block runs over all the positions its rows see, so there is
// one partial per (row, head) and the combine only normalises and gates it
__global__ void __launch_bounds__(ATT_THREADS) k_attn_part_prompt(const float* __restrict__ qg, int ldq, const __half* __restrict__ kc,
                                                                  const __half* __restrict__ vc, float* __restrict__ acc_out,
                                                                  AttPartial* __restrict__ mz_out, int T, int nq, int nkv, const int* __restrict__ pos0p) {
    extern __shared__ __align__(16) uint8_t smem[];
    attn_part_body_t<ATP_ROWS, ATP_MQ, false, true>(qg, ldq, kc, vc, acc_out, mz_out, T, nq, nkv, *pos0p, nullptr, 0, 1, (int) blockIdx.y,
                                                    (int) blockIdx.z * ATP_ROWS, (int) threadIdx.x, smem, SyncBlock());
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
    FNX_REQUIRE(T >= 1 && (depth ? T <= FNX_MAX_ROWS : T <= 65535), "fnx_attn_prep_append: %d rows", T);
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
    const size_t smem = attn_part_smem();
    if (int rc = set_smem_limit((const void*) k_attn_part, (int) attn_part_smem())) return rc;
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

extern "C" size_t fnx_attn_prompt_scratch_bytes(int T, int nq, int hd) { return (size_t) T * nq * ((size_t) hd * sizeof(float) + sizeof(AttPartial)); }

namespace fnxb {
bool attn_prompt_tc_fits(int nq, int nkv, int hd);
int attn_prompt_tc_launch(const float* qg, int ldq, const __half* kc, const __half* vc, float* out, int T, int nq, int nkv, const int* pos0, unsigned* err,
                          cudaStream_t st);
}  // namespace fnxb

extern "C" int fnx_attn_prompt(const float* qg, int ldq, const void* kc, const void* vc, float* out, int T, int nq, int nkv, int hd, const int* pos0,
                               void* scratch, unsigned* err, int use_mma_sync, fnx_stream st) {
    FNX_REQUIRE(qg && kc && vc && out && pos0 && scratch, "fnx_attn_prompt: null pointer");
    FNX_REQUIRE(T >= 1 && T <= 65535, "fnx_attn_prompt: %d rows", T);
    FNX_REQUIRE(hd == ATT_THREADS, "fnx_attn_prompt: head dim %d (this build: %d)", hd, ATT_THREADS);
    FNX_REQUIRE(nkv >= 1 && nq % nkv == 0 && nq / nkv <= ATT_MAXQ, "fnx_attn_prompt: %d q heads over %d KV heads", nq, nkv);
    if (!use_mma_sync && attn_prompt_tc_fits(nq, nkv, hd)) {
        FNX_REQUIRE(ldq % 4 == 0 && ((uintptr_t) qg & 15) == 0 && ((uintptr_t) kc & 15) == 0 && ((uintptr_t) vc & 15) == 0 && ((uintptr_t) out & 15) == 0,
                    "fnx_attn_prompt: rows and caches must be 16-byte aligned");
        return attn_prompt_tc_launch(qg, ldq, (const __half*) kc, (const __half*) vc, out, T, nq, nkv, pos0, err, as_stream(st));
    }
    float* acc = (float*) scratch;
    AttPartial* mz = (AttPartial*) (acc + (size_t) T * nq * hd);
    if (int rc = set_smem_limit((const void*) k_attn_part_prompt, (int) attn_prompt_smem())) return rc;
    k_attn_part_prompt<<<dim3(1, nkv, (T + ATP_ROWS - 1) / ATP_ROWS), ATT_THREADS, attn_prompt_smem(), as_stream(st)>>>(qg, ldq, (const __half*) kc, (const __half*) vc, acc, mz,
                                                                                                                     T, nq, nkv, pos0);
    FNX_LAUNCH_OK("fnx_attn_prompt (partials)");
    k_attn_combine<<<dim3(nq, T), hd * ATC_G, 0, as_stream(st)>>>(acc, mz, qg, ldq, out, nq, hd, 1);
    FNX_LAUNCH_OK("fnx_attn_prompt (combine)");
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
        if (int rc2 = set_smem_limit((const void*) k_attn_part, (int) attn_part_smem())) return rc2;
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
    const size_t smem = attn_part_smem();
    cudaError_t le = launch_k(k_attn_part, dim3(S, nkv, (T + ATT_ROWS - 1) / ATT_ROWS), dim3(ATT_THREADS), smem, as_stream(st), qg, ldq,
                              (const __half*) kc, (const __half*) vc, acc, mz, T, nq, nkv, hd, pos0, parent);
    if (le != cudaSuccess) return fail(FNX_E_CUDA, "k_attn_part: launch failed: %s", cudaGetErrorString(le));
    FNX_LAUNCH_OK("fnx_attn_static (partials)");
    le = launch_k(k_attn_combine, dim3(nq, T), dim3(hd * ATC_G), 0, as_stream(st), acc, mz, qg, ldq, out, nq, hd, S);
    if (le != cudaSuccess) return fail(FNX_E_CUDA, "k_attn_combine: launch failed: %s", cudaGetErrorString(le));
    FNX_LAUNCH_OK("fnx_attn_static (combine)");
    return FNX_OK;
}

// ---- batched lanes (see k_attn_prep_append_lanes)
extern "C" int fnx_attn_prep_append_lanes(float* qg, int ldq, float* k, int ldk, const float* v, int ldv, const float* q_norm, const float* k_norm,
                                          void* kc_base, void* vc_base, size_t seq_stride_rows, int n_lanes, int max_lane_rows, int nq, int nkv, int hd,
                                          int nrot, const int* pos, const int* lane_seq, const int* lane_row0, float eps, float rope_base, fnx_stream st) {
    FNX_REQUIRE(qg && k && v && q_norm && k_norm && kc_base && vc_base && pos && lane_seq && lane_row0, "fnx_attn_prep_append_lanes: null pointer");
    FNX_REQUIRE(n_lanes >= 1 && n_lanes <= FNX_MAX_ROWS && max_lane_rows >= 1 && max_lane_rows <= FNX_MAX_ROWS, "fnx_attn_prep_append_lanes: %d lanes of up to %d rows",
                n_lanes, max_lane_rows);
    FNX_REQUIRE(hd % 32 == 0 && hd <= 1024 && nrot <= hd && nrot % 2 == 0, "fnx_attn_prep_append_lanes: head dim %d, rotary %d", hd, nrot);
    const cudaError_t le = launch_k(k_attn_prep_append_lanes, dim3(nq + 2 * nkv, max_lane_rows, n_lanes), dim3(hd), hd * sizeof(float), as_stream(st), qg, ldq, k, ldk,
                                    v, ldv, q_norm, k_norm, (__half*) kc_base, (__half*) vc_base, seq_stride_rows * (size_t) nkv * hd, nq, nkv, hd, nrot, pos, lane_seq,
                                    lane_row0, eps, rope_base);
    if (le != cudaSuccess) return fail(FNX_E_CUDA, "k_attn_prep_append_lanes: launch failed: %s", cudaGetErrorString(le));
    FNX_LAUNCH_OK("fnx_attn_prep_append_lanes");
    return FNX_OK;
}

extern "C" int fnx_attn_lanes(const float* qg, int ldq, const void* kc_base, const void* vc_base, size_t seq_stride_rows, float* out, int T, int n_lanes,
                              int nq, int nkv, int hd, const int* pos, const int* lane_seq, const int* lane_row0, void* scratch, fnx_stream st) {
    FNX_REQUIRE(qg && kc_base && vc_base && out && pos && lane_seq && lane_row0 && scratch, "fnx_attn_lanes: null pointer");
    FNX_REQUIRE(T >= 1 && T <= FNX_MAX_ROWS && n_lanes >= 1 && n_lanes <= T, "fnx_attn_lanes: %d rows in %d lanes", T, n_lanes);
    FNX_REQUIRE(hd == ATT_THREADS, "fnx_attn_lanes: head dim %d (this build: %d)", hd, ATT_THREADS);
    FNX_REQUIRE(nkv >= 1 && nq % nkv == 0 && nq / nkv <= ATT_MAXQ, "fnx_attn_lanes: %d q heads over %d KV heads", nq, nkv);
    const int S = attn_splits(nkv);
    FNX_REQUIRE(S <= 256, "fnx_attn_lanes: %d splits", S);
    float* acc = (float*) scratch;
    AttPartial* mz = (AttPartial*) (acc + (size_t) T * nq * S * hd);
    if (int rc = set_smem_limit((const void*) k_attn_part_lanes, (int) attn_part_smem())) return rc;
    cudaError_t le = launch_k(k_attn_part_lanes, dim3(S, nkv, n_lanes), dim3(ATT_THREADS), attn_part_smem(), as_stream(st), qg, ldq, (const __half*) kc_base,
                              (const __half*) vc_base, seq_stride_rows * (size_t) nkv * hd, acc, mz, nq, nkv, pos, lane_seq, lane_row0);
    if (le != cudaSuccess) return fail(FNX_E_CUDA, "k_attn_part_lanes: launch failed: %s", cudaGetErrorString(le));
    FNX_LAUNCH_OK("fnx_attn_lanes (partials)");
    le = launch_k(k_attn_combine, dim3(nq, T), dim3(hd * ATC_G), 0, as_stream(st), acc, mz, qg, ldq, out, nq, hd, S);
    if (le != cudaSuccess) return fail(FNX_E_CUDA, "k_attn_combine: launch failed: %s", cudaGetErrorString(le));
    FNX_LAUNCH_OK("fnx_attn_lanes (combine)");
    return FNX_OK;
}
