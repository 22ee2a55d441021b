// Shared helpers of the fnx_b200 kernels: error reporting, warp reductions, bounded mbarrier waits, Philox.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/fnx_b200.h"

namespace fnxb {

// ---- host-side error text (per thread), returned by fnx_last_error()
char* error_buf();
int fail(int code, const char* fmt, ...);

#define FNX_CUDA_OK(expr)                                                                                   \
    do {                                                                                                    \
        cudaError_t e_ = (expr);                                                                            \
        if (e_ != cudaSuccess) return ::fnxb::fail(FNX_E_CUDA, "%s: %s (%s:%d)", #expr, cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)
#define FNX_LAUNCH_OK(what)                                                                                 \
    do {                                                                                                    \
        cudaError_t e_ = cudaGetLastError();                                                                \
        if (e_ != cudaSuccess) return ::fnxb::fail(FNX_E_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e_)); \
    } while (0)
#define FNX_REQUIRE(cond, ...)                                      \
    do {                                                            \
        if (!(cond)) return ::fnxb::fail(FNX_E_ARG, __VA_ARGS__);   \
    } while (0)

#define FNX_TRY(expr)                  \
    do {                               \
        int rc_ = (expr);              \
        if (rc_ != FNX_OK) return rc_; \
    } while (0)

inline cudaStream_t as_stream(fnx_stream s) { return (cudaStream_t) s; }
int sm_count();
// raises a kernel's dynamic shared-memory limit on the current device, once per (device, kernel)
int set_smem_limit(const void* kernel, int bytes);
// Programmatic dependent launch: every kernel of the window is launched so that it may start while its predecessor
// in the stream drains.  A kernel does whatever does not depend on earlier kernels (its tables, its barriers, bulk
// copies of weights), then pdl_wait() before it touches anything an earlier kernel wrote.  Off unless FNX_PDL=1:
// inside the window's CUDA graph the overlap measured slower than plain stream order on B200.
bool pdl_enabled();
#if defined(__CUDACC__)
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

#if defined(__CUDACC__)
// ---- programmatic dependent launch (no-ops when the launch carried no such dependency)
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- warp helpers
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.0f + expf(-x)); }

// ---- shared-memory barriers for bulk async copies.  Every wait is bounded: after `limit` polls it gives up and
// the caller records FNX_ERR_TIMEOUT instead of hanging the GPU.
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// true when the phase completed, false when the poll limit ran out
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity, unsigned limit = 4000000u) {
    for (unsigned i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// global -> shared bulk copy (dst, src 16-byte aligned, bytes a multiple of 16), completion on `bar`
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- Philox4x32-10 (Salmon et al., SC'11), the published round constants
__host__ __device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                                                       uint32_t (&out)[4]) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t) 0xD2511F53u * c0, p1 = (uint64_t) 0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t) (p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t) p1;
        const uint32_t n2 = (uint32_t) (p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t) p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}
// the acceptance stream: uniform in [0,1) addressed by (seed, seq, step, slot)
__host__ __device__ __forceinline__ double philox_uniform(uint64_t seed, uint32_t seq, uint32_t step, uint32_t slot) {
    uint32_t o[4];
    philox4x32_10(slot, step, seq, 0u, (uint32_t) seed, (uint32_t) (seed >> 32), o);
    const uint64_t hi = o[0] >> 5, lo = o[1] >> 6;
    return (double) ((hi << 26) | lo) * (1.0 / 9007199254740992.0);
}
#endif

}  // namespace fnxb
