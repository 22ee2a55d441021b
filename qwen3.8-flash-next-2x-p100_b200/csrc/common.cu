// Host-side plumbing shared by every entry point: the per-thread error text and device facts.
#include "fnx_common.cuh"

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <set>
#include <utility>

namespace fnxb {

char* error_buf() {
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buf(), 512, fmt, ap);
    va_end(ap);
    return code;
}

// the current device's SM count (remembered per device: one process may drive several)
int sm_count() {
    constexpr int MAXD = 64;
    static int n[MAXD];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAXD) return 148;
    if (!n[dev]) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        n[dev] = v;
    }
    return n[dev];
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device attribute of a kernel: set once per (device, kernel)
int set_smem_limit(const void* kernel, int bytes) {
    static std::mutex mu;
    static std::set<std::pair<int, const void*>> done;
    int dev = 0;
    FNX_CUDA_OK(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    if (done.count({dev, kernel})) return FNX_OK;
    FNX_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    done.insert({dev, kernel});
    return FNX_OK;
}

bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* v = getenv("FNX_PDL");
        on = v && v[0] == '1';
    }
    return on != 0;
}

}  // namespace fnxb

extern "C" const char* fnx_last_error(void) { return fnxb::error_buf(); }
extern "C" int fnx_version(void) { return 100; }
