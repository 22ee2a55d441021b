// Host-side plumbing shared by every entry point: the per-thread error text and device facts.
#include "fnx_common.cuh"

#include <cstdlib>
#include <cstring>

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

int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
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
