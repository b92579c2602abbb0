// Error plumbing shared by the extern "C" entry points of libvlgpu.
#include <cstdarg>
#include <cstdio>

#include "vl_common.cuh"

namespace {
thread_local char g_error[512] = "";
}

void vl_set_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

// SMs of the current device (asked once per device; 148 on a B200): launch-size caps are
// multiples of it.
int vl_sm_count()
{
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return 148;
        cached[dev] = sms;
    }
    return cached[dev];
}

extern "C" const char* vl_last_error(void) { return g_error; }

extern "C" int vl_abi_version(void) { return 4; }
