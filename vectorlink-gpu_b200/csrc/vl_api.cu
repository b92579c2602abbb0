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

extern "C" const char* vl_last_error(void) { return g_error; }

extern "C" int vl_abi_version(void) { return 2; }
