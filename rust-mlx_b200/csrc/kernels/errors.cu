// The error channel of the C interface: the last message of the calling thread.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_error[1024] = "";

void rmx_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

RMX_API const char* rmx_last_error() { return g_error; }

// The compute capability the library needs; the loader compares it with the device's.
RMX_API int rmx_required_sm() { return 100; }

static bool g_dependent_launch = true;
bool rmx_dependent_launch_enabled() { return g_dependent_launch; }
// Switch programmatic dependent launch of this library's kernels on or off (on by default).
RMX_API void rmx_set_dependent_launch(int on) { g_dependent_launch = on != 0; }
