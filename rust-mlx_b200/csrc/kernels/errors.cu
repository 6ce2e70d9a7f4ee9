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
