// The error text of a library's entry points: an entry point that refuses its arguments or whose launch fails leaves
// a message here and returns non-zero; the Python side reads it with frb_last_error().  Every library of kernels is
// linked with its own copy of this file.
#include <stdarg.h>

#include "common.cuh"

static thread_local char g_error[1024] = "";

void frb_set_error(const char* fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, args);
    va_end(args);
}

FRB_API const char* frb_last_error() { return g_error; }

FRB_API int frb_abi_version() { return 4; }
