// Error reporting shared by the C entry points.
#include <cstdlib>
#include <cstring>

#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>

static thread_local char g_error[512] = "";

void llmp_set_error(const char* fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, args);
    va_end(args);
}

int llmp_check_launch(const char* what) {
    const cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) return 0;
    llmp_set_error("%s: launch failed: %s", what, cudaGetErrorString(err));
    return 2;
}

LLMP_API const char* llmp_last_error() { return g_error; }

// Version of the entry-point signatures; the Python bindings refuse a library built from other sources.
LLMP_API int llmp_abi_version() { return 1; }

bool llmp_pdl_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* v = getenv("LLMP_B200_PDL");
        enabled = (v && strcmp(v, "0") == 0) ? 0 : 1;
    }
    return enabled == 1;
}
