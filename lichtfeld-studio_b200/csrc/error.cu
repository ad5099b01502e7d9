// Error bookkeeping for the C ABI.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace lfs {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(e));
        return LFS_ECUDA;
    }
    return LFS_OK;
}

const char* last_error() { return g_err; }

}  // namespace lfs
