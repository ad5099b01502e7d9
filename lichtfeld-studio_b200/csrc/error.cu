// Error bookkeeping for the C ABI.
#include <cstdarg>
#include <cstdio>
#include <vector>

#include <nvtx3/nvToolsExt.h>   // header-only: ranges cost nothing unless a profiler attached its injection library

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

int num_sms() {
    static int cached[64] = {};   // per device ordinal; 0 = not read yet
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

namespace {
struct ProfRec { const char* name; cudaEvent_t a, b; };
bool g_prof = false;   // bracket every launch with two CUDA events
bool g_nvtx = false;   // open an NVTX range (the LFS_TIMED name) around every launch
std::vector<ProfRec> g_recs;
}  // namespace

KernelTimer::KernelTimer(const char* name, cudaStream_t st) : name_(name), st_(st), a_(nullptr), b_(nullptr), nvtx_(g_nvtx) {
    if (nvtx_) nvtxRangePushA(name);
    if (!g_prof) return;
    cudaEvent_t a, b;
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return;
    cudaEventRecord(a, st);
    a_ = a; b_ = b;
}
KernelTimer::~KernelTimer() {
    if (nvtx_) nvtxRangePop();
    if (!a_) return;
    cudaEventRecord(reinterpret_cast<cudaEvent_t>(b_), st_);
    g_recs.push_back(ProfRec{name_, reinterpret_cast<cudaEvent_t>(a_), reinterpret_cast<cudaEvent_t>(b_)});
}

void profile_enable(bool events, bool nvtx) {
    for (auto& r : g_recs) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
    g_recs.clear();
    g_prof = events;
    g_nvtx = nvtx;
}
int profile_collect(int max_records, const char** names, float* ms) {
    int n = 0;
    for (auto& r : g_recs) {
        if (n >= max_records) break;
        if (cudaEventSynchronize(r.b) != cudaSuccess) break;
        float t = 0.f;
        cudaEventElapsedTime(&t, r.a, r.b);
        names[n] = r.name;
        ms[n] = t;
        ++n;
    }
    return n;
}

}  // namespace lfs
