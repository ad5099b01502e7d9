// lfs_mcmc_classify_noalloc: the dead / alive classification of the MCMC densification step with its
// scratch memory inside the library instead of in a caller-provided workspace.
//
// Who needs this: a host that may not allocate device memory at the point where it runs the
// densification step. Two such callers exist around this path. (1) A trainer that shares the GPU with
// a live viewer thread refines the model while holding the render lock; an allocation there (even one
// served by a caching allocator that has to grow) can synchronise the whole device and stall the frame
// in flight, so that code path is written to allocate nothing. (2) A plugin host that hands this
// library a fixed memory budget at start-up and forbids any later growth cannot size a workspace for a
// step whose Gaussian count changes from call to call. For both, the scratch below is reserved once,
// when the library is loaded, and never changes size.
//
// Cost and limits: every GPU that loads the library holds kScratchBytes (about 2.1 MB) until the
// process exits. At most LFS_NOALLOC_MAX_GAUSSIANS Gaussians per call. All calls on one device share
// the same scratch, which keeps whatever the previous call left in it; two calls that overlap on the
// GPU (different streams, or different host threads) race on it and give wrong lists.
#include "elementwise.cuh"

namespace lfs {
namespace {

constexpr int kMaxN = LFS_NOALLOC_MAX_GAUSSIANS;
constexpr size_t kFlagsOff = 0;                                     // int32[kMaxN]  dead flag per Gaussian
constexpr size_t kOffsOff = kFlagsOff + sizeof(int32_t) * kMaxN;    // int32[kMaxN]  exclusive prefix of the flags
constexpr size_t kTotalOff = kOffsOff + sizeof(int32_t) * kMaxN;    // int32[64]     number of dead Gaussians
constexpr size_t kSumsOff = kTotalOff + 256;                        // uint32[...]   per-block sums of the prefix scan
constexpr size_t kScratchBytes = kSumsOff + sizeof(uint32_t) * (kScanBlocks + 320);

// In host code this name is only a handle for cudaGetSymbolAddress: it is NOT a device address and must
// never be passed to a kernel or used in pointer arithmetic on the host.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_addr[kMaxDevices] = {};  // device address of g_scratch, per device, filled on first use

// Device address of the CURRENT device's copy of the scratch array. The first call on a device resolves it
// with cudaGetSymbolAddress (that device must be current, which it is: we ask which one is current). The caller's
// stream must belong to that same device; the entry point cannot check this from a bare stream handle.
// Two host threads that make their first call at the same time both store the same address, which is harmless.
int scratch_base(unsigned char** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_error("lfs_mcmc_classify_noalloc: cudaGetDevice failed or device index out of range (%s)",
                  e == cudaSuccess ? "index" : cudaGetErrorString(e));
        return LFS_ECUDA;
    }
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_scratch);
        if (e != cudaSuccess || p == nullptr) {
            set_error("lfs_mcmc_classify_noalloc: cudaGetSymbolAddress failed (%s)", cudaGetErrorString(e));
            return LFS_ECUDA;
        }
        g_scratch_addr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_scratch_addr[dev];
    return LFS_OK;
}

}  // namespace
}  // namespace lfs

using namespace lfs;

extern "C" int lfs_mcmc_classify_noalloc(int N, const float* opacity_raw, const float* rotation_raw, float min_opacity,
                                         int64_t* dead_indices, int64_t* alive_indices, float* alive_opacities,
                                         int32_t* counts_dev, void* stream) {
    LFS_REQUIRE(N >= 0, "bad size");
    if (N > kMaxN) {
        set_error("lfs_mcmc_classify_noalloc: N = %d exceeds the built-in scratch (at most %d Gaussians); "
                  "use lfs_mcmc_classify with a caller-provided workspace", N, kMaxN);
        return LFS_ECAPACITY;
    }
    LFS_REQUIRE(counts_dev != nullptr, "null pointer");
    if (N > 0) LFS_REQUIRE(opacity_raw && rotation_raw && dead_indices && alive_indices && alive_opacities, "null pointer");
    LFS_REQUIRE((reinterpret_cast<uintptr_t>(rotation_raw) & 15) == 0, "rotation_raw must be 16-byte aligned");
    unsigned char* base = nullptr;
    const int rc = scratch_base(&base);
    if (rc != LFS_OK) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int32_t* flags = reinterpret_cast<int32_t*>(base + kFlagsOff);
    int32_t* offs = reinterpret_cast<int32_t*>(base + kOffsOff);
    int32_t* total = reinterpret_cast<int32_t*>(base + kTotalOff);
    SortScratch s;
    s.hist = nullptr;  // only the prefix scan runs here; it does not touch the radix histogram
    s.block_sums = reinterpret_cast<uint32_t*>(base + kSumsOff);
    // The scratch still holds the previous call's flags, prefix and count. Flags and prefix are rewritten
    // for [0, N) before they are read; the count is the one value a reader could see stale, so clear it.
    if (cudaMemsetAsync(total, 0, 64 * sizeof(int32_t), st) != cudaSuccess) return check_launch("lfs_mcmc_classify_noalloc");
    return launch_mcmc_classify(N, opacity_raw, rotation_raw, min_opacity, dead_indices, alive_indices, alive_opacities,
                                counts_dev, flags, offs, total, s, st);
}
