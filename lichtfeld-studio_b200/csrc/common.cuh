// Shared declarations of the lfs_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lfs_b200.h"

namespace lfs {

// ---------------------------------------------------------------------------------------------
// Error reporting: every entry point returns a status and leaves a message for lfs_last_error().
// ---------------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int check_launch(const char* what);

// Opt-in per-kernel timing (lfs_profile_enable): when on, a KernelTimer brackets a launch with two
// CUDA events on the launching stream; lfs_profile_collect returns the elapsed times. With the NVTX bit it opens an
// NVTX range of the same name around the launch for timeline tools. Off by default and free when off.
struct KernelTimer {
    KernelTimer(const char* name, cudaStream_t st);
    ~KernelTimer();
    const char* name_;
    cudaStream_t st_;
    void* a_;
    void* b_;
    bool nvtx_;
};
#define LFS_TIMED(name, st) ::lfs::KernelTimer lfs_kernel_timer_(name, st)

#define LFS_REQUIRE(cond, msg)                         \
    do {                                               \
        if (!(cond)) {                                 \
            ::lfs::set_error("%s: %s", __func__, msg); \
            return LFS_EINVAL;                         \
        }                                              \
    } while (0)

// Persistent / grid-stride kernels are sized in multiples of the SM count of the current device (148 on a B200),
// read once per device from cudaDevAttrMultiProcessorCount.
int num_sms();

inline int grid_for(int64_t n, int block, int max_blocks_per_sm = 8) {
    int64_t g = (n + block - 1) / block;
    const int64_t cap = (int64_t)num_sms() * max_blocks_per_sm;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

// ---------------------------------------------------------------------------------------------
// Per-camera constants derived once per call by camera_setup_kernel from the row-major
// world-to-camera matrix and the intrinsics (global shutter).
// ---------------------------------------------------------------------------------------------
struct CamDev {
    float qw, qx, qy, qz;  // quat_cast of the rotation block
    float tx, ty, tz;      // translation column
    float Rinv[9];         // mat3_cast(inverse(q)), row-major
    float ro[3];           // world ray origin = -Rinv * t
    float campos[3];       // -R^T t (what inverse(viewmat)[:3,3] gives), used for SH directions
    float fx, fy, cx, cy;
    float k[4];            // fisheye radial coefficients
    float dist[12];        // OpenCV pinhole distortion: k1..k6, p1, p2, s1..s4 (model == LFS_PINHOLE_OPENCV)
    float max_angle;       // fisheye
    float approx_b1;       // fisheye: linear term of the crude backward polynomial
    int W, H, model;
    int rs_type;           // ShutterType of the reference: 0..3 rolling (top-to-bottom, left-to-right, bottom-to-top,
                           // right-to-left), 4 global
    // rolling shutter: end-of-frame pose (equal to the start pose without one) and the centre-of-frame pose that
    // gives the depth of a Gaussian (gsplat/ProjectionUT3DGSFused.cu:73-77)
    int has_end;
    float q1w, q1x, q1y, q1z, t1x, t1y, t1z;
    float qcw, qcx, qcy, qcz, tcx, tcy, tcz;
};
constexpr int LFS_SHUTTER_GLOBAL = 4;

// Internal model id: LFS_PINHOLE with any of the three distortion tensors present selects the OpenCV pinhole
// model (gsplat/ProjectionUT3DGSFused.cu:91-113); it never crosses the C ABI.
constexpr int LFS_PINHOLE_OPENCV = 4;
inline int effective_model(int model, const float* radial, const float* tangential, const float* thin_prism) {
    return (model == LFS_PINHOLE && (radial || tangential || thin_prism)) ? LFS_PINHOLE_OPENCV : model;
}

// One packed 64-byte record per Gaussian for the rasterizer:
//   r0 = (M00, M01, M02, gro.x)   M = diag(1/scale) * R^T
//   r1 = (M10, M11, M12, gro.y)   gro = M * (ray_origin - mean)
//   r2 = (M20, M21, M22, gro.z)
//   r3 = (red, green, blue, opacity)
constexpr int kRecordFloats = 16;

// Host-side launchers shared between translation units (all asynchronous on `st`).
// radial: [C,4] for LFS_FISHEYE, [C,6] for LFS_PINHOLE; tangential [C,2] and thin_prism [C,4] only for LFS_PINHOLE.
// viewmats1 [C,4,4] or null (no end pose), rs_type = ShutterType (4 = global)
int launch_camera_setup(int C, const float* viewmats, const float* viewmats1, int rs_type, const float* Ks, const float* radial,
                        const float* tangential, const float* thin_prism, int W, int H, int model, CamDev* cams,
                        cudaStream_t st);

// ---- sort.cu -------------------------------------------------------------------------------
struct SortScratch {
    uint32_t* hist;       // [kRadixBlocks * 256]
    uint32_t* block_sums; // [kScanBlocks + 1]
};
// Capacity of the scratch arrays; the launches use min(4 x SM count, capacity) blocks.
constexpr int kRadixBlocks = 1024;
constexpr int kScanBlocks = 1024;
size_t sort_scratch_bytes();

// Stable LSD radix sort of (key, value) uint32 pairs over key bits [0, key_bits). n is read from
// *n_dev when n_dev != nullptr (device-side count, bounded by n_max), else n_max is the count.
// Returns the index (0 or 1) of the buffer pair holding the result.
int radix_sort_pairs(uint32_t* keys[2], uint32_t* vals[2], const int32_t* n_dev, int64_t n_max, int key_bits,
                     const SortScratch& scratch, cudaStream_t st);

// out[i] = exclusive prefix sum of gather(i) = src[idx ? idx[i] : i]; total written to *total_dev.
int exclusive_scan_gather(const int32_t* src, const uint32_t* idx, int64_t n, int32_t* out, int32_t* total_dev,
                          const SortScratch& scratch, cudaStream_t st);

// One 16-byte store to an NVSwitch multicast address: the switch writes it into the same offset of every GPU bound to the
// multicast object (this GPU included), so a broadcast leaves this GPU's NVLink ports once instead of once per peer.
__device__ __forceinline__ void multimem_st4(float* mc, const float4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}
__device__ __forceinline__ void multimem_st1(float* mc, const float v) {
    asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc), "f"(v) : "memory");
}

}  // namespace lfs
