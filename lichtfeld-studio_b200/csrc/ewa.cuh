// Launchers of the EWA (default, non --gut) rasterizer: ewa.cu (per-Gaussian stage, built without FMA contraction)
// and ewa_raster.cu (blend forward / backward and the per-Gaussian gradient stage).
#pragma once

#include "common.cuh"

namespace lfs {

struct EwaCamera {       // passed by value to the kernels
    const float* w2c;    // device [4,4] row-major world-to-camera matrix (the first three rows are used)
    const float* campos; // device [3] camera position in world space
    float fx, fy, cx, cy, near_plane, far_plane;
    int W, H, tw, th;
    int active_sh_bases, total_rest;  // SH bases in use (1, 4, 9, 16), rows stored per Gaussian in shN
};

// preprocess_cu: activations, 3-D and 2-D covariance, exact tile count, SH colour; packed record, depth sort key
// (0xFFFFFFFF when culled), zeroed gradient accumulators, visible count.
int launch_ewa_preprocess(int N, const lfs_splats& p, const EwaCamera& cam,
                          int32_t* n_touched, ushort4* bounds, float4* records, uint32_t* sort_keys, uint32_t* sort_vals,
                          float4* accum, int32_t* n_visible, cudaStream_t st);

struct EwaBlendArgs {
    const float4* records;        // [N*3]
    const uint32_t* instance_ids; // depth-sorted Gaussian index per instance, grouped by tile
    const int32_t* tile_offsets;  // [tw*th + 1]
    const int32_t* overflow;      // device flag: lists incomplete, draw nothing (may be null)
    const float* background;      // [3] or null
    int W, H, tw, th;
    const int32_t* tile_order = nullptr;  // [tw*th] or null: CTA b works on tile tile_order[b] (longest lists first)
};
// image [3,H,W] (background included), alpha [H,W], n_contrib [H,W] = 1 + list position of the last contributor
int launch_ewa_blend_fwd(const EwaBlendArgs& a, float* image, float* alpha, int32_t* n_contrib, cudaStream_t st);
// accum [N*12]: per Gaussian (d mean2d 2, d conic 3, sum alpha dL/dalpha 1, d colour 3, pad 3), zeroed by the forward
int launch_ewa_blend_bwd(const EwaBlendArgs& a, const float* alpha, const int32_t* n_contrib, const float* grad_image,
                         const float* grad_alpha, float* accum, cudaStream_t st);
// preprocess_backward_cu + SH backward; writes all N rows of the six gradient tensors (zeros for culled Gaussians)
// or adds to them; densification_info [2,N] may be null.
int launch_ewa_epilogue(int N, int K, const lfs_splats& p, const EwaCamera& cam, const int32_t* n_touched, const float4* records,
                        const float* accum, const lfs_splats& g, int accumulate, float* densification_info, float* grad_w2c, cudaStream_t st);

}  // namespace lfs
