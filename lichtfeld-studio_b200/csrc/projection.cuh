// Launchers of the per-Gaussian stage (projection.cu).
#pragma once

#include "common.cuh"

namespace lfs {

struct ProjParams {
    float eps2d, near_plane, far_plane, radius_clip;
    float alpha, beta, kappa, margin;
    bool require_all;
};

inline ProjParams make_proj_params(float eps2d, float near_plane, float far_plane, float radius_clip,
                                   const lfs_ut_params& ut) {
    ProjParams p;
    p.eps2d = eps2d; p.near_plane = near_plane; p.far_plane = far_plane; p.radius_clip = radius_clip;
    p.alpha = ut.alpha; p.beta = ut.beta; p.kappa = ut.kappa; p.margin = ut.in_image_margin_factor;
    p.require_all = ut.require_all_sigma_points_valid != 0;
    return p;
}

int launch_projection_ut(int C, int N, const float* means, const float* quats, const float* scales,
                         const float* opacities, const float* viewmats, const float* viewmats1, int rs_type, const float* Ks,
                         const float* radial, const float* tangential, const float* thin_prism, int W, int H, const ProjParams& pp,
                         int model, int32_t* radii,
                         float* means2d, float* depths, float* conics, float* compensations, cudaStream_t st);

// colours [N, channels] with channels 1 (extra only), 3 (rgb) or 4 (rgb + extra); accum / accum_extra (may be null)
// are zeroed for the backward.
int launch_pack_records(int N, const float* means, const float* quats, const float* scales, const float* colors, int channels,
                        const float* opacities, const CamDev* cam, float4* records, uint4* bounds, float4* accum,
                        float* accum_extra, cudaStream_t st);

// Per-render switches of the fused path (FusedRasterizationSettings, src/training/rasterization/rasterizer_autograd.hpp).
struct PackOptions {
    float scaling_modifier = 1.0f;  // scales are multiplied by it before projection and blending
    int calc_compensations = 0;     // antialiased: blended opacity = opacity * sqrt(det(cov) / det(cov + eps2d I))
    int want_rgb = 1;               // 0 in the depth-only render modes: SH colours are not evaluated
};

// model: the effective (internal) model id, see effective_model(); rolling: the camera has a rolling shutter or an end pose
int launch_project_pack(int N, int K, int sh_degree, const lfs_splats& p, const CamDev* cam, const ProjParams& pp,
                        const PackOptions& opt, int model, int rolling, int tile_size, int tw, int th, int32_t* radii, float* means2d, float* depths,
                        int32_t* tiles, uint32_t* sort_keys, uint32_t* sort_vals, float4* records, uint4* bounds, float4* accum,
                        int32_t* n_visible, cudaStream_t st);

// colours (SH + 0.5, clamped at 0) of the visible Gaussians into records[g*4+3].xyz
int launch_sh_color(int N, int K, int sh_degree, const lfs_splats& p, const CamDev* cam, const int32_t* radii, float4* records,
                    cudaStream_t st);

int launch_tile_count(int64_t total, const float* means2d, const int32_t* radii, int tile_size, int tw, int th,
                      int32_t* tiles, cudaStream_t st);

}  // namespace lfs
