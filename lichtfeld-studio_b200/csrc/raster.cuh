// Launchers of the rasterizer stage (raster.cu).
#pragma once

#include "common.cuh"

namespace lfs {

struct RasterArgs {
    const CamDev* cam;            // one camera
    const float4* records;        // [N] packed 64-byte records
    const uint4* bounds;          // [N] (x box, y box, rejection exponent, 0): inclusive pixel box (lo | hi << 16)
                                  //     outside of which alpha < 1/255, and -ln(255 opacity) - margin as float bits
    const uint32_t* flatten_ids;  // depth-sorted Gaussian index per instance
    const int32_t* tile_offsets;  // [tw*th] first instance of each tile
    const int32_t* n_isects_dev;  // device-side instance count, or null to use n_isects_host
    int64_t n_isects_host;
    const float* background;      // [3] or null
    const int32_t* overflow;      // device flag: when set the lists are incomplete and nothing is drawn (may be null)
    int W, H, tw, th, model;
};

int launch_raster_fwd(const RasterArgs& a, float* render, float* alphas, int32_t* last_ids, cudaStream_t st);
int launch_raster_bwd(const RasterArgs& a, const float* render_alphas, const int32_t* last_ids, const float* v_render,
                      const float* v_alphas, float* accum, cudaStream_t st);
int launch_grad_epilogue_op(int N, const CamDev* cam, const float* accum, const float* means, const float* quats,
                            const float* scales, float* v_means, float* v_quats, float* v_scales, float* v_colors,
                            float* v_opacities, cudaStream_t st);
int launch_grad_epilogue_fused(int N, int K, int sh_degree, const CamDev* cam, const float* accum,
                               const float4* records, const int32_t* radii, const lfs_splats& p, const lfs_splats& g,
                               int accumulate, cudaStream_t st);

}  // namespace lfs
