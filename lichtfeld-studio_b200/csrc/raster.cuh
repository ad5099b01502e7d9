// Launchers of the rasterizer stage (raster.cu).
#pragma once

#include "common.cuh"

namespace lfs {

struct RasterArgs {
    const CamDev* cam;            // one camera
    const float4* records;        // [N] packed 64-byte records
    const uint4* bounds;          // [N] (x box, y box, rejection exponent, extra): inclusive pixel box (lo | hi << 16)
                                  //     outside of which alpha < 1/255, -ln(255 opacity) - margin as float bits, and the
                                  //     value blended into the last channel when channels is 1 or 4 (the depth)
    const uint32_t* flatten_ids;  // depth-sorted Gaussian index per instance
    const int32_t* tile_offsets;  // [tw*th] first instance of each tile
    const int32_t* n_isects_dev;  // device-side instance count, or null to use n_isects_host
    int64_t n_isects_host;
    const float* background;      // [3] or null
    const int32_t* overflow;      // device flag: when set the lists are incomplete and nothing is drawn (may be null)
    int W, H, tw, th, model;
    int channels = 3;             // 3 = colour; 1 = extra only; 4 = colour + extra
    int normalize = 0;            // divide the extra channel by max(alpha, 1e-10) on output (expected depth)
    const uint8_t* masks = nullptr;  // [tw*th] or null: tiles labelled 0 show the background and get no gradient
    const int32_t* tile_order = nullptr;  // [tw*th] or null: CTA b works on tile tile_order[b] (longest lists first)
    int rolling = 0;              // the camera has a rolling shutter or an end pose: per-pixel ray origins
};

// extra_sum [H*W] (may be null unless a.normalize): the blended, undivided last channel, kept for the backward.
int launch_raster_fwd(const RasterArgs& a, float* render, float* alphas, int32_t* last_ids, float* extra_sum, cudaStream_t st);
// accum_extra [N] (zeroed by the caller) receives the gradient of the per-Gaussian extra value; null drops it.
int launch_raster_bwd(const RasterArgs& a, const float* render_alphas, const int32_t* last_ids, const float* extra_sum,
                      const float* v_render, const float* v_alphas, float* accum, float* accum_extra, cudaStream_t st);
int launch_grad_epilogue_op(int N, const CamDev* cam, const float* accum, const float* means, const float* quats,
                            const float* scales, int channels, const float* accum_extra, float* v_means, float* v_quats,
                            float* v_scales, float* v_colors, float* v_opacities, cudaStream_t st);
// In-place Adam of the five small groups inside the gradient stage: index 0..4 = means, sh0, scaling_raw, rotation_raw,
// opacity_raw. step_size = lr * bias_correction1_rcp.
struct AdamSmall {
    float* p[5]; float* m[5]; float* v[5];
    float step_size[5];
    float beta1, beta2, eps, bc2_sqrt_rcp, grad_scale;
};
// adam != nullptr: no gradient tensor is written (g is ignored); each Gaussian's row of 16 sums in `accum` receives the six
// floats of its rank-1 shN factors and the small groups are updated in place (one camera per step only).
int launch_grad_epilogue_fused(int N, int K, int sh_degree, const CamDev* cam, const float* accum,
                               const float4* records, const int32_t* radii, const lfs_splats& p, const lfs_splats& g,
                               int accumulate, float scaling_modifier, int sh_factors, cudaStream_t st,
                               const AdamSmall* adam = nullptr);
// Adam on the shN tensor with the gradient rows rebuilt from the sh0 gradient of a one-camera backward
// (g_shN[k][c] = Y_k(direction) * g_sh0[c] / Y_0); p, m, v are the shN parameter and moment tensors [N, K-1, 3].
// campos: device [3], the camera position in world space that the backward used.
int launch_adam_sh_rank1(int N, int K, int sh_degree, const float* campos, const float* means, const float* g_sh0, float* p,
                         float* m, float* v, float step_size, float beta1, float beta2, float eps, float bc2_sqrt_rcp,
                         float grad_scale, cudaStream_t st, const float* factors = nullptr, int factor_stride = 0);
// factors != nullptr: the (colour gradient, unit direction) rows written by the gradient stage, `factor_stride` floats
// apart, replace campos / means / g_sh0.

struct AdamRank1 {
    float* p; float* m; float* v;
    float step_size, beta1, beta2, eps, bc2_sqrt_rcp, grad_scale;
    int vec;  // the three pointers are 16-byte aligned
};
// Data-parallel rank-1 shN update (see dp_sh_rank1_kernel). factors[i] / shN[i]: peer-mapped factor buffer [N,6] and shN
// parameter tensor of rank (own + i) % world; [lo, lo + n) this rank's element range of the shN tensor; m / v its moments.
constexpr int kRank1MaxPeers = 8;
struct DpRank1 {
    const float* factors[kRank1MaxPeers];
    float* shN[kRank1MaxPeers];
    float* mc_shN;             // NVSwitch multicast address of the shN tensor, or nullptr: plain peer stores
    int64_t lo, n;
    float* m; float* v;
    AdamRank1 adam;   // p / m / v unused here
    int world, N, vec;
};
int launch_dp_sh_rank1(int K, int sh_degree, const DpRank1& A, int ctas_per_sm, cudaStream_t st);

}  // namespace lfs
