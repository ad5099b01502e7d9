/*
 * lfs_gsplat_ops.h — the operator API of gsplat/Ops.h:12-270 (namespace gsplat, at::Tensor in,
 * std::tuple<at::Tensor, ...> out) served by the lfs_b200 C ABI.
 *
 * Host-side C++ for libtorch programs: lichtfeld-studio_b200/csrc/ops_shim.cpp defines these twelve functions
 * with the reference's names, argument order, defaults and error behaviour (TORCH_CHECK failures where the
 * reference checks, c10::Error for a failing C-ABI call), allocates every output with ATen on the inputs' device and
 * launches on at::cuda::getCurrentCUDAStream(), like the reference wrappers (gsplat/Projection.cpp:22,
 * gsplat/Intersect.cpp:15, gsplat/Rasterization.cpp:20 / :135 / :279 / :470, gsplat/SphericalHarmonics.cpp:15,
 * gsplat/Relocation.cpp:15, gsplat/QuatToRotmat.cpp).
 *
 * Inside the reference tree the shim is compiled against the reference's own gsplat/Ops.h instead of this header
 * (define LFS_SHIM_USE_REFERENCE_HEADERS): it then replaces gsplat_backend at link time and nothing above Ops.h
 * changes. This header repeats the three small types of gsplat/Common.h:46-51 and gsplat/Cameras.h:16-61 that the
 * signatures need, so that the shim also builds where the reference tree (and glm) is not available.
 */
#pragma once

#include <ATen/core/Tensor.h>
#include <c10/util/Optional.h>

#include <cstdint>
#include <tuple>

/* gsplat/Cameras.h:16-22 */
enum class ShutterType {
    ROLLING_TOP_TO_BOTTOM,
    ROLLING_LEFT_TO_RIGHT,
    ROLLING_BOTTOM_TO_TOP,
    ROLLING_RIGHT_TO_LEFT,
    GLOBAL
};

/* gsplat/Cameras.h:27-45 */
struct UnscentedTransformParameters {
    float alpha = 0.1f;
    float beta = 2.f;
    float kappa = 0.f;
    float in_image_margin_factor = 0.1f;
    bool require_all_sigma_points_valid = true;
};

namespace gsplat {

    /* gsplat/Common.h:46-51 */
    enum CameraModelType { PINHOLE = 0, ORTHO = 1, FISHEYE = 2, EQUIRECTANGULAR = 3 };

    at::Tensor spherical_harmonics_fwd(const uint32_t degrees_to_use, const at::Tensor dirs, const at::Tensor coeffs,
                                       const at::optional<at::Tensor> masks);
    std::tuple<at::Tensor, at::Tensor> spherical_harmonics_bwd(const uint32_t K, const uint32_t degrees_to_use,
                                                               const at::Tensor dirs, const at::Tensor coeffs,
                                                               const at::optional<at::Tensor> masks, const at::Tensor v_colors,
                                                               bool compute_v_dirs);
    std::tuple<at::Tensor, at::Tensor, at::Tensor> intersect_tile(const at::Tensor means2d, const at::Tensor radii,
                                                                  const at::Tensor depths,
                                                                  const at::optional<at::Tensor> camera_ids,
                                                                  const at::optional<at::Tensor> gaussian_ids, const uint32_t C,
                                                                  const uint32_t tile_size, const uint32_t tile_width,
                                                                  const uint32_t tile_height, const bool sort);
    at::Tensor intersect_offset(const at::Tensor isect_ids, const uint32_t C, const uint32_t tile_width,
                                const uint32_t tile_height);
    at::Tensor quats_to_rotmats(const at::Tensor quats);
    std::tuple<at::Tensor, at::Tensor> relocation(at::Tensor opacities, at::Tensor scales, at::Tensor ratios, at::Tensor binoms,
                                                  const int n_max);
    void add_noise(at::Tensor raw_opacities, at::Tensor raw_scales, at::Tensor raw_quats, at::Tensor noise, at::Tensor means,
                   const float current_lr);
    std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> projection_ut_3dgs_fused(
        const at::Tensor means, const at::Tensor quats, const at::Tensor scales, const at::optional<at::Tensor> opacities,
        const at::Tensor viewmats0, const at::optional<at::Tensor> viewmats1, const at::Tensor Ks, const uint32_t image_width,
        const uint32_t image_height, const float eps2d, const float near_plane, const float far_plane, const float radius_clip,
        const bool calc_compensations, const CameraModelType camera_model, const UnscentedTransformParameters ut_params,
        ShutterType rs_type, const at::optional<at::Tensor> radial_coeffs, const at::optional<at::Tensor> tangential_coeffs,
        const at::optional<at::Tensor> thin_prism_coeffs);
    std::tuple<at::Tensor, at::Tensor, at::Tensor> rasterize_to_pixels_from_world_3dgs_fwd(
        const at::Tensor means, const at::Tensor quats, const at::Tensor scales, const at::Tensor colors, const at::Tensor opacities,
        const at::optional<at::Tensor> backgrounds, const at::optional<at::Tensor> masks, const uint32_t image_width,
        const uint32_t image_height, const uint32_t tile_size, const at::Tensor viewmats0, const at::optional<at::Tensor> viewmats1,
        const at::Tensor Ks, const CameraModelType camera_model, const UnscentedTransformParameters ut_params, ShutterType rs_type,
        const at::optional<at::Tensor> radial_coeffs, const at::optional<at::Tensor> tangential_coeffs,
        const at::optional<at::Tensor> thin_prism_coeffs, const at::Tensor tile_offsets, const at::Tensor flatten_ids);
    std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> rasterize_to_pixels_from_world_3dgs_bwd(
        const at::Tensor means, const at::Tensor quats, const at::Tensor scales, const at::Tensor colors, const at::Tensor opacities,
        const at::optional<at::Tensor> backgrounds, const at::optional<at::Tensor> masks, const uint32_t image_width,
        const uint32_t image_height, const uint32_t tile_size, const at::Tensor viewmats0, const at::optional<at::Tensor> viewmats1,
        const at::Tensor Ks, const CameraModelType camera_model, const UnscentedTransformParameters ut_params, ShutterType rs_type,
        const at::optional<at::Tensor> radial_coeffs, const at::optional<at::Tensor> tangential_coeffs,
        const at::optional<at::Tensor> thin_prism_coeffs, const at::Tensor tile_offsets, const at::Tensor flatten_ids,
        const at::Tensor render_alphas, const at::Tensor last_ids, const at::Tensor v_render_colors,
        const at::Tensor v_render_alphas);
    std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor>
    rasterize_from_world_with_sh_fwd(
        const at::Tensor means, const at::Tensor quats, const at::Tensor scales, const at::Tensor opacities, const at::Tensor sh_coeffs,
        const uint32_t sh_degree, const at::optional<at::Tensor> backgrounds, const at::optional<at::Tensor> masks,
        const uint32_t image_width, const uint32_t image_height, const uint32_t tile_size, const at::Tensor viewmats0,
        const at::optional<at::Tensor> viewmats1, const at::Tensor Ks, const CameraModelType camera_model, const float eps2d,
        const float near_plane, const float far_plane, const float radius_clip, const float scaling_modifier,
        const bool calc_compensations, const int render_mode, const UnscentedTransformParameters ut_params, ShutterType rs_type,
        const at::optional<at::Tensor> radial_coeffs, const at::optional<at::Tensor> tangential_coeffs,
        const at::optional<at::Tensor> thin_prism_coeffs);
    std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> rasterize_from_world_with_sh_bwd(
        const at::Tensor means, const at::Tensor quats, const at::Tensor scales, const at::Tensor opacities, const at::Tensor sh_coeffs,
        const uint32_t sh_degree, const at::optional<at::Tensor> backgrounds, const at::optional<at::Tensor> masks,
        const uint32_t image_width, const uint32_t image_height, const uint32_t tile_size, const at::Tensor viewmats0,
        const at::optional<at::Tensor> viewmats1, const at::Tensor Ks, const CameraModelType camera_model, const float eps2d,
        const float near_plane, const float far_plane, const float radius_clip, const float scaling_modifier,
        const bool calc_compensations, const int render_mode, const UnscentedTransformParameters ut_params, ShutterType rs_type,
        const at::optional<at::Tensor> radial_coeffs, const at::optional<at::Tensor> tangential_coeffs,
        const at::optional<at::Tensor> thin_prism_coeffs, const at::Tensor render_alphas, const at::Tensor last_ids,
        const at::Tensor tile_offsets, const at::Tensor flatten_ids, const at::Tensor colors, const at::Tensor radii,
        const at::Tensor means2d, const at::Tensor depths, const at::Tensor compensations, const at::Tensor v_render_colors,
        const at::Tensor v_render_alphas);

} // namespace gsplat
