// namespace gsplat of gsplat/Ops.h:12-270 on top of the lfs_b200 C ABI: C++ host code for libtorch programs.
//
// Each function validates its tensors the way the reference wrapper does (CHECK_INPUT: CUDA + contiguous,
// gsplat/Common.h:12-17), allocates its outputs with ATen on the inputs' device, launches on the current CUDA stream
// and turns a failing C-ABI call into a c10::Error, so that code written against the reference's Ops.h links
// against this translation unit instead of gsplat_backend and behaves the same. The two fused operators
// (rasterize_from_world_with_sh_fwd / _bwd) keep the reference's ATen glue between the operator calls
// (gsplat/Rasterization.cpp:326-466, :527-641).
//
// Differences that a caller can observe: packed mode (camera_ids / gaussian_ids) and compute_v_dirs raise, like the
// features the reference's trainer never requests; the ORTHO camera raises; outputs the reference leaves
// uninitialised for culled Gaussians are left uninitialised here as well.
#ifdef LFS_SHIM_USE_REFERENCE_HEADERS
#include "Ops.h"
#else
#include "lfs_gsplat_ops.h"
#endif

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "lfs_b200.h"

namespace gsplat {

    namespace {

        void check_input(const at::Tensor& t, const char* name, at::ScalarType dtype = at::kFloat) {
            TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
            TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
            TORCH_CHECK(t.scalar_type() == dtype, name, " has the wrong dtype");
        }

        void ok(int rc, const char* what) { TORCH_CHECK(rc == LFS_OK, what, ": ", lfs_last_error()); }

        void* stream() { return at::cuda::getCurrentCUDAStream().stream(); }

        const float* fptr(const at::optional<at::Tensor>& t) {
            return (t.has_value() && t->defined() && t->numel() > 0) ? t->data_ptr<float>() : nullptr;
        }

        lfs_ut_params ut(const UnscentedTransformParameters& p) {
            return lfs_ut_params{p.alpha, p.beta, p.kappa, p.in_image_margin_factor, p.require_all_sigma_points_valid ? 1 : 0};
        }

        at::Tensor workspace(size_t nbytes, const at::Tensor& like) {
            return at::empty({(int64_t)std::max<size_t>(nbytes, 256)}, like.options().dtype(at::kByte));
        }

        // Distortion coefficient tensors in the widths the C ABI reads: pinhole radial [C,6] (the reference kernel reads six
        // floats whatever the tensor holds, gsplat/RasterizeToPixelsFromWorld3DGSFwd.cu:105-107), tangential [C,2], thin
        // prism [C,4]; fisheye radial [C,4]. Narrower tensors are zero-padded.
        struct Coeffs {
            at::Tensor radial, tangential, thin_prism;
            const float *r = nullptr, *t = nullptr, *p = nullptr;
        };
        at::Tensor widen(const at::optional<at::Tensor>& t, int64_t n) {
            if (!t.has_value() || !t->defined() || t->numel() == 0) return at::Tensor();
            check_input(*t, "distortion coefficients");
            auto x = t->reshape({-1, t->size(-1)});
            TORCH_CHECK(x.size(-1) <= n, "at most ", n, " distortion coefficients, got ", x.size(-1));
            if (x.size(-1) == n) return x.contiguous();
            return at::constant_pad_nd(x, {0, n - x.size(-1)}, 0).contiguous();
        }
        Coeffs camera_args(CameraModelType camera_model, ShutterType rs_type, const at::optional<at::Tensor>& viewmats1,
                           const at::optional<at::Tensor>& radial, const at::optional<at::Tensor>& tangential,
                           const at::optional<at::Tensor>& thin_prism) {
            if (viewmats1.has_value() && viewmats1->defined()) check_input(*viewmats1, "viewmats1");
            TORCH_CHECK(camera_model == CameraModelType::PINHOLE || camera_model == CameraModelType::FISHEYE ||
                            camera_model == CameraModelType::EQUIRECTANGULAR,
                        "camera model must be PINHOLE, FISHEYE or EQUIRECTANGULAR");
            Coeffs c;
            if (camera_model == CameraModelType::EQUIRECTANGULAR) {
                TORCH_CHECK(rs_type == ShutterType::GLOBAL && fptr(viewmats1) == nullptr && fptr(radial) == nullptr &&
                                fptr(tangential) == nullptr && fptr(thin_prism) == nullptr,
                            "the equirectangular model has a global shutter and no distortion coefficients");
                return c;
            }
            if (camera_model == CameraModelType::PINHOLE) {
                c.radial = widen(radial, 6);
                c.tangential = widen(tangential, 2);
                c.thin_prism = widen(thin_prism, 4);
            } else {
                TORCH_CHECK(fptr(tangential) == nullptr && fptr(thin_prism) == nullptr,
                            "tangential / thin-prism coefficients belong to the pinhole model");
                c.radial = widen(radial, 4);
            }
            c.r = c.radial.defined() ? c.radial.data_ptr<float>() : nullptr;
            c.t = c.tangential.defined() ? c.tangential.data_ptr<float>() : nullptr;
            c.p = c.thin_prism.defined() ? c.thin_prism.data_ptr<float>() : nullptr;
            return c;
        }

        at::Tensor mask_bytes(const at::optional<at::Tensor>& masks, uint32_t W, uint32_t H, uint32_t tile) {
            if (!masks.has_value() || !masks->defined() || masks->numel() == 0) return at::Tensor();
            const int64_t tw = (W + tile - 1) / tile, th = (H + tile - 1) / tile;
            TORCH_CHECK(masks->is_cuda() && masks->scalar_type() == at::kBool && masks->numel() == tw * th,
                        "masks must be a CUDA bool tensor [1, ", th, ", ", tw, "]");
            return masks->contiguous().view(at::kByte);
        }

    } // namespace

    at::Tensor spherical_harmonics_fwd(const uint32_t degrees_to_use, const at::Tensor dirs, const at::Tensor coeffs,
                                       const at::optional<at::Tensor> masks) {
        const c10::cuda::OptionalCUDAGuard guard(device_of(dirs));
        check_input(dirs, "dirs");
        check_input(coeffs, "coeffs");
        TORCH_CHECK(coeffs.size(-1) == 3 && dirs.size(-1) == 3, "dirs [..., 3], coeffs [..., K, 3]");
        const int64_t K = coeffs.size(-2), n = dirs.numel() / 3;
        // coefficients may be shared by all cameras ([1, N, K, 3] against dirs [C, N, 3])
        at::Tensor cf = coeffs;
        if (coeffs.numel() != n * K * 3) cf = coeffs.expand({dirs.size(0), coeffs.size(-3), K, 3}).contiguous();
        TORCH_CHECK(cf.numel() == n * K * 3, "coeffs do not match dirs");
        at::Tensor m;
        if (masks.has_value() && masks->defined()) {
            TORCH_CHECK(masks->is_cuda() && masks->scalar_type() == at::kBool, "masks must be a CUDA bool tensor");
            m = masks->contiguous().view(at::kByte);
        }
        at::Tensor colors = at::empty_like(dirs);
        ok(lfs_spherical_harmonics_fwd((int)n, (int)K, (int)degrees_to_use, dirs.data_ptr<float>(), cf.data_ptr<float>(),
                                       m.defined() ? m.data_ptr<uint8_t>() : nullptr, colors.data_ptr<float>(), stream()),
           "spherical_harmonics_fwd");
        return colors;
    }

    std::tuple<at::Tensor, at::Tensor> spherical_harmonics_bwd(const uint32_t K, const uint32_t degrees_to_use, const at::Tensor dirs,
                                                               const at::Tensor coeffs, const at::optional<at::Tensor> masks,
                                                               const at::Tensor v_colors, bool compute_v_dirs) {
        const c10::cuda::OptionalCUDAGuard guard(device_of(dirs));
        TORCH_CHECK(!compute_v_dirs, "compute_v_dirs is not supported (the training path never requests it)");
        check_input(dirs, "dirs");
        check_input(v_colors, "v_colors");
        (void)coeffs;
        const int64_t n = dirs.numel() / 3;
        at::Tensor m;
        if (masks.has_value() && masks->defined()) m = masks->contiguous().view(at::kByte);
        auto shape = dirs.sizes().vec();
        shape.back() = K;
        shape.push_back(3);
        at::Tensor v_coeffs = at::empty(shape, dirs.options());
        ok(lfs_spherical_harmonics_bwd((int)n, (int)K, (int)degrees_to_use, dirs.data_ptr<float>(),
                                       m.defined() ? m.data_ptr<uint8_t>() : nullptr, v_colors.data_ptr<float>(),
                                       v_coeffs.data_ptr<float>(), stream()),
           "spherical_harmonics_bwd");
        return std::make_tuple(v_coeffs, at::Tensor());
    }

    std::tuple<at::Tensor, at::Tensor, at::Tensor> intersect_tile(const at::Tensor means2d, const at::Tensor radii, const at::Tensor depths,
                                                                  const at::optional<at::Tensor> camera_ids,
                                                                  const at::optional<at::Tensor> gaussian_ids, const uint32_t C,
                                                                  const uint32_t tile_size, const uint32_t tile_width,
                                                                  const uint32_t tile_height, const bool sort) {
        const c10::cuda::OptionalCUDAGuard guard(device_of(means2d));
        check_input(means2d, "means2d");
        check_input(radii, "radii", at::kInt);
        check_input(depths, "depths");
        TORCH_CHECK(!camera_ids.has_value() && !gaussian_ids.has_value() && means2d.dim() == 3, "packed mode is not supported");
        const int64_t N = means2d.size(1);
        at::Tensor tiles_per_gauss = at::empty_like(depths, depths.options().dtype(at::kInt));
        at::Tensor n_dev = at::zeros({1}, depths.options().dtype(at::kLong));
        ok(lfs_intersect_tile_count((int)C, (int)N, means2d.data_ptr<float>(), radii.data_ptr<int32_t>(), (int)tile_size, (int)tile_width,
                                    (int)tile_height, tiles_per_gauss.data_ptr<int32_t>(), n_dev.data_ptr<int64_t>(), stream()),
           "intersect_tile (count)");
        const int64_t n_isects = n_dev.item<int64_t>();   // the same host read as gsplat/Intersect.cpp:76
        at::Tensor isect_ids = at::empty({n_isects}, depths.options().dtype(at::kLong));
        at::Tensor flatten_ids = at::empty({n_isects}, depths.options().dtype(at::kInt));
        if (n_isects > 0) {
            at::Tensor ws = workspace(lfs_intersect_tile_workspace_bytes((int)C, (int)N, n_isects), depths);
            ok(lfs_intersect_tile_emit((int)C, (int)N, means2d.data_ptr<float>(), radii.data_ptr<int32_t>(), depths.data_ptr<float>(),
                                       tiles_per_gauss.data_ptr<int32_t>(), (int)tile_size, (int)tile_width, (int)tile_height, sort ? 1 : 0,
                                       n_isects, isect_ids.data_ptr<int64_t>(), flatten_ids.data_ptr<int32_t>(), ws.data_ptr(),
                                       (size_t)ws.numel(), stream()),
               "intersect_tile (emit)");
        }
        return std::make_tuple(tiles_per_gauss, isect_ids, flatten_ids);
    }

    at::Tensor intersect_offset(const at::Tensor isect_ids, const uint32_t C, const uint32_t tile_width, const uint32_t tile_height) {
        const c10::cuda::OptionalCUDAGuard guard(device_of(isect_ids));
        check_input(isect_ids, "isect_ids", at::kLong);
        at::Tensor offsets = at::empty({(int64_t)C, (int64_t)tile_height, (int64_t)tile_width}, isect_ids.options().dtype(at::kInt));
        ok(lfs_intersect_offset(isect_ids.numel(), isect_ids.data_ptr<int64_t>(), (int)C, (int)tile_width, (int)tile_height,
                                offsets.data_ptr<int32_t>(), stream()),
           "intersect_offset");
        return offsets;
    }

    at::Tensor quats_to_rotmats(const at::Tensor quats) {
        const c10::cuda::OptionalCUDAGuard guard(device_of(quats));
        check_input(quats, "quats");
        at::Tensor out = at::empty({quats.size(0), 3, 3}, quats.options());
        ok(lfs_quats_to_rotmats((int)quats.size(0), quats.data_ptr<float>(), out.data_ptr<float>(), stream()), "quats_to_rotmats");
        return out;
    }

    std::tuple<at::Tensor, at::Tensor> relocation(at::Tensor opacities, at::Tensor scales, at::Tensor ratios, at::Tensor binoms,
                                                  const int n_max) {
        const c10::cuda::OptionalCUDAGuard guard(device_of(opacities));
        check_input(opacities, "opacities");
        check_input(scales, "scales");
        check_input(ratios, "ratios", at::kInt);
        check_input(binoms, "binoms");
        at::Tensor new_opacities = at::empty_like(opacities), new_scales = at::empty_like(scales);
        ok(lfs_relocation((int)opacities.size(0), opacities.data_ptr<float>(), scales.data_ptr<float>(), ratios.data_ptr<int32_t>(),
                          binoms.data_ptr<float>(), n_max, new_opacities.data_ptr<float>(), new_scales.data_ptr<float>(), stream()),
           "relocation");
        return std::make_tuple(new_opacities, new_scales);
    }

    void add_noise(at::Tensor raw_opacities, at::Tensor raw_scales, at::Tensor raw_quats, at::Tensor noise, at::Tensor means,
                   const float current_lr) {
        const c10::cuda::OptionalCUDAGuard guard(device_of(means));
        check_input(raw_opacities, "raw_opacities");
        check_input(raw_scales, "raw_scales");
        check_input(raw_quats, "raw_quats");
        check_input(noise, "noise");
        check_input(means, "means");
        ok(lfs_add_noise((int)means.size(0), raw_opacities.data_ptr<float>(), raw_scales.data_ptr<float>(), raw_quats.data_ptr<float>(),
                         noise.data_ptr<float>(), means.data_ptr<float>(), current_lr, stream()),
           "add_noise");
    }

    std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> projection_ut_3dgs_fused(
        const at::Tensor means, const at::Tensor quats, const at::Tensor scales, const at::optional<at::Tensor> opacities,
        const at::Tensor viewmats0, const at::optional<at::Tensor> viewmats1, const at::Tensor Ks, const uint32_t image_width,
        const uint32_t image_height, const float eps2d, const float near_plane, const float far_plane, const float radius_clip,
        const bool calc_compensations, const CameraModelType camera_model, const UnscentedTransformParameters ut_params,
        ShutterType rs_type, const at::optional<at::Tensor> radial_coeffs, const at::optional<at::Tensor> tangential_coeffs,
        const at::optional<at::Tensor> thin_prism_coeffs) {
        const c10::cuda::OptionalCUDAGuard guard(device_of(means));
        check_input(means, "means");
        check_input(quats, "quats");
        check_input(scales, "scales");
        check_input(viewmats0, "viewmats0");
        check_input(Ks, "Ks");
        if (opacities.has_value() && opacities->defined()) check_input(*opacities, "opacities");
        const Coeffs co = camera_args(camera_model, rs_type, viewmats1, radial_coeffs, tangential_coeffs, thin_prism_coeffs);
        const int64_t N = means.size(0), C = viewmats0.size(0);
        auto opt = means.options();
        at::Tensor radii = at::empty({C, N, 2}, opt.dtype(at::kInt));
        at::Tensor means2d = at::empty({C, N, 2}, opt), depths = at::empty({C, N}, opt), conics = at::empty({C, N, 3}, opt);
        at::Tensor compensations;
        if (calc_compensations) compensations = at::zeros({C, N}, opt);
        ok(lfs_projection_ut_3dgs_fused((int)C, (int)N, means.data_ptr<float>(), quats.data_ptr<float>(), scales.data_ptr<float>(),
                                        fptr(opacities), viewmats0.data_ptr<float>(), fptr(viewmats1), Ks.data_ptr<float>(),
                                        (int)image_width, (int)image_height, eps2d, near_plane, far_plane, radius_clip, (int)camera_model,
                                        ut(ut_params), (int)rs_type, co.r, co.t, co.p, radii.data_ptr<int32_t>(), means2d.data_ptr<float>(),
                                        depths.data_ptr<float>(), conics.data_ptr<float>(),
                                        compensations.defined() ? compensations.data_ptr<float>() : nullptr, stream()),
           "projection_ut_3dgs_fused");
        return std::make_tuple(radii, means2d, depths, conics, compensations);
    }

    std::tuple<at::Tensor, at::Tensor, at::Tensor> rasterize_to_pixels_from_world_3dgs_fwd(
        const at::Tensor means, const at::Tensor quats, const at::Tensor scales, const at::Tensor colors, const at::Tensor opacities,
        const at::optional<at::Tensor> backgrounds, const at::optional<at::Tensor> masks, const uint32_t image_width,
        const uint32_t image_height, const uint32_t tile_size, const at::Tensor viewmats0, const at::optional<at::Tensor> viewmats1,
        const at::Tensor Ks, const CameraModelType camera_model, const UnscentedTransformParameters ut_params, ShutterType rs_type,
        const at::optional<at::Tensor> radial_coeffs, const at::optional<at::Tensor> tangential_coeffs,
        const at::optional<at::Tensor> thin_prism_coeffs, const at::Tensor tile_offsets, const at::Tensor flatten_ids) {
        const c10::cuda::OptionalCUDAGuard guard(device_of(means));
        (void)ut_params;
        check_input(means, "means");
        check_input(quats, "quats");
        check_input(scales, "scales");
        check_input(colors, "colors");
        check_input(opacities, "opacities");
        check_input(viewmats0, "viewmats0");
        check_input(Ks, "Ks");
        check_input(tile_offsets, "tile_offsets", at::kInt);
        check_input(flatten_ids, "flatten_ids", at::kInt);
        const Coeffs co = camera_args(camera_model, rs_type, viewmats1, radial_coeffs, tangential_coeffs, thin_prism_coeffs);
        const int64_t CH = colors.size(-1);
        TORCH_CHECK(CH == 1 || CH == 3 || CH == 4, "Unsupported number of channels: ", CH);
        // the reference kernels index means[g] with the flattened [C*N] id and are only correct for one camera
        TORCH_CHECK(viewmats0.size(0) == 1 && tile_offsets.size(0) == 1, "only one camera per rasterize call is supported");
        TORCH_CHECK(opacities.dim() == 2, "packed mode is not supported");
        at::Tensor mb = mask_bytes(masks, image_width, image_height, tile_size);
        const int64_t N = means.size(0), H = image_height, W = image_width;
        auto opt = means.options();
        at::Tensor renders = at::empty({1, H, W, CH}, opt), alphas = at::empty({1, H, W, 1}, opt);
        at::Tensor last_ids = at::empty({1, H, W}, opt.dtype(at::kInt));
        const float* bg = fptr(backgrounds);
        if (bg) TORCH_CHECK(backgrounds->numel() >= CH, "backgrounds must have ", CH, " channels");
        at::Tensor ws = workspace(lfs_rasterize_workspace_bytes((int)N), means);
        ok(lfs_rasterize_to_pixels_from_world_3dgs_fwd(
               (int)N, flatten_ids.numel(), (int)CH, means.data_ptr<float>(), quats.data_ptr<float>(), scales.data_ptr<float>(),
               colors.data_ptr<float>(), opacities.data_ptr<float>(), bg, mb.defined() ? mb.data_ptr<uint8_t>() : nullptr, (int)W, (int)H,
               (int)tile_size, viewmats0.data_ptr<float>(), fptr(viewmats1), Ks.data_ptr<float>(), (int)camera_model, (int)rs_type, co.r, co.t,
               co.p, tile_offsets.data_ptr<int32_t>(), flatten_ids.data_ptr<int32_t>(), renders.data_ptr<float>(), alphas.data_ptr<float>(),
               last_ids.data_ptr<int32_t>(), ws.data_ptr(), (size_t)ws.numel(), stream()),
           "rasterize_to_pixels_from_world_3dgs_fwd");
        return std::make_tuple(renders, alphas, last_ids);
    }

    std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> rasterize_to_pixels_from_world_3dgs_bwd(
        const at::Tensor means, const at::Tensor quats, const at::Tensor scales, const at::Tensor colors, const at::Tensor opacities,
        const at::optional<at::Tensor> backgrounds, const at::optional<at::Tensor> masks, const uint32_t image_width,
        const uint32_t image_height, const uint32_t tile_size, const at::Tensor viewmats0, const at::optional<at::Tensor> viewmats1,
        const at::Tensor Ks, const CameraModelType camera_model, const UnscentedTransformParameters ut_params, ShutterType rs_type,
        const at::optional<at::Tensor> radial_coeffs, const at::optional<at::Tensor> tangential_coeffs,
        const at::optional<at::Tensor> thin_prism_coeffs, const at::Tensor tile_offsets, const at::Tensor flatten_ids,
        const at::Tensor render_alphas, const at::Tensor last_ids, const at::Tensor v_render_colors, const at::Tensor v_render_alphas) {
        const c10::cuda::OptionalCUDAGuard guard(device_of(means));
        (void)ut_params;
        check_input(means, "means");
        check_input(quats, "quats");
        check_input(scales, "scales");
        check_input(colors, "colors");
        check_input(opacities, "opacities");
        check_input(render_alphas, "render_alphas");
        check_input(last_ids, "last_ids", at::kInt);
        check_input(v_render_colors, "v_render_colors");
        check_input(v_render_alphas, "v_render_alphas");
        check_input(tile_offsets, "tile_offsets", at::kInt);
        check_input(flatten_ids, "flatten_ids", at::kInt);
        const Coeffs co = camera_args(camera_model, rs_type, viewmats1, radial_coeffs, tangential_coeffs, thin_prism_coeffs);
        const int64_t CH = colors.size(-1);
        TORCH_CHECK(CH == 1 || CH == 3 || CH == 4, "Unsupported number of channels: ", CH);
        TORCH_CHECK(viewmats0.size(0) == 1 && tile_offsets.size(0) == 1, "only one camera per rasterize call is supported");
        TORCH_CHECK(opacities.dim() == 2, "packed mode is not supported");
        at::Tensor mb = mask_bytes(masks, image_width, image_height, tile_size);
        const int64_t N = means.size(0);
        at::Tensor v_means = at::empty_like(means), v_quats = at::empty_like(quats), v_scales = at::empty_like(scales);
        at::Tensor v_colors = at::empty_like(colors), v_opacities = at::empty_like(opacities);
        at::Tensor ws = workspace(lfs_rasterize_workspace_bytes((int)N), means);
        ok(lfs_rasterize_to_pixels_from_world_3dgs_bwd(
               (int)N, flatten_ids.numel(), (int)CH, means.data_ptr<float>(), quats.data_ptr<float>(), scales.data_ptr<float>(),
               colors.data_ptr<float>(), opacities.data_ptr<float>(), fptr(backgrounds), mb.defined() ? mb.data_ptr<uint8_t>() : nullptr,
               (int)image_width, (int)image_height, (int)tile_size, viewmats0.data_ptr<float>(), fptr(viewmats1), Ks.data_ptr<float>(),
               (int)camera_model, (int)rs_type, co.r, co.t, co.p, tile_offsets.data_ptr<int32_t>(), flatten_ids.data_ptr<int32_t>(),
               render_alphas.data_ptr<float>(), last_ids.data_ptr<int32_t>(), v_render_colors.data_ptr<float>(),
               v_render_alphas.data_ptr<float>(), v_means.data_ptr<float>(), v_quats.data_ptr<float>(), v_scales.data_ptr<float>(),
               v_colors.data_ptr<float>(), v_opacities.data_ptr<float>(), ws.data_ptr(), (size_t)ws.numel(), stream()),
           "rasterize_to_pixels_from_world_3dgs_bwd");
        return std::make_tuple(v_means, v_quats, v_scales, v_colors, v_opacities);
    }

    std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor>
    rasterize_from_world_with_sh_fwd(
        const at::Tensor means, const at::Tensor quats, const at::Tensor scales, const at::Tensor opacities_in, const at::Tensor sh_coeffs,
        const uint32_t sh_degree, const at::optional<at::Tensor> backgrounds, const at::optional<at::Tensor> masks,
        const uint32_t image_width, const uint32_t image_height, const uint32_t tile_size, const at::Tensor viewmats0,
        const at::optional<at::Tensor> viewmats1, const at::Tensor Ks, const CameraModelType camera_model, const float eps2d,
        const float near_plane, const float far_plane, const float radius_clip, const float scaling_modifier,
        const bool calc_compensations, const int render_mode, const UnscentedTransformParameters ut_params, ShutterType rs_type,
        const at::optional<at::Tensor> radial_coeffs, const at::optional<at::Tensor> tangential_coeffs,
        const at::optional<at::Tensor> thin_prism_coeffs) {
        const c10::cuda::OptionalCUDAGuard guard(device_of(means));
        TORCH_CHECK(render_mode >= 0 && render_mode <= 4, "render_mode must be 0=RGB, 1=D, 2=ED, 3=RGB_D or 4=RGB_ED");
        check_input(sh_coeffs, "sh_coeffs");
        at::Tensor opacities = (opacities_in.dim() == 2 && opacities_in.size(1) == 1) ? opacities_in.squeeze(-1) : opacities_in;
        const uint32_t C = viewmats0.size(0);
        // gsplat/Rasterization.cpp:326-349
        auto scaled_scales = scales * scaling_modifier;
        auto proj = projection_ut_3dgs_fused(means, quats, scaled_scales, opacities, viewmats0, viewmats1, Ks, image_width, image_height, eps2d,
                                             near_plane, far_plane, radius_clip, calc_compensations, camera_model, ut_params, rs_type,
                                             radial_coeffs, tangential_coeffs, thin_prism_coeffs);
        auto radii = std::get<0>(proj), means2d = std::get<1>(proj), depths = std::get<2>(proj), compensations = std::get<4>(proj);
        // :358-393
        auto viewmat_inv = at::inverse(viewmats0);
        auto campos = viewmat_inv.index({"...", at::indexing::Slice(at::indexing::None, 3), 3});
        auto dirs = (means.unsqueeze(0) - campos.unsqueeze(1)).contiguous();
        auto radii_masks = (radii > 0).all(-1);
        auto shs = sh_coeffs.unsqueeze(0);
        at::Tensor colors;
        if (render_mode == 0 || render_mode == 3 || render_mode == 4) {
            auto rgb = spherical_harmonics_fwd(sh_degree, dirs, shs, radii_masks);
            rgb = at::clamp_min(rgb + 0.5f, 0.0f);
            colors = render_mode == 0 ? rgb : at::cat({rgb, depths.unsqueeze(-1)}, -1);
        } else {
            colors = depths.unsqueeze(-1);
        }
        colors = colors.contiguous();
        // :396-407
        auto final_opacities = opacities.unsqueeze(0);
        if (calc_compensations && compensations.defined() && compensations.numel() > 0) final_opacities = final_opacities * compensations;
        at::Tensor final_bg;
        if (backgrounds.has_value() && backgrounds->defined() && backgrounds->numel() > 0) final_bg = backgrounds.value();
        else final_bg = at::empty({0}, means.options().dtype(at::kFloat));
        // :409-424
        const uint32_t tile_width = (image_width + tile_size - 1) / tile_size, tile_height = (image_height + tile_size - 1) / tile_size;
        auto isect = intersect_tile(means2d, radii, depths, at::nullopt, at::nullopt, C, tile_size, tile_width, tile_height, true);
        auto flatten_ids = std::get<2>(isect);
        auto isect_offsets = intersect_offset(std::get<1>(isect), C, tile_width, tile_height).reshape({C, tile_height, tile_width});
        // :426-452
        auto raster = rasterize_to_pixels_from_world_3dgs_fwd(means, quats, scaled_scales, colors, final_opacities.contiguous(), final_bg, masks,
                                                              image_width, image_height, tile_size, viewmats0, viewmats1, Ks, camera_model,
                                                              ut_params, rs_type, radial_coeffs, tangential_coeffs, thin_prism_coeffs,
                                                              isect_offsets, flatten_ids);
        return std::make_tuple(std::get<0>(raster), std::get<1>(raster), radii, means2d, depths, colors, isect_offsets, flatten_ids,
                               std::get<2>(raster), compensations);
    }

    std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> rasterize_from_world_with_sh_bwd(
        const at::Tensor means, const at::Tensor quats, const at::Tensor scales, const at::Tensor opacities_in, const at::Tensor sh_coeffs,
        const uint32_t sh_degree, const at::optional<at::Tensor> backgrounds, const at::optional<at::Tensor> masks,
        const uint32_t image_width, const uint32_t image_height, const uint32_t tile_size, const at::Tensor viewmats0,
        const at::optional<at::Tensor> viewmats1, const at::Tensor Ks, const CameraModelType camera_model, const float eps2d,
        const float near_plane, const float far_plane, const float radius_clip, const float scaling_modifier,
        const bool calc_compensations, const int render_mode, const UnscentedTransformParameters ut_params, ShutterType rs_type,
        const at::optional<at::Tensor> radial_coeffs, const at::optional<at::Tensor> tangential_coeffs,
        const at::optional<at::Tensor> thin_prism_coeffs, const at::Tensor render_alphas, const at::Tensor last_ids,
        const at::Tensor tile_offsets, const at::Tensor flatten_ids, const at::Tensor colors, const at::Tensor radii,
        const at::Tensor means2d, const at::Tensor depths, const at::Tensor compensations, const at::Tensor v_render_colors,
        const at::Tensor v_render_alphas) {
        const c10::cuda::OptionalCUDAGuard guard(device_of(means));
        (void)eps2d; (void)near_plane; (void)far_plane; (void)radius_clip; (void)means2d; (void)depths;
        at::Tensor opacities = (opacities_in.dim() == 2 && opacities_in.size(1) == 1) ? opacities_in.squeeze(-1) : opacities_in;
        // gsplat/Rasterization.cpp:527-541
        at::Tensor final_bg;
        if (backgrounds.has_value() && backgrounds->defined() && backgrounds->numel() > 0) final_bg = backgrounds.value();
        else final_bg = at::empty({0}, means.options().dtype(at::kFloat));
        auto final_opacities = opacities.unsqueeze(0);
        if (calc_compensations && compensations.defined() && compensations.numel() > 0) final_opacities = final_opacities * compensations;
        auto scaled_scales = scales * scaling_modifier;
        // :543-575
        auto g = rasterize_to_pixels_from_world_3dgs_bwd(means, quats, scaled_scales, colors, final_opacities.contiguous(), final_bg, masks,
                                                         image_width, image_height, tile_size, viewmats0, viewmats1, Ks, camera_model, ut_params,
                                                         rs_type, radial_coeffs, tangential_coeffs, thin_prism_coeffs, tile_offsets, flatten_ids,
                                                         render_alphas, last_ids, v_render_colors, v_render_alphas);
        auto v_colors = std::get<3>(g);
        // :577-630 (the depth channel's per-Gaussian gradient is dropped, as in the reference)
        at::Tensor v_sh_coeffs;
        if (render_mode == 0 || render_mode == 3 || render_mode == 4) {
            const auto rgb_slice = at::indexing::Slice(at::indexing::None, 3);
            at::Tensor v_rgb = render_mode == 0 ? v_colors : v_colors.index({"...", rgb_slice});
            at::Tensor rgb = render_mode == 0 ? colors : colors.index({"...", rgb_slice});
            auto viewmat_inv = at::inverse(viewmats0);
            auto campos = viewmat_inv.index({"...", at::indexing::Slice(at::indexing::None, 3), 3});
            auto dirs = (means.unsqueeze(0) - campos.unsqueeze(1)).contiguous();
            auto radii_masks = (radii > 0).all(-1);
            auto shs = sh_coeffs.unsqueeze(0);
            auto v_pre = v_rgb.clone();
            v_pre.masked_fill_(rgb <= 0.0f, 0.0f);
            const uint32_t K = sh_coeffs.size(1);
            auto sh_grads = spherical_harmonics_bwd(K, sh_degree, dirs.reshape({-1, 3}), shs.reshape({-1, (int64_t)K, 3}),
                                                    radii_masks.reshape({-1}), v_pre.reshape({-1, 3}).contiguous(), false);
            v_sh_coeffs = std::get<0>(sh_grads).reshape({(int64_t)viewmats0.size(0), -1, (int64_t)K, 3}).sum(0);
        } else {
            v_sh_coeffs = at::zeros({means.size(0), sh_coeffs.size(1), 3}, sh_coeffs.options());
        }
        // :633
        return std::make_tuple(std::get<0>(g), std::get<1>(g), std::get<2>(g) * scaling_modifier, std::get<4>(g), v_sh_coeffs);
    }

} // namespace gsplat
