"""Host-side mirror of the reference operator API (namespace gsplat, gsplat/Ops.h:12-270) over the
C ABI: same function names, argument order and meaning, outputs allocated by the callee on the
input's device, `RuntimeError` where the reference raises through TORCH_CHECK
(gsplat/Common.h:12-17). torch is used for device memory and the current stream only."""
from __future__ import annotations

import torch

from . import _capi as capi
from ._capi import UTParams, call, ptr

CameraModelType = type("CameraModelType", (), dict(PINHOLE=0, ORTHO=1, FISHEYE=2, EQUIRECTANGULAR=3))
ShutterType = type("ShutterType", (), dict(ROLLING_TOP_TO_BOTTOM=0, ROLLING_LEFT_TO_RIGHT=1, ROLLING_BOTTOM_TO_TOP=2,
                                           ROLLING_RIGHT_TO_LEFT=3, GLOBAL=4))
UnscentedTransformParameters = UTParams


def _stream():
    return capi.vp(torch.cuda.current_stream().cuda_stream)


def _check_input(t, name, dtype=torch.float32):
    """CHECK_INPUT of gsplat/Common.h:12-17."""
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}")


def _ws(nbytes, device):
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def _only_global_pinhole_fisheye(camera_model, rs_type, viewmats1, tangential_coeffs, thin_prism_coeffs, radial_coeffs):
    """Checks the camera arguments and returns the three coefficient tensors in the widths the C ABI reads:
    pinhole radial [C,6] (zero-padded: the reference kernel reads six floats whatever the tensor holds), tangential
    [C,2], thin prism [C,4]; fisheye radial [C,4]."""
    if int(rs_type) not in (0, 1, 2, 3, 4):
        raise RuntimeError("rs_type must be a ShutterType")
    if viewmats1 is not None:
        _check_input(viewmats1, "viewmats1")
    if camera_model not in (CameraModelType.PINHOLE, CameraModelType.FISHEYE, CameraModelType.EQUIRECTANGULAR):
        raise RuntimeError("camera model must be PINHOLE, FISHEYE or EQUIRECTANGULAR")
    if camera_model == CameraModelType.EQUIRECTANGULAR:
        if int(rs_type) != 4 or viewmats1 is not None or radial_coeffs is not None or tangential_coeffs is not None or thin_prism_coeffs is not None:
            raise RuntimeError("the equirectangular model has a global shutter and no distortion coefficients")
        return None, None, None
    if camera_model == CameraModelType.FISHEYE and (tangential_coeffs is not None or thin_prism_coeffs is not None):
        raise RuntimeError("tangential / thin-prism coefficients belong to the pinhole model")

    def widen(t, n):
        if t is None:
            return None
        _check_input(t, "distortion coefficients")
        t = t.reshape(-1, t.shape[-1])
        if t.shape[-1] > n:
            raise RuntimeError(f"at most {n} coefficients, got {t.shape[-1]}")
        return t if t.shape[-1] == n else torch.nn.functional.pad(t, (0, n - t.shape[-1])).contiguous()

    if camera_model == CameraModelType.PINHOLE:
        return widen(radial_coeffs, 6), widen(tangential_coeffs, 2), widen(thin_prism_coeffs, 4)
    return widen(radial_coeffs, 4), None, None


# gsplat/Ops.h:12-17
def spherical_harmonics_fwd(degrees_to_use, dirs, coeffs, masks=None):
    _check_input(dirs, "dirs"); _check_input(coeffs, "coeffs")
    if masks is not None:
        _check_input(masks, "masks", None)
    K = coeffs.shape[-2]
    n = dirs.numel() // 3
    if coeffs.numel() != n * K * 3:
        raise RuntimeError("coeffs must have shape [..., K, 3] matching dirs")
    colors = torch.empty_like(dirs)
    m = None if masks is None else masks.reshape(-1).to(torch.uint8)
    call("lfs_spherical_harmonics_fwd", n, K, int(degrees_to_use), ptr(dirs), ptr(coeffs), ptr(m), ptr(colors), _stream())
    return colors


# gsplat/Ops.h:18-25
def spherical_harmonics_bwd(K, degrees_to_use, dirs, coeffs, masks, v_colors, compute_v_dirs=False):
    if compute_v_dirs:
        raise RuntimeError("compute_v_dirs is not supported (the training path never requests it)")
    _check_input(dirs, "dirs"); _check_input(v_colors, "v_colors")
    n = dirs.numel() // 3
    v_coeffs = torch.empty(tuple(dirs.shape[:-1]) + (K, 3), dtype=torch.float32, device=dirs.device)
    m = None if masks is None else masks.reshape(-1).to(torch.uint8)
    call("lfs_spherical_harmonics_bwd", n, int(K), int(degrees_to_use), ptr(dirs), ptr(m), ptr(v_colors), ptr(v_coeffs), _stream())
    return v_coeffs, None


# gsplat/Ops.h:28-38
def intersect_tile(means2d, radii, depths, camera_ids, gaussian_ids, C, tile_size, tile_width, tile_height, sort=True):
    _check_input(means2d, "means2d"); _check_input(radii, "radii", torch.int32); _check_input(depths, "depths")
    if means2d.dim() == 2:
        raise RuntimeError("packed mode is not supported")
    N = means2d.numel() // 2 // max(C, 1)
    dev = means2d.device
    tiles_per_gauss = torch.empty(depths.shape, dtype=torch.int32, device=dev)
    n_dev = torch.zeros(1, dtype=torch.int64, device=dev)
    call("lfs_intersect_tile_count", C, N, ptr(means2d), ptr(radii), tile_size, tile_width, tile_height,
         ptr(tiles_per_gauss), ptr(n_dev), _stream())
    n_isects = int(n_dev.item())  # the same host read as gsplat/Intersect.cpp:76
    isect_ids = torch.empty(n_isects, dtype=torch.int64, device=dev)
    flatten_ids = torch.empty(n_isects, dtype=torch.int32, device=dev)
    if n_isects:
        nbytes = capi.lib().lfs_intersect_tile_workspace_bytes(C, N, n_isects)
        ws = _ws(nbytes, dev)
        call("lfs_intersect_tile_emit", C, N, ptr(means2d), ptr(radii), ptr(depths), ptr(tiles_per_gauss), tile_size,
             tile_width, tile_height, 1 if sort else 0, n_isects, ptr(isect_ids), ptr(flatten_ids), ptr(ws), ws.numel(), _stream())
    return tiles_per_gauss, isect_ids, flatten_ids


# gsplat/Ops.h:39-43
def intersect_offset(isect_ids, C, tile_width, tile_height):
    _check_input(isect_ids, "isect_ids", torch.int64)
    offsets = torch.empty((C, tile_height, tile_width), dtype=torch.int32, device=isect_ids.device)
    call("lfs_intersect_offset", isect_ids.numel(), ptr(isect_ids), C, tile_width, tile_height, ptr(offsets), _stream())
    return offsets


# gsplat/Ops.h:45-48
def quats_to_rotmats(quats):
    _check_input(quats, "quats")
    out = torch.empty((quats.shape[0], 3, 3), dtype=torch.float32, device=quats.device)
    call("lfs_quats_to_rotmats", quats.shape[0], ptr(quats), ptr(out), _stream())
    return out


# gsplat/Ops.h:50-57
def relocation(opacities, scales, ratios, binoms, n_max):
    for t, n in ((opacities, "opacities"), (scales, "scales"), (binoms, "binoms")):
        _check_input(t, n)
    _check_input(ratios, "ratios", torch.int32)
    new_opacities = torch.empty_like(opacities)
    new_scales = torch.empty_like(scales)
    call("lfs_relocation", opacities.shape[0], ptr(opacities), ptr(scales), ptr(ratios), ptr(binoms), int(n_max),
         ptr(new_opacities), ptr(new_scales), _stream())
    return new_opacities, new_scales


# gsplat/Ops.h:59-65 (in place on means)
def add_noise(raw_opacities, raw_scales, raw_quats, noise, means, current_lr):
    for t, n in ((raw_opacities, "raw_opacities"), (raw_scales, "raw_scales"), (raw_quats, "raw_quats"),
                 (noise, "noise"), (means, "means")):
        _check_input(t, n)
    call("lfs_add_noise", means.shape[0], ptr(raw_opacities), ptr(raw_scales), ptr(raw_quats), ptr(noise), ptr(means),
         float(current_lr), _stream())


# gsplat/Ops.h:67-95
def projection_ut_3dgs_fused(means, quats, scales, opacities, viewmats0, viewmats1, Ks, image_width, image_height, eps2d,
                             near_plane, far_plane, radius_clip, calc_compensations, camera_model,
                             ut_params=None, rs_type=ShutterType.GLOBAL, radial_coeffs=None, tangential_coeffs=None,
                             thin_prism_coeffs=None):
    for t, n in ((means, "means"), (quats, "quats"), (scales, "scales"), (viewmats0, "viewmats0"), (Ks, "Ks")):
        _check_input(t, n)
    if opacities is not None:
        _check_input(opacities, "opacities")
    radial_coeffs, tangential_coeffs, thin_prism_coeffs = _only_global_pinhole_fisheye(
        camera_model, rs_type, viewmats1, tangential_coeffs, thin_prism_coeffs, radial_coeffs)
    ut = ut_params or UTParams()
    N, Cn, dev = means.shape[0], viewmats0.shape[0], means.device
    radii = torch.empty((Cn, N, 2), dtype=torch.int32, device=dev)
    means2d = torch.empty((Cn, N, 2), dtype=torch.float32, device=dev)
    depths = torch.empty((Cn, N), dtype=torch.float32, device=dev)
    conics = torch.empty((Cn, N, 3), dtype=torch.float32, device=dev)
    comps = torch.zeros((Cn, N), dtype=torch.float32, device=dev) if calc_compensations else None
    call("lfs_projection_ut_3dgs_fused", Cn, N, ptr(means), ptr(quats), ptr(scales), ptr(opacities), ptr(viewmats0), ptr(viewmats1),
         ptr(Ks), int(image_width), int(image_height), float(eps2d), float(near_plane), float(far_plane), float(radius_clip),
         int(camera_model), ut, int(rs_type), ptr(radial_coeffs), ptr(tangential_coeffs), ptr(thin_prism_coeffs), ptr(radii), ptr(means2d), ptr(depths), ptr(conics), ptr(comps), _stream())
    return radii, means2d, depths, conics, comps


def _one_camera(viewmats0, Ks, tile_offsets, opacities):
    if viewmats0.shape[0] != 1 or tile_offsets.shape[0] != 1:
        # the reference kernels index means[g] with the flattened [C*N] id and are only correct for C = 1
        raise RuntimeError("only one camera per rasterize call is supported")
    if opacities.dim() == 1:
        raise RuntimeError("packed mode is not supported")


def _tile_masks(masks, image_width, image_height, tile_size):
    """[C, tile_h, tile_w] bool -> contiguous uint8 view (the C ABI takes bytes)."""
    if masks is None:
        return None
    tw, th = (int(image_width) + tile_size - 1) // tile_size, (int(image_height) + tile_size - 1) // tile_size
    if masks.numel() != tw * th or masks.dtype != torch.bool or not masks.is_cuda:
        raise RuntimeError(f"masks must be a CUDA bool tensor [1, {th}, {tw}]")
    return masks.contiguous().view(torch.uint8)


# gsplat/Ops.h:97-125
def rasterize_to_pixels_from_world_3dgs_fwd(means, quats, scales, colors, opacities, backgrounds, masks, image_width,
                                            image_height, tile_size, viewmats0, viewmats1, Ks, camera_model,
                                            ut_params=None, rs_type=ShutterType.GLOBAL, radial_coeffs=None,
                                            tangential_coeffs=None, thin_prism_coeffs=None, tile_offsets=None,
                                            flatten_ids=None):
    for t, n in ((means, "means"), (quats, "quats"), (scales, "scales"), (colors, "colors"), (opacities, "opacities"),
                 (viewmats0, "viewmats0"), (Ks, "Ks")):
        _check_input(t, n)
    _check_input(tile_offsets, "tile_offsets", torch.int32); _check_input(flatten_ids, "flatten_ids", torch.int32)
    radial_coeffs, tangential_coeffs, thin_prism_coeffs = _only_global_pinhole_fisheye(
        camera_model, rs_type, viewmats1, tangential_coeffs, thin_prism_coeffs, radial_coeffs)
    CH = int(colors.shape[-1])
    if CH not in (1, 3, 4):
        raise RuntimeError(f"Unsupported number of channels: {CH}")
    masks = _tile_masks(masks, image_width, image_height, tile_size)
    _one_camera(viewmats0, Ks, tile_offsets, opacities)
    N, dev = means.shape[0], means.device
    H, W = int(image_height), int(image_width)
    renders = torch.empty((1, H, W, CH), dtype=torch.float32, device=dev)
    alphas = torch.empty((1, H, W, 1), dtype=torch.float32, device=dev)
    last_ids = torch.empty((1, H, W), dtype=torch.int32, device=dev)
    bg = backgrounds if (backgrounds is not None and backgrounds.numel() > 0) else None
    ws = _ws(capi.lib().lfs_rasterize_workspace_bytes(N), dev)
    if bg is not None and bg.numel() < CH:
        raise RuntimeError(f"backgrounds must have {CH} channels")
    call("lfs_rasterize_to_pixels_from_world_3dgs_fwd", N, flatten_ids.numel(), CH, ptr(means), ptr(quats), ptr(scales), ptr(colors),
         ptr(opacities), ptr(bg), ptr(masks), W, H, int(tile_size), ptr(viewmats0), ptr(viewmats1), ptr(Ks), int(camera_model),
         int(rs_type), ptr(radial_coeffs),
         ptr(tangential_coeffs), ptr(thin_prism_coeffs), ptr(tile_offsets), ptr(flatten_ids), ptr(renders), ptr(alphas), ptr(last_ids), ptr(ws), ws.numel(), _stream())
    return renders, alphas, last_ids


# gsplat/Ops.h:127-160
def rasterize_to_pixels_from_world_3dgs_bwd(means, quats, scales, colors, opacities, backgrounds, masks, image_width,
                                            image_height, tile_size, viewmats0, viewmats1, Ks, camera_model,
                                            ut_params=None, rs_type=ShutterType.GLOBAL, radial_coeffs=None,
                                            tangential_coeffs=None, thin_prism_coeffs=None, tile_offsets=None,
                                            flatten_ids=None, render_alphas=None, last_ids=None, v_render_colors=None,
                                            v_render_alphas=None):
    for t, n in ((means, "means"), (quats, "quats"), (scales, "scales"), (colors, "colors"), (opacities, "opacities"),
                 (render_alphas, "render_alphas"), (v_render_colors, "v_render_colors"), (v_render_alphas, "v_render_alphas")):
        _check_input(t, n)
    _check_input(last_ids, "last_ids", torch.int32)
    radial_coeffs, tangential_coeffs, thin_prism_coeffs = _only_global_pinhole_fisheye(
        camera_model, rs_type, viewmats1, tangential_coeffs, thin_prism_coeffs, radial_coeffs)
    CH = int(colors.shape[-1])
    if CH not in (1, 3, 4):
        raise RuntimeError(f"Unsupported number of channels: {CH}")
    masks = _tile_masks(masks, image_width, image_height, tile_size)
    _one_camera(viewmats0, Ks, tile_offsets, opacities)
    N, dev = means.shape[0], means.device
    v_means, v_quats, v_scales = torch.empty_like(means), torch.empty_like(quats), torch.empty_like(scales)
    v_colors, v_opacities = torch.empty_like(colors), torch.empty_like(opacities)
    bg = backgrounds if (backgrounds is not None and backgrounds.numel() > 0) else None
    ws = _ws(capi.lib().lfs_rasterize_workspace_bytes(N), dev)
    call("lfs_rasterize_to_pixels_from_world_3dgs_bwd", N, flatten_ids.numel(), CH, ptr(means), ptr(quats), ptr(scales), ptr(colors),
         ptr(opacities), ptr(bg), ptr(masks), int(image_width), int(image_height), int(tile_size), ptr(viewmats0), ptr(viewmats1), ptr(Ks),
         int(camera_model), int(rs_type), ptr(radial_coeffs), ptr(tangential_coeffs), ptr(thin_prism_coeffs), ptr(tile_offsets), ptr(flatten_ids), ptr(render_alphas), ptr(last_ids), ptr(v_render_colors),
         ptr(v_render_alphas), ptr(v_means), ptr(v_quats), ptr(v_scales), ptr(v_colors), ptr(v_opacities), ptr(ws), ws.numel(),
         _stream())
    return v_means, v_quats, v_scales, v_colors, v_opacities


# src/training/kernels/ssim.cu:431 / :476
def fusedssim(C1, C2, img1, img2, train=True):
    _check_input(img1, "img1"); _check_input(img2, "img2")
    B, CH, H, W = img1.shape
    if B != 1:
        raise RuntimeError("batch size must be 1")
    outs = [torch.empty_like(img1) for _ in range(4 if train else 1)]
    p = [ptr(o) for o in outs] + [None] * (4 - len(outs))
    call("lfs_fusedssim", CH, H, W, float(C1), float(C2), ptr(img1), ptr(img2), *p, _stream())
    e = torch.empty(0, device=img1.device)
    return tuple(outs) if train else (outs[0], e, e, e)


def fusedssim_backward(C1, C2, img1, img2, dL_dmap, dm_dmu1, dm_dsigma1_sq, dm_dsigma12):
    for t, n in ((img1, "img1"), (img2, "img2"), (dL_dmap, "dL_dmap")):
        _check_input(t, n)
    B, CH, H, W = img1.shape
    out = torch.empty_like(img1)
    call("lfs_fusedssim_backward", CH, H, W, float(C1), float(C2), ptr(img1), ptr(img2), ptr(dL_dmap), ptr(dm_dmu1),
         ptr(dm_dsigma1_sq), ptr(dm_dsigma12), ptr(out), _stream())
    return out


# src/training/fastgs/optimizer/src/adam_api.cu:8 adam_step_wrapper
def adam_step_wrapper(param, exp_avg, exp_avg_sq, param_grad, lr, beta1, beta2, eps, bias_correction1_rcp,
                      bias_correction2_sqrt_rcp):
    for t, n in ((param, "param"), (exp_avg, "exp_avg"), (exp_avg_sq, "exp_avg_sq"), (param_grad, "param_grad")):
        _check_input(t, n)
    call("lfs_adam_step", ptr(param), ptr(exp_avg), ptr(exp_avg_sq), ptr(param_grad), param.numel(), float(lr), float(beta1),
         float(beta2), float(eps), float(bias_correction1_rcp), float(bias_correction2_sqrt_rcp), _stream())


# gsplat/Ops.h:162-270: the fused operator pair, composed from the operator-level entry points with
# the same torch glue as gsplat/Rasterization.cpp:326-466 / :527-641 (all five render modes, compensations, masks).
def rasterize_from_world_with_sh_fwd(means, quats, scales, opacities, sh_coeffs, sh_degree, backgrounds, masks, image_width,
                                     image_height, tile_size, viewmats0, viewmats1, Ks, camera_model, eps2d, near_plane,
                                     far_plane, radius_clip, scaling_modifier, calc_compensations, render_mode,
                                     ut_params=None, rs_type=ShutterType.GLOBAL, radial_coeffs=None, tangential_coeffs=None,
                                     thin_prism_coeffs=None):
    if render_mode not in (0, 1, 2, 3, 4):
        raise RuntimeError("render_mode must be 0=RGB, 1=D, 2=ED, 3=RGB_D or 4=RGB_ED")
    if opacities.dim() == 2:
        opacities = opacities.squeeze(-1)
    Cn = viewmats0.shape[0]
    scaled = scales * scaling_modifier if scaling_modifier != 1.0 else scales
    radii, means2d, depths, conics, comps = projection_ut_3dgs_fused(
        means, quats, scaled, opacities, viewmats0, viewmats1, Ks, image_width, image_height, eps2d, near_plane, far_plane,
        radius_clip, bool(calc_compensations), camera_model, ut_params, rs_type, radial_coeffs, tangential_coeffs, thin_prism_coeffs)
    Rm, t = viewmats0[:, :3, :3], viewmats0[:, :3, 3]
    campos = -(Rm.double().transpose(1, 2) @ t.double().unsqueeze(-1)).squeeze(-1).float()  # inverse(viewmat)[:3, 3]
    dirs = (means.unsqueeze(0) - campos.unsqueeze(1)).contiguous()
    radii_masks = (radii > 0).all(-1)
    if render_mode in (0, 3, 4):
        rgb = spherical_harmonics_fwd(sh_degree, dirs, sh_coeffs.unsqueeze(0).expand(Cn, -1, -1, -1).contiguous(), radii_masks)
        colors = torch.clamp_min(rgb + 0.5, 0.0)
        if render_mode != 0:
            colors = torch.cat([colors, depths.unsqueeze(-1)], -1)
    else:
        colors = depths.unsqueeze(-1)
    colors = colors.contiguous()
    final_opacities = opacities.unsqueeze(0)
    if calc_compensations and comps is not None and comps.numel() > 0:
        final_opacities = final_opacities * comps
    tw, th = (image_width + tile_size - 1) // tile_size, (image_height + tile_size - 1) // tile_size
    tiles_per_gauss, isect_ids, flatten_ids = intersect_tile(means2d, radii, depths, None, None, Cn, tile_size, tw, th, True)
    offsets = intersect_offset(isect_ids, Cn, tw, th)
    renders, alphas, last_ids = rasterize_to_pixels_from_world_3dgs_fwd(
        means, quats, scaled, colors, final_opacities.contiguous(), backgrounds, masks, image_width, image_height, tile_size,
        viewmats0, viewmats1, Ks, camera_model, ut_params, rs_type, radial_coeffs, tangential_coeffs, thin_prism_coeffs,
        offsets, flatten_ids)
    return renders, alphas, radii, means2d, depths, colors, offsets, flatten_ids, last_ids, comps


def rasterize_from_world_with_sh_bwd(means, quats, scales, opacities, sh_coeffs, sh_degree, backgrounds, masks, image_width,
                                     image_height, tile_size, viewmats0, viewmats1, Ks, camera_model, eps2d, near_plane,
                                     far_plane, radius_clip, scaling_modifier, calc_compensations, render_mode, ut_params,
                                     rs_type, radial_coeffs, tangential_coeffs, thin_prism_coeffs, render_alphas, last_ids,
                                     tile_offsets, flatten_ids, colors, radii, means2d, depths, compensations,
                                     v_render_colors, v_render_alphas):
    if opacities.dim() == 2:
        opacities = opacities.squeeze(-1)
    Cn = viewmats0.shape[0]
    scaled = scales * scaling_modifier if scaling_modifier != 1.0 else scales
    final_opacities = opacities.unsqueeze(0)
    if calc_compensations and compensations is not None and compensations.numel() > 0:
        final_opacities = final_opacities * compensations
    v_means, v_quats, v_scales, v_colors, v_opac = rasterize_to_pixels_from_world_3dgs_bwd(
        means, quats, scaled, colors, final_opacities.contiguous(), backgrounds, masks, image_width, image_height, tile_size,
        viewmats0, viewmats1, Ks, camera_model, ut_params, rs_type, radial_coeffs, tangential_coeffs, thin_prism_coeffs,
        tile_offsets, flatten_ids, render_alphas, last_ids, v_render_colors, v_render_alphas)
    Rm, t = viewmats0[:, :3, :3], viewmats0[:, :3, 3]
    campos = -(Rm.double().transpose(1, 2) @ t.double().unsqueeze(-1)).squeeze(-1).float()
    dirs = (means.unsqueeze(0) - campos.unsqueeze(1)).contiguous()
    radii_masks = (radii > 0).all(-1)
    K = sh_coeffs.shape[1]
    if render_mode in (0, 3, 4):
        # the depth channel's per-Gaussian gradient is dropped (gsplat/Rasterization.cpp:575-590)
        v_pre = v_colors[..., :3].clone()
        v_pre.masked_fill_(colors[..., :3] <= 0.0, 0.0)
        v_sh, _ = spherical_harmonics_bwd(K, sh_degree, dirs.reshape(-1, 3), None, radii_masks.reshape(-1),
                                          v_pre.reshape(-1, 3).contiguous(), False)
        v_sh = v_sh.reshape(Cn, -1, K, 3).sum(0)
    else:
        v_sh = torch.zeros_like(sh_coeffs)
    return v_means, v_quats, v_scales * scaling_modifier, v_opac.squeeze(0), v_sh
