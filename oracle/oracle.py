"""TEST INFRASTRUCTURE — ctypes front end of the scalar CPU oracle (oracle/lfs_oracle.cpp).

Only tests, the smoke check and the benchmark's CPU-baseline / reference arm may import this
module. The product (the CUDA library and its host mirror) never does.

Parity status: PARITY UNPINNED by the reference's own tests — the reference ships no golden
vectors or known-answer tests for this path and has no CPU implementation. See the header of
lfs_oracle.cpp.

The orchestration functions below restate the reference's torch glue:
  * activations: src/core/splat_data.cpp:267-286 (sigmoid / exp / F.normalize / cat(sh0, shN))
  * forward:     gsplat/Rasterization.cpp:326-466
  * backward:    gsplat/Rasterization.cpp:527-641
  * image:       src/training/rasterization/rasterizer.cpp:205 (clamp + permute)
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "_build" / "liblfs_oracle.so"
_SRC = _HERE / "lfs_oracle.cpp"


def build(force: bool = False) -> Path:
    """Compile the oracle with gcc (IEEE float32, no contraction, OpenMP)."""
    srcs = [_SRC, _SRC.with_name("lfs_oracle_ewa.cpp")]
    if force or not _SO.exists() or _SO.stat().st_mtime < max(s.stat().st_mtime for s in srcs):
        _SO.parent.mkdir(exist_ok=True)
        subprocess.check_call(
            ["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC",
             "-o", str(_SO)] + [str(s) for s in srcs])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build()))
        _lib.orc_intersect_count.restype = C.c_int64
        _lib.orc_rasterize_fwd_ch.restype = C.c_int64
        _lib.orc_rasterize_bwd_ch.restype = C.c_int64
        _lib.orc_photometric_loss.restype = C.c_float
        _lib.orc_num_threads.restype = C.c_int
        _lib.orc_ewa_lists.restype = C.c_int64
    return _lib


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


f = C.c_float
i32 = C.c_int
u32 = C.c_uint32
i64 = C.c_int64

UT_DEFAULT = np.array([0.1, 2.0, 0.0, 0.1, 1.0], dtype=np.float32)
PINHOLE, ORTHO, FISHEYE, EQUIRECTANGULAR = 0, 1, 2, 3


def num_threads() -> int:
    return int(lib().orc_num_threads())


def use_all_cores() -> int:
    """Launchers such as torch.distributed.run export OMP_NUM_THREADS=1; the timed CPU baseline wants every host core.
    Sets the OpenMP thread count of the loaded library to the number of cores this process may run on."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    fn = lib().omp_set_num_threads          # resolved through the library's OpenMP runtime dependency
    fn.argtypes, fn.restype = [C.c_int], None
    fn(int(n))
    return num_threads()


# ------------------------------------------------------------------ operators
def projection_ut_3dgs_fused(means, quats, scales, opacities, viewmats, Ks, W, H, eps2d=0.3,
                             near=0.01, far=1e4, radius_clip=0.0, calc_compensations=False,
                             camera_model=PINHOLE, ut=UT_DEFAULT, radial_coeffs=None):
    means, quats, scales = _f32(means), _f32(quats), _f32(scales)
    opacities, viewmats, Ks = _f32(opacities), _f32(viewmats), _f32(Ks)
    radial_coeffs = _f32(radial_coeffs)
    N, Cn = means.shape[0], viewmats.shape[0]
    radii = np.zeros((Cn, N, 2), np.int32)
    means2d = np.zeros((Cn, N, 2), np.float32)
    depths = np.zeros((Cn, N), np.float32)
    conics = np.zeros((Cn, N, 3), np.float32)
    comps = np.zeros((Cn, N), np.float32) if calc_compensations else None
    lib().orc_projection_ut_3dgs_fused(
        i32(Cn), i32(N), _p(means), _p(quats), _p(scales), _p(opacities), _p(viewmats), _p(Ks),
        i32(W), i32(H), f(eps2d), f(near), f(far), f(radius_clip), i32(camera_model),
        _p(_f32(ut)), _p(radial_coeffs), _p(radii), _p(means2d), _p(depths), _p(conics), _p(comps))
    return radii, means2d, depths, conics, comps


def spherical_harmonics_fwd(degree, dirs, coeffs, masks=None):
    dirs, coeffs = _f32(dirs), _f32(coeffs)
    n, K = dirs.reshape(-1, 3).shape[0], coeffs.shape[-2]
    colors = np.zeros((n, 3), np.float32)
    m = None if masks is None else np.ascontiguousarray(masks.reshape(-1), np.uint8)
    lib().orc_spherical_harmonics_fwd(i32(n), i32(K), i32(degree), _p(dirs), _p(coeffs), _p(m), _p(colors))
    return colors.reshape(dirs.shape)


def spherical_harmonics_bwd(K, degree, dirs, masks, v_colors):
    dirs, v_colors = _f32(dirs), _f32(v_colors)
    n = dirs.reshape(-1, 3).shape[0]
    v_coeffs = np.zeros((n, K, 3), np.float32)
    m = None if masks is None else np.ascontiguousarray(masks.reshape(-1), np.uint8)
    lib().orc_spherical_harmonics_bwd(i32(n), i32(K), i32(degree), _p(dirs), _p(m), _p(v_colors), _p(v_coeffs))
    return v_coeffs


def intersect_tile(means2d, radii, depths, Cn, tile_size, tw, th, sort=True):
    means2d, depths = _f32(means2d), _f32(depths)
    radii = np.ascontiguousarray(radii, np.int32)
    N = means2d.size // 2 // Cn
    tpg = np.zeros((Cn, N), np.int32)
    n = int(lib().orc_intersect_count(i32(Cn), i32(N), _p(means2d), _p(radii), u32(tile_size), u32(tw), u32(th), _p(tpg)))
    ids = np.zeros(n, np.int64)
    flat = np.zeros(n, np.int32)
    lib().orc_intersect_emit_sort(i32(Cn), i32(N), _p(means2d), _p(radii), _p(depths), u32(tile_size), u32(tw), u32(th),
                                  i32(1 if sort else 0), i64(n), _p(ids), _p(flat))
    return tpg, ids, flat


def intersect_offset(isect_ids, Cn, tw, th):
    isect_ids = np.ascontiguousarray(isect_ids, np.int64)
    off = np.zeros((Cn, th, tw), np.int32)
    lib().orc_intersect_offset(i64(isect_ids.size), _p(isect_ids), i32(Cn), u32(tw), u32(th), _p(off))
    return off


def rasterize_fwd(means, quats, scales, colors, opacities, background, W, H, tile_size, viewmat, K,
                  tile_offsets, flatten_ids, camera_model=PINHOLE, radial=None, tile_range=(0, -1), masks=None):
    """One camera (the reference kernel supports C = 1 only). colors is [N, CH] with CH in 1..4.
    Returns render [H,W,CH], alpha [H,W,1], last_ids [H,W] and the number of (pixel, entry) pairs visited."""
    a = [_f32(x) for x in (means, quats, scales, colors, opacities)]
    CH = a[3].shape[-1] if a[3].ndim == 2 else 1
    bg = _f32(background)
    mk = None if masks is None else np.ascontiguousarray(masks, np.uint8)
    render = np.zeros((H, W, CH), np.float32)
    alpha = np.zeros((H, W, 1), np.float32)
    last = np.zeros((H, W), np.int32)
    to = np.ascontiguousarray(tile_offsets, np.int32)
    fl = np.ascontiguousarray(flatten_ids, np.int32)
    npairs = lib().orc_rasterize_fwd_ch(
        i32(a[0].shape[0]), i64(fl.size), i32(CH), _p(a[0]), _p(a[1]), _p(a[2]), _p(a[3]), _p(a[4]), _p(bg), _p(mk),
        i32(W), i32(H), i32(tile_size), _p(_f32(viewmat)), _p(_f32(K)), i32(camera_model), _p(_f32(radial)),
        _p(to), _p(fl), _p(render), _p(alpha), _p(last), i32(tile_range[0]), i32(tile_range[1]))
    return render, alpha, last, int(npairs)


def rasterize_bwd(means, quats, scales, colors, opacities, background, W, H, tile_size, viewmat, K,
                  tile_offsets, flatten_ids, render_alphas, last_ids, v_render_colors, v_render_alphas,
                  camera_model=PINHOLE, radial=None, tile_range=(0, -1), masks=None):
    a = [_f32(x) for x in (means, quats, scales, colors, opacities)]
    N = a[0].shape[0]
    CH = a[3].shape[-1] if a[3].ndim == 2 else 1
    mk = None if masks is None else np.ascontiguousarray(masks, np.uint8)
    bg = _f32(background)
    to = np.ascontiguousarray(tile_offsets, np.int32)
    fl = np.ascontiguousarray(flatten_ids, np.int32)
    v_means = np.zeros((N, 3), np.float32)
    v_quats = np.zeros((N, 4), np.float32)
    v_scales = np.zeros((N, 3), np.float32)
    v_colors = np.zeros((N, CH), np.float32)
    v_opac = np.zeros((N,), np.float32)
    npairs = lib().orc_rasterize_bwd_ch(
        i32(N), i64(fl.size), i32(CH), _p(a[0]), _p(a[1]), _p(a[2]), _p(a[3]), _p(a[4]), _p(bg), _p(mk),
        i32(W), i32(H), i32(tile_size), _p(_f32(viewmat)), _p(_f32(K)), i32(camera_model), _p(_f32(radial)),
        _p(to), _p(fl), _p(_f32(render_alphas)), _p(np.ascontiguousarray(last_ids, np.int32)),
        _p(_f32(v_render_colors)), _p(_f32(v_render_alphas)),
        _p(v_means), _p(v_quats), _p(v_scales), _p(v_colors), _p(v_opac), i32(tile_range[0]), i32(tile_range[1]))
    return v_means, v_quats, v_scales, v_colors, v_opac, int(npairs)


def fusedssim(img1, img2, C1=0.01 ** 2, C2=0.03 ** 2):
    img1, img2 = _f32(img1), _f32(img2)
    CH, H, W = img1.shape
    outs = [np.zeros_like(img1) for _ in range(4)]
    lib().orc_fusedssim_fwd(i32(CH), i32(H), i32(W), f(C1), f(C2), _p(img1), _p(img2), *[_p(o) for o in outs])
    return outs


def fusedssim_backward(img1, img2, dL_dmap, dm1, ds1, ds12):
    img1 = _f32(img1)
    CH, H, W = img1.shape
    out = np.zeros_like(img1)
    lib().orc_fusedssim_bwd(i32(CH), i32(H), i32(W), _p(img1), _p(_f32(img2)), _p(_f32(dL_dmap)),
                            _p(_f32(dm1)), _p(_f32(ds1)), _p(_f32(ds12)), _p(out))
    return out


def photometric_loss(render_hwc, target_chw, lambda_dssim=0.2, want_grad=True):
    render_hwc, target_chw = _f32(render_hwc), _f32(target_chw)
    H, W, _ = render_hwc.shape
    g = np.zeros_like(render_hwc) if want_grad else None
    l1, ss = C.c_float(), C.c_float()
    loss = lib().orc_photometric_loss(i32(H), i32(W), f(lambda_dssim), _p(render_hwc), _p(target_chw), _p(g),
                                      C.byref(l1), C.byref(ss))
    return float(loss), g, float(l1.value), float(ss.value)


def adam_step(param, exp_avg, exp_avg_sq, grad, lr, beta1, beta2, eps, step_count):
    """In place. Bias terms in double on the host as src/training/optimizers/fused_adam.cpp:78-79."""
    bc1 = 1.0 / (1.0 - beta1 ** step_count)
    bc2 = 1.0 / np.sqrt(1.0 - beta2 ** step_count)
    for a in (param, exp_avg, exp_avg_sq):
        assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    lib().orc_adam_step(i64(param.size), _p(param), _p(exp_avg), _p(exp_avg_sq), _p(_f32(grad)),
                        f(lr), f(beta1), f(beta2), f(eps), f(bc1), f(bc2))


def binoms_table(n_max=51):
    """src/training/strategies/mcmc.cpp:459-472: running float product."""
    b = np.zeros((n_max, n_max), np.float32)
    for n in range(n_max):
        for k in range(n + 1):
            v = np.float32(1.0)
            for i in range(k):
                v = np.float32(v * (np.float32(n - i) / np.float32(i + 1)))
            b[n, k] = v
    return b


def relocation(opacities, scales, ratios, binoms, n_max):
    opacities, scales, binoms = _f32(opacities), _f32(scales), _f32(binoms)
    ratios = np.ascontiguousarray(ratios, np.int32)
    n = opacities.shape[0]
    no = np.zeros(n, np.float32)
    ns = np.zeros((n, 3), np.float32)
    lib().orc_relocation(i32(n), _p(opacities), _p(scales), _p(ratios), _p(binoms), i32(n_max), _p(no), _p(ns))
    return no, ns


def add_noise(raw_opacities, raw_scales, raw_quats, noise, means, current_lr):
    """In place on means."""
    assert means.dtype == np.float32 and means.flags["C_CONTIGUOUS"]
    lib().orc_add_noise(i32(means.shape[0]), _p(_f32(raw_opacities)), _p(_f32(raw_scales)), _p(_f32(raw_quats)),
                        _p(_f32(noise)), _p(means), f(current_lr))


def quats_to_rotmats(quats):
    quats = _f32(quats)
    out = np.zeros((quats.shape[0], 3, 3), np.float32)
    lib().orc_quats_to_rotmats(i32(quats.shape[0]), _p(quats), _p(out))
    return out


def campos(viewmat):
    out = np.zeros(3, np.float32)
    lib().orc_campos(_p(_f32(viewmat)), _p(out))
    return out


def cam_point_to_image(model, K, W, H, dist, p, margin=0.1):
    out = np.zeros(2, np.float32)
    ok = lib().orc_cam_point_to_image(i32(model), _p(_f32(K)), i32(W), i32(H), _p(_f32(dist)), _p(_f32(p)), C.c_float(margin), _p(out))
    return out, bool(ok)


def image_to_cam_ray(model, K, W, H, dist, px, py):
    ray = np.zeros(3, np.float32)
    ok = lib().orc_image_to_cam_ray(i32(model), _p(_f32(K)), i32(W), i32(H), _p(_f32(dist)), C.c_float(px), C.c_float(py), _p(ray))
    return ray, bool(ok)


GLOBAL_SHUTTER = 4   # ShutterType of gsplat/Cameras.h: 0 top-to-bottom, 1 left-to-right, 2 bottom-to-top, 3 right-to-left, 4 global


class shutter:
    """Context manager: the projection / rasterizer calls inside use a rolling shutter between the start pose (their
    viewmat argument) and `viewmat1` (the reference's viewmats1), ShutterType `rs_type`."""

    def __init__(self, viewmat1, rs_type):
        self.vm1, self.type = (None if viewmat1 is None else _f32(viewmat1).reshape(4, 4)), int(rs_type)

    def __enter__(self):
        lib().orc_set_shutter(_p(self.vm1), i32(self.type))
        return self

    def __exit__(self, *exc):
        lib().orc_set_shutter(None, i32(GLOBAL_SHUTTER))
        return False


def pack_distortion(radial=None, tangential=None, thin_prism=None):
    """The 12-float OpenCV pinhole distortion block this oracle takes in place of the reference's three optional
    tensors (k1..k6, p1, p2, s1..s4); shorter inputs are zero-padded. None when all three are absent."""
    if radial is None and tangential is None and thin_prism is None:
        return None
    d = np.zeros(12, np.float32)
    for off, n, a in ((0, 6, radial), (6, 2, tangential), (8, 4, thin_prism)):
        if a is not None:
            a = np.asarray(a, np.float32).reshape(-1)
            d[off:off + min(n, a.size)] = a[:n]
    return d


# ------------------------------------------------------------------ activations
def act_opacity(raw):
    return (1.0 / (1.0 + np.exp(-raw.astype(np.float64)))).astype(np.float32).reshape(-1)


def act_scale(raw):
    return np.exp(raw.astype(np.float64)).astype(np.float32)


def act_quat(raw):
    raw = raw.astype(np.float32)
    n2 = ((raw[:, 0] * raw[:, 0] + raw[:, 1] * raw[:, 1]) + raw[:, 2] * raw[:, 2]) + raw[:, 3] * raw[:, 3]
    nrm = np.maximum(np.sqrt(n2), np.float32(1e-12)).astype(np.float32)
    return (raw / nrm[:, None]).astype(np.float32), nrm


# ------------------------------------------------------------------ orchestration
def render_fwd(params, viewmat, K, W, H, sh_degree, background=None, camera_model=PINHOLE, radial=None,
               tile_size=16, eps2d=0.3, near=0.01, far=1e4, tile_range=(0, -1), render_mode=0,
               calc_compensations=False, scaling_modifier=1.0, tile_masks=None):
    """gsplat::rasterize_from_world_with_sh_fwd (gsplat/Rasterization.cpp:279-468) for one camera on raw SplatData
    parameters, followed by the render-mode post-processing of rasterize()
    (src/training/rasterization/rasterizer.cpp:171-198).
    params: dict(means, sh0, shN, scaling_raw, rotation_raw, opacity_raw). render_mode: 0 RGB, 1 D, 2 ED, 3 RGB_D,
    4 RGB_ED. background has as many entries as the render has channels."""
    means = _f32(params["means"])
    opac = act_opacity(params["opacity_raw"])
    scales = act_scale(params["scaling_raw"])
    if scaling_modifier != 1.0:
        scales = (scales * np.float32(scaling_modifier)).astype(np.float32)
    quats, qnorm = act_quat(params["rotation_raw"])
    sh = np.concatenate([params["sh0"], params["shN"]], axis=1).astype(np.float32)
    vm = _f32(viewmat).reshape(1, 4, 4)
    Kc = _f32(K).reshape(1, 3, 3)
    rc = None if radial is None else _f32(radial).reshape(1, -1)
    radii, means2d, depths, conics, comps = projection_ut_3dgs_fused(
        means, quats, scales, opac, vm, Kc, W, H, eps2d, near, far, 0.0, bool(calc_compensations), camera_model, UT_DEFAULT, rc)
    cp = campos(vm[0])
    dirs = (means - cp[None, :]).astype(np.float32)
    masks = (radii[0] > 0).all(-1)
    if render_mode in (0, 3, 4):
        rgb = spherical_harmonics_fwd(sh_degree, dirs, sh, masks)
        colors = np.maximum(rgb + np.float32(0.5), np.float32(0.0)).astype(np.float32)
        colors[~masks] = 0.0
        if render_mode != 0:
            colors = np.concatenate([colors, depths[0][:, None]], axis=1).astype(np.float32)
    else:
        colors = np.ascontiguousarray(depths[0][:, None], np.float32)
    final_opac = (opac * comps[0]).astype(np.float32) if calc_compensations else opac
    tw, th = (W + tile_size - 1) // tile_size, (H + tile_size - 1) // tile_size
    tpg, ids, flat = intersect_tile(means2d, radii, depths, 1, tile_size, tw, th, True)
    offs = intersect_offset(ids, 1, tw, th)
    render, alpha, last, npairs = rasterize_fwd(means, quats, scales, colors, final_opac, background, W, H, tile_size,
                                                vm[0], Kc[0], offs[0], flat, camera_model, rc, tile_range, tile_masks)
    out = dict(render=render, alpha=alpha, last_ids=last, radii=radii[0], means2d=means2d[0], depths=depths[0],
               colors=colors, tile_offsets=offs[0], flatten_ids=flat, isect_ids=ids, tiles_per_gauss=tpg[0],
               masks=masks, dirs=dirs, opac=opac, final_opac=final_opac, scales=scales, quats=quats, qnorm=qnorm, sh=sh,
               n_pairs_fwd=npairs, conics=conics[0], render_mode=render_mode, tile_masks=tile_masks)
    if render_mode != 0:
        acc = render[..., -1:]
        if render_mode in (2, 4):
            depth = (acc / np.maximum(alpha, np.float32(1e-10))).astype(np.float32)
            if tile_masks is not None:
                # masked tiles: the reference divides by an alpha it never wrote there; defined here as "no division"
                off = np.kron(~np.asarray(tile_masks, bool), np.ones((tile_size, tile_size), bool))[:H, :W]
                depth[off] = acc[off]
            out["depth"] = depth
        else:
            out["depth"] = acc
        out["image"] = render[..., :3] if render_mode in (3, 4) else None
    else:
        out["image"], out["depth"] = render, None
    return out


def render_bwd(params, fwd, viewmat, K, W, H, sh_degree, v_render, v_alpha=None, background=None,
               camera_model=PINHOLE, radial=None, tile_size=16, tile_range=(0, -1)):
    """gsplat::rasterize_from_world_with_sh_bwd (gsplat/Rasterization.cpp:470-642) followed by the activation
    backward; returns gradients w.r.t. the six raw parameter tensors. v_render has the channels of fwd["render"]; in
    the expected-depth modes its last channel is the gradient of the DIVIDED depth and the chain rule of
    depth = sum / clamp_min(alpha, 1e-10) (rasterizer.cpp:186-198, as autograd would apply it) comes first."""
    means = _f32(params["means"])
    mode = fwd.get("render_mode", 0)
    v_render = _f32(v_render).copy()
    v_alpha = np.zeros((H, W, 1), np.float32) if v_alpha is None else _f32(v_alpha).copy()
    if mode in (2, 4):
        a = fwd["alpha"]
        ac = np.maximum(a, np.float32(1e-10))
        vd = v_render[..., -1:]
        v_alpha = (v_alpha + np.where(a > 1e-10, -fwd["render"][..., -1:] / (ac * ac) * vd, 0.0)).astype(np.float32)
        v_render[..., -1:] = vd / ac
    rc = None if radial is None else _f32(radial).reshape(1, -1)
    v_means, v_quats, v_scales, v_colors, v_opac, npairs = rasterize_bwd(
        means, fwd["quats"], fwd["scales"], fwd["colors"], fwd["final_opac"], background, W, H, tile_size,
        viewmat, K, fwd["tile_offsets"], fwd["flatten_ids"], fwd["alpha"], fwd["last_ids"], v_render, v_alpha,
        camera_model, rc, tile_range, fwd.get("tile_masks"))
    K_sh = fwd["sh"].shape[1]
    if mode in (0, 3, 4):
        v_pre = v_colors[:, :3].copy()
        v_pre[fwd["colors"][:, :3] <= 0.0] = 0.0
        v_sh = spherical_harmonics_bwd(K_sh, sh_degree, fwd["dirs"], fwd["masks"], v_pre)
    else:
        v_sh = np.zeros((means.shape[0], K_sh, 3), np.float32)
    # the opacity gradient is taken w.r.t. the compensated opacity and passed on unchanged; v_scales is w.r.t.
    # the modified scale = exp(raw) * modifier (Rasterization.cpp:626), whose derivative w.r.t. raw is itself
    o, s, q, nrm = fwd["opac"], fwd["scales"], fwd["quats"], fwd["qnorm"]
    g_opacity = (v_opac * (o * (np.float32(1.0) - o))).astype(np.float32).reshape(-1, 1)
    g_scaling = (v_scales * s).astype(np.float32)
    dq = (v_quats * q).sum(-1, keepdims=True).astype(np.float32)
    g_rotation = ((v_quats - q * dq) / nrm[:, None]).astype(np.float32)
    return dict(means=v_means, sh0=np.ascontiguousarray(v_sh[:, :1]), shN=np.ascontiguousarray(v_sh[:, 1:]),
                scaling_raw=g_scaling, rotation_raw=g_rotation, opacity_raw=g_opacity,
                v_colors=v_colors, v_opacities=v_opac, v_quats=v_quats, v_scales=v_scales, n_pairs_bwd=npairs)


# ------------------------------------------------------------------ EWA (default, non --gut) rasterizer
def ewa_forward(params, w2c, cam_position, W, H, fx, fy, cx, cy, active_sh_bases, background=None, near=0.01, far=1e10):
    """fast_rasterize (src/training/rasterization/fast_rasterizer.cpp:13-71) for one camera on raw SplatData parameters:
    preprocess -> lists -> blend. Returns image [3,H,W] (with background), alpha [H,W] and the intermediate state."""
    means = _f32(params["means"])
    N = means.shape[0]
    sh0, shN = _f32(params["sh0"]).reshape(N, 3), _f32(params["shN"])
    total_rest = shN.shape[1] if shN.ndim == 3 else 0
    n_touched = np.zeros(N, np.int32)
    bounds = np.zeros((N, 4), np.int32)
    mean2d = np.zeros((N, 2), np.float32)
    conic_opacity = np.zeros((N, 4), np.float32)
    color = np.zeros((N, 3), np.float32)
    depth = np.zeros(N, np.float32)
    w2c, cam_position = _f32(w2c), _f32(cam_position)
    f = lambda v: C.c_float(float(v))
    lib().orc_ewa_preprocess(i32(N), _p(means), _p(_f32(params["scaling_raw"])), _p(_f32(params["rotation_raw"])),
                             _p(_f32(params["opacity_raw"]).reshape(-1)), _p(sh0), _p(shN), _p(w2c), _p(cam_position),
                             i32(active_sh_bases), i32(total_rest), i32(W), i32(H), f(fx), f(fy), f(cx), f(cy), f(near), f(far),
                             _p(n_touched), _p(bounds), _p(mean2d), _p(conic_opacity), _p(color), _p(depth))
    gw, gh = (W + 15) // 16, (H + 15) // 16
    ids = np.zeros(max(int(n_touched.sum()), 1), np.int32)
    offs = np.zeros(gw * gh + 1, np.int32)
    n = lib().orc_ewa_lists(i32(N), _p(n_touched), _p(bounds), _p(mean2d), _p(conic_opacity), _p(depth), i32(W), i32(H), _p(ids), _p(offs))
    ids = ids[:n]
    image = np.zeros((3, H, W), np.float32)
    alpha = np.zeros((H, W), np.float32)
    n_contrib = np.zeros((H, W), np.int32)
    bg = _f32(background)
    lib().orc_ewa_blend_fwd(i32(W), i32(H), _p(ids if n else np.zeros(1, np.int32)), _p(offs), _p(mean2d), _p(conic_opacity), _p(color),
                            _p(bg), _p(image), _p(alpha), _p(n_contrib))
    return dict(image=image, alpha=alpha, n_contrib=n_contrib, n_touched=n_touched, bounds=bounds, mean2d=mean2d,
                conic_opacity=conic_opacity, color=color, depth=depth, instance_ids=ids, tile_offsets=offs, background=bg,
                cam=(w2c, cam_position, W, H, fx, fy, cx, cy, active_sh_bases, total_rest))


def ewa_backward(params, fwd, grad_image, grad_alpha=None, densification_info=None):
    """FastGSRasterize::backward (fast_rasterizer_autograd.cpp:88-165) incl. the background term of fast_rasterize;
    grad_image [3,H,W] is w.r.t. the final image. Returns gradients w.r.t. the six raw tensors; densification_info
    [2,N] is updated in place when given."""
    w2c, cam_position, W, H, fx, fy, cx, cy, active, total_rest = fwd["cam"]
    means = _f32(params["means"])
    N = means.shape[0]
    gm2, gcon, gop, gcol = (np.zeros((N, 2), np.float32), np.zeros((N, 3), np.float32), np.zeros(N, np.float32),
                            np.zeros((N, 3), np.float32))
    ids = fwd["instance_ids"] if fwd["instance_ids"].size else np.zeros(1, np.int32)
    lib().orc_ewa_blend_bwd(i32(N), i32(W), i32(H), _p(ids), _p(fwd["tile_offsets"]), _p(fwd["mean2d"]), _p(fwd["conic_opacity"]),
                            _p(fwd["color"]), _p(fwd["background"]), _p(fwd["alpha"]), _p(fwd["n_contrib"]), _p(_f32(grad_image)),
                            _p(_f32(grad_alpha)), _p(gm2), _p(gcon), _p(gop), _p(gcol))
    shN = _f32(params["shN"])
    g_means, g_scales, g_rot = np.zeros((N, 3), np.float32), np.zeros((N, 3), np.float32), np.zeros((N, 4), np.float32)
    g_sh0, g_shN = np.zeros((N, 1, 3), np.float32), np.zeros_like(shN)
    g_cam = np.zeros((N, 3), np.float32)
    f = lambda v: C.c_float(float(v))
    lib().orc_ewa_preprocess_bwd(i32(N), _p(means), _p(_f32(params["scaling_raw"])), _p(_f32(params["rotation_raw"])), _p(shN),
                                 _p(w2c), _p(cam_position), _p(fwd["n_touched"]), _p(gm2), _p(gcon), _p(gcol), i32(active),
                                 i32(total_rest), i32(W), i32(H), f(fx), f(fy), f(cx), f(cy), _p(g_means), _p(g_scales), _p(g_rot),
                                 _p(g_sh0), _p(g_shN), _p(densification_info), _p(g_cam))
    # camera-pose gradient (kernels_backward.cuh:160-173): sum of (camera-space mean gradient) x (mean, 1), rows 0..2
    grad_w2c = np.zeros((4, 4), np.float64)
    grad_w2c[:3, :3] = g_cam.astype(np.float64).T @ means.astype(np.float64)
    grad_w2c[:3, 3] = g_cam.astype(np.float64).sum(0)
    vis = fwd["n_touched"] > 0
    gop = np.where(vis, gop, 0).astype(np.float32)
    return dict(means=g_means, sh0=g_sh0, shN=g_shN, scaling_raw=g_scales, rotation_raw=g_rot, opacity_raw=gop.reshape(N, 1),
                grad_mean2d=gm2, grad_conic=gcon, grad_color=gcol, grad_w2c=grad_w2c.astype(np.float32))
