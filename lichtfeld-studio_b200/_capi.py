"""ctypes binding of liblfs_b200.so (include/lfs_b200.h). The CUDA library is the product; this
module only loads it and declares the signatures. There is no fallback: if the library is missing
or a call fails, an exception is raised."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "liblfs_b200.so"

LFS_OK, LFS_EINVAL, LFS_ECAPACITY, LFS_ECUDA, LFS_EUNSUPPORTED = 0, -1, -2, -3, -4
PINHOLE, ORTHO, FISHEYE, EQUIRECTANGULAR = 0, 1, 2, 3
LFS_DP_MAX_WORLD, LFS_DP_FLAG_SLOTS = 16, 8
LFS_DP_FLAG_WORDS = LFS_DP_MAX_WORLD * LFS_DP_FLAG_SLOTS


class UTParams(C.Structure):
    """gsplat/Cameras.h:27-45 UnscentedTransformParameters."""
    _fields_ = [("alpha", C.c_float), ("beta", C.c_float), ("kappa", C.c_float),
                ("in_image_margin_factor", C.c_float), ("require_all_sigma_points_valid", C.c_int)]

    def __init__(self, alpha=0.1, beta=2.0, kappa=0.0, in_image_margin_factor=0.1, require_all_sigma_points_valid=True):
        super().__init__(alpha, beta, kappa, in_image_margin_factor, 1 if require_all_sigma_points_valid else 0)


class Splats(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")]


class RenderConfig(C.Structure):
    _fields_ = [("N", C.c_int), ("sh_coeffs", C.c_int), ("sh_degree", C.c_int), ("image_width", C.c_int),
                ("image_height", C.c_int), ("tile_size", C.c_int), ("camera_model", C.c_int),
                ("eps2d", C.c_float), ("near_plane", C.c_float), ("far_plane", C.c_float), ("radius_clip", C.c_float),
                ("ut", UTParams), ("isect_capacity", C.c_int64), ("render_mode", C.c_int), ("calc_compensations", C.c_int),
                ("scaling_modifier", C.c_float), ("tile_masks", C.c_void_p), ("radial_coeffs", C.c_void_p),
                ("tangential_coeffs", C.c_void_p), ("thin_prism_coeffs", C.c_void_p), ("shutter", C.c_int),
                ("viewmat_end", C.c_void_p)]


class EwaConfig(C.Structure):
    _fields_ = [("N", C.c_int), ("sh_coeffs", C.c_int), ("active_sh_bases", C.c_int), ("image_width", C.c_int),
                ("image_height", C.c_int), ("focal_x", C.c_float), ("focal_y", C.c_float), ("center_x", C.c_float),
                ("center_y", C.c_float), ("near_plane", C.c_float), ("far_plane", C.c_float), ("instance_capacity", C.c_int64)]


class EwaView(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("n_touched", "bounds", "records", "instance_ids", "tile_offsets", "n_contrib")]


class RenderView(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("radii", "means2d", "depths", "tiles_per_gauss", "tile_offsets",
                                          "flatten_ids", "last_ids", "records")]


class AdamSegment(C.Structure):
    _fields_ = [("param", C.c_void_p), ("exp_avg", C.c_void_p), ("exp_avg_sq", C.c_void_p), ("grad", C.c_void_p),
                ("n", C.c_int64), ("lr", C.c_float)]


class DpSegment(C.Structure):
    _fields_ = [("offset", C.c_int64), ("n", C.c_int64), ("exp_avg", C.c_void_p), ("exp_avg_sq", C.c_void_p), ("lr", C.c_float)]


class LfsError(RuntimeError):
    pass


_lib = None
vp, i32, i64, f32, sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

_SIGNATURES = {
    "lfs_projection_ut_3dgs_fused": [i32, i32, vp, vp, vp, vp, vp, vp, vp, i32, i32, f32, f32, f32, f32, i32, UTParams, i32, vp, vp, vp,
                                     vp, vp, vp, vp, vp, vp],
    "lfs_spherical_harmonics_fwd": [i32, i32, i32, vp, vp, vp, vp, vp],
    "lfs_spherical_harmonics_bwd": [i32, i32, i32, vp, vp, vp, vp, vp],
    "lfs_intersect_tile_count": [i32, i32, vp, vp, i32, i32, i32, vp, vp, vp],
    "lfs_intersect_tile_emit": [i32, i32, vp, vp, vp, vp, i32, i32, i32, i32, i64, vp, vp, vp, sz, vp],
    "lfs_intersect_offset": [i64, vp, i32, i32, i32, vp, vp],
    "lfs_rasterize_to_pixels_from_world_3dgs_fwd": [i32, i64, i32, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, vp, i32, i32, vp, vp, vp,
                                                    vp, vp, vp, vp, vp, vp, sz, vp],
    "lfs_rasterize_to_pixels_from_world_3dgs_bwd": [i32, i64, i32, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, vp, i32, i32, vp, vp, vp,
                                                    vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp],
    "lfs_fusedssim": [i32, i32, i32, f32, f32, vp, vp, vp, vp, vp, vp, vp],
    "lfs_fusedssim_backward": [i32, i32, i32, f32, f32, vp, vp, vp, vp, vp, vp, vp, vp],
    "lfs_adam_step": [vp, vp, vp, vp, i64, f32, f32, f32, f32, f32, f32, vp],
    "lfs_relocation": [i32, vp, vp, vp, vp, i32, vp, vp, vp],
    "lfs_add_noise": [i32, vp, vp, vp, vp, vp, f32, vp],
    "lfs_quats_to_rotmats": [i32, vp, vp, vp],
    "lfs_ewa_forward": [C.POINTER(EwaConfig), C.POINTER(Splats), vp, vp, vp, vp, vp, vp, vp, sz, vp],
    "lfs_ewa_backward": [C.POINTER(EwaConfig), C.POINTER(Splats), vp, vp, vp, vp, vp, vp, C.POINTER(Splats), i32, vp, vp, vp, sz, vp],
    "lfs_ewa_adam_step_rank1_sh": [C.POINTER(EwaConfig), C.POINTER(Splats), vp, C.POINTER(Splats), C.POINTER(Splats), C.POINTER(Splats),
                                   C.POINTER(C.c_float), C.c_double, C.c_double, C.c_double, i64, i32, f32, vp],
    "lfs_ewa_workspace_view": [C.POINTER(EwaConfig), vp, sz, C.POINTER(EwaView)],
    "lfs_ply_pack_rows": [i32, i32, C.POINTER(Splats), vp, vp],
    "lfs_ply_unpack_rows": [i32, i32, vp, C.POINTER(Splats), vp],
    "lfs_render_forward": [C.POINTER(RenderConfig), C.POINTER(Splats), vp, vp, vp, vp, vp, vp, vp, sz, vp],
    "lfs_render_forward_lists": [C.POINTER(RenderConfig), C.POINTER(Splats), vp, vp, vp, sz, vp],
    "lfs_render_forward_lists_event": [C.POINTER(RenderConfig), C.POINTER(Splats), vp, vp, vp, vp, sz, vp],
    "lfs_render_forward_shade": [C.POINTER(RenderConfig), C.POINTER(Splats), vp, vp, vp, vp, vp, sz, vp],
    "lfs_render_backward": [C.POINTER(RenderConfig), C.POINTER(Splats), vp, vp, vp, vp, C.POINTER(Splats), i32, vp, sz, vp],
    "lfs_render_backward_adam": [C.POINTER(RenderConfig), C.POINTER(Splats), vp, vp, vp, vp, C.POINTER(Splats), C.POINTER(Splats),
                                 C.POINTER(C.c_float), C.c_double, C.c_double, C.c_double, i64, i32, f32, vp, sz, vp],
    "lfs_render_workspace_view": [C.POINTER(RenderConfig), vp, sz, C.POINTER(RenderView)],
    "lfs_photometric_loss": [i32, i32, f32, f32, vp, vp, vp, vp, vp, sz, vp],
    "lfs_background_gradient": [i32, i32, i32, vp, vp, vp, vp, sz, vp],
    "lfs_adam_step_splats": [i32, i32, C.POINTER(Splats), C.POINTER(Splats), C.POINTER(Splats), C.POINTER(Splats),
                             C.POINTER(C.c_float), C.c_double, C.c_double, C.c_double, i64, i32, i64, i64, f32, vp],
    "lfs_adam_step_splats_rank1_sh": [C.POINTER(RenderConfig), C.POINTER(Splats), C.POINTER(Splats), C.POINTER(Splats),
                                      C.POINTER(Splats), C.POINTER(C.c_float), C.c_double, C.c_double, C.c_double, i64, i32, f32,
                                      vp, sz, vp],
    "lfs_regularization": [i32, vp, vp, f32, f32, vp, vp, vp, vp],
    "lfs_adam_step_segments": [i32, C.POINTER(AdamSegment), C.c_double, C.c_double, C.c_double, i64, f32, i32, vp],
    "lfs_dp_reduce_adam_broadcast": [i32, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), vp, i32, C.POINTER(DpSegment), C.c_double,
                                     C.c_double, C.c_double, i64, f32, i32, vp],
    "lfs_dp_signal": [i32, C.POINTER(C.c_void_p), i32, i32, i32, vp],
    "lfs_dp_wait": [i32, vp, i32, i32, C.c_uint64, vp, vp],
    "lfs_dp_barrier": [i32, C.POINTER(C.c_void_p), i32, i32, i32, C.c_uint64, vp, vp],
    "lfs_dp_sh_rank1_adam_broadcast": [i32, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), vp, i32, i32, i32, i64, i64, vp, vp, f32,
                                       C.c_double, C.c_double, C.c_double, i64, f32, i32, vp],
    "lfs_mcmc_classify": [i32, vp, vp, f32, vp, vp, vp, vp, vp, sz, vp],
    "lfs_mcmc_classify_noalloc": [i32, vp, vp, f32, vp, vp, vp, vp, vp],
    "lfs_mcmc_map_indices": [i32, vp, vp, vp, vp],
    "lfs_mcmc_gather_ratios": [i32, i32, vp, vp, vp, i32, vp, vp, vp, vp, vp],
    "lfs_mcmc_apply": [i32, i32, i32, vp, vp, vp, vp, f32, C.POINTER(Splats), C.POINTER(Splats), C.POINTER(Splats), vp],
}
_SIZE_FUNCS = {
    "lfs_intersect_tile_workspace_bytes": [i32, i32, i64],
    "lfs_rasterize_workspace_bytes": [i32],
    "lfs_render_workspace_bytes": [C.POINTER(RenderConfig)],
    "lfs_ewa_workspace_bytes": [C.POINTER(EwaConfig)],
    "lfs_photometric_loss_workspace_bytes": [i32, i32],
    "lfs_mcmc_workspace_bytes": [i32],
}
EXPORTED = sorted(list(_SIGNATURES) + list(_SIZE_FUNCS) + ["lfs_last_error", "lfs_build_info", "lfs_profile_enable",
                                                          "lfs_profile_collect"])


def lib():
    """Loads the shared library once. Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise LfsError(f"{LIB_PATH} is missing: run `python lichtfeld-studio_b200/build.py` (needs nvcc). "
                           "There is no CPU or PyTorch fallback.")
        l = C.CDLL(str(LIB_PATH))
        for name, args in _SIGNATURES.items():
            fn = getattr(l, name)
            fn.argtypes, fn.restype = args, C.c_int
        for name, args in _SIZE_FUNCS.items():
            fn = getattr(l, name)
            fn.argtypes, fn.restype = args, C.c_size_t
        l.lfs_last_error.restype = C.c_char_p
        l.lfs_build_info.restype = C.c_char_p
        _lib = l
    return _lib


def call(name: str, *args):
    rc = getattr(lib(), name)(*args)
    if rc != LFS_OK:
        raise LfsError(f"{name} failed ({rc}): {lib().lfs_last_error().decode()}")


def profile_enable(on: bool, nvtx: bool = False):
    """on: CUDA events around every launch (profile_collect); nvtx: an NVTX range of the same name around every launch."""
    rc = lib().lfs_profile_enable((1 if on else 0) | (2 if nvtx else 0))
    if rc != LFS_OK:
        raise LfsError(f"lfs_profile_enable failed ({rc})")


def profile_collect(max_records: int = 4096):
    """[(kernel name, milliseconds)] in launch order since profile_enable(True)."""
    names = (C.c_char_p * max_records)()
    ms = (C.c_float * max_records)()
    n = lib().lfs_profile_collect(max_records, names, ms)
    return [(names[i].decode(), float(ms[i])) for i in range(n)]


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else C.c_void_p(t.data_ptr())


def splats_struct(d) -> Splats:
    return Splats(*(d[k].data_ptr() if d.get(k) is not None else None
                    for k in ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")))
