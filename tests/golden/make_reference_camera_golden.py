"""Writes reference_cameras.npz: renders of the REFERENCE'S OWN CUDA build (oracle/_ref/lfs_reference.so, built by
oracle/ref_build.py from the reference's unmodified sources) for the camera features and render modes of
gsplat::rasterize_from_world_with_sh_fwd (gsplat/Rasterization.cpp:279-468) that the training-step golden does not
exercise: OpenCV distortion, fisheye with radial coefficients, rolling shutter, the depth render modes, the antialiased
compensation and the scaling modifier. Inputs are the 512 Gaussians and the 64x48 camera of tiny_step.npz; every case
stores the operator's first two outputs (render_colors, render_alphas) and radii, and for seven of them the gradients of
rasterize_from_world_with_sh_bwd for seeded output gradients. These vectors pin the CPU oracle to the
reference for those features where no GPU is available (tests/test_cpu.py).

Needs a GPU and the built reference module:

    python tests/golden/make_reference_camera_golden.py [output.npz]      (default: tests/golden/reference_cameras.npz)
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
NAMES = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")

RADIAL = np.array([-0.22, 0.06, -0.004, 0.01, 0.002, 0.0], np.float32)
TANGENTIAL = np.array([0.0015, -0.002], np.float32)
THIN_PRISM = np.array([0.0008, 0.0, -0.0005, 0.0002], np.float32)
FISHEYE_RADIAL = np.array([0.03, -0.008, 0.002, 0.0], np.float32)
BG4 = np.array([0.15, 0.25, 0.05, 0.0], np.float32)


def end_pose(vm, dt=(0.25, -0.10, 0.05), angle=0.04):
    c, s = np.cos(angle), np.sin(angle)
    Rz = np.array([[c, -s, 0], [s, c, 0], [0, 0, 1]], np.float32)
    vm1 = vm.copy()
    vm1[:3, :3] = Rz @ vm[:3, :3]
    vm1[:3, 3] = vm[:3, 3] + np.array(dt, np.float32)
    return vm1


# name -> (camera_model, render_mode, antialiased, scaling_modifier, rs_type (4 = global), distortion?, fisheye radial?)
CASES = {
    "dist_full": dict(model=0, mode=0, aa=False, smod=1.0, rs=4, dist=True, fish=False),
    "dist_rgbd": dict(model=0, mode=3, aa=False, smod=1.0, rs=4, dist=True, fish=False),
    "fisheye": dict(model=2, mode=0, aa=False, smod=1.0, rs=4, dist=False, fish=True),
    "rolling_tb": dict(model=0, mode=0, aa=False, smod=1.0, rs=0, dist=False, fish=False),
    "rolling_lr_rgbd": dict(model=0, mode=3, aa=False, smod=1.0, rs=1, dist=False, fish=False),
    "mode_d": dict(model=0, mode=1, aa=False, smod=1.0, rs=4, dist=False, fish=False),
    "mode_ed": dict(model=0, mode=2, aa=False, smod=1.0, rs=4, dist=False, fish=False),
    "mode_rgb_ed_aa": dict(model=0, mode=4, aa=True, smod=1.0, rs=4, dist=False, fish=False),
    "antialiased_smod": dict(model=0, mode=0, aa=True, smod=0.7, rs=4, dist=False, fish=False),
    "antialiased": dict(model=0, mode=0, aa=True, smod=1.0, rs=4, dist=False, fish=False),
}
# cases whose backward (gsplat::rasterize_from_world_with_sh_bwd, gsplat/Rasterization.cpp:470-642) is stored too: the
# operator's gradients w.r.t. means, quats, scales, opacities and SH coefficients for seeded output gradients
BACKWARD_CASES = ("dist_full", "dist_rgbd", "fisheye", "rolling_tb", "rolling_lr_rgbd", "mode_d", "antialiased")


def output_gradients(name, H, W, ch):
    """Seeded v_render [H,W,ch] and v_alpha [H,W,1] of a case (the CPU test draws the same ones)."""
    rng = np.random.default_rng(sum(name.encode()))
    return (rng.normal(size=(H, W, ch)).astype(np.float32) * 1e-2), (rng.normal(size=(H, W, 1)).astype(np.float32) * 1e-3)


def channels(mode):
    return {0: 3, 1: 1, 2: 1, 3: 4, 4: 4}[mode]


def background(mode):
    ch = channels(mode)
    return BG4[:3].copy() if ch == 3 else (BG4[:1].copy() if ch == 1 else BG4.copy())


def build():
    import torch
    from oracle import reference as R
    ref = R.load()
    dev = "cuda:0"
    T = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    g = np.load(os.path.join(HERE, "tiny_step.npz"))
    P = {k: g[f"in_{k}"] for k in NAMES}
    W, H, deg = (int(x) for x in g["in_size"])
    vm, K = g["in_viewmat"], g["in_K"]
    vm1 = end_pose(vm)
    means, q, s, o, sh = R.activated(P)
    out = dict(viewmat_end=vm1, radial=RADIAL, tangential=TANGENTIAL, thin_prism=THIN_PRISM, fisheye_radial=FISHEYE_RADIAL, bg4=BG4)
    for name, c in CASES.items():
        bg = background(c["mode"])
        radial = RADIAL[None] if c["dist"] else (FISHEYE_RADIAL[None] if c["fish"] else None)
        tang = TANGENTIAL[None] if c["dist"] else None
        prism = THIN_PRISM[None] if c["dist"] else None
        res = ref.rasterize_from_world_with_sh_fwd(
            means, q, s, o, sh, deg, T(bg[None]), None, W, H, 16, T(vm[None]), T(vm1[None]) if c["rs"] != 4 else None, T(K[None]),
            c["model"], 0.3, 0.01, 10000.0, 0.0, float(c["smod"]), bool(c["aa"]), int(c["mode"]), None, int(c["rs"]), T(radial), T(tang),
            T(prism))
        out[name + "_render"] = res[0][0].cpu().numpy()
        out[name + "_alpha"] = res[1][0].cpu().numpy()
        out[name + "_radii"] = res[2][0].cpu().numpy()
        if name in BACKWARD_CASES:
            render, alpha, radii, means2d, depths, colors, offsets, flat, last_ids, comps = res
            v_r, v_a = output_gradients(name, H, W, channels(c["mode"]))
            comps_t = comps if comps is not None else torch.empty(0, device=dev)
            b = ref.rasterize_from_world_with_sh_bwd(
                means, q, s, o, sh, deg, T(bg[None]), None, W, H, 16, T(vm[None]), T(vm1[None]) if c["rs"] != 4 else None, T(K[None]),
                c["model"], 0.3, 0.01, 10000.0, 0.0, float(c["smod"]), bool(c["aa"]), int(c["mode"]), None, int(c["rs"]), T(radial), T(tang),
                T(prism), alpha, last_ids, offsets, flat, colors, radii, means2d, depths, comps_t, T(v_r[None]), T(v_a[None]))
            for key, t in zip(("v_means", "v_quats", "v_scales", "v_opacities", "v_sh_coeffs"), b):
                out[f"{name}_{key}"] = t.cpu().numpy()
    torch.cuda.synchronize()
    return out


if __name__ == "__main__":
    path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_cameras.npz")
    np.savez_compressed(path, **build())
    print(path, os.path.getsize(path), "bytes")
