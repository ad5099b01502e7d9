"""Seeded synthetic scenes, cameras and targets with the shapes and value distributions of the
benchmark configurations (stand-ins for the Mip-NeRF-360 inputs the reference's eval scripts use;
nothing from that dataset is reproduced).

Random numbers come from a counter-based SplitMix64 stream per (seed, tensor id): uniform = top 24
bits / 2^24, normal = Box-Muller using both outputs in order. Everything is float32, row-major, in
the reference's SplatData layouts (src/core/splat_data.hpp:104-109): means [N,3], sh0 [N,1,3],
shN [N,K-1,3], scaling_raw [N,3] (log), rotation_raw [N,4] (wxyz, unnormalised), opacity_raw [N,1]
(logit).
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = x + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _stream(seed: int, tensor_id: int, n: int) -> np.ndarray:
    base = _splitmix64(np.array([seed * 1000003 + tensor_id], dtype=np.uint64))[0]
    with np.errstate(over="ignore"):
        ctr = base + np.arange(1, n + 1, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15)
    return _splitmix64(ctr)


def uniform(seed: int, tensor_id: int, n: int) -> np.ndarray:
    """U[0,1) with 24-bit resolution, float32."""
    return ((_stream(seed, tensor_id, n) >> np.uint64(40)).astype(np.float32) / np.float32(1 << 24))


def normal(seed: int, tensor_id: int, n: int) -> np.ndarray:
    """Standard normal, float32, Box-Muller on consecutive uniform pairs."""
    m = (n + 1) // 2
    bits = _stream(seed, tensor_id, 2 * m) >> np.uint64(40)
    u1 = (bits[0::2].astype(np.float64) + 1.0) / float(1 << 24)  # (0,1]
    u2 = bits[1::2].astype(np.float64) / float(1 << 24)
    r = np.sqrt(-2.0 * np.log(u1))
    out = np.empty(2 * m, np.float64)
    out[0::2] = r * np.cos(2.0 * np.pi * u2)
    out[1::2] = r * np.sin(2.0 * np.pi * u2)
    return out[:n].astype(np.float32)


# tensor ids
_T_MEANS, _T_SCALE, _T_QUAT, _T_OPAC, _T_SH0, _T_SHN, _T_CENTRES = range(7)


def make_gaussians(n: int, seed: int, layout: str, sh_degree: int) -> dict:
    """layout: 'cube' (cfg1: U[-1,1]^3, log-scale N(-4,0.5), logit N(0,1)),
    'clusters' (cfg2-4: 64 isotropic clusters sigma 0.3 in [-3,3]^3, log-scale N(-4.5,0.6),
    logit N(-1,1)), 'wide' (cfg5: U[-10,10]^3, log-scale N(-5,0.7), logit N(-1,1))."""
    K = (sh_degree + 1) ** 2
    if layout == "cube":
        means = uniform(seed, _T_MEANS, 3 * n).reshape(n, 3) * np.float32(2.0) - np.float32(1.0)
        ls_mu, ls_sd, op_mu = -4.0, 0.5, 0.0
    elif layout == "clusters":
        centres = uniform(seed, _T_CENTRES, 64 * 3).reshape(64, 3) * np.float32(4.2) - np.float32(2.1)
        means = centres[np.arange(n) % 64] + normal(seed, _T_MEANS, 3 * n).reshape(n, 3) * np.float32(0.3)
        means = np.clip(means, -3.0, 3.0).astype(np.float32)
        ls_mu, ls_sd, op_mu = -4.5, 0.6, -1.0
    elif layout == "wide":
        means = uniform(seed, _T_MEANS, 3 * n).reshape(n, 3) * np.float32(20.0) - np.float32(10.0)
        ls_mu, ls_sd, op_mu = -5.0, 0.7, -1.0
    else:
        raise ValueError(layout)
    scaling_raw = (normal(seed, _T_SCALE, 3 * n).reshape(n, 3) * np.float32(ls_sd) + np.float32(ls_mu))
    rotation_raw = normal(seed, _T_QUAT, 4 * n).reshape(n, 4)
    rotation_raw = rotation_raw / np.maximum(np.linalg.norm(rotation_raw, axis=1, keepdims=True), 1e-12)
    opacity_raw = (normal(seed, _T_OPAC, n).reshape(n, 1) + np.float32(op_mu))
    sh0 = normal(seed, _T_SH0, 3 * n).reshape(n, 1, 3) * np.float32(0.5)
    shN = normal(seed, _T_SHN, 3 * n * (K - 1)).reshape(n, K - 1, 3) * np.float32(0.05)
    f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)
    return dict(means=f32(means), sh0=f32(sh0), shN=f32(shN), scaling_raw=f32(scaling_raw),
                rotation_raw=f32(rotation_raw), opacity_raw=f32(opacity_raw))


def look_at_origin(pos) -> np.ndarray:
    """World-to-camera [R|t] (row-major 4x4) of a camera at `pos` looking at the origin, z-up world:
    forward f = -p/|p|, right r = norm(f x up), down d = f x r, R rows = (r, d, f), t = -R p."""
    p = np.asarray(pos, np.float64)
    fwd = -p / np.linalg.norm(p)
    up = np.array([0.0, 0.0, 1.0])
    r = np.cross(fwd, up)
    r /= np.linalg.norm(r)
    d = np.cross(fwd, r)
    R = np.stack([r, d, fwd])
    vm = np.eye(4)
    vm[:3, :3] = R
    vm[:3, 3] = -R @ p
    return vm.astype(np.float32)


def hemisphere_poses(n_poses: int, radius: float) -> np.ndarray:
    """Golden-angle spiral on the upper hemisphere: h_i = 0.1 + 0.8 (i + 1/2)/n, phi_i = i * 2.399963."""
    out = np.zeros((n_poses, 4, 4), np.float32)
    for i in range(n_poses):
        h = 0.1 + 0.8 * (i + 0.5) / n_poses
        phi = i * 2.399963
        s = np.sqrt(1.0 - h * h)
        out[i] = look_at_origin(radius * np.array([s * np.cos(phi), s * np.sin(phi), h]))
    return out


def intrinsics(fx, fy, cx, cy) -> np.ndarray:
    return np.array([[fx, 0, cx], [0, fy, cy], [0, 0, 1]], np.float32)


CONFIGS = {
    # name: N, layout, sh_degree, W, H, fx, n_poses, radius, camera_model
    "tiny": dict(n=16384, layout="cube", sh_degree=0, W=256, H=256, fx=300.0, n_poses=1, radius=4.0, model=0),
    "train_1m": dict(n=1_000_000, layout="clusters", sh_degree=3, W=1296, H=840, fx=1150.0, n_poses=200, radius=5.0, model=0),
    "mcmc_3m": dict(n=3_000_000, layout="clusters", sh_degree=3, W=1296, H=840, fx=1150.0, n_poses=200, radius=5.0, model=0),
    "dp_3m": dict(n=3_000_000, layout="clusters", sh_degree=3, W=1600, H=1064, fx=1420.0, n_poses=400, radius=6.0, model=0),
    "wide_4k": dict(n=6_000_000, layout="wide", sh_degree=3, W=3840, H=2160, fx=2800.0, n_poses=32, radius=12.0, model=0),
    "wide_fisheye": dict(n=6_000_000, layout="wide", sh_degree=3, W=1920, H=1920, fx=960.0 / (np.pi / 2), n_poses=32, radius=12.0, model=2),
}


def make_cameras(cfg: dict):
    if cfg["n_poses"] == 1:
        vm = np.eye(4, dtype=np.float32)
        vm[2, 3] = cfg["radius"]  # R = I, t = (0,0,radius): camera at (0,0,-radius) looking at the origin
        poses = vm[None]
    else:
        poses = hemisphere_poses(cfg["n_poses"], cfg["radius"])
    K = intrinsics(cfg["fx"], cfg["fx"], cfg["W"] / 2.0, cfg["H"] / 2.0)
    return poses, K


def pose_index(step: int, n_poses: int) -> int:
    return (step * 7919) % n_poses
