"""Writes tests/golden/tiny_step.npz: inputs and oracle outputs of one small training step, used as a regression
anchor for the oracle (CPU test) and as a second check of the CUDA path (GPU test).

The reference project ships no golden vectors for this path and its CUDA sources cannot be built or run where this
script runs, so these vectors come from the CPU oracle (oracle/lfs_oracle.cpp), not from the reference itself:
they pin the oracle against drift, they do not pin it to the reference.

Run from the repository root:  python tests/golden/make_golden.py"""
import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def build():
    from oracle import oracle as orc
    orc.build()
    synth = importlib.import_module("lichtfeld-studio_b200").synth
    n, W, H, deg = 512, 64, 48, 2
    cfg = dict(n=n, layout="cube", sh_degree=deg, W=W, H=H, fx=80.0, n_poses=1, radius=4.0, model=0)
    P = synth.make_gaussians(n, 42, "cube", deg)
    P["scaling_raw"] = (P["scaling_raw"] + np.float32(2.0)).astype(np.float32)   # larger splats: longer tile lists
    poses, K = synth.make_cameras(cfg)
    vm = poses[0]
    bg = np.array([0.15, 0.25, 0.05], np.float32)
    out = {f"in_{k}": v for k, v in P.items()}
    out.update(in_viewmat=vm, in_K=K, in_bg=bg, in_size=np.array([W, H, deg], np.int32))
    fwd = orc.render_fwd(P, vm, K, W, H, deg, background=bg)
    rng = np.random.default_rng(7)
    target = rng.random((3, H, W)).astype(np.float32)
    loss, g, l1, ssim = orc.photometric_loss(fwd["render"], target, 0.2)
    bwd = orc.render_bwd(P, fwd, vm, K, W, H, deg, g, background=bg)
    out.update(in_target=target, radii=fwd["radii"], means2d=fwd["means2d"], depths=fwd["depths"], visible=fwd["masks"],
               tiles_per_gauss=fwd["tiles_per_gauss"], flatten_ids=fwd["flatten_ids"], tile_offsets=fwd["tile_offsets"],
               render=fwd["render"], alpha=fwd["alpha"], last_ids=fwd["last_ids"], loss=np.array([loss, l1, ssim], np.float32),
               v_render=g)
    for k in ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw"):
        out[f"grad_{k}"] = bwd[k]
    # distorted camera and depth mode: lists and images only
    dist = orc.pack_distortion([-0.2, 0.05], [0.001, -0.002], None)
    fd = orc.render_fwd(P, vm, K, W, H, deg, background=np.append(bg, 0).astype(np.float32), radial=dist, render_mode=4)
    out.update(in_dist=dist, dist_radii=fd["radii"], dist_flatten_ids=fd["flatten_ids"], dist_render=fd["render"], dist_depth=fd["depth"])
    # MCMC relocation and one Adam step
    ratios = (1 + np.arange(64) % 9).astype(np.int32)
    op = (0.05 + 0.9 * rng.random(64)).astype(np.float32)
    sc = np.exp(rng.normal(-3, 0.5, size=(64, 3))).astype(np.float32)
    no, ns = orc.relocation(op, sc, ratios, orc.binoms_table(51), 51)
    out.update(in_reloc_opacity=op, in_reloc_scale=sc, in_reloc_ratios=ratios, reloc_opacity=no, reloc_scale=ns)
    p = rng.normal(size=257).astype(np.float32); m = (rng.normal(size=257) * 1e-2).astype(np.float32)
    v = (rng.random(257) * 1e-4).astype(np.float32); gr = (rng.normal(size=257) * 1e-2).astype(np.float32)
    out.update(in_adam_p=p.copy(), in_adam_m=m.copy(), in_adam_v=v.copy(), in_adam_g=gr)
    orc.adam_step(p, m, v, gr, 1e-3, 0.9, 0.999, 1e-15, 5)
    out.update(adam_p=p, adam_m=m, adam_v=v)
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tiny_step.npz")
    np.savez_compressed(path, **build())
    print(path, os.path.getsize(path), "bytes")
