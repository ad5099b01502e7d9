"""Writes reference_step.npz: outputs of the REFERENCE'S OWN CUDA build (oracle/_ref/lfs_reference.so, the reference's
unmodified kernels compiled by oracle/ref_build.py) for the inputs stored in tiny_step.npz (one small training step
of 512 Gaussians at 64x48, SH degree 2), plus its relocation, Adam, SSIM and EWA results on seeded inputs and an
equirectangular render of the same Gaussians from inside the scene. These are
the vectors that pin the CPU oracle to the reference where no GPU is available (tests/test_cpu.py) and a second
anchor for the CUDA library (tests/test_gpu_golden.py).

Needs a GPU and the built reference module:

    python tests/golden/make_reference_golden.py [output.npz]      (default: tests/golden/reference_step.npz)
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
NAMES = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")


def build():
    import torch
    from oracle import reference as R
    ref = R.load()
    dev = "cuda:0"
    T = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    g = np.load(os.path.join(HERE, "tiny_step.npz"))
    P = {k: g[f"in_{k}"] for k in NAMES}
    W, H, deg = (int(x) for x in g["in_size"])
    vm, K, bg, target = g["in_viewmat"], g["in_K"], g["in_bg"], g["in_target"]
    out = {}
    # operator by operator, on the activated parameters
    means, q, s, o, sh = R.activated(P)
    vmt, Kt = T(vm[None]), T(K[None])
    radii, means2d, depths, conics, comps = ref.projection_ut_3dgs_fused(means, q, s, o, vmt, None, Kt, W, H, 0.3, 0.01, 1e4, 0.0, True, 0,
                                                                         None, 4, None, None, None)
    tw, th = (W + 15) // 16, (H + 15) // 16
    tiles_per_gauss, isect_ids, flatten_ids = ref.intersect_tile(means2d, radii, depths, None, None, 1, 16, tw, th, True)
    tile_offsets = ref.intersect_offset(isect_ids, 1, tw, th)
    vis = (radii > 0).all(-1)
    out.update(radii=radii[0].cpu().numpy(), visible=vis[0].cpu().numpy(), means2d=means2d[0].cpu().numpy(), depths=depths[0].cpu().numpy(),
               conics=conics[0].cpu().numpy(), compensations=comps[0].cpu().numpy(), tiles_per_gauss=tiles_per_gauss[0].cpu().numpy(),
               isect_ids=isect_ids.cpu().numpy(), flatten_ids=flatten_ids.cpu().numpy(), tile_offsets=tile_offsets[0].cpu().numpy())
    # the training step through the reference's autograd nodes
    r = R.step_outputs(P, vm, K, W, H, deg, bg, target, 0.2, True, None)
    out.update(image=r["image"], alpha=r["alpha"], loss=np.float32(r["loss"]))
    for k in NAMES:
        out[f"grad_{k}"] = r[f"grad_{k}"]
    # loss pieces on the stored target
    img = T(np.clip(r["image"], 0, 1)[None])
    tgt = T(target[None])
    ssim_map, dm1, ds1, ds12 = ref.fusedssim(1e-4, 9e-4, img, tgt, True)
    out.update(ssim_map=ssim_map[0].cpu().numpy(), ssim_dm_dmu1=dm1[0].cpu().numpy())
    # the default (EWA) path on the same inputs
    e = R.step_outputs(P, vm, K, W, H, deg, bg, target, 0.2, False, None)
    out.update(ewa_image=e["image"], ewa_alpha=e["alpha"], ewa_loss=np.float32(e["loss"]))
    for k in NAMES:
        out[f"ewa_grad_{k}"] = e[f"grad_{k}"]
    # camera-pose gradient of the EWA path (kernels_backward.cuh:160-173): the same loss with a pose that requires a gradient
    t2 = R.make_trainer(P, [0.0] * 6, deg)
    vm_t = T(vm[None]).clone().requires_grad_(True)
    rr2 = t2.fast_rasterize(vm_t, float(K[0, 0]), float(K[1, 1]), float(K[0, 2]), float(K[1, 2]), W, H, T(bg))
    ref.photometric_loss(rr2.image, T(target), 0.2).backward()
    out.update(ewa_grad_w2c=vm_t.grad[0].cpu().numpy())
    # relocation and Adam on tiny_step's inputs
    from oracle import oracle as orc
    no, ns = ref.relocation(T(g["in_reloc_opacity"]), T(g["in_reloc_scale"]), T(g["in_reloc_ratios"]), T(orc.binoms_table(51)), 51)
    out.update(reloc_opacity=no.cpu().numpy(), reloc_scale=ns.cpu().numpy())
    p, m, v = T(g["in_adam_p"]), T(g["in_adam_m"]), T(g["in_adam_v"])
    ref.adam_step_wrapper(p, m, v, T(g["in_adam_g"]), 1e-3, 0.9, 0.999, 1e-15, float(1.0 / (1.0 - 0.9 ** 5)), float(1.0 / np.sqrt(1.0 - 0.999 ** 5)))
    out.update(adam_p=p.cpu().numpy(), adam_m=m.cpu().numpy(), adam_v=v.cpu().numpy())
    # add_noise and quats_to_rotmats
    rng = np.random.default_rng(11)
    noise = rng.normal(size=P["means"].shape).astype(np.float32)
    moved = T(P["means"].copy())
    ref.add_noise(T(P["opacity_raw"]), T(P["scaling_raw"]), T(P["rotation_raw"]), T(noise), moved, 80.0)
    out.update(in_noise=noise, noise_means=moved.cpu().numpy(), rotmats=ref.quats_to_rotmats(T(P["rotation_raw"])).cpu().numpy())
    # EQUIRECTANGULAR camera (gsplat/Cameras.cuh:1003-1039) with the camera INSIDE the cube of Gaussians, so that the back
    # hemisphere (negative depths) is populated: the reference's rasterize() from the raw parameters, 64x32
    eq_vm = np.eye(4, dtype=np.float32)
    eq_vm[:3, 3] = [0.05, -0.02, 0.1]
    We, He = 64, 32
    t = R.make_trainer(P, [0.0] * 6, deg)
    rr = t.render_no_grad(True, T(eq_vm[None]), Kt, We, He, T(bg), 3)
    pe = ref.projection_ut_3dgs_fused(means, q, s, o, T(eq_vm[None]), None, Kt, We, He, 0.3, 0.01, 1e4, 0.0, False, 3, None, 4, None, None, None)
    out.update(eq_viewmat=eq_vm, eq_size=np.array([We, He], np.int32), eq_image=rr.image.cpu().numpy(), eq_alpha=rr.alpha.cpu().numpy(),
               eq_radii=pe[0][0].cpu().numpy(), eq_means2d=pe[1][0].cpu().numpy(), eq_depths=pe[2][0].cpu().numpy())
    torch.cuda.synchronize()
    return out


if __name__ == "__main__":
    path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_step.npz")
    np.savez_compressed(path, **build())
    print(path, os.path.getsize(path), "bytes")
