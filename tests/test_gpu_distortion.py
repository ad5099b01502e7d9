"""OpenCV pinhole distortion (radial k1..k6, tangential p1 p2, thin prism s1..s4; gsplat/Cameras.cuh:474-755) in the
unscented-transform projection (forward model) and the rasterizer's pixel rays (Newton inversion), at the operator
level and through the fused path, against the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import make_scene, rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAMES = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")

RADIAL = np.array([-0.22, 0.06, -0.004, 0.01, 0.002, 0.0], np.float32)
TANGENTIAL = np.array([0.0015, -0.002], np.float32)
THIN_PRISM = np.array([0.0008, 0.0, -0.0005, 0.0002], np.float32)
CASES = [
    dict(radial=RADIAL, tangential=TANGENTIAL, thin_prism=THIN_PRISM),   # FULL_OPENCV + thin prism
    dict(radial=RADIAL[:2], tangential=TANGENTIAL, thin_prism=None),     # COLMAP OPENCV: 2 + 2 coefficients
    dict(radial=RADIAL[:1], tangential=None, thin_prism=None),           # SIMPLE_RADIAL
    dict(radial=None, tangential=TANGENTIAL, thin_prism=None),           # only one of the three tensors present
]


def T(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def check_image(a, b, tol=1e-4):
    diff = np.abs(a - b).reshape(a.shape[0] * a.shape[1], -1).max(-1)
    assert (diff > tol).sum() <= 2 and np.quantile(diff, 0.9999) < tol, diff.max()


@pytest.mark.parametrize("case", CASES)
def test_projection_with_distortion_is_bit_exact(pkg, orc, synth, case):
    P = synth.make_gaussians(20000, 5, "cube", 0)
    q, _ = orc.act_quat(P["rotation_raw"])
    s, o = orc.act_scale(P["scaling_raw"]) * 3, orc.act_opacity(P["opacity_raw"])
    vm = synth.look_at_origin([0.4, -1.9, 0.6])[None]   # close: wide field of view, strong distortion at the borders
    K = synth.intrinsics(210.0, 205.0, 162.0, 118.0)[None]
    W, H = 320, 240
    dist = orc.pack_distortion(**case)
    ref = orc.projection_ut_3dgs_fused(P["means"], q, s, o, vm, K, W, H, camera_model=0, radial_coeffs=dist[None])
    b = lambda a: None if a is None else T(np.asarray(a, np.float32)[None])
    out = pkg.ops.projection_ut_3dgs_fused(T(P["means"]), T(q), T(s), T(o), T(vm), None, T(K), W, H, 0.3, 0.01, 1e4, 0.0, False, 0,
                                           radial_coeffs=b(case["radial"]), tangential_coeffs=b(case["tangential"]),
                                           thin_prism_coeffs=b(case["thin_prism"]))
    assert np.array_equal(out[0].cpu().numpy(), ref[0])
    vis = (ref[0][0] > 0).all(-1)
    assert 2000 < vis.sum() < vis.size
    for k in (1, 2, 3):
        assert np.array_equal(out[k].cpu().numpy()[0][vis].view(np.uint32), ref[k][0][vis].view(np.uint32)), k
    # the distortion really moved things: compare with the distortion-free projection
    plain = orc.projection_ut_3dgs_fused(P["means"], q, s, o, vm, K, W, H)
    both = vis & (plain[0][0] > 0).all(-1)
    assert np.abs(plain[1][0][both] - ref[1][0][both]).max() > 1.0


@pytest.mark.parametrize("case,mode", [(CASES[0], 0), (CASES[1], 3), (CASES[2], 0)])
def test_fused_path_with_distortion(pkg, orc, synth, case, mode):
    tr = pkg.trainer
    n, W, H, deg = 12000, 200, 150, 2
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=8, fx=140.0)
    dist = orc.pack_distortion(**case)
    CH = 3 if mode == 0 else 4
    bg = np.array([0.1, 0.3, 0.2, 0.0], np.float32)[:CH]
    fwd = orc.render_fwd(P, vm, K, W, H, deg, background=bg, radial=dist, render_mode=mode)
    model = tr.SplatData(n, (deg + 1) ** 2, DEV).load(P)
    grads = model.like()
    rast = tr.Rasterizer(model, W, H, deg, render_mode=mode)
    cam = tr.Camera(T(vm), T(K), W, H, radial=T(case["radial"]), tangential=T(case["tangential"]), thin_prism=T(case["thin_prism"]))
    out = rast.forward(cam, T(bg))
    st = rast.state()
    assert np.array_equal(st["radii"].cpu().numpy(), fwd["radii"])
    assert np.array_equal(st["flatten_ids"].cpu().numpy(), fwd["flatten_ids"])
    assert np.array_equal(st["tile_offsets"].cpu().numpy()[:-1], fwd["tile_offsets"].reshape(-1))
    check_image(out.image.cpu().numpy(), fwd["image"])
    check_image(out.alpha.cpu().numpy(), fwd["alpha"])
    rng = np.random.default_rng(2)
    v_r = rng.normal(size=(H, W, CH)).astype(np.float32) * 1e-3
    if CH == 4:
        v_r[..., -1] /= max(1.0, float(fwd["depths"][fwd["masks"]].max()))
    v_a = rng.normal(size=(H, W, 1)).astype(np.float32) * 1e-3
    bwd = orc.render_bwd(P, fwd, vm, K, W, H, deg, v_r, v_a, background=bg, radial=dist)
    rast.backward(T(v_r), grads, T(bg), T(v_a))
    for name in NAMES:
        assert rel_l2(grads.tensor(name).cpu().numpy(), bwd[name]) < 1e-3, name
    # the same camera without distortion gives a visibly different picture
    plain = orc.render_fwd(P, vm, K, W, H, deg, background=bg, render_mode=mode)
    assert np.abs(plain["image"] - fwd["image"]).max() > 0.05


def test_zero_coefficients_equal_the_plain_pinhole(pkg, synth):
    """All-zero coefficient tensors select the OpenCV model (as in the reference) and must draw the same picture:
    the Newton inversion starts at the solution."""
    tr = pkg.trainer
    n, W, H, deg = 8000, 160, 120, 1
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=1)
    model = tr.SplatData(n, (deg + 1) ** 2, DEV).load(P)
    rast = tr.Rasterizer(model, W, H, deg)
    a = rast.forward(tr.Camera(T(vm), T(K), W, H), None).image.clone()
    b = rast.forward(tr.Camera(T(vm), T(K), W, H, radial=torch.zeros(4, device=DEV)), None).image.clone()
    assert float((a - b).abs().max()) < 1e-5


def test_operator_rasterize_with_distortion(pkg, orc, synth):
    n, W, H, deg = 6000, 150, 100, 1
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=4, fx=110.0)
    case = CASES[0]
    dist = orc.pack_distortion(**case)
    fwd = orc.render_fwd(P, vm, K, W, H, deg, radial=dist)
    means, q, s, o, col = P["means"], fwd["quats"], fwd["scales"], fwd["opac"], fwd["colors"]
    b = lambda a: T(np.asarray(a, np.float32)[None])
    args = [T(means), T(q), T(s), T(col[None]), T(o[None]), None, None, W, H, 16, T(vm[None]), None, T(K[None]), 0]
    kw = dict(radial_coeffs=b(case["radial"]), tangential_coeffs=b(case["tangential"]), thin_prism_coeffs=b(case["thin_prism"]),
              tile_offsets=T(fwd["tile_offsets"][None]), flatten_ids=T(fwd["flatten_ids"]))
    ren, alp, last = pkg.ops.rasterize_to_pixels_from_world_3dgs_fwd(*args, **kw)
    check_image(ren.cpu().numpy()[0], fwd["render"])
    rng = np.random.default_rng(1)
    v_r = rng.normal(size=(H, W, 3)).astype(np.float32) * 1e-3
    v_a = rng.normal(size=(H, W, 1)).astype(np.float32) * 1e-3
    ref = orc.rasterize_bwd(means, q, s, col, o, None, W, H, 16, vm, K, fwd["tile_offsets"], fwd["flatten_ids"], fwd["alpha"],
                            fwd["last_ids"], v_r, v_a, radial=dist)
    out = pkg.ops.rasterize_to_pixels_from_world_3dgs_bwd(*args, **kw, render_alphas=T(fwd["alpha"][None]),
                                                          last_ids=T(fwd["last_ids"][None]), v_render_colors=T(v_r[None]),
                                                          v_render_alphas=T(v_a[None]))
    for name, a, r in zip(("v_means", "v_quats", "v_scales", "v_colors", "v_opacities"), out, ref[:5]):
        assert rel_l2(a.cpu().numpy().reshape(r.shape), r) < 1e-3, name
