"""Rolling shutter (gsplat/Cameras.cuh:253-413: pose interpolated by image row / column, iterative projection of the
sigma points, per-pixel ray origins) at the operator level and through the fused path, against the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import make_scene, rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAMES = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")


def T(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def end_pose(vm, dt=(0.25, -0.10, 0.05), angle=0.04):
    c, s = np.cos(angle), np.sin(angle)
    Rz = np.array([[c, -s, 0], [s, c, 0], [0, 0, 1]], np.float32)
    vm1 = vm.copy()
    vm1[:3, :3] = Rz @ vm[:3, :3]
    vm1[:3, 3] = vm[:3, 3] + np.array(dt, np.float32)
    return vm1


def check_image(a, b, tol=1e-4):
    diff = np.abs(a - b).reshape(a.shape[0] * a.shape[1], -1).max(-1)
    assert (diff > tol).sum() <= 2 and np.quantile(diff, 0.9999) < tol, diff.max()


@pytest.mark.parametrize("rs_type,model", [(0, 0), (1, 0), (2, 2), (3, 0), (4, 0)])
def test_projection_with_rolling_shutter(pkg, orc, synth, rs_type, model):
    P = synth.make_gaussians(12000, 5, "cube", 0)
    q, _ = orc.act_quat(P["rotation_raw"])
    s, o = orc.act_scale(P["scaling_raw"]) * 3, orc.act_opacity(P["opacity_raw"])
    vm = synth.look_at_origin([0.4, -2.4, 0.6])
    vm1 = end_pose(vm)
    K = synth.intrinsics(210.0, 205.0, 162.0, 118.0) if model == 0 else synth.intrinsics(120.0, 120.0, 160.0, 120.0)
    W, H = 320, 240
    with orc.shutter(vm1, rs_type):
        ref = orc.projection_ut_3dgs_fused(P["means"], q, s, o, vm[None], K[None], W, H, camera_model=model)
    out = pkg.ops.projection_ut_3dgs_fused(T(P["means"]), T(q), T(s), T(o), T(vm[None]), T(vm1[None]), T(K[None]), W, H, 0.3, 0.01,
                                           1e4, 0.0, False, model, rs_type=rs_type)
    # slerp's acos / sin and (fisheye) atan2 go through double on both sides: allow a vanishing number of last-bit flips
    mism = (out[0].cpu().numpy() != ref[0]).any(-1).sum()
    assert mism <= 2, mism
    vis = (ref[0][0] > 0).all(-1) & (out[0].cpu().numpy()[0] > 0).all(-1)
    assert vis.sum() > 2000
    assert np.abs(out[1].cpu().numpy()[0][vis] - ref[1][0][vis]).max() < 2e-3
    assert np.abs(out[2].cpu().numpy()[0][vis] - ref[2][0][vis]).max() < 1e-5
    plain = orc.projection_ut_3dgs_fused(P["means"], q, s, o, vm[None], K[None], W, H, camera_model=model)
    both = vis & (plain[0][0] > 0).all(-1)
    if rs_type != 4:   # a global shutter projects with the start pose (only the depth comes from the centre pose)
        assert np.abs(plain[1][0][both] - ref[1][0][both]).max() > 1.0    # the motion moved the projections
    else:
        assert np.array_equal(plain[1][0][both], ref[1][0][both]) and np.abs(plain[2][0][both] - ref[2][0][both]).max() > 1e-3


@pytest.mark.parametrize("shutter,mode", [(1, 0), (2, 0), (1, 3)])
def test_fused_path_with_rolling_shutter(pkg, orc, synth, shutter, mode):
    tr = pkg.trainer
    n, W, H, deg = 10000, 176, 128, 2
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=8, fx=150.0)
    vm1 = end_pose(vm)
    CH = 3 if mode == 0 else 4
    bg = np.array([0.1, 0.3, 0.2, 0.0], np.float32)[:CH]
    with orc.shutter(vm1, shutter - 1):
        fwd = orc.render_fwd(P, vm, K, W, H, deg, background=bg, render_mode=mode)
    model = tr.SplatData(n, (deg + 1) ** 2, DEV).load(P)
    grads = model.like()
    rast = tr.Rasterizer(model, W, H, deg, render_mode=mode)
    cam = tr.Camera(T(vm), T(K), W, H, shutter=shutter, viewmat_end=T(vm1))
    out = rast.forward(cam, T(bg))
    st = rast.state()
    mism = (st["radii"].cpu().numpy() != fwd["radii"]).any(-1).sum()
    assert mism <= 2, mism
    if mism == 0:
        assert np.array_equal(st["flatten_ids"].cpu().numpy(), fwd["flatten_ids"])
        check_image(out.image.cpu().numpy(), fwd["image"])
        check_image(out.alpha.cpu().numpy(), fwd["alpha"])
        rng = np.random.default_rng(2)
        v_r = rng.normal(size=(H, W, CH)).astype(np.float32) * 1e-3
        if CH == 4:
            v_r[..., -1] /= max(1.0, float(fwd["depths"][fwd["masks"]].max()))
        v_a = rng.normal(size=(H, W, 1)).astype(np.float32) * 1e-3
        with orc.shutter(vm1, shutter - 1):
            bwd = orc.render_bwd(P, fwd, vm, K, W, H, deg, v_r, v_a, background=bg)
        rast.backward(T(v_r), grads, T(bg), T(v_a))
        for name in NAMES:
            assert rel_l2(grads.tensor(name).cpu().numpy(), bwd[name]) < 1e-3, name
    plain = orc.render_fwd(P, vm, K, W, H, deg, background=bg, render_mode=mode)
    assert np.abs(plain["image"] - fwd["image"]).max() > 0.05


def test_end_pose_equal_to_start_pose_is_the_global_render(pkg, synth):
    tr = pkg.trainer
    n, W, H, deg = 6000, 128, 96, 1
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=1)
    model = tr.SplatData(n, 4, DEV).load(P)
    rast = tr.Rasterizer(model, W, H, deg)
    a = rast.forward(tr.Camera(T(vm), T(K), W, H), None).image.clone()
    b = rast.forward(tr.Camera(T(vm), T(K), W, H, shutter=1, viewmat_end=T(vm)), None).image.clone()
    assert float((a - b).abs().max()) < 2e-5
