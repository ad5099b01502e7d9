"""Edge cases of the fused paths: no Gaussians, nothing visible, one-pixel and sub-tile images, SH degree 4,
a single Gaussian covering the whole image, repeated forwards on one workspace."""
import numpy as np
import pytest
import torch

from conftest import make_scene, rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAMES = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")


def T(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


@pytest.mark.parametrize("path", ["gut", "ewa"])
def test_no_gaussians_and_nothing_visible(pkg, synth, path):
    tr = pkg.trainer
    W, H = 40, 24
    cfg, P, vm, K = make_scene(synth, 64, W, H, 1, seed=0)
    bg = torch.tensor([0.2, 0.4, 0.6], device=DEV)
    make = (lambda m: tr.Rasterizer(m, W, H, 1)) if path == "gut" else (lambda m: tr.FastRasterizer(m, W, H, 1))
    expect = (lambda img: img) if path == "gut" else (lambda img: img.permute(1, 2, 0))
    # capacity reserved but no live rows
    model = tr.SplatData(0, 4, DEV, capacity=64)
    rast = make(model)
    out = rast.forward(tr.Camera(T(vm), T(K), W, H), bg)
    assert torch.allclose(expect(out.image), bg.expand(H, W, 3)) and float(out.alpha.abs().max()) == 0
    assert out.status.cpu().tolist()[:3] == [0, 0, 0]
    grads = model.like()
    g = torch.ones_like(out.image)
    rast.backward(g, grads, bg)
    # everything behind the camera
    P["means"][:, 2] = -50.0
    model = tr.SplatData(64, 4, DEV).load(P)
    rast = make(model)
    out = rast.forward(tr.Camera(T(vm), T(K), W, H), bg)
    assert torch.allclose(expect(out.image), bg.expand(H, W, 3)) and out.status.cpu().tolist()[:3] == [0, 0, 0]
    grads = model.like()
    grads.flat.fill_(7.0)
    rast.backward(torch.ones_like(out.image), grads, bg)
    assert float(grads.flat[: 64 * model.row_floats].abs().max()) == 0.0   # overwritten with zeros


@pytest.mark.parametrize("W,H", [(1, 1), (5, 3), (17, 16), (16, 33)])
def test_small_and_ragged_images(pkg, orc, synth, W, H):
    tr = pkg.trainer
    n, deg = 300, 2
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=3, fx=12.0)
    P["scaling_raw"] += 1.0
    bg = np.array([0.3, 0.2, 0.1], np.float32)
    model = tr.SplatData(n, 9, DEV).load(P)
    # gut path
    fwd = orc.render_fwd(P, vm, K, W, H, deg, background=bg)
    rast = tr.Rasterizer(model, W, H, deg)
    out = rast.forward(tr.Camera(T(vm), T(K), W, H), T(bg))
    assert np.abs(out.image.cpu().numpy() - fwd["render"]).max() < 2e-4
    rng = np.random.default_rng(0)
    v = rng.normal(size=(H, W, 3)).astype(np.float32)
    bwd = orc.render_bwd(P, fwd, vm, K, W, H, deg, v, background=bg)
    grads = model.like()
    rast.backward(T(v), grads, T(bg))
    for name in NAMES:
        assert rel_l2(grads.tensor(name).cpu().numpy(), bwd[name]) < 2e-3, name
    # EWA path
    f2 = orc.ewa_forward(P, vm, orc.campos(vm), W, H, K[0, 0], K[1, 1], K[0, 2], K[1, 2], 9, background=bg)
    fr = tr.FastRasterizer(model, W, H, deg)
    o2 = fr.forward(tr.Camera(T(vm), T(K), W, H), T(bg))
    assert np.abs(o2.image.cpu().numpy() - f2["image"]).max() < 2e-4
    v2 = np.ascontiguousarray(v.transpose(2, 0, 1))
    b2 = orc.ewa_backward(P, f2, v2)
    g2 = model.like()
    fr.backward(T(v2), g2, T(bg))
    for name in NAMES:
        assert rel_l2(g2.tensor(name).cpu().numpy(), b2[name]) < 2e-3, name


def test_sh_degree_four_and_repeated_forwards(pkg, orc, synth):
    tr = pkg.trainer
    n, W, H, deg = 2000, 96, 64, 4
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=5)
    model = tr.SplatData(n, 25, DEV).load(P)
    rast = tr.Rasterizer(model, W, H, deg)
    cam = tr.Camera(T(vm), T(K), W, H)
    fwd = orc.render_fwd(P, vm, K, W, H, deg)
    imgs = [rast.forward(cam, None).image.clone() for _ in range(3)]
    assert torch.equal(imgs[0], imgs[1]) and torch.equal(imgs[1], imgs[2])   # same workspace, bit-identical
    assert np.abs(imgs[0].cpu().numpy() - fwd["render"]).max() < 2e-4
    v = np.random.default_rng(1).normal(size=(H, W, 3)).astype(np.float32)
    bwd = orc.render_bwd(P, fwd, vm, K, W, H, deg, v)
    grads = model.like()
    rast.backward(T(v), grads)
    for name in NAMES:
        assert rel_l2(grads.tensor(name).cpu().numpy(), bwd[name]) < 1e-3, name


def test_one_huge_gaussian_covers_every_tile(pkg, orc, synth):
    """A Gaussian larger than the image lands in every tile list (gut: radius box; EWA: exact test says yes everywhere)."""
    tr = pkg.trainer
    W, H = 130, 70
    cfg, P, vm, K = make_scene(synth, 4, W, H, 0, seed=1)
    P["means"][:] = 0.0
    P["means"][1:, 2] = -100.0           # the other three are behind the camera
    P["scaling_raw"][0] = np.log(3.0)
    P["opacity_raw"][0] = 2.0
    model = tr.SplatData(4, 1, DEV).load(P)
    tiles = ((W + 15) // 16) * ((H + 15) // 16)
    for rast in (tr.Rasterizer(model, W, H, 0), tr.FastRasterizer(model, W, H, 0)):
        out = rast.forward(tr.Camera(T(vm), T(K), W, H), None)
        assert out.status.cpu().tolist()[:3] == [0, tiles, 1]
        assert float(out.alpha.min()) > 0.5


def test_profiling_modes(pkg, synth):
    """lfs_profile_enable: CUDA-event records per launch, NVTX ranges (no records; free without an attached profiler), both,
    and a rejected flag value. The images do not depend on the mode."""
    tr, capi = pkg.trainer, pkg._capi
    W, H = 96, 64
    cfg, P, vm, K = make_scene(synth, 3000, W, H, 1, seed=1)
    model = tr.SplatData(3000, 4, DEV).load(P)
    rast = tr.Rasterizer(model, W, H, 1)
    cam, bg = tr.Camera(T(vm), T(K), W, H), torch.zeros(3, device=DEV)
    base = rast.forward(cam, bg).image.clone()
    try:
        capi.profile_enable(True)
        img = rast.forward(cam, bg).image.clone()
        recs = capi.profile_collect()
        assert torch.equal(img, base) and {"project_pack", "raster_fwd"} <= {n for n, _ in recs} and all(ms >= 0 for _, ms in recs)
        capi.profile_enable(False, nvtx=True)
        img = rast.forward(cam, bg).image.clone()
        assert torch.equal(img, base) and capi.profile_collect() == []
        capi.profile_enable(True, nvtx=True)
        rast.forward(cam, bg)
        assert len(capi.profile_collect()) == len(recs)
        assert capi.lib().lfs_profile_enable(4) == capi.LFS_EINVAL
    finally:
        capi.profile_enable(False)
    assert capi.profile_collect() == []
