"""Render modes (D / ED / RGB_D / RGB_ED), antialiased compensations, scaling modifier and tile masks
(gsplat/Rasterization.cpp:373-399, src/training/rasterization/rasterizer.cpp:171-198,
gsplat/RasterizeToPixelsFromWorld3DGSFwd.cu:147-155) against the CPU oracle, at the operator level
(colours with 1 and 4 channels) and through the fused path from raw parameters."""
import numpy as np
import pytest
import torch

from conftest import make_scene, rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAMES = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def check_image(a, b, tol=1e-4, scale=1.0):
    diff = np.abs(a - b).reshape(a.shape[0] * a.shape[1], -1).max(-1) / scale
    assert (diff > tol).sum() <= 2 and np.quantile(diff, 0.9999) < tol, diff.max()


def tile_mask(W, H, seed=0):
    tw, th = (W + 15) // 16, (H + 15) // 16
    m = np.random.default_rng(seed).random((th, tw)) > 0.3
    m[0, 0] = False
    return m


@pytest.mark.parametrize("CH,masked", [(1, False), (4, False), (4, True), (3, True)])
def test_operator_channels_and_masks(pkg, orc, synth, CH, masked):
    n, W, H, deg = 6000, 150, 100, 1
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=4)
    fwd0 = orc.render_fwd(P, vm, K, W, H, deg)
    means, q, s, o = P["means"], fwd0["quats"], fwd0["scales"], fwd0["opac"]
    rng = np.random.default_rng(7)
    col = {1: fwd0["depths"][:, None], 3: fwd0["colors"], 4: np.concatenate([fwd0["colors"], fwd0["depths"][:, None]], 1)}[CH]
    col = np.ascontiguousarray(col, np.float32)
    bg = rng.random(CH).astype(np.float32)
    masks = tile_mask(W, H) if masked else None
    ren_ref, alp_ref, last_ref, _ = orc.rasterize_fwd(means, q, s, col, o, bg, W, H, 16, vm, K, fwd0["tile_offsets"],
                                                       fwd0["flatten_ids"], masks=masks)
    args = [T(means), T(q), T(s), T(col[None]), T(o[None]), T(bg[None]), None if masks is None else T(masks[None]), W, H, 16,
            T(vm[None]), None, T(K[None]), 0]
    kw = dict(tile_offsets=T(fwd0["tile_offsets"][None]), flatten_ids=T(fwd0["flatten_ids"]))
    ren, alp, last = pkg.ops.rasterize_to_pixels_from_world_3dgs_fwd(*args, **kw)
    dscale = max(1.0, float(fwd0["depths"][fwd0["masks"]].max())) if CH != 3 else 1.0
    check_image(ren.cpu().numpy()[0], ren_ref, scale=dscale)
    check_image(alp.cpu().numpy()[0], alp_ref)
    assert (last.cpu().numpy()[0] != last_ref).sum() <= 2
    if masked:
        off = np.kron(~masks, np.ones((16, 16), bool))[:H, :W]
        assert np.array_equal(ren.cpu().numpy()[0][off], np.broadcast_to(bg, (int(off.sum()), CH)))
        assert (alp.cpu().numpy()[0][off] == 0).all()
    v_r = rng.normal(size=(H, W, CH)).astype(np.float32) * 1e-3
    if CH != 3:
        v_r[..., -1] /= dscale   # keep the depth channel's weight comparable to a colour channel's
    v_a = rng.normal(size=(H, W, 1)).astype(np.float32) * 1e-3
    ref = orc.rasterize_bwd(means, q, s, col, o, bg, W, H, 16, vm, K, fwd0["tile_offsets"], fwd0["flatten_ids"], alp_ref, last_ref,
                            v_r, v_a, masks=masks)
    out = pkg.ops.rasterize_to_pixels_from_world_3dgs_bwd(*args, **kw, render_alphas=T(alp_ref[None]), last_ids=T(last_ref[None]),
                                                          v_render_colors=T(v_r[None]), v_render_alphas=T(v_a[None]))
    for name, a, b in zip(("v_means", "v_quats", "v_scales", "v_colors", "v_opacities"), out, ref[:5]):
        a = a.cpu().numpy().reshape(b.shape)
        assert rel_l2(a, b) < 1e-3, name
    vc = out[3].cpu().numpy().reshape(n, CH)
    for k in range(CH):  # every colour channel on its own (the depth channel is much larger than the others)
        assert rel_l2(vc[:, k], ref[3][:, k]) < 1e-3, k


@pytest.mark.parametrize("mode,aa,modifier,masked", [
    (1, False, 1.0, False), (2, False, 1.0, False), (3, True, 1.0, False), (4, False, 0.8, True), (0, True, 1.3, True)])
def test_fused_render_modes(pkg, orc, synth, mode, aa, modifier, masked):
    tr = pkg.trainer
    n, W, H, deg = 8000, 170, 120, 2
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=6)
    CH = {0: 3, 1: 1, 2: 1, 3: 4, 4: 4}[mode]
    rng = np.random.default_rng(mode)
    bg = rng.random(CH).astype(np.float32) * 0.5
    masks = tile_mask(W, H, 3) if masked else None
    fwd = orc.render_fwd(P, vm, K, W, H, deg, background=bg, render_mode=mode, calc_compensations=aa,
                         scaling_modifier=modifier, tile_masks=masks)
    model = tr.SplatData(n, (deg + 1) ** 2, DEV).load(P)
    grads = model.like()
    rast = tr.Rasterizer(model, W, H, deg, render_mode=mode, antialiased=aa, scaling_modifier=modifier)
    rast.set_tile_masks(None if masks is None else T(masks))
    cam = tr.Camera(T(vm), T(K), W, H)
    out = rast.forward(cam, T(bg))
    st = rast.state()
    assert np.array_equal(st["radii"].cpu().numpy(), fwd["radii"])
    assert np.array_equal(st["flatten_ids"].cpu().numpy(), fwd["flatten_ids"])
    vis = fwd["masks"]
    assert np.abs(st["records"].cpu().numpy()[vis][:, 15] - fwd["final_opac"][vis]).max() < 1e-6
    dmax = max(1.0, float(fwd["depths"][vis].max()))
    check_image(out.alpha.cpu().numpy(), fwd["alpha"])
    if mode in (0, 3, 4):
        check_image(out.image.cpu().numpy(), fwd["image"])
    if mode != 0:
        check_image(out.depth.cpu().numpy(), fwd["depth"], scale=dmax)
    # backward: random output gradients on every channel and on alpha
    v_r = rng.normal(size=(H, W, CH)).astype(np.float32) * 1e-3
    if CH != 3:
        v_r[..., -1] /= dmax
    v_a = rng.normal(size=(H, W, 1)).astype(np.float32) * 1e-3
    bwd = orc.render_bwd(P, fwd, vm, K, W, H, deg, v_r, v_a, background=bg)
    rast.backward(T(v_r), grads, T(bg), T(v_a))
    for name in NAMES:
        a = grads.tensor(name).cpu().numpy()
        if mode in (1, 2) and name in ("sh0", "shN"):
            assert (a == 0).all(), name   # depth-only modes: no colour gradient
        else:
            assert rel_l2(a, bwd[name]) < 1e-3, name


def test_expected_depth_of_an_opaque_wall_is_its_distance(pkg, synth):
    """Property with a closed form: Gaussians spread on the plane z = 0 seen from distance 4 render an expected depth of
    about 4 wherever the wall is opaque, whatever the opacities are (ED = sum(w z) / sum(w))."""
    tr = pkg.trainer
    n, W, H = 20000, 128, 128
    cfg, P, vm, K = make_scene(synth, n, W, H, 0, seed=2)
    P["means"][:, 2] = 0.0
    P["scaling_raw"][:] = np.log(0.03)
    model = tr.SplatData(n, 1, DEV).load(P)
    rast = tr.Rasterizer(model, W, H, 0, render_mode=tr.RENDER_ED)
    out = rast.forward(tr.Camera(T(vm), T(K), W, H), None)
    d, a = out.depth.cpu().numpy()[..., 0], out.alpha.cpu().numpy()[..., 0]
    solid = a > 0.5
    assert solid.sum() > 1000
    zc = d[solid]
    # the depth of a Gaussian is its centre's camera z (4 on the wall)
    assert np.abs(zc - 4.0).max() < 1e-3


def test_background_gradient_matches_the_autograd_node(pkg, synth):
    """v_bg_color = (v_render_colors * (1 - render_alphas)).sum over the image (rasterizer_autograd.cpp:206-209), against the
    same expression in torch (float64 sum) and against a finite difference of the render in the background colour."""
    tr = pkg.trainer
    n, W, H, deg = 4000, 90, 70, 1
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=8)
    model = tr.SplatData(n, 4, DEV).load(P)
    for mode, ch in ((tr.RENDER_RGB, 3), (tr.RENDER_RGB_D, 4)):
        rast = tr.Rasterizer(model, W, H, deg, render_mode=mode)
        bg = torch.tensor([0.3, 0.6, 0.1, 0.0][:ch], device=DEV)
        cam = tr.Camera(T(vm), T(K), W, H)
        out = rast.forward(cam, bg)
        gen = torch.Generator(device=DEV).manual_seed(ch)
        v = torch.randn((H, W, ch), generator=gen, device=DEV)
        got = rast.background_gradient(v)
        want = (v.double() * (1.0 - out.alpha.double())).sum((0, 1))
        assert torch.allclose(got.double(), want, rtol=1e-5, atol=1e-5)
        # d(sum v * render)/d(bg_0) by a central difference (the render is linear in the background)
        r0 = out.render.clone()
        bg2 = bg.clone(); bg2[0] += 0.5
        r1 = rast.forward(cam, bg2).render
        fd = float(((r1 - r0).double() * v.double()).sum() / 0.5)
        assert abs(fd - float(want[0])) < 1e-3 * max(1.0, abs(float(want[0])))
