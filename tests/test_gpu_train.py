"""End-to-end parity of the fused training path (raw SplatData parameters -> image -> loss ->
raw-parameter gradients -> Adam) against the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import make_scene, rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LRS = [1.6e-4, 2.5e-3, 1.25e-4, 5e-3, 1e-3, 5e-2]
NAMES = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _run(pkg, orc, synth, n, W, H, deg, seed, bg, fx=300.0, n_cams=1):
    tr = pkg.trainer
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=seed, fx=fx)
    _, P2, _, _ = make_scene(synth, n, W, H, deg, seed=seed + 1000, fx=fx)
    fwd = orc.render_fwd(P, vm, K, W, H, deg, background=bg)
    target = np.ascontiguousarray(np.clip(orc.render_fwd(P2, vm, K, W, H, deg, background=bg)["render"], 0, 1).transpose(2, 0, 1))
    loss_ref, g_ref, _, _ = orc.photometric_loss(fwd["render"], target, 0.2)
    bwd = orc.render_bwd(P, fwd, vm, K, W, H, deg, g_ref, background=bg)

    model = tr.SplatData(n, (deg + 1) ** 2, DEV).load(P)
    grads, m, v = model.like(), model.like(), model.like()
    rast = tr.Rasterizer(model, W, H, deg)
    lossfn = tr.PhotometricLoss(W, H, DEV)
    cam = tr.Camera(T(vm), T(K), W, H)
    tbg = None if bg is None else T(bg)
    out = rast.forward(cam, tbg)
    loss, v_render = lossfn(out.image, T(target))
    rast.backward(v_render, grads, tbg)
    st = rast.state()
    return dict(P=P, fwd=fwd, bwd=bwd, loss_ref=loss_ref, g_ref=g_ref, model=model, grads=grads, m=m, v=v, rast=rast, out=out,
                loss=loss, v_render=v_render, state=st, target=target, cam=cam, tbg=tbg, lossfn=lossfn)


@pytest.mark.parametrize("n,W,H,deg,seed,bg", [
    (16384, 256, 256, 0, 0, np.zeros(3, np.float32)),      # the tiny benchmark configuration
    (20000, 250, 170, 3, 3, np.array([0.2, 0.5, 0.1], np.float32)),  # ragged image, SH degree 3, background
    (3000, 64, 48, 2, 9, None),                            # no background
])
def test_fused_step_matches_oracle(pkg, orc, synth, n, W, H, deg, seed, bg):
    r = _run(pkg, orc, synth, n, W, H, deg, seed, bg)
    fwd, st = r["fwd"], r["state"]
    # tile lists from raw parameters: bit-exact
    assert np.array_equal(st["radii"].cpu().numpy(), fwd["radii"])
    assert np.array_equal(st["tiles_per_gauss"].cpu().numpy(), fwd["tiles_per_gauss"])
    assert st["n_isects"] == fwd["flatten_ids"].size
    assert np.array_equal(st["flatten_ids"].cpu().numpy(), fwd["flatten_ids"])
    assert np.array_equal(st["tile_offsets"].cpu().numpy()[:-1], fwd["tile_offsets"].reshape(-1))
    vis = fwd["masks"]
    assert np.array_equal(st["means2d"].cpu().numpy()[vis].view(np.uint32), fwd["means2d"][vis].view(np.uint32))
    assert np.array_equal(st["depths"].cpu().numpy()[vis].view(np.uint32), fwd["depths"][vis].view(np.uint32))
    status = r["out"].status.cpu().numpy()
    assert status[0] == 0 and status[2] == vis.sum()
    # colours (clamped SH) and image
    assert np.abs(st["records"].cpu().numpy()[vis][:, 12:15] - fwd["colors"][vis]).max() < 2e-5
    diff = np.abs(r["out"].image.cpu().numpy() - fwd["render"]).max(-1)
    assert (diff > 1e-4).sum() <= 2 and np.quantile(diff, 0.9999) < 1e-4, diff.max()
    assert np.abs(r["out"].alpha.cpu().numpy() - fwd["alpha"]).max() < 5e-3
    assert (st["last_ids"].cpu().numpy() != fwd["last_ids"]).sum() <= 2
    # loss and gradients
    assert abs(float(r["loss"][0].item()) - r["loss_ref"]) < 1e-5
    for name in ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw"):
        a = r["grads"].tensor(name).cpu().numpy()
        if a.size:
            assert rel_l2(a, r["bwd"][name]) < 1e-3, name
    # Adam on the oracle side with the oracle's gradients
    tr = pkg.trainer
    tr.adam_step_splats(r["model"], r["m"], r["v"], r["grads"], LRS, 1)
    for gi, name in enumerate(("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")):
        p = r["P"][name].copy().reshape(-1)
        if p.size == 0:
            continue
        mm, vv = np.zeros_like(p), np.zeros_like(p)
        orc.adam_step(p, mm, vv, r["grads"].tensor(name).cpu().numpy().reshape(-1), LRS[gi], 0.9, 0.999, 1e-15, 1)
        assert np.allclose(r["model"].tensor(name).cpu().numpy().reshape(-1), p, rtol=1e-5, atol=1e-8), name


def test_accumulate_and_row_range(pkg, orc, synth):
    r = _run(pkg, orc, synth, 3000, 64, 48, 1, 21, np.zeros(3, np.float32))
    tr = pkg.trainer
    g1 = {k: t.clone() for k, t in r["grads"].tensors().items()}
    # a second camera pass (same camera here) accumulated on top: forward, then backward with accumulate
    r["rast"].forward(r["cam"], r["tbg"])
    r["rast"].backward(r["v_render"], r["grads"], r["tbg"], accumulate=True)
    for k, t in r["grads"].tensors().items():
        # atomic summation order differs run to run, so compare in norm rather than element by element
        assert rel_l2(t.cpu().numpy(), (2 * g1[k]).cpu().numpy()) < 1e-4, k
    # sharded Adam: two half ranges == one full range
    a, b = r["model"], r["model"].like()
    b.flat.copy_(a.flat)
    ma, va, mb, vb = a.like(), a.like(), a.like(), a.like()
    tr.adam_step_splats(a, ma, va, r["grads"], LRS, 3, grad_scale=0.5)
    half = a.size // 2 + 1
    tr.adam_step_splats(b, mb, vb, r["grads"], LRS, 3, first_row=0, n_rows=half, grad_scale=0.5)
    tr.adam_step_splats(b, mb, vb, r["grads"], LRS, 3, first_row=half, n_rows=a.size - half, grad_scale=0.5)
    assert torch.equal(a.flat, b.flat) and torch.equal(ma.flat, mb.flat) and torch.equal(va.flat, vb.flat)
    # skip_shN leaves the shN group untouched
    c = a.like(); c.flat.copy_(a.flat)
    tr.adam_step_splats(c, ma, va, r["grads"], LRS, 4, skip_shN=True)
    assert torch.equal(c.tensor("shN"), a.tensor("shN")) and not torch.equal(c.tensor("means"), a.tensor("means"))


def test_isect_overflow_is_reported(pkg, orc, synth):
    tr = pkg.trainer
    cfg, P, vm, K = make_scene(synth, 4000, 96, 96, 0, seed=2)
    model = tr.SplatData(4000, 1, DEV).load(P)
    rast = tr.Rasterizer(model, 96, 96, 0, isect_capacity=100)
    out = rast.forward(tr.Camera(T(vm), T(K), 96, 96), None)
    torch.cuda.synchronize()
    st = out.status.cpu().numpy()
    assert st[0] == 1 and st[1] > 100


def test_split_forward_and_split_adam_equal_the_fused_calls(pkg, synth):
    """forward_lists + forward_shade == forward and Adam(geometry groups) + Adam(colour groups) == Adam(all), bit for bit."""
    tr = pkg.trainer
    n, W, H, deg = 12000, 200, 120, 3
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=12)
    model = tr.SplatData(n, 16, DEV).load(P)
    cam = tr.Camera(T(vm), T(K), W, H)
    bg = T(np.array([0.3, 0.1, 0.6], np.float32))
    a = tr.Rasterizer(model, W, H, deg)
    b = tr.Rasterizer(model, W, H, deg)
    out_a = a.forward(cam, bg)
    b.forward_lists(cam)
    out_b = b.forward_shade(bg)
    assert torch.equal(out_a.image, out_b.image) and torch.equal(out_a.alpha, out_b.alpha)
    sa, sb = a.state(), b.state()
    vis = (sa["radii"] > 0).all(-1)   # records of culled Gaussians are never written
    assert torch.equal(sa["radii"], sb["radii"]) and torch.equal(sa["records"][vis], sb["records"][vis])
    # the same lists with an event recorded between the projection kernel and the sorting kernels: work of another stream
    # that waits for it starts no earlier than the projection's end
    c = tr.Rasterizer(model, W, H, deg)
    ev = torch.cuda.Event()
    with pytest.raises(RuntimeError, match="no handle"):
        c.forward_lists(cam, projected_event=ev)
    ev.record()
    side = torch.cuda.Stream()
    c.forward_lists(cam, projected_event=ev)
    with torch.cuda.stream(side):
        side.wait_event(ev)
        radii_seen = c.state()["radii"].clone()           # written by the projection kernel
    out_c = c.forward_shade(bg)
    torch.cuda.synchronize()
    assert ev.query() and torch.equal(out_a.image, out_c.image) and torch.equal(radii_seen, sa["radii"])
    rng = np.random.default_rng(0)
    v = T(rng.normal(size=(H, W, 3)).astype(np.float32))
    ga, gb = model.like(), model.like()
    a.backward(v, ga, bg)
    b.backward(v, gb, bg)
    for name in NAMES:
        assert rel_l2(ga.tensor(name).cpu().numpy(), gb.tensor(name).cpu().numpy()) < 1e-5, name
    m1, v1, m2, v2 = model.like(), model.like(), model.like(), model.like()
    model2 = tr.SplatData(n, 16, DEV).load(P)
    tr.adam_step_splats(model, m1, v1, ga, LRS, 3)
    tr.adam_step_groups(model2, m2, v2, ga, LRS, 3, tr.GEOMETRY_GROUPS)
    tr.adam_step_groups(model2, m2, v2, ga, LRS, 3, tr.COLOR_GROUPS)
    assert torch.equal(model.flat, model2.flat) and torch.equal(m1.flat, m2.flat) and torch.equal(v1.flat, v2.flat)


@pytest.mark.parametrize("n,W,H,deg,skip_shN", [(12000, 200, 120, 3, False), (5003, 97, 61, 2, False), (5003, 97, 61, 3, True),
                                                 (4001, 80, 64, 0, False)])
def test_rank1_sh_adam_equals_materialised_gradient(pkg, synth, n, W, H, deg, skip_shN):
    """backward(write_shN=False) + lfs_adam_step_splats_rank1_sh == backward + lfs_adam_step_splats: the shN gradient
    rows rebuilt inside the optimizer from the sh0 gradient equal the materialised ones up to rounding."""
    tr = pkg.trainer
    K = (deg + 1) ** 2
    cfg, P, vm, Kmat = make_scene(synth, n, W, H, deg, seed=21)
    cam = tr.Camera(T(vm), T(Kmat), W, H)
    bg = T(np.array([0.3, 0.1, 0.6], np.float32))
    rng = np.random.default_rng(5)
    v_render = T(rng.normal(size=(H, W, 3)).astype(np.float32))
    models, moments = [], []
    for _ in range(2):
        model = tr.SplatData(n, K, DEV).load(P)
        m, v = model.like(), model.like()
        # non-zero moments make the update a smooth function of the gradient (no sign flips on tiny gradients)
        gen = torch.Generator(device=DEV).manual_seed(77)
        m.flat.copy_(torch.randn(m.flat.shape, generator=gen, device=DEV) * 1e-3)
        v.flat.copy_(torch.rand(v.flat.shape, generator=gen, device=DEV) * 1e-4 + 1e-6)
        models.append(model); moments.append((m, v))
    ra, rb = tr.Rasterizer(models[0], W, H, deg), tr.Rasterizer(models[1], W, H, deg)
    ra.forward(cam, bg)
    ga = models[0].like()
    ra.backward(v_render, ga, bg)
    tr.adam_step_splats(models[0], moments[0][0], moments[0][1], ga, LRS, 3, skip_shN=skip_shN, grad_scale=0.5)
    rb.forward(cam, bg)
    gb = models[1].like()
    if K > 1:
        gb.tensor("shN").fill_(123.0)
    rb.backward(v_render, gb, bg, write_shN=False)
    if K > 1:
        assert bool((gb.tensor("shN") == 123.0).all())       # not written
    rb.adam_step_rank1_sh(moments[1][0], moments[1][1], gb, LRS, 3, skip_shN=skip_shN, grad_scale=0.5)
    vis = (ra.state()["radii"] > 0).all(-1)
    assert 0 < int(vis.sum()) < n
    worst = {}
    for name in NAMES:
        pa, pb = models[0].tensor(name), models[1].tensor(name)
        if pa.numel() == 0:
            continue
        p0 = torch.from_numpy(np.ascontiguousarray(P[name], dtype=np.float32)).reshape(pa.shape).to(DEV)
        d_a, d_b = (pa - p0).cpu().numpy(), (pb - p0).cpu().numpy()
        if name == "shN" and skip_shN:
            assert not d_a.any() and not d_b.any()
        else:
            assert np.abs(d_a).max() > 0
            # the steps are ~1e-5 of the parameter values, so float32 subtraction alone costs ~1e-4 here; the moments
            # below carry the gradient at full precision
            assert rel_l2(d_b, d_a) < 1e-3, name
        for k in range(2):
            worst[(name, k)] = rel_l2(moments[1][k].tensor(name).cpu().numpy(), moments[0][k].tensor(name).cpu().numpy())
    assert max(worst.values()) < 1e-5, worst
    # Gaussians that were not visible take a zero gradient in both paths: identical rows
    hidden = (~vis).cpu().numpy()
    if K > 1 and not skip_shN:
        assert np.array_equal(models[1].tensor("shN").cpu().numpy()[hidden], models[0].tensor("shN").cpu().numpy()[hidden])
        assert np.array_equal(moments[1][0].tensor("shN").cpu().numpy()[hidden], moments[0][0].tensor("shN").cpu().numpy()[hidden])


@pytest.mark.parametrize("n,W,H,deg,skip_shN", [(12000, 200, 120, 3, False), (5003, 97, 61, 2, False), (5003, 97, 61, 3, True),
                                                 (4001, 80, 64, 0, False)])
def test_backward_adam_equals_backward_then_adam(pkg, synth, n, W, H, deg, skip_shN):
    """lfs_render_backward_adam == lfs_render_backward + lfs_adam_step_splats up to the rounding of the atomic sums."""
    tr = pkg.trainer
    K = (deg + 1) ** 2
    cfg, P, vm, Kmat = make_scene(synth, n, W, H, deg, seed=23)
    cam = tr.Camera(T(vm), T(Kmat), W, H)
    bg = T(np.array([0.3, 0.1, 0.6], np.float32))
    v_render = T(np.random.default_rng(6).normal(size=(H, W, 3)).astype(np.float32))
    res = []
    for fused in (False, True):
        model = tr.SplatData(n, K, DEV).load(P)
        m, v = model.like(), model.like()
        gen = torch.Generator(device=DEV).manual_seed(78)
        m.flat.copy_(torch.randn(m.flat.shape, generator=gen, device=DEV) * 1e-3)
        v.flat.copy_(torch.rand(v.flat.shape, generator=gen, device=DEV) * 1e-4 + 1e-6)
        rast = tr.Rasterizer(model, W, H, deg)
        rast.forward(cam, bg)
        if fused:
            rast.backward_adam(v_render, m, v, LRS, 3, bg, skip_shN=skip_shN, grad_scale=0.5)
        else:
            grads = model.like()
            rast.backward(v_render, grads, bg)
            tr.adam_step_splats(model, m, v, grads, LRS, 3, skip_shN=skip_shN, grad_scale=0.5)
        res.append((model, m, v, (rast.state()["radii"] > 0).all(-1)))
    vis = res[0][3]
    assert 0 < int(vis.sum()) < n
    worst = {}
    for name in NAMES:
        pa, pb = res[0][0].tensor(name), res[1][0].tensor(name)
        if pa.numel() == 0:
            continue
        p0 = torch.from_numpy(np.ascontiguousarray(P[name], dtype=np.float32)).reshape(pa.shape).to(DEV)
        d_a, d_b = (pa - p0).cpu().numpy(), (pb - p0).cpu().numpy()
        if name == "shN" and skip_shN:
            assert not d_a.any() and not d_b.any()
        else:
            assert np.abs(d_a).max() > 0
            assert rel_l2(d_b, d_a) < 1e-3, name      # float32 subtraction of ~1e-5 steps; the moments are the sharp check
        for k in (1, 2):
            worst[(name, k)] = rel_l2(res[1][k].tensor(name).cpu().numpy(), res[0][k].tensor(name).cpu().numpy())
    assert max(worst.values()) < 1e-5, worst
    hidden = (~vis).cpu().numpy()
    for name in ("means", "opacity_raw"):
        assert np.array_equal(res[1][1].tensor(name).cpu().numpy()[hidden], res[0][1].tensor(name).cpu().numpy()[hidden])
        assert np.array_equal(res[1][0].tensor(name).cpu().numpy()[hidden], res[0][0].tensor(name).cpu().numpy()[hidden])


def test_state_with_reserved_capacity(pkg, orc, synth):
    """state() reads the workspace with the layout of the last forward (N = live rows), also when the model reserves
    more rows than it holds and the row count is not a multiple of four."""
    tr = pkg.trainer
    n, W, H, deg = 5001, 96, 80, 1
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=4)
    bg = np.zeros(3, np.float32)
    fwd = orc.render_fwd(P, vm, K, W, H, deg, background=bg)
    model = tr.SplatData(n, (deg + 1) ** 2, DEV, capacity=n + 1003).load(P)
    assert model.capacity != model.size
    rast = tr.Rasterizer(model, W, H, deg)
    rast.forward(tr.Camera(T(vm), T(K), W, H), T(bg))
    st = rast.state()
    vis = fwd["masks"]
    assert np.array_equal(st["radii"].cpu().numpy(), fwd["radii"])
    assert np.array_equal(st["means2d"].cpu().numpy()[vis].view(np.uint32), fwd["means2d"][vis].view(np.uint32))
    assert np.array_equal(st["depths"].cpu().numpy()[vis].view(np.uint32), fwd["depths"][vis].view(np.uint32))
    assert np.array_equal(st["tiles_per_gauss"].cpu().numpy(), fwd["tiles_per_gauss"])
    assert np.array_equal(st["flatten_ids"].cpu().numpy(), fwd["flatten_ids"])
    assert np.array_equal(st["tile_offsets"].cpu().numpy()[:-1], fwd["tile_offsets"].reshape(-1))
    assert (st["last_ids"].cpu().numpy() != fwd["last_ids"]).sum() <= 2


def test_equirectangular_fused_path_matches_oracle(pkg, orc, synth):
    """CameraModelType::EQUIRECTANGULAR through the fused path against the CPU oracle (whose equirectangular model is pinned
    to its pinhole model by a CPU test): camera inside the scene, so Gaussians behind the camera (negative depth) are drawn
    too. atan2f / asinf of the device and of the host's libm differ in the last bit, so the per-Gaussian values are compared
    with a bound instead of bit for bit and a few Gaussians may change tiles."""
    tr = pkg.trainer
    n, W, H, deg = 8000, 256, 128, 2
    P = synth.make_gaussians(n, 6, "cube", deg)
    P["scaling_raw"] = (P["scaling_raw"] + np.float32(0.7)).astype(np.float32)
    vm = np.eye(4, dtype=np.float32)
    vm[:3, 3] = [0.05, -0.02, 0.1]
    K = synth.intrinsics(100.0, 100.0, W / 2, H / 2)
    bg = np.array([0.2, 0.1, 0.3], np.float32)
    fwd = orc.render_fwd(P, vm, K, W, H, deg, background=bg, camera_model=orc.EQUIRECTANGULAR)
    assert (fwd["depths"][fwd["masks"]] < 0).sum() > 100           # the back hemisphere is populated
    model = tr.SplatData(n, (deg + 1) ** 2, DEV).load(P)
    rast = tr.Rasterizer(model, W, H, deg)
    cam = tr.Camera(T(vm), T(K), W, H, camera_model=pkg._capi.EQUIRECTANGULAR)
    out = rast.forward(cam, T(bg))
    st = rast.state()
    vis = fwd["masks"]
    assert (st["radii"].cpu().numpy() != fwd["radii"]).any(-1).sum() <= n // 500
    assert np.abs(st["means2d"].cpu().numpy()[vis] - fwd["means2d"][vis]).max() < 2e-2   # a few ulp of a coordinate near 256
    assert abs(st["n_isects"] - fwd["flatten_ids"].size) <= fwd["flatten_ids"].size // 1000
    diff = np.abs(out.image.cpu().numpy() - fwd["render"]).max(-1)
    assert (diff > 1e-4).mean() < 2e-3 and np.quantile(diff, 0.99) < 1e-4, (diff.max(), (diff > 1e-4).mean())
    rng = np.random.default_rng(3)
    v = rng.normal(size=(H, W, 3)).astype(np.float32) * 1e-3
    bwd = orc.render_bwd(P, fwd, vm, K, W, H, deg, v, background=bg, camera_model=orc.EQUIRECTANGULAR)
    grads = model.like()
    rast.backward(T(v), grads, T(bg))
    for name in NAMES:
        a = grads.tensor(name).cpu().numpy()
        if a.size:
            assert rel_l2(a, bwd[name]) < 2e-3, name
