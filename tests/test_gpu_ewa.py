"""The EWA rasterizer of the default (non --gut) trainer path (src/training/fastgs/rasterization/, glue in
src/training/rasterization/fast_rasterizer.cpp) against the CPU oracle: per-Gaussian records and exact tile lists
bit for bit, image / alpha within float tolerance, raw-parameter gradients and the densification statistics."""
import numpy as np
import pytest
import torch

from conftest import make_scene, rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAMES = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")


def T(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def run(pkg, orc, synth, n, W, H, deg, active_deg, seed, bg, fx=300.0, scale_shift=0.0, cap=None):
    tr = pkg.trainer
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=seed, fx=fx)
    P["scaling_raw"] = (P["scaling_raw"] + np.float32(scale_shift)).astype(np.float32)
    campos = orc.campos(vm)
    fwd = orc.ewa_forward(P, vm, campos, W, H, K[0, 0], K[1, 1], K[0, 2], K[1, 2], (active_deg + 1) ** 2, background=bg)
    model = tr.SplatData(n, (deg + 1) ** 2, DEV).load(P)
    rast = tr.FastRasterizer(model, W, H, active_deg, instance_capacity=cap)
    cam = tr.Camera(T(vm), T(K), W, H)
    out = rast.forward(cam, T(bg))
    return dict(P=P, fwd=fwd, model=model, rast=rast, out=out, cam=cam, vm=vm, K=K)


@pytest.mark.parametrize("n,W,H,deg,active,seed,bg,shift", [
    (16384, 256, 256, 0, 0, 0, None, 0.0),
    (20000, 250, 170, 3, 3, 3, np.array([0.2, 0.5, 0.1], np.float32), 0.8),   # ragged image, SH degree 3, background
    (5000, 100, 60, 3, 1, 9, np.array([1.0, 1.0, 1.0], np.float32), 2.0),     # active degree below the stored one, big splats
])
def test_ewa_forward_backward_match_oracle(pkg, orc, synth, n, W, H, deg, active, seed, bg, shift):
    r = run(pkg, orc, synth, n, W, H, deg, active, seed, bg, scale_shift=shift)
    fwd, st = r["fwd"], r["rast"].state()
    # per-Gaussian stage and lists: bit-exact
    assert np.array_equal(st["n_touched"].cpu().numpy(), fwd["n_touched"])
    vis = fwd["n_touched"] > 0
    assert 0 < vis.sum()
    assert np.array_equal(st["bounds"].cpu().numpy()[vis].astype(np.int32), fwd["bounds"][vis])
    assert np.array_equal(st["mean2d"].cpu().numpy()[vis].view(np.uint32), fwd["mean2d"][vis].view(np.uint32))
    assert np.array_equal(st["conic_opacity"].cpu().numpy()[vis].view(np.uint32), fwd["conic_opacity"][vis].view(np.uint32))
    assert st["n_instances"] == fwd["instance_ids"].size == int(fwd["n_touched"].sum())
    assert np.array_equal(st["instance_ids"].cpu().numpy(), fwd["instance_ids"])
    assert np.array_equal(st["tile_offsets"].cpu().numpy(), fwd["tile_offsets"])
    status = r["out"].status.cpu().numpy()
    assert status[0] == 0 and status[1] == fwd["instance_ids"].size and status[2] == vis.sum()
    assert np.abs(st["color"].cpu().numpy()[vis] - np.maximum(fwd["color"][vis], 0)).max() < 2e-5
    # image
    diff = np.abs(r["out"].image.cpu().numpy() - fwd["image"]).max(0)
    assert (diff > 1e-4).sum() <= 2 and np.quantile(diff, 0.9999) < 1e-4, diff.max()
    assert np.abs(r["out"].alpha.cpu().numpy()[0] - fwd["alpha"]).max() < 5e-3
    assert (st["n_contrib"].cpu().numpy() != fwd["n_contrib"]).sum() <= 2
    # backward with random output gradients; densification statistics accumulate on top of what is there
    rng = np.random.default_rng(seed)
    gi = rng.normal(size=(3, H, W)).astype(np.float32) * 1e-3
    ga = rng.normal(size=(H, W)).astype(np.float32) * 1e-3
    dens0 = rng.random((2, n)).astype(np.float32)
    dens_ref = dens0.copy()
    bwd = orc.ewa_backward(r["P"], fwd, gi, ga, dens_ref)
    grads = r["model"].like()
    dens = T(dens0)
    gw = torch.full((4, 4), 7.0, device=DEV)      # overwritten, not added to
    r["rast"].backward(T(gi), grads, T(bg), T(ga[None]), densification_info=dens, grad_w2c=gw)
    for name in NAMES:
        a = grads.tensor(name).cpu().numpy()
        if a.size:
            assert rel_l2(a, bwd[name]) < 1e-3, name
            assert (a[~vis] == 0).all(), name
    d = dens.cpu().numpy()
    assert np.array_equal(d[0], dens_ref[0]) and np.allclose(d[1], dens_ref[1], rtol=2e-3, atol=1e-6)
    # camera-pose gradient (kernels_backward.cuh:160-173): rows 0..2, float32 sums of ~N terms against a float64 sum
    gw = gw.cpu().numpy()
    assert (gw[3] == 0).all() and rel_l2(gw[:3], bwd["grad_w2c"][:3]) < 1e-3, (gw, bwd["grad_w2c"])
    # the gradients of the Gaussians do not depend on whether the pose gradient was asked for
    grads2 = r["model"].like()
    r["rast"].forward(r["cam"], T(bg))
    r["rast"].backward(T(gi), grads2, T(bg), T(ga[None]))
    assert rel_l2(grads2.flat.cpu().numpy(), grads.flat.cpu().numpy()) < 1e-5    # the blend backward sums with atomics


def test_ewa_accumulate_and_overflow(pkg, orc, synth):
    tr = pkg.trainer
    bg = np.array([0.1, 0.2, 0.3], np.float32)
    r = run(pkg, orc, synth, 8000, 128, 96, 2, 2, 5, bg, scale_shift=1.0)
    rng = np.random.default_rng(0)
    gi = T(rng.normal(size=(3, 96, 128)).astype(np.float32) * 1e-3)
    g1, g2 = r["model"].like(), r["model"].like()
    r["rast"].backward(gi, g1, T(bg))
    g2.flat.copy_(g1.flat)
    r["rast"].forward(r["cam"], T(bg))
    gw1, gw2 = torch.zeros(4, 4, device=DEV), torch.zeros(4, 4, device=DEV)
    r["rast"].backward(gi, g2, T(bg), accumulate=True, grad_w2c=gw2)   # adds the same gradient once more
    for name in NAMES:
        assert rel_l2(g2.tensor(name).cpu().numpy(), 2.0 * g1.tensor(name).cpu().numpy()) < 1e-4, name
    r["rast"].forward(r["cam"], T(bg))
    r["rast"].backward(gi, g1.like(), T(bg), grad_w2c=gw1)
    r["rast"].forward(r["cam"], T(bg))
    r["rast"].backward(gi, g1.like(), T(bg), accumulate=True, grad_w2c=gw2)   # pose gradient: added to with `accumulate`
    assert float(gw1.abs().max()) > 0 and rel_l2(gw2.cpu().numpy(), 2.0 * gw1.cpu().numpy()) < 1e-4
    # capacity too small: the overflow flag is raised, nothing is drawn, the backward leaves zeros
    n_inst = int(r["out"].status[1].item())
    small = tr.FastRasterizer(r["model"], 128, 96, 2, instance_capacity=n_inst // 2)
    out = small.forward(r["cam"], T(bg))
    assert int(out.status[0].item()) == 1
    assert torch.allclose(out.image, T(bg)[:, None, None].expand(3, 96, 128)) and float(out.alpha.abs().max()) == 0.0
    g3 = r["model"].like()
    small.backward(gi, g3, T(bg))
    assert float(g3.tensor("means").abs().max()) == 0.0


def test_default_strategy_trains_on_the_ewa_path(pkg, synth):
    """The default trainer loop: fast_rasterize -> loss -> backward (fills densification_info) -> DefaultStrategy."""
    tr, st = pkg.trainer, pkg.strategy
    n, W, H, deg = 4000, 128, 96, 1
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=2)
    model = tr.SplatData(n, (deg + 1) ** 2, DEV, capacity=4 * n).load(P)
    s = st.DefaultStrategy(model)
    s.initialize(st.DefaultStrategy.Parameters(sh_degree=deg, start_refine=2, refine_every=3, iterations=100, grad_threshold=1e-7))
    rast = tr.FastRasterizer(model, W, H, deg, instance_capacity=64 * 4 * n)
    lossfn = tr.PhotometricLoss(W, H, DEV, 0.2)
    cam = tr.Camera(T(vm), T(K), W, H)
    bg = torch.zeros(3, device=DEV)
    target = torch.rand((3, H, W), generator=torch.Generator().manual_seed(0)).to(DEV)
    losses = []
    for it in range(1, 8):
        out = rast.forward(cam, bg)
        loss, v_hwc = lossfn(out.image.permute(1, 2, 0).contiguous(), target)
        s.grads.size = model.size
        if s.densification_info.shape[-1] != model.size:
            s.densification_info = torch.zeros((2, model.size), device=DEV)
        rast.backward(v_hwc.permute(2, 0, 1).contiguous(), s.grads, bg, densification_info=s.densification_info)
        losses.append(float(loss[0]))
        s.post_backward(it)
        s.step(it)
    assert losses[1] < losses[0] and all(np.isfinite(losses))
    assert model.size > n   # the statistics written by the backward drove a densification step


@pytest.mark.parametrize("n,W,H,deg,active", [(12000, 200, 120, 3, 3), (5003, 97, 61, 3, 1)])
def test_ewa_rank1_sh_adam_equals_materialised_gradient(pkg, synth, n, W, H, deg, active):
    """backward(write_shN=False) + lfs_ewa_adam_step_rank1_sh == backward + lfs_adam_step_splats on the EWA path."""
    tr = pkg.trainer
    lrs = [1.6e-4, 2.5e-3, 1.25e-4, 5e-3, 1e-3, 5e-2]
    K = (deg + 1) ** 2
    cfg, P, vm, Kmat = make_scene(synth, n, W, H, deg, seed=14)
    P["scaling_raw"] = (P["scaling_raw"] + np.float32(0.8)).astype(np.float32)
    cam = tr.Camera(T(vm), T(Kmat), W, H)
    bg = T(np.array([0.3, 0.1, 0.6], np.float32))
    g_img = T(np.random.default_rng(3).normal(size=(3, H, W)).astype(np.float32))
    res = []
    for rank1 in (False, True):
        model = tr.SplatData(n, K, DEV).load(P)
        m, v = model.like(), model.like()
        gen = torch.Generator(device=DEV).manual_seed(77)
        m.flat.copy_(torch.randn(m.flat.shape, generator=gen, device=DEV) * 1e-3)
        v.flat.copy_(torch.rand(v.flat.shape, generator=gen, device=DEV) * 1e-4 + 1e-6)
        rast = tr.FastRasterizer(model, W, H, active)
        rast.forward(cam, bg)
        grads = model.like()
        if rank1:
            grads.tensor("shN").fill_(7.0)
            rast.backward(g_img, grads, bg, write_shN=False)
            assert bool((grads.tensor("shN") == 7.0).all())
            rast.adam_step_rank1_sh(m, v, grads, lrs, 3, grad_scale=0.5)
        else:
            rast.backward(g_img, grads, bg)
            tr.adam_step_splats(model, m, v, grads, lrs, 3, grad_scale=0.5)
        res.append((model, m, v))
    worst = {}
    for name in NAMES:
        for k in (1, 2):
            a, b = res[0][k].tensor(name).cpu().numpy(), res[1][k].tensor(name).cpu().numpy()
            worst[(name, k)] = rel_l2(b, a)
        p0 = T(P[name]).reshape(res[0][0].tensor(name).shape)
        d_a, d_b = (res[0][0].tensor(name) - p0).cpu().numpy(), (res[1][0].tensor(name) - p0).cpu().numpy()
        assert np.abs(d_a).max() > 0
        assert rel_l2(d_b, d_a) < 1e-3, name
    assert max(worst.values()) < 1e-5, worst


def test_ewa_state_with_reserved_capacity(pkg, orc, synth):
    """FastRasterizer.state() uses the layout of the last forward when the model reserves more rows than it holds."""
    tr = pkg.trainer
    n, W, H, deg = 5001, 96, 80, 1
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=4)
    P["scaling_raw"] = (P["scaling_raw"] + np.float32(1.0)).astype(np.float32)
    fwd = orc.ewa_forward(P, vm, orc.campos(vm), W, H, K[0, 0], K[1, 1], K[0, 2], K[1, 2], 4, background=None)
    model = tr.SplatData(n, 4, DEV, capacity=n + 1003).load(P)
    rast = tr.FastRasterizer(model, W, H, deg)
    rast.forward(tr.Camera(T(vm), T(K), W, H), None)
    st = rast.state()
    vis = fwd["n_touched"] > 0
    assert np.array_equal(st["n_touched"].cpu().numpy(), fwd["n_touched"])
    assert np.array_equal(st["bounds"].cpu().numpy()[vis].astype(np.int32), fwd["bounds"][vis])
    assert np.array_equal(st["mean2d"].cpu().numpy()[vis].view(np.uint32), fwd["mean2d"][vis].view(np.uint32))
    assert np.array_equal(st["instance_ids"].cpu().numpy(), fwd["instance_ids"])
    assert np.array_equal(st["tile_offsets"].cpu().numpy(), fwd["tile_offsets"])
    assert (st["n_contrib"].cpu().numpy() != fwd["n_contrib"]).sum() <= 2
