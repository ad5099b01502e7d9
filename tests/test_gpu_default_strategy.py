"""DefaultStrategy (src/training/strategies/default_strategy.cpp) on the GPU: split() with given noise against a
numpy restatement built on the oracle's quats_to_rotmats; grow_gs / prune_gs row bookkeeping; a few training
steps through the strategy interface."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAMES = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")


def make(pkg, synth, n=3000, deg=2, cap=None, **kw):
    st, tr = pkg.strategy, pkg.trainer
    P = synth.make_gaussians(n, 11, "clusters", deg)
    model = tr.SplatData(n, (deg + 1) ** 2, DEV, capacity=cap or 3 * n).load(P)
    s = st.DefaultStrategy(model)
    s.initialize(st.DefaultStrategy.Parameters(sh_degree=deg, **kw))
    return s, P


@pytest.mark.parametrize("revised", [False, True])
def test_split_matches_restatement(pkg, synth, orc, revised):
    n = 3000
    s, P = make(pkg, synth, n, revised_opacity=revised)
    rng = np.random.default_rng(3)
    sel = rng.random(n) < 0.2
    k = int(sel.sum())
    noise = rng.normal(size=(2, k, 3)).astype(np.float32)
    s._optimizer.exp_avg.flat.fill_(1.0)
    s._optimizer.exp_avg_sq.flat.fill_(2.0)
    s.split(torch.from_numpy(sel).to(DEV), torch.from_numpy(noise).to(DEV))

    q = P["rotation_raw"][sel].astype(np.float64)
    q = (q / np.linalg.norm(q, axis=-1, keepdims=True)).astype(np.float32)
    R = orc.quats_to_rotmats(q).astype(np.float64)
    sc = np.exp(P["scaling_raw"][sel].astype(np.float64))
    samples = np.einsum("nij,nj,bnj->bni", R, sc, noise.astype(np.float64))
    exp = {}
    for name in NAMES:
        rest, x = P[name][~sel], P[name][sel]
        if name == "means":
            new = (x[None].astype(np.float64) + samples).reshape(-1, 3)
        elif name == "scaling_raw":
            new = np.tile(np.log(sc / 1.6), (2, 1))
        elif name == "opacity_raw" and revised:
            o = 1.0 / (1.0 + np.exp(-x.astype(np.float64)))
            o = 1.0 - np.sqrt(1.0 - o)
            new = np.tile(np.log(o / (1.0 - o)), (2, 1))
        else:
            new = np.tile(x, (2,) + (1,) * (x.ndim - 1))
        exp[name] = np.concatenate([rest.astype(np.float64), new.reshape((2 * k,) + rest.shape[1:])], 0)
    sd = s.get_model()
    assert sd.size == n + k and s._optimizer.exp_avg.size == n + k
    for name in NAMES:
        got = sd.tensor(name).cpu().numpy()
        # float32 arithmetic of exp / log / einsum against float64: a few ulp of the operands
        assert np.allclose(got, exp[name], rtol=2e-5, atol=2e-5), name
        if name in ("sh0", "shN", "rotation_raw") or (name == "opacity_raw" and not revised):
            assert np.array_equal(got, exp[name].astype(np.float32)), name   # copied rows are bit-identical
        m = s._optimizer.exp_avg.tensor(name)
        assert bool(m[: n - k].eq(1).all()) and bool(m[n - k:].eq(0).all()), name
        v = s._optimizer.exp_avg_sq.tensor(name)
        assert bool(v[: n - k].eq(2).all()) and bool(v[n - k:].eq(0).all()), name


def test_grow_then_prune_counts(pkg, synth):
    n = 3000
    s, P = make(pkg, synth, n, grow_scale3d=0.02)
    sd = s.get_model()
    scales = np.exp(P["scaling_raw"]).max(-1)
    info = torch.zeros((2, n), device=DEV)
    info[0] = 2.0
    hot = np.arange(n) % 3 == 0
    info[1, torch.from_numpy(hot).to(DEV)] = 2.0 * 0.001
    s.densification_info = info
    small = scales <= 0.02
    n_dup, n_split = int((hot & small).sum()), int((hot & ~small).sum())
    assert n_dup > 0 and n_split > 0
    s.grow_gs(600)
    assert sd.size == n + n_dup + n_split
    # duplicated rows sit after the originals and before the split products
    kept = (~(hot & ~small)).nonzero()[0]
    assert np.array_equal(sd.tensor("sh0")[: kept.size].cpu().numpy().reshape(kept.size, -1), P["sh0"][kept].reshape(kept.size, -1))
    op = torch.sigmoid(sd.tensor("opacity_raw")).reshape(-1)
    n_low = int((op < 0.005).sum())
    before = sd.size
    s.prune_gs(600)
    assert sd.size == before - n_low
    assert bool((torch.sigmoid(sd.tensor("opacity_raw")) >= 0.005).all())


def test_strategy_drives_training_steps(pkg, synth):
    """post_backward / step through the IStrategy surface with the fused renderer: the loss falls, sizes stay in step."""
    tr = pkg.trainer
    cfg = synth.CONFIGS["tiny"]
    n, W, H, deg = cfg["n"], cfg["W"], cfg["H"], cfg["sh_degree"]
    st = pkg.strategy
    P = synth.make_gaussians(n, 0, cfg["layout"], deg)
    model = tr.SplatData(n, (deg + 1) ** 2, DEV, capacity=4 * n).load(P)
    s = st.DefaultStrategy(model)
    s.initialize(st.DefaultStrategy.Parameters(sh_degree=deg, start_refine=2, refine_every=3, iterations=100))
    poses, K = synth.make_cameras(cfg)
    rast = tr.Rasterizer(model, W, H, deg, isect_capacity=64 * 4 * n)
    loss = tr.PhotometricLoss(W, H, DEV, 0.2)
    cam = tr.Camera(torch.from_numpy(poses[0]).to(DEV), torch.from_numpy(K).to(DEV), W, H)
    bg = torch.zeros(3, device=DEV)
    gt = torch.rand((3, H, W), generator=torch.Generator().manual_seed(0)).to(DEV)
    vals = []
    for it in range(1, 10):
        out = rast.forward(cam, bg)
        l, v_render = loss(out.image, gt)
        s.grads.size = model.size
        rast.backward(v_render, s.grads, bg)
        vals.append(float(l[0]))
        if s.is_refining(it):
            # stand-in for the EWA rasterizer's image-plane statistics: the norm of the mean gradient
            g = s.grads.tensor("means").norm(dim=-1)
            s.densification_info = torch.stack([torch.ones_like(g), g * 0 + 1e-3 * (torch.arange(model.size, device=DEV) % 7 == 0)])
        s.post_backward(it)
        s.step(it)
    assert model.size > n and s._optimizer.exp_avg.size == model.size
    assert vals[1] < vals[0] and all(np.isfinite(vals))   # the first two steps run before any refinement


def test_refinement_iteration_skips_adam(pkg, synth):
    """An iteration whose post_backward rewrites the rows runs no Adam and does not count the step, as in the reference:
    update_param_with_optimizer installs new leaf tensors without .grad, so FusedAdam::step `continue`s before
    step_count++ (src/training/optimizers/fused_adam.cpp:46-48). Checked against a numpy oracle that applies the row
    surgery to parameters and moments and skips the optimizer."""
    n = 2000
    s, P = make(pkg, synth, n, grow_scale3d=0.02)
    sd = s.get_model()
    names = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")
    # one ordinary step first, so that the moments are non-trivial
    gen = torch.Generator(device=DEV).manual_seed(5)
    s.grads.size = sd.size
    s.grads.flat.normal_(generator=gen)
    s.grads.flat.mul_(1e-3)
    s.step(501)
    assert s._optimizer.step_count == 1
    before = {k: {nm: b.tensor(nm).clone() for nm in names} for k, b in (("p", sd), ("m", s._optimizer.exp_avg), ("v", s._optimizer.exp_avg_sq))}
    lr0 = s._optimizer.lr[0]
    # refinement iteration: duplicate every seventh Gaussian (all count as small by a generous threshold)
    s._params.grow_scale3d = 1e9
    info = torch.zeros((2, n), device=DEV)
    info[0] = 1.0
    hot = torch.arange(n, device=DEV) % 7 == 0
    info[1, hot] = 1.0
    s.densification_info = info
    s.grads.flat.normal_(generator=gen)          # this iteration's (now stale) gradients
    s.grow_gs(600)
    k = int(hot.sum())
    assert sd.size == n + k
    s.step(600)
    assert s._optimizer.step_count == 1                       # not counted
    assert s._optimizer.lr[0] == lr0 * s._scheduler.gamma     # the scheduler still ran
    idx = hot.nonzero().squeeze(-1)
    for nm in names:
        exp_p = torch.cat([before["p"][nm], before["p"][nm].index_select(0, idx)], 0)
        assert torch.equal(sd.tensor(nm), exp_p), nm
        for key, buf in (("m", s._optimizer.exp_avg), ("v", s._optimizer.exp_avg_sq)):
            exp_m = torch.cat([before[key][nm], torch.zeros_like(before[key][nm].index_select(0, idx))], 0)
            assert torch.equal(buf.tensor(nm), exp_m), (nm, key)
    # the following iteration steps again
    s.grads.size = sd.size
    s.grads.flat.normal_(generator=gen)
    s.step(601)
    assert s._optimizer.step_count == 2
    assert not torch.equal(sd.tensor("means")[:n], before["p"]["means"])
