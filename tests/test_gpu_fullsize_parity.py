"""Parity AT THE BENCHMARK SIZES, against the reference's own CUDA build (oracle/_ref) and against the CPU oracle:

  * config 2: one full training step of 1,000,000 Gaussians at 1296x840 (projection, lists, image, loss, the six
    raw-parameter gradients);
  * config 3: the MCMC refine step on 3,000,000 Gaussians with torch's CUDA generator seeded alike on both sides
    (dead / alive lists, sampled indices, ratios, moved rows, noise);
  * config 5: the forward of 6,000,000 Gaussians at 3840x2160 (pinhole) and 1920x1920 (180 degree fisheye), one pose
    each.

The measured mismatch counts are printed (run pytest with -s to see them)."""
import numpy as np
import pytest
import torch

from conftest import rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAMES = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


@pytest.fixture(scope="module")
def R():
    from oracle import ref_build, reference
    if not reference.available():
        if ref_build.reference_root() is None:
            pytest.skip("oracle/_ref is not built and there is no reference checkout to build it from")
        ref_build.build()
    return reference


def test_train_1m_step_against_reference_and_oracle(pkg, orc, synth, R):
    tr = pkg.trainer
    cfg = synth.CONFIGS["train_1m"]
    n, W, H, deg = cfg["n"], cfg["W"], cfg["H"], cfg["sh_degree"]
    P = synth.make_gaussians(n, 0, cfg["layout"], deg)
    poses, K = synth.make_cameras(cfg)
    vm = poses[synth.pose_index(3, cfg["n_poses"])]
    bg = np.array([0.1, 0.2, 0.3], np.float32)
    # target: the held-out Gaussian set of the benchmark, rendered by the reference
    held = R.make_trainer(synth.make_gaussians(n, 1000, cfg["layout"], deg), [0.0] * 6, deg)
    target = held.render_no_grad(True, T(vm[None]), T(K[None]), W, H, T(bg), 0).image.contiguous()
    del held
    # reference, twice: its float atomics make its own gradients vary from run to run
    t = R.make_trainer(P, [0.0] * 6, deg)
    image, alpha, loss_ref = t.forward_backward(True, T(vm[None]), T(K[None]), W, H, T(bg), target, 0.2)
    g_ref = [g.clone() for g in t.grads()]
    t.zero_grad()
    t.forward_backward(True, T(vm[None]), T(K[None]), W, H, T(bg), target, 0.2)
    for name, g0, g1 in zip(NAMES, g_ref, t.grads()):
        print(f"  grad {name}: reference run 1 vs run 2 rel-L2 {rel_l2(g1.cpu().numpy(), g0.cpu().numpy()):.2e}")
    rr = t.render_no_grad(True, T(vm[None]), T(K[None]), W, H, T(bg), 0)
    radii_ref = rr.radii[0]
    # this library
    model = tr.SplatData(n, 16, DEV).load(P)
    grads = model.like()
    rast = tr.Rasterizer(model, W, H, deg, isect_capacity=12 * n)
    lossfn = tr.PhotometricLoss(W, H, DEV)
    out = rast.forward(tr.Camera(T(vm), T(K), W, H), T(bg))
    loss, v_render = lossfn(out.image, target)
    rast.backward(v_render, grads, T(bg))
    st = rast.state()
    vis_ref, vis = (radii_ref > 0).all(-1), (st["radii"] > 0).all(-1)
    n_vis_mism = int((vis_ref != vis).sum())
    n_radii_mism = int((radii_ref != st["radii"]).any(-1).sum())
    both = vis & vis_ref
    m2_diff = float((rr.means2d[0][both] - st["means2d"][both]).abs().max())
    d = (out.image.permute(2, 0, 1).clamp(0, 1) - image).abs().amax(0)
    n_px = int((d > 1e-4).sum())
    print(f"\ntrain_1m vs reference CUDA: visible {int(vis_ref.sum())}, visibility mismatches {n_vis_mism}, radii mismatches {n_radii_mism}, "
          f"means2d max diff {m2_diff:.4f} px, pixels > 1e-4: {n_px} of {W * H} (max {float(d.max()):.2e}), "
          f"loss {float(loss[0]):.8f} vs {float(loss_ref):.8f}")
    assert n_vis_mism <= n // 10000 and n_radii_mism <= n // 1000 and m2_diff < 0.1
    # every pixel walks hundreds of Gaussians here, each with a hard cut at alpha = 1/255 (and a list that may differ by the
    # Gaussians whose radius moved): a cut that falls the other way changes the pixel by up to ~4e-3. Measured: 739 of
    # 1,088,640 pixels above 1e-4, maximum 5e-3, loss equal to 8 digits.
    assert n_px <= W * H // 500 and float(torch.quantile(d.flatten()[:: 7], 0.998)) < 1e-4 and float(d.max()) < 2e-2
    assert abs(float(loss[0]) - float(loss_ref)) < 1e-6
    rels = {}
    for name, g in zip(NAMES, g_ref):
        rels[name] = rel_l2(grads.tensor(name).cpu().numpy(), g.cpu().numpy())
        print(f"  grad {name}: rel-L2 vs reference {rels[name]:.2e}")
    g_ref_np = {name: g.cpu().numpy() for name, g in zip(NAMES, g_ref)}
    del t, g_ref
    # the CPU oracle on the same step: lists bit-exact, image, loss, gradients
    orc.use_all_cores()
    fwd = orc.render_fwd(P, vm, K, W, H, deg, background=bg)
    assert np.array_equal(st["radii"].cpu().numpy(), fwd["radii"])
    assert np.array_equal(st["tiles_per_gauss"].cpu().numpy(), fwd["tiles_per_gauss"])
    assert np.array_equal(st["flatten_ids"].cpu().numpy(), fwd["flatten_ids"])
    assert np.array_equal(st["tile_offsets"].cpu().numpy()[:-1], fwd["tile_offsets"].reshape(-1))
    vo = fwd["masks"]
    assert np.array_equal(st["means2d"].cpu().numpy()[vo].view(np.uint32), fwd["means2d"][vo].view(np.uint32))
    do = np.abs(out.image.cpu().numpy() - fwd["render"]).max(-1)
    da = np.abs(out.alpha.cpu().numpy() - fwd["alpha"]).max(-1)
    print(f"train_1m vs CPU oracle: lists bit-exact (I = {fwd['flatten_ids'].size}), pixels > 1e-4: {(do > 1e-4).sum()} (max {do.max():.2e}), "
          f"alpha > 1e-4: {(da > 1e-4).sum()}, last_ids mismatches {(st['last_ids'].cpu().numpy() != fwd['last_ids']).sum()}")
    assert (do > 1e-4).sum() <= W * H // 2000 and np.quantile(do, 0.999) < 1e-4
    assert (da > 1e-4).sum() <= W * H // 2000
    lo, g_o, _, _ = orc.photometric_loss(fwd["render"], target.cpu().numpy(), 0.2)
    assert abs(lo - float(loss[0])) < 1e-6
    bwd = orc.render_bwd(P, fwd, vm, K, W, H, deg, g_o, background=bg)
    for name in NAMES:
        rel = rel_l2(grads.tensor(name).cpu().numpy(), bwd[name])
        print(f"  grad {name}: rel-L2 library vs oracle {rel:.2e}; oracle vs reference {rel_l2(bwd[name], g_ref_np[name]):.2e}")
        assert rel < 1e-3, name
    # Against the fast-math reference the bar at this size is 2e-3: its own gradients are 1.06e-3 (means) away from its
    # arithmetic evaluated in IEEE float32 (the oracle column above) while two runs of the reference differ by 1e-7, i.e. the
    # distance is the reference's approximate exp / rsqrt / division acting on the alpha = 1/255 cut, not summation order.
    # Library and oracle, which round every operation once, agree to 3e-4 here and to 1e-3 everywhere.
    for name in NAMES:
        assert rels[name] < 2e-3, (name, rels[name])


def test_mcmc_refine_3m_against_reference(pkg, synth, R):
    """Config 3 at size. torch.multinomial on CUDA builds its cumulative distribution with a parallel float scan whose
    summation order varies from launch to launch, so the reference does not reproduce its OWN draw bit for bit at this size
    (measured below). The contract is therefore split: (a) with this library's own draw (same seed, same generator, same
    weights) the sampled indices differ from the reference's in no larger a fraction than two runs of the reference
    differ from each other; (b) GIVEN the reference's draw, everything downstream - dead / alive lists, ratios, which
    rows are copied where, the moments - equals the reference bit for bit, and the relocated opacities / scales agree to
    the reference's fast-math pow (2e-3 relative)."""
    tr, st = pkg.trainer, pkg.strategy
    cfg = synth.CONFIGS["mcmc_3m"]
    n, deg = cfg["n"], cfg["sh_degree"]
    P = synth.make_gaussians(n, 0, cfg["layout"], deg)
    P["opacity_raw"][np.arange(n) % 20 == 7] = -6.0
    cap = int(np.float32(1.05) * np.float32(n)) + 64

    def ours(mode, ref_last=None):
        model = tr.SplatData(n, (deg + 1) ** 2, DEV, capacity=cap).load(P)
        s = st.MCMC(model)
        s.initialize(st.OptimizationParameters(max_cap=cap, sh_degree=deg))
        s._optimizer.exp_avg.flat.fill_(1.0)
        s._optimizer.exp_avg_sq.flat.fill_(2.0)
        torch.manual_seed(1234)
        if mode == "relocate":
            k = s.relocate_gs(None if ref_last is None else ref_last["relocate_sampled_local"])
            return s, model, k, s._dead[:k].clone(), s._sampled[:k].clone(), s._ratios[:k].clone()
        k = s.add_new_gs(None if ref_last is None else ref_last["add_sampled"])
        return s, model, k, None, None, s._ratios[:k].clone()

    def theirs(mode):
        m = R.McmcReference(P, 0.005, cap, DEV)
        for k in NAMES:
            m.m[k].fill_(1.0)
            m.v[k].fill_(2.0)
        torch.manual_seed(1234)
        k = m.relocate_gs() if mode == "relocate" else m.add_new_gs()
        return m, k

    for mode in ("relocate", "add"):
        key = "relocate_sampled" if mode == "relocate" else "add_sampled"
        m, k_ref = theirs(mode)
        m2, _ = theirs(mode)
        self_diff = int((m.last[key] != m2.last[key]).sum())
        del m2
        # (a) own draw
        s, model, k, dead, sampled, ratios = ours(mode)
        assert k == k_ref and k > 100000
        if mode == "relocate":
            assert torch.equal(dead, m.last["dead_indices"])
            own_diff = int((sampled != m.last[key]).sum())
        else:
            own_diff = -1   # the growth draw is not kept by the strategy; its effect is covered by (b)
        print(f"\nmcmc_3m {mode}: {k} draws; reference vs reference differing indices {self_diff}; library vs reference {own_diff}")
        # measured: 14,177 of 150,022 indices differ between two runs of the reference itself, 13,806 between library and reference
        assert own_diff <= 1.5 * self_diff + 100
        del s, model
        # (b) the reference's draw injected: bit-exact bookkeeping
        s, model, k, dead, sampled, ratios = ours(mode, m.last)
        if mode == "relocate":
            assert torch.equal(dead, m.last["dead_indices"]) and torch.equal(sampled, m.last["relocate_sampled"])
            assert torch.equal(ratios, m.last["relocate_ratios"])
        else:
            assert torch.equal(ratios, m.last["add_ratios"])
        size = n + (k if mode == "add" else 0)
        assert model.size == size and m.p["means"].shape[0] == size
        touched = torch.zeros(size, dtype=torch.bool, device=DEV)
        touched[m.last[key]] = True
        if mode == "relocate":
            touched[m.last["dead_indices"]] = True
        else:
            touched[n:] = True
        for name in NAMES:
            a, b = model.tensor(name), m.p[name]
            if name in ("means", "sh0", "shN", "rotation_raw"):
                assert torch.equal(a, b), name                                   # copied rows: bit-identical
            else:
                assert torch.equal(a[~touched], b[~touched]), name
                assert float(((a - b).abs() / b.abs().clamp_min(1e-6)).max()) < 2e-3, name
            assert torch.equal(s._optimizer.exp_avg.tensor(name), m.m[name]), name
            assert torch.equal(s._optimizer.exp_avg_sq.tensor(name), m.v[name]), name
        del s, model, m
    # noise on identical state with the same generator state
    model = tr.SplatData(n, (deg + 1) ** 2, DEV, capacity=cap).load(P)
    s = st.MCMC(model)
    s.initialize(st.OptimizationParameters(max_cap=cap, sh_degree=deg))
    m = R.McmcReference(P, 0.005, cap, DEV)
    torch.manual_seed(99)
    s.inject_noise()
    torch.manual_seed(99)
    m.inject_noise(float(np.float32(s._optimizer.lr[0])) * 5e5)
    assert rel_l2((model.tensor("means") - T(P["means"])).cpu().numpy(), (m.p["means"] - T(P["means"])).cpu().numpy()) < 1e-4


@pytest.mark.parametrize("workload", ["wide_4k", "wide_fisheye"])
def test_wide_forward_against_reference(pkg, synth, R, workload):
    tr = pkg.trainer
    cfg = synth.CONFIGS[workload]
    n, W, H, deg, cm = cfg["n"], cfg["W"], cfg["H"], cfg["sh_degree"], cfg["model"]
    P = synth.make_gaussians(n, 0, cfg["layout"], deg)
    poses, K = synth.make_cameras(cfg)
    vm = poses[5]
    bg = np.zeros(3, np.float32)
    t = R.make_trainer(P, [0.0] * 6, deg)
    rr = t.render_no_grad(True, T(vm[None]), T(K[None]), W, H, T(bg), cm)
    model = tr.SplatData(n, 16, DEV).load(P)
    rast = tr.Rasterizer(model, W, H, deg, camera_model=cm, isect_capacity=4 * n)
    out = rast.forward(tr.Camera(T(vm), T(K), W, H, camera_model=cm), T(bg))
    st = rast.state()
    assert int(out.status[0]) == 0
    radii_ref = rr.radii[0]
    vis_ref, vis = (radii_ref > 0).all(-1), (st["radii"] > 0).all(-1)
    n_vis_mism = int((vis_ref != vis).sum())
    n_radii_mism = int((radii_ref != st["radii"]).any(-1).sum())
    both = vis & vis_ref
    m2_diff = float((rr.means2d[0][both] - st["means2d"][both]).abs().max())
    d = (out.image.permute(2, 0, 1).clamp(0, 1) - rr.image).abs().amax(0)
    n_px = int((d > 1e-4).sum())
    print(f"\n{workload} vs reference CUDA: visible {int(vis_ref.sum())}, I = {st['n_isects']}, visibility mismatches {n_vis_mism}, "
          f"radii mismatches {n_radii_mism}, means2d max diff {m2_diff:.4f} px, pixels > 1e-4: {n_px} of {W * H} (max {float(d.max()):.2e})")
    # measured: 4K pinhole 32 visibility / 4,924 radius mismatches of 2.31 M visible, 0.39 % of the pixels above 1e-4 (max 1.8e-2);
    # fisheye 1,202 / 12,878 of 5.86 M, 1.75 % of the pixels. Each differing pixel is a contribution at the alpha = 1/255 cut
    # (or a Gaussian whose box moved by one tile) that one side takes and the other drops.
    assert n_vis_mism <= n // 2000 and n_radii_mism <= n // 300
    assert n_px <= W * H // 40 and float(torch.quantile(d.flatten()[:: 31], 0.97)) < 1e-4 and float(d.max()) < 5e-2
    # lists from the REFERENCE's projection through this library's intersect: equal to the reference's own lists
    ref = R.load()
    tw, th = (W + 15) // 16, (H + 15) // 16
    ia = ref.intersect_tile(rr.means2d, rr.radii, rr.depths, None, None, 1, 16, tw, th, True)
    ib = pkg.ops.intersect_tile(rr.means2d, rr.radii, rr.depths, None, None, 1, 16, tw, th, True)
    for k in range(3):
        assert torch.equal(ia[k], ib[k]), k
