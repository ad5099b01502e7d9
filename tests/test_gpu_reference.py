"""Parity against the REFERENCE ITSELF: the reference's unmodified CUDA sources of this path, built by
oracle/ref_build.py into oracle/_ref/lfs_reference.so (flags of the reference: -O3 --use_fast_math), run on the
same seeded inputs as the CUDA library of this repository and as the CPU oracle.

What is compared, and how tight:
  * integer / index work (tile counts, sort keys, tile lists, offsets) on identical inputs: bit-exact;
  * projection from raw parameters: the reference evaluates `__logf` / fast division under --use_fast_math while this
    library and the oracle round every operation once (IEEE, no contraction), so radii may differ for a handful of
    Gaussians whose extent lands within rounding of an integer; the count is asserted to stay below 0.1 % and
    means2d within 0.02 px (measured: 2 of 16,384 and 0.0045 px);
  * images 1e-4 max-abs except the few pixels where an alpha lands within rounding of the 1/255 cut on one side
    only (at most 8 pixels may exceed it), gradients 1e-3 relative L2, loss 1e-6.
"""
import numpy as np
import pytest
import torch

from conftest import make_scene, rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LRS = [1.6e-4, 2.5e-3, 1.25e-4, 5e-3, 1e-3, 5e-2]
NAMES = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")
SCENES = [(16384, 256, 256, 0, 0, (0.0, 0.0, 0.0)), (20000, 250, 170, 3, 3, (0.2, 0.5, 0.1))]


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


@pytest.fixture(scope="module")
def ref(R):
    return R.load()


def _projection_inputs(R, synth, n, W, H, deg, seed):
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=seed)
    means, q, s, o, sh = R.activated(P)
    return P, vm, K, means, q, s, o, sh, T(vm[None]), T(K[None])


@pytest.mark.parametrize("n,W,H,deg,seed,bg", SCENES)
def test_projection_against_reference(pkg, orc, synth, R, ref, n, W, H, deg, seed, bg):
    P, vm, K, means, q, s, o, sh, vmt, Kt = _projection_inputs(R, synth, n, W, H, deg, seed)
    a = ref.projection_ut_3dgs_fused(means, q, s, o, vmt, None, Kt, W, H, 0.3, 0.01, 1e4, 0.0, True, 0, None, 4, None, None, None)
    b = pkg.ops.projection_ut_3dgs_fused(means, q, s, o, vmt, None, Kt, W, H, 0.3, 0.01, 1e4, 0.0, True, 0)
    qn, _ = orc.act_quat(P["rotation_raw"])
    c = orc.projection_ut_3dgs_fused(P["means"], qn, orc.act_scale(P["scaling_raw"]), orc.act_opacity(P["opacity_raw"]), vm[None], K[None],
                                     W, H, calc_compensations=True)
    ra = a[0].cpu().numpy()[0]
    va = (ra > 0).all(-1)
    assert va.sum() > 1000
    for name, radii, m2, dep, con, comp in (("library", b[0].cpu().numpy()[0], b[1].cpu().numpy()[0], b[2].cpu().numpy()[0],
                                             b[3].cpu().numpy()[0], b[4].cpu().numpy()[0]),
                                            ("oracle", c[0][0], c[1][0], c[2][0], c[3][0], c[4][0])):
        vb = (radii > 0).all(-1)
        assert (va != vb).sum() <= max(1, n // 2000), name                      # visibility set
        assert (ra != radii).any(-1).sum() <= max(2, n // 1000), name          # radii (fast-math log / division)
        both = va & vb
        assert np.abs(a[1].cpu().numpy()[0][both] - m2[both]).max() < 0.02, name
        assert np.array_equal(a[2].cpu().numpy()[0][both].view(np.uint32), dep[both].view(np.uint32)), name   # depths: bit-exact
        assert rel_l2(con[both], a[3].cpu().numpy()[0][both]) < 1e-3, name
        assert np.abs(a[4].cpu().numpy()[0][both] - comp[both]).max() < 1e-3, name


@pytest.mark.parametrize("n,W,H,deg,seed,bg", SCENES)
def test_tile_lists_bit_exact_against_reference(pkg, orc, synth, R, ref, n, W, H, deg, seed, bg):
    """intersect_tile / intersect_offset fed with the reference's own projection outputs: every integer output
    equals the reference's (and the oracle's) bit for bit, sorted and unsorted."""
    P, vm, K, means, q, s, o, sh, vmt, Kt = _projection_inputs(R, synth, n, W, H, deg, seed)
    a = ref.projection_ut_3dgs_fused(means, q, s, o, vmt, None, Kt, W, H, 0.3, 0.01, 1e4, 0.0, False, 0, None, 4, None, None, None)
    tw, th = (W + 15) // 16, (H + 15) // 16
    for sort in (True, False):
        ia = ref.intersect_tile(a[1], a[0], a[2], None, None, 1, 16, tw, th, sort)
        ib = pkg.ops.intersect_tile(a[1], a[0], a[2], None, None, 1, 16, tw, th, sort)
        ic = orc.intersect_tile(a[1].cpu().numpy(), a[0].cpu().numpy(), a[2].cpu().numpy(), 1, 16, tw, th, sort)
        assert ia[2].numel() > 10000
        for k in range(3):
            assert torch.equal(ia[k], ib[k]), (sort, k)
            assert np.array_equal(ic[k], ia[k].cpu().numpy()), (sort, k)
    ia = ref.intersect_tile(a[1], a[0], a[2], None, None, 1, 16, tw, th, True)
    oa = ref.intersect_offset(ia[1], 1, tw, th)
    assert torch.equal(oa, pkg.ops.intersect_offset(ia[1], 1, tw, th))
    assert np.array_equal(orc.intersect_offset(ia[1].cpu().numpy(), 1, tw, th), oa.cpu().numpy())


@pytest.mark.parametrize("n,W,H,deg,seed,bg", SCENES)
def test_sh_and_rasterizer_operators_against_reference(pkg, synth, R, ref, n, W, H, deg, seed, bg):
    """SH forward / backward and the rasterizer pair on IDENTICAL inputs (the reference's projection and lists)."""
    ops = pkg.ops
    P, vm, K, means, q, s, o, sh, vmt, Kt = _projection_inputs(R, synth, n, W, H, deg, seed)
    a = ref.projection_ut_3dgs_fused(means, q, s, o, vmt, None, Kt, W, H, 0.3, 0.01, 1e4, 0.0, False, 0, None, 4, None, None, None)
    tw, th = (W + 15) // 16, (H + 15) // 16
    ia = ref.intersect_tile(a[1], a[0], a[2], None, None, 1, 16, tw, th, True)
    oa = ref.intersect_offset(ia[1], 1, tw, th)
    campos = torch.inverse(vmt)[:, :3, 3]
    dirs = (means[None] - campos[:, None]).contiguous()
    masks = (a[0] > 0).all(-1)
    shc = sh[None].contiguous()
    ca = ref.spherical_harmonics_fwd(deg, dirs, shc, masks)
    cb = ops.spherical_harmonics_fwd(deg, dirs, shc, masks)
    assert float((ca - cb)[masks].abs().max()) < 1e-6
    gen = torch.Generator(device=DEV).manual_seed(seed)
    vcol = torch.randn(ca.shape, generator=gen, device=DEV)
    ga = ref.spherical_harmonics_bwd(sh.shape[1], deg, dirs, shc, masks, vcol, False)[0]
    gb = ops.spherical_harmonics_bwd(sh.shape[1], deg, dirs, None, masks, vcol, False)[0]
    assert float((ga - gb).abs().max()) < 1e-6
    colors = torch.clamp_min(ca + 0.5, 0.0)
    colors[~masks] = 0
    bgt = T(np.asarray([bg], np.float32))
    common = (means, q, s, colors.contiguous(), o[None].contiguous(), bgt, None, W, H, 16, vmt, None, Kt, 0, None, 4, None, None, None,
              oa, ia[2])
    fa = ref.rasterize_to_pixels_from_world_3dgs_fwd(*common)
    fb = ops.rasterize_to_pixels_from_world_3dgs_fwd(*common)
    d = (fa[0] - fb[0]).abs().amax(-1)
    assert int((d > 1e-4).sum()) <= 8 and float(torch.quantile(d.flatten(), 0.9995)) < 1e-4, float(d.max())
    assert int(((fa[1] - fb[1]).abs() > 1e-4).sum()) <= 8
    assert int((fa[2] != fb[2]).sum()) <= 8
    vr = torch.randn(fa[0].shape, generator=gen, device=DEV)
    va = torch.randn(fa[1].shape, generator=gen, device=DEV) * 0.1
    ba = ref.rasterize_to_pixels_from_world_3dgs_bwd(*common, fa[1], fa[2], vr, va)
    bb = ops.rasterize_to_pixels_from_world_3dgs_bwd(*common, fa[1], fa[2], vr, va)
    for name, x, y in zip(("v_means", "v_quats", "v_scales", "v_colors", "v_opacities"), ba, bb):
        assert rel_l2(y.cpu().numpy(), x.cpu().numpy()) < 1e-3, name


def test_loss_optimizer_mcmc_operators_against_reference(pkg, orc, R, ref):
    ops = pkg.ops
    gen = torch.Generator(device=DEV).manual_seed(7)
    H, W = 170, 250
    img1 = torch.rand((1, 3, H, W), generator=gen, device=DEV)
    img2 = torch.rand((1, 3, H, W), generator=gen, device=DEV)
    sa, sb = ref.fusedssim(1e-4, 9e-4, img1, img2, True), ops.fusedssim(1e-4, 9e-4, img1, img2, True)
    for x, y in zip(sa, sb):
        assert float((x - y).abs().max()) < 3e-5
    dl = torch.randn(img1.shape, generator=gen, device=DEV)
    ga = ref.fusedssim_backward(1e-4, 9e-4, img1, img2, dl, *sa[1:])
    gb = ops.fusedssim_backward(1e-4, 9e-4, img1, img2, dl, *sa[1:])
    assert float((ga - gb).abs().max()) < 1e-5
    # the whole photometric loss and its gradient through the reference's autograd function
    lossfn = pkg.trainer.PhotometricLoss(W, H, DEV, 0.2)
    render = (torch.rand((H, W, 3), generator=gen, device=DEV) * 1.4 - 0.2).contiguous()   # some values outside [0, 1]
    chw = render.permute(2, 0, 1).clamp(0, 1).contiguous().requires_grad_(True)
    l_ref = ref.photometric_loss(chw, img2[0], 0.2)
    l_ref.backward()
    l, v_render = lossfn(render, img2[0].contiguous())
    assert abs(float(l[0]) - float(l_ref.detach())) < 1e-6
    inside = ((render >= 0) & (render <= 1)).permute(2, 0, 1)
    g_ref = (chw.grad * inside).permute(1, 2, 0)        # the clamp passes no gradient outside [0, 1]
    assert rel_l2(v_render.cpu().numpy(), g_ref.cpu().numpy()) < 1e-4
    # Adam
    p = torch.randn(100003, generator=gen, device=DEV)
    g = torch.randn(p.shape, generator=gen, device=DEV) * 1e-3
    m1 = torch.randn(p.shape, generator=gen, device=DEV) * 1e-3
    v1 = torch.rand(p.shape, generator=gen, device=DEV) * 1e-6
    pa, ma, va = p.clone(), m1.clone(), v1.clone()
    pb, mb, vb = p.clone(), m1.clone(), v1.clone()
    bc1, bc2 = 1.0 / (1 - 0.9 ** 7), 1.0 / np.sqrt(1 - 0.999 ** 7)
    ref.adam_step_wrapper(pa, ma, va, g, 1e-3, 0.9, 0.999, 1e-15, bc1, bc2)
    ops.adam_step_wrapper(pb, mb, vb, g, 1e-3, 0.9, 0.999, 1e-15, bc1, bc2)
    assert float((pa - pb).abs().max()) < 5e-7 and rel_l2(mb.cpu().numpy(), ma.cpu().numpy()) < 1e-6
    assert rel_l2(vb.cpu().numpy(), va.cpu().numpy()) < 1e-6
    # relocation (eq. 9), noise, rotation matrices
    M = 50000
    op_ = torch.rand(M, generator=gen, device=DEV) * 0.98 + 0.01
    sc_ = torch.rand((M, 3), generator=gen, device=DEV) * 0.1 + 1e-3
    ratios = torch.randint(1, 52, (M,), generator=gen, device=DEV, dtype=torch.int32)
    binoms = T(orc.binoms_table(51))
    xa, xb = ref.relocation(op_, sc_, ratios, binoms, 51), ops.relocation(op_, sc_, ratios, binoms, 51)
    assert float(((xa[0] - xb[0]).abs() / xa[0].abs().clamp_min(1e-12)).max()) < 1e-3     # the reference's pow is fast-math
    assert float(((xa[1] - xb[1]).abs() / xa[1].abs().clamp_min(1e-12)).max()) < 1e-3
    xo = orc.relocation(op_.cpu().numpy(), sc_.cpu().numpy(), ratios.cpu().numpy(), orc.binoms_table(51), 51)
    assert np.abs(xo[0] - xa[0].cpu().numpy()).max() < 1e-3 * float(xa[0].abs().max())
    ro = torch.randn((M, 1), generator=gen, device=DEV)
    rs = torch.randn((M, 3), generator=gen, device=DEV) - 4
    rq = torch.randn((M, 4), generator=gen, device=DEV)
    nz = torch.randn((M, 3), generator=gen, device=DEV)
    ma_, mb_ = torch.zeros((M, 3), device=DEV), torch.zeros((M, 3), device=DEV)
    ref.add_noise(ro, rs, rq, nz, ma_, 80.0)
    ops.add_noise(ro, rs, rq, nz, mb_, 80.0)
    assert rel_l2(mb_.cpu().numpy(), ma_.cpu().numpy()) < 1e-5
    assert float((ref.quats_to_rotmats(rq) - ops.quats_to_rotmats(rq)).abs().max()) < 1e-6
    # regularizers: loss values and accumulated gradients
    sraw = (torch.randn((M, 3), generator=gen, device=DEV) - 4).requires_grad_(True)
    oraw = torch.randn((M, 1), generator=gen, device=DEV).requires_grad_(True)
    sraw.grad, oraw.grad = torch.zeros_like(sraw), torch.zeros_like(oraw)
    ls = ref.exp_l1_regularization_with_grad(sraw, 0.01)
    lo = ref.sigmoid_l1_regularization_with_grad(oraw, 0.01)
    tr = pkg.trainer
    model, grads = tr.SplatData(M, 1, DEV), tr.SplatData(M, 1, DEV)
    model.tensor("scaling_raw").copy_(sraw.detach())
    model.tensor("opacity_raw").copy_(oraw.detach())
    out = tr.regularization(model, grads, 0.01, 0.01).tolist()
    assert abs(out[0] - ls) < 1e-6 and abs(out[1] - lo) < 1e-6
    assert rel_l2(grads.tensor("scaling_raw").cpu().numpy(), sraw.grad.cpu().numpy()) < 1e-5
    assert rel_l2(grads.tensor("opacity_raw").cpu().numpy(), oraw.grad.cpu().numpy()) < 1e-5


def _reference_step(R, P, P2, vm, K, W, H, deg, bg, gut=True):
    target = R.make_trainer(P2, [0.0] * 6, deg).render_no_grad(True, T(vm[None]), T(K[None]), W, H, T(bg), 0).image.contiguous()
    return target, R.step_outputs(P, vm, K, W, H, deg, bg, target.cpu().numpy(), 0.2, gut, None)


@pytest.mark.parametrize("n,W,H,deg,seed,bg", SCENES)
def test_training_step_against_reference(pkg, orc, synth, R, n, W, H, deg, seed, bg):
    """rasterize() + compute_photometric_loss + backward through the reference's own autograd nodes, against the fused
    path of this library AND against the CPU oracle: image, loss, all six raw-parameter gradients."""
    tr = pkg.trainer
    bg = np.asarray(bg, np.float32)
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=seed)
    _, P2, _, _ = make_scene(synth, n, W, H, deg, seed=seed + 1000)
    target, r = _reference_step(R, P, P2, vm, K, W, H, deg, bg)
    model = tr.SplatData(n, (deg + 1) ** 2, DEV).load(P)
    grads = model.like()
    rast = tr.Rasterizer(model, W, H, deg)
    lossfn = tr.PhotometricLoss(W, H, DEV)
    out = rast.forward(tr.Camera(T(vm), T(K), W, H), T(bg))
    loss, v_render = lossfn(out.image, target)
    rast.backward(v_render, grads, T(bg))
    d = np.abs(np.clip(out.image.cpu().numpy().transpose(2, 0, 1), 0, 1) - r["image"]).max(0)
    assert (d > 1e-4).sum() <= 8 and np.quantile(d, 0.9995) < 1e-4, d.max()
    assert (np.abs(out.alpha.cpu().numpy()[..., 0] - r["alpha"][0]) > 1e-4).sum() <= 8
    assert abs(float(loss[0]) - r["loss"]) < 1e-6
    for name in NAMES:
        a = grads.tensor(name).cpu().numpy()
        if a.size:
            assert rel_l2(a, r["grad_" + name]) < 1e-3, name
    # the oracle against the reference: this is what pins the oracle
    fwd = orc.render_fwd(P, vm, K, W, H, deg, background=bg)
    lo, g_ref, _, _ = orc.photometric_loss(fwd["render"], target.cpu().numpy(), 0.2)
    bwd = orc.render_bwd(P, fwd, vm, K, W, H, deg, g_ref, background=bg)
    d = np.abs(np.clip(fwd["render"].transpose(2, 0, 1), 0, 1) - r["image"]).max(0)
    assert (d > 1e-4).sum() <= 8 and np.quantile(d, 0.9995) < 1e-4, d.max()
    assert abs(lo - r["loss"]) < 1e-6
    for name in NAMES:
        if bwd[name].size:
            assert rel_l2(bwd[name], r["grad_" + name]) < 1e-3, name


def test_fused_adam_class_against_reference(pkg, synth, R):
    """FusedAdam::step of the reference (its own class: lazy state, per-group rates, shN skipped up to iteration 1000,
    ExponentialLR on the means) for three iterations with given gradients, against strategy.FusedAdam + ExponentialLR."""
    tr, st = pkg.trainer, pkg.strategy
    n, deg = 3000, 2
    P = synth.make_gaussians(n, 5, "clusters", deg)
    t = R.make_trainer(P, LRS, deg, iterations=30000)
    model = tr.SplatData(n, (deg + 1) ** 2, DEV).load(P)
    opt = st.FusedAdam(model, LRS, (0.9, 0.999), 1e-15)
    sched = st.ExponentialLR(opt, 0.01 ** (1.0 / 30000), 0)
    grads = model.like()
    gen = torch.Generator(device=DEV).manual_seed(3)
    for it in (999, 1000, 1001):
        for name, p in zip(NAMES, t.params()):
            g = torch.randn(p.shape, generator=gen, device=DEV) * 1e-2
            p.grad = g.clone()
            grads.tensor(name).copy_(g)
        t.optimizer_step(it)
        opt.step(it, grads)
        sched.step()
    for name, p, (m, v, count) in zip(NAMES, t.params(), t.moments()):
        assert count == 3, name
        assert rel_l2(model.tensor(name).cpu().numpy() - P[name].reshape(p.shape), p.detach().cpu().numpy() - P[name].reshape(p.shape)) < 1e-5, name
        assert rel_l2(opt.exp_avg.tensor(name).cpu().numpy(), m.cpu().numpy()) < 1e-5, name
        assert rel_l2(opt.exp_avg_sq.tensor(name).cpu().numpy(), v.cpu().numpy()) < 1e-5, name


def test_ewa_step_against_reference(pkg, synth, R):
    """The default (non --gut) path: fast_rasterize() + loss + backward of the reference against lfs_ewa_forward /
    lfs_ewa_backward. Kept at 20,000 Gaussians: the reference's own forward of this path fails on the host (garbage bucket
    count, `numel: integer multiplication overflow`) from about 200,000 Gaussians in this toolchain."""
    tr = pkg.trainer
    n, W, H, deg, seed = 20000, 250, 170, 3, 3
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=seed)
    bg = np.array([0.1, 0.2, 0.3], np.float32)
    target = torch.rand((3, H, W), generator=torch.Generator().manual_seed(2)).to(DEV)
    r = R.step_outputs(P, vm, K, W, H, deg, bg, target.cpu().numpy(), 0.2, False, None)
    model = tr.SplatData(n, (deg + 1) ** 2, DEV).load(P)
    grads = model.like()
    rast = tr.FastRasterizer(model, W, H, deg)
    out = rast.forward(tr.Camera(T(vm), T(K), W, H), T(bg))
    d = np.abs(out.image.cpu().numpy() - r["image"]).max(0)
    assert (d > 1e-4).sum() <= 8 and np.quantile(d, 0.9995) < 1e-4, d.max()
    assert (np.abs(out.alpha.cpu().numpy() - r["alpha"]) > 1e-4).sum() <= 8
    lossfn = tr.PhotometricLoss(W, H, DEV)
    loss, v_hwc = lossfn(out.image.permute(1, 2, 0).contiguous(), target)
    rast.backward(v_hwc.permute(2, 0, 1).contiguous(), grads, T(bg))
    assert abs(float(loss[0]) - r["loss"]) < 1e-6
    for name in NAMES:
        a = grads.tensor(name).cpu().numpy()
        if a.size:
            assert rel_l2(a, r["grad_" + name]) < 1e-3, name


def test_ewa_pose_gradient_against_reference(pkg, synth, R):
    """grad_w2c of FastGSRasterize::backward (kernels_backward.cuh:160-173, returned when w2c requires a gradient) against
    lfs_ewa_backward's: both sum ~N float32 terms with atomics in arbitrary order, hence the relative bound."""
    tr = pkg.trainer
    n, W, H, deg, seed = 20000, 250, 170, 3, 3
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=seed)
    bg = np.array([0.1, 0.2, 0.3], np.float32)
    G = (torch.randn((3, H, W), generator=torch.Generator().manual_seed(4)) * 1e-3).to(DEV)
    trn = R.make_trainer(P, [0.0] * 6, deg)
    vm_t = T(vm[None]).clone().requires_grad_(True)
    rr = trn.fast_rasterize(vm_t, float(K[0, 0]), float(K[1, 1]), float(K[0, 2]), float(K[1, 2]), W, H, T(bg))
    (rr.image * G).sum().backward()
    ref_gw = vm_t.grad[0].cpu().numpy()
    assert np.abs(ref_gw[:3]).max() > 0 and (ref_gw[3] == 0).all()
    model = tr.SplatData(n, (deg + 1) ** 2, DEV).load(P)
    rast = tr.FastRasterizer(model, W, H, deg)
    rast.forward(tr.Camera(T(vm), T(K), W, H), T(bg))
    gw = torch.zeros(4, 4, device=DEV)
    rast.backward(G, model.like(), T(bg), grad_w2c=gw)
    gw = gw.cpu().numpy()
    assert (gw[3] == 0).all() and rel_l2(gw[:3], ref_gw[:3]) < 1e-3, (gw, ref_gw)


def test_equirectangular_camera_against_reference(pkg, synth, R, ref):
    """CameraModelType::EQUIRECTANGULAR (gsplat/Cameras.cuh:1003-1039): the whole sphere on a 2:1 image, no near-plane cull,
    Gaussians behind the camera carry a negative depth whose bit pattern sorts after every positive one
    (gsplat/IntersectTile.cu:96-98). Projection, lists, forward image and the backward of the operator pair against the
    reference itself, with the camera INSIDE the scene so that every direction is populated."""
    ops = pkg.ops
    n, W, H, deg = 20000, 256, 128, 2
    P = synth.make_gaussians(n, 6, "cube", deg)
    P["scaling_raw"] = (P["scaling_raw"] + np.float32(0.7)).astype(np.float32)
    means, q, s, o, sh = R.activated(P)
    vm = np.eye(4, dtype=np.float32)
    vm[:3, 3] = [0.05, -0.02, 0.1]                      # camera close to the centre of the cube of Gaussians
    K = synth.intrinsics(100.0, 100.0, W / 2, H / 2)    # unused by the model, passed like the trainer does
    vmt, Kt = T(vm[None]), T(K[None])
    a = ref.projection_ut_3dgs_fused(means, q, s, o, vmt, None, Kt, W, H, 0.3, 0.01, 1e4, 0.0, False, 3, None, 4, None, None, None)
    b = ops.projection_ut_3dgs_fused(means, q, s, o, vmt, None, Kt, W, H, 0.3, 0.01, 1e4, 0.0, False, 3)
    va, vb = (a[0] > 0).all(-1), (b[0] > 0).all(-1)
    assert int(va.sum()) > 5000 and int((a[2][va] < 0).sum()) > 1000          # behind the camera too
    assert int((va != vb).sum()) <= n // 1000 and int((a[0] != b[0]).any(-1).sum()) <= n // 500
    both = va & vb
    assert float((a[1][both] - b[1][both]).abs().max()) < 0.05
    assert torch.equal(a[2][both], b[2][both])
    # lists from the reference's projection: bit-exact, negative depths included
    tw, th = (W + 15) // 16, (H + 15) // 16
    ia = ref.intersect_tile(a[1], a[0], a[2], None, None, 1, 16, tw, th, True)
    ib = ops.intersect_tile(a[1], a[0], a[2], None, None, 1, 16, tw, th, True)
    assert all(torch.equal(x, y) for x, y in zip(ia, ib)) and ia[2].numel() > 20000
    oa = ref.intersect_offset(ia[1], 1, tw, th)
    assert torch.equal(oa, ops.intersect_offset(ia[1], 1, tw, th))
    # rasterizer pair on identical inputs
    gen = torch.Generator(device=DEV).manual_seed(2)
    colors = torch.rand((1, n, 3), generator=gen, device=DEV)
    common = (means, q, s, colors, o[None].contiguous(), T(np.array([[0.1, 0.2, 0.3]], np.float32)), None, W, H, 16, vmt, None, Kt, 3,
              None, 4, None, None, None, oa, ia[2])
    fa = ref.rasterize_to_pixels_from_world_3dgs_fwd(*common)
    fb = ops.rasterize_to_pixels_from_world_3dgs_fwd(*common)
    d = (fa[0] - fb[0]).abs().amax(-1)
    assert int((d > 1e-4).sum()) <= 8 and float(torch.quantile(d.flatten(), 0.9995)) < 1e-4, float(d.max())
    vr = torch.randn(fa[0].shape, generator=gen, device=DEV)
    va_ = torch.randn(fa[1].shape, generator=gen, device=DEV) * 0.1
    ba = ref.rasterize_to_pixels_from_world_3dgs_bwd(*common, fa[1], fa[2], vr, va_)
    bb = ops.rasterize_to_pixels_from_world_3dgs_bwd(*common, fa[1], fa[2], vr, va_)
    for name, x, y in zip(("v_means", "v_quats", "v_scales", "v_colors", "v_opacities"), ba, bb):
        assert rel_l2(y.cpu().numpy(), x.cpu().numpy()) < 1e-3, name
    # the fused path from raw parameters against the reference's rasterize()
    tr = pkg.trainer
    t = R.make_trainer(P, [0.0] * 6, deg)
    bg = T(np.array([0.1, 0.2, 0.3], np.float32))
    rr = t.render_no_grad(True, vmt, Kt, W, H, bg, 3)
    model = tr.SplatData(n, (deg + 1) ** 2, DEV).load(P)
    rast = tr.Rasterizer(model, W, H, deg, camera_model=3)
    out = rast.forward(tr.Camera(T(vm), T(K), W, H, camera_model=3), bg)
    d = (out.image.permute(2, 0, 1).clamp(0, 1) - rr.image).abs().amax(0)
    assert int((d > 1e-4).sum()) <= 40 and float(torch.quantile(d.flatten(), 0.998)) < 1e-4, float(d.max())
