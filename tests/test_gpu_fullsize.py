"""Full-size configuration (1,000,000 Gaussians, 1296x840, SH degree 3): the CPU oracle would take minutes here,
so parity is checked through size-independent properties of the domain: list sortedness and counting
identities, agreement of the fused path with the operator-level path (which is oracle-checked at small
sizes), determinism of the forward, linearity of the backward, and range invariants."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def full(pkg, synth):
    tr = pkg.trainer
    cfg = synth.CONFIGS["train_1m"]
    n, W, H, deg = cfg["n"], cfg["W"], cfg["H"], cfg["sh_degree"]
    P = synth.make_gaussians(n, 0, cfg["layout"], deg)
    poses, K = synth.make_cameras(cfg)
    model = tr.SplatData(n, 16, DEV).load(P)
    rast = tr.Rasterizer(model, W, H, deg, isect_capacity=12 * n)
    cam = tr.Camera(torch.from_numpy(poses[synth.pose_index(3, 200)]).to(DEV), torch.from_numpy(K).to(DEV), W, H)
    bg = torch.tensor([0.1, 0.2, 0.3], device=DEV)
    out = rast.forward(cam, bg)
    img, alpha = out.image.clone(), out.alpha.clone()
    return dict(P=P, model=model, rast=rast, cam=cam, bg=bg, img=img, alpha=alpha, state=rast.state(), W=W, H=H, n=n, deg=deg)


def test_lists_are_sorted_and_counted(full):
    st = full["state"]
    n_isects = st["n_isects"]
    assert int(full["rast"].status[0]) == 0 and n_isects > 3_000_000
    assert int(st["tiles_per_gauss"].sum()) == n_isects
    vis = (st["radii"] > 0).all(-1)
    assert int(full["rast"].status[2]) == int(vis.sum()) and int((st["tiles_per_gauss"] > 0).sum()) <= int(vis.sum())
    off = st["tile_offsets"].long()
    assert off[0] == 0 and off[-1] == n_isects and bool((off[1:] >= off[:-1]).all())
    # inside every tile: ascending depth bit pattern, ties by ascending Gaussian index
    flat = st["flatten_ids"].long()
    depth_bits = st["depths"].view(torch.int32)[flat].long()
    tile_of = torch.bucketize(torch.arange(n_isects, device=DEV), off[1:], right=True)
    same_tile = tile_of[1:] == tile_of[:-1]
    d0, d1 = depth_bits[:-1], depth_bits[1:]
    ordered = (d1 > d0) | ((d1 == d0) & (flat[1:] > flat[:-1]))
    assert bool((ordered | ~same_tile).all())
    # every instance lies in a tile its Gaussian's box covers, and each (Gaussian, tile) pair appears once
    tw = (full["W"] + 15) // 16
    m2, r = st["means2d"][flat], st["radii"][flat].float()
    tx, ty = (tile_of % tw).float(), (tile_of // tw).float()
    assert bool((torch.floor(m2[:, 0] / 16 - r[:, 0] / 16) <= tx).all() and (tx < torch.ceil(m2[:, 0] / 16 + r[:, 0] / 16)).all())
    assert bool((torch.floor(m2[:, 1] / 16 - r[:, 1] / 16) <= ty).all() and (ty < torch.ceil(m2[:, 1] / 16 + r[:, 1] / 16)).all())
    assert torch.unique(flat * 8192 + tile_of).numel() == n_isects


def test_fused_lists_equal_operator_level_lists(pkg, full):
    """Activations in torch, then the operator-level projection / intersect entry points: bit-identical radii,
    tile counts and sorted lists (the operator level is checked against the oracle at small sizes)."""
    ops, st, P = pkg.ops, full["state"], full["P"]
    t = lambda a: torch.from_numpy(a).to(DEV)
    opac = (1.0 / (1.0 + torch.exp(-t(P["opacity_raw"]).double()))).float().reshape(-1)
    scales = torch.exp(t(P["scaling_raw"]).double()).float()
    q = t(P["rotation_raw"])
    n2 = ((q[:, 0] * q[:, 0] + q[:, 1] * q[:, 1]) + q[:, 2] * q[:, 2]) + q[:, 3] * q[:, 3]
    quats = q / torch.clamp_min(torch.sqrt(n2), 1e-12)[:, None]
    W, H = full["W"], full["H"]
    radii, means2d, depths, conics, _ = ops.projection_ut_3dgs_fused(
        t(P["means"]), quats.contiguous(), scales.contiguous(), opac.contiguous(), full["cam"].viewmat[None].contiguous(), None,
        full["cam"].K[None].contiguous(), W, H, 0.3, 0.01, 1e4, 0.0, False, 0)
    assert torch.equal(radii[0], st["radii"])
    tw, th = (W + 15) // 16, (H + 15) // 16
    tpg, ids, flat = ops.intersect_tile(means2d, radii, depths, None, None, 1, 16, tw, th, True)
    assert torch.equal(tpg[0], st["tiles_per_gauss"]) and torch.equal(flat, st["flatten_ids"])
    assert torch.equal(ops.intersect_offset(ids, 1, tw, th).reshape(-1), st["tile_offsets"][:-1])
    assert bool((ids[1:] >= ids[:-1]).all())  # 64-bit keys ascending


def test_forward_is_deterministic_and_in_range(full):
    out = full["rast"].forward(full["cam"], full["bg"])
    assert torch.equal(out.image, full["img"]) and torch.equal(out.alpha, full["alpha"])
    a = full["alpha"]
    assert float(a.min()) >= 0.0 and float(a.max()) <= 1.0 and float(a.mean()) > 0.2
    assert bool(torch.isfinite(full["img"]).all()) and float(full["img"].min()) >= 0.0
    # compositing identity: with a black background the image can only get darker by (1 - alpha) * bg
    out0 = full["rast"].forward(full["cam"], None)
    diff = full["img"] - out0.image - (1 - a) * full["bg"]
    assert float(diff.abs().max()) < 1e-5
    full["rast"].forward(full["cam"], full["bg"])  # leave the workspace in the state the next test expects


def test_backward_is_linear_in_the_output_gradient(pkg, full):
    tr = pkg.trainer
    rast, model = full["rast"], full["model"]
    g = torch.Generator(device=DEV).manual_seed(5)
    v1 = torch.randn(full["H"], full["W"], 3, device=DEV, generator=g) * 1e-3
    v2 = torch.randn(full["H"], full["W"], 3, device=DEV, generator=g) * 1e-3
    outs = []
    for v in (v1, v2, 2.0 * v1 - 0.5 * v2):
        rast.forward(full["cam"], full["bg"])
        grads = model.like()
        rast.backward(v.contiguous(), grads, full["bg"])
        outs.append(grads.flat.clone())
    lin = 2.0 * outs[0] - 0.5 * outs[1]
    rel = float((outs[2] - lin).norm() / lin.norm())
    assert rel < 1e-4, rel
    assert bool(torch.isfinite(outs[2]).all())
    # Gaussians that are not visible get exactly zero gradient in every group
    vis = (full["state"]["radii"] > 0).all(-1)
    grads = model.like(); grads.flat.copy_(outs[2])
    for name in ("means", "shN", "opacity_raw"):
        assert float(grads.tensor(name)[~vis].abs().max()) == 0.0


def test_rank1_sh_update_equals_materialised_gradient_update(pkg, full):
    """At full size: Adam moments after backward(write_shN=False) + the rank-1 shN update equal those after the plain
    backward + Adam (the gradient rows rebuilt inside the optimizer are the materialised ones up to rounding)."""
    tr = pkg.trainer
    rast, model = full["rast"], full["model"]
    lrs = [1.6e-4, 2.5e-3, 1.25e-4, 5e-3, 1e-3, 5e-2]
    g = torch.Generator(device=DEV).manual_seed(9)
    v = (torch.randn(full["H"], full["W"], 3, device=DEV, generator=g) * 1e-3).contiguous()
    saved = model.flat.clone()
    moments = []
    for rank1 in (False, True):
        model.flat.copy_(saved)
        m, s = model.like(), model.like()
        rast.forward(full["cam"], full["bg"])
        grads = model.like()
        if rank1:
            rast.backward(v, grads, full["bg"], write_shN=False)
            rast.adam_step_rank1_sh(m, s, grads, lrs, 1)
        else:
            rast.backward(v, grads, full["bg"])
            tr.adam_step_splats(model, m, s, grads, lrs, 1)
        moments.append((m.flat.clone(), s.flat.clone()))
    model.flat.copy_(saved)
    for k in range(2):
        a, b = moments[0][k], moments[1][k]
        assert float(a.abs().max()) > 0
        assert float((a - b).norm() / a.norm()) < 1e-5, k
