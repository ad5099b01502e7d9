"""Drop-in check of the C++ operator shim (lichtfeld-studio_b200/csrc/ops_shim.cpp: namespace gsplat of gsplat/Ops.h over
the C ABI). ONE call sequence - the one rasterize() and the autograd node make (rasterizer.cpp:90-205,
rasterizer_autograd.cpp:11-215): fused forward, then fused backward with the saved tensors - is run twice with the very
same arguments: through the reference's own build (oracle/_ref) and through the shim. Both modules expose the same
bindings (csrc/gsplat_ops_pybind.inc), so the driver below cannot tell them apart. Also checks that every operator of the
shim returns what the ctypes mirror (ops.py) returns, bit for bit, since both sit on the same C ABI."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import make_scene, rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = Path(__file__).resolve().parents[1]


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


@pytest.fixture(scope="module")
def shim():
    spec = importlib.util.spec_from_file_location("_lfs_build", ROOT / "lichtfeld-studio_b200" / "build.py")
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    return b.load_shim()


@pytest.fixture(scope="module")
def R():
    from oracle import ref_build, reference
    if not reference.available():
        if ref_build.reference_root() is None:
            pytest.skip("oracle/_ref is not built and there is no reference checkout to build it from")
        ref_build.build()
    return reference


def rasterize_sequence(mod, act, vm, K, W, H, deg, bg, render_mode, antialiased, v_render, v_alpha, scaling_modifier=1.0):
    """What FusedRasterizationWithSHFunction::forward / ::backward call, on any module with the Ops.h operators."""
    means, quats, scales, opac, sh = act
    fwd = mod.rasterize_from_world_with_sh_fwd(means, quats, scales, opac, sh, deg, bg, None, W, H, 16, vm, None, K, 0, 0.3, 0.01, 10000.0,
                                               0.0, scaling_modifier, antialiased, render_mode, None, 4, None, None, None)
    render, alpha, radii, means2d, depths, colors, offsets, flat, last_ids, comps = fwd
    comps_t = comps if comps is not None else torch.empty(0, device=DEV)
    bwd = mod.rasterize_from_world_with_sh_bwd(means, quats, scales, opac, sh, deg, bg, None, W, H, 16, vm, None, K, 0, 0.3, 0.01, 10000.0,
                                               0.0, scaling_modifier, antialiased, render_mode, None, 4, None, None, None, alpha, last_ids,
                                               offsets, flat, colors, radii, means2d, depths, comps_t, v_render, v_alpha)
    return fwd, bwd


@pytest.mark.parametrize("render_mode,antialiased,smod", [(0, False, 1.0), (4, True, 1.3)])
def test_shim_drops_in_for_the_reference_call_sequence(pkg, synth, R, shim, render_mode, antialiased, smod):
    n, W, H, deg = 20000, 250, 170, 3
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=3)
    act = R.activated(P)
    ch = 3 if render_mode == 0 else 4
    bg = T(np.array([[0.2, 0.5, 0.1, 0.0][:ch]], np.float32))
    vmt, Kt = T(vm[None]), T(K[None])
    gen = torch.Generator(device=DEV).manual_seed(1)
    v_render = torch.randn((1, H, W, ch), generator=gen, device=DEV) * 1e-2
    v_alpha = torch.randn((1, H, W, 1), generator=gen, device=DEV) * 1e-3
    fa, ba = rasterize_sequence(R.load(), act, vmt, Kt, W, H, deg, bg, render_mode, antialiased, v_render, v_alpha, smod)
    fb, bb = rasterize_sequence(shim, act, vmt, Kt, W, H, deg, bg, render_mode, antialiased, v_render, v_alpha, smod)
    # same shapes and dtypes for every returned tensor (the tile list's length follows the radii, which may differ by one
    # for a couple of Gaussians against the fast-math reference)
    for k, (x, y) in enumerate(zip(list(fa) + list(ba), list(fb) + list(bb))):
        if x is None or y is None or x.numel() == 0:
            continue
        assert x.dtype == y.dtype and x.dim() == y.dim()
        if k != 7:
            assert x.shape == y.shape, k
    assert abs(fa[7].numel() - fb[7].numel()) <= 64
    vis = (fa[2] > 0).all(-1)
    assert int(((fb[2] > 0).all(-1) != vis).sum()) <= n // 2000 and int((fa[2] != fb[2]).any(-1).sum()) <= n // 1000
    d = (fa[0][..., :3] - fb[0][..., :3]).abs().amax(-1)
    assert int((d > 1e-4).sum()) <= 8 and float(torch.quantile(d.flatten(), 0.9995)) < 1e-4
    assert int(((fa[1] - fb[1]).abs() > 1e-4).sum()) <= 8
    for name, x, y in zip(("v_means", "v_quats", "v_scales", "v_opacities", "v_sh_coeffs"), ba, bb):
        assert rel_l2(y.cpu().numpy(), x.cpu().numpy()) < 1e-3, name


def test_shim_operators_equal_the_ctypes_mirror(pkg, synth, R, shim):
    """Both host layers call the same C ABI: identical bits from identical inputs."""
    ops = pkg.ops
    n, W, H, deg = 8000, 128, 96, 2
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=5)
    means, q, s, o, sh = R.activated(P)
    vmt, Kt = T(vm[None]), T(K[None])
    a = shim.projection_ut_3dgs_fused(means, q, s, o, vmt, None, Kt, W, H, 0.3, 0.01, 1e4, 0.0, True, 0, None, 4, None, None, None)
    b = ops.projection_ut_3dgs_fused(means, q, s, o, vmt, None, Kt, W, H, 0.3, 0.01, 1e4, 0.0, True, 0)
    vis = (a[0] > 0).all(-1)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1][vis], b[1][vis]) and torch.equal(a[2][vis], b[2][vis])
    tw, th = (W + 15) // 16, (H + 15) // 16
    ia = shim.intersect_tile(a[1], a[0], a[2], None, None, 1, 16, tw, th, True)
    ib = ops.intersect_tile(a[1], a[0], a[2], None, None, 1, 16, tw, th, True)
    assert all(torch.equal(x, y) for x, y in zip(ia, ib))
    oa = shim.intersect_offset(ia[1], 1, tw, th)
    assert torch.equal(oa, ops.intersect_offset(ia[1], 1, tw, th))
    campos = torch.inverse(vmt)[:, :3, 3]
    dirs = (means[None] - campos[:, None]).contiguous()
    ca = shim.spherical_harmonics_fwd(deg, dirs, sh[None].contiguous(), vis)
    assert torch.equal(ca[vis], ops.spherical_harmonics_fwd(deg, dirs, sh[None].contiguous(), vis)[vis])
    colors = torch.clamp_min(ca + 0.5, 0.0)
    colors[~vis] = 0
    common = (means, q, s, colors.contiguous(), o[None].contiguous(), None, None, W, H, 16, vmt, None, Kt, 0, None, 4, None, None, None, oa, ia[2])
    fa, fb = shim.rasterize_to_pixels_from_world_3dgs_fwd(*common), ops.rasterize_to_pixels_from_world_3dgs_fwd(*common)
    assert all(torch.equal(x, y) for x, y in zip(fa, fb))
    rq = torch.randn((100, 4), device=DEV)
    assert torch.equal(shim.quats_to_rotmats(rq), ops.quats_to_rotmats(rq))
    # error behaviour: the reference's TORCH_CHECKs surface as RuntimeError
    with pytest.raises(RuntimeError, match="CUDA"):
        shim.quats_to_rotmats(torch.zeros(4, 4))
    with pytest.raises(RuntimeError, match="PINHOLE, FISHEYE or EQUIRECTANGULAR"):
        shim.projection_ut_3dgs_fused(means, q, s, o, vmt, None, Kt, W, H, 0.3, 0.01, 1e4, 0.0, True, 1, None, 4, None, None, None)
