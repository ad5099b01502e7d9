"""CPU-only checks: the oracle against analytic cases, finite differences and the committed outputs of the reference's
own CUDA build (tests/golden/reference_step.npz; the reference itself ships no golden vectors for this path), the seeded
generator, the host-side logic and the C ABI surface."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

from conftest import make_scene, rel_l2

ROOT = Path(__file__).resolve().parents[1]


def test_abi_exports_every_declared_symbol(pkg):
    header = (ROOT / "include" / "lfs_b200.h").read_text()
    declared = set(re.findall(r"\b(lfs_[a-z0-9_]+)\s*\(", header))
    declared -= {"lfs_status", "lfs_camera_model"}
    lib = ctypes.CDLL(str(pkg._capi.LIB_PATH))
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, missing
    assert set(pkg._capi.EXPORTED) == declared
    assert b"sm_100a" in pkg._capi.lib().lfs_build_info()


def test_ops_shim_module_loads_and_exposes_every_operator():
    """The C++ operator shim (namespace gsplat of gsplat/Ops.h over the C ABI) builds against libtorch, loads next to the
    library and exposes the twelve operators declared in include/lfs_gsplat_ops.h; without a GPU a call fails with the
    reference's own check message instead of computing anything."""
    import importlib.util
    import torch
    spec = importlib.util.spec_from_file_location("_lfs_build", ROOT / "lichtfeld-studio_b200" / "build.py")
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    b.build_shim()
    shim = b.load_shim()
    header = (ROOT / "include" / "lfs_gsplat_ops.h").read_text()
    declared = set(re.findall(r"\b(spherical_harmonics_\w+|intersect_\w+|quats_to_rotmats|relocation|add_noise|projection_ut_3dgs_fused|"
                              r"rasterize_\w+)\s*\(", header))
    assert len(declared) == 12
    for name in declared:
        assert hasattr(shim, name), name
    with pytest.raises(RuntimeError, match="CUDA"):
        shim.quats_to_rotmats(torch.zeros(4, 4))


def test_synth_is_deterministic_and_distributed(synth):
    a = synth.make_gaussians(5000, 0, "clusters", 3)
    b = synth.make_gaussians(5000, 0, "clusters", 3)
    c = synth.make_gaussians(5000, 1, "clusters", 3)
    for k in a:
        assert np.array_equal(a[k], b[k]) and not np.array_equal(a[k], c[k])
    assert a["shN"].shape == (5000, 15, 3) and a["opacity_raw"].shape == (5000, 1)
    assert abs(a["scaling_raw"].mean() + 4.5) < 0.05 and abs(a["scaling_raw"].std() - 0.6) < 0.05
    assert abs(np.linalg.norm(a["rotation_raw"], axis=1) - 1).max() < 1e-5
    assert np.abs(a["means"]).max() <= 3.0
    n = synth.normal(3, 9, 200001)
    assert abs(n.mean()) < 0.01 and abs(n.std() - 1) < 0.01
    poses = synth.hemisphere_poses(200, 5.0)
    R = poses[:, :3, :3]
    assert np.abs(R @ R.transpose(0, 2, 1) - np.eye(3)).max() < 1e-6
    campos = -np.einsum("nji,nj->ni", R, poses[:, :3, 3])
    assert np.abs(np.linalg.norm(campos, axis=1) - 5).max() < 1e-5 and (campos[:, 2] > 0).all()


def test_oracle_projection_analytic(orc):
    """A small isotropic Gaussian on the optical axis projects to the principal point with covariance
    (f s / z)^2 + eps2d and radius ceil(min(3.33, sqrt(2 ln(255 o))) * sigma)."""
    vm = np.eye(4, dtype=np.float32); vm[2, 3] = 4.0
    K = np.array([[300, 0, 128], [0, 300, 128], [0, 0, 1]], np.float32)
    s, o = 0.01, 0.8
    radii, m2, d, conics, comp = orc.projection_ut_3dgs_fused(
        np.zeros((1, 3), np.float32), np.array([[1, 0, 0, 0]], np.float32), np.full((1, 3), s, np.float32),
        np.array([o], np.float32), vm[None], K[None], 256, 256, calc_compensations=True)
    var = (300 * s / 4.0) ** 2
    assert np.allclose(m2[0, 0], [128, 128], atol=1e-3) and abs(d[0, 0] - 4.0) < 1e-6
    assert abs(1 / conics[0, 0, 0] - (var + 0.3)) < 2e-3 and abs(conics[0, 0, 1]) < 1e-3
    assert abs(comp[0, 0] - var / (var + 0.3)) < 2e-3
    ext = min(3.33, np.sqrt(2 * np.log(o * comp[0, 0] * 255)))
    assert radii[0, 0, 0] == int(np.ceil(ext * np.sqrt(var + 0.3)))
    # behind the camera / beyond the far plane / almost transparent -> culled
    for mean, op in (([0, 0, -5], 0.8), ([0, 0, 2e4], 0.8), ([0, 0, 0], 0.001)):
        r = orc.projection_ut_3dgs_fused(np.array([mean], np.float32), np.array([[1, 0, 0, 0]], np.float32),
                                         np.full((1, 3), s, np.float32), np.array([op], np.float32), vm[None], K[None], 256, 256)[0]
        assert (r == 0).all()


def test_oracle_intersect_hand_case(orc):
    """One Gaussian covering tiles (1..2, 0..1) of a 4x3 grid, one culled, one clipped at the top-left corner."""
    m2 = np.array([[[30.0, 10.0], [5.0, 5.0], [-3.0, -2.0]]], np.float32)
    r = np.array([[[10, 8], [0, 4], [6, 6]]], np.int32)
    d = np.array([[2.0, 1.0, 0.5]], np.float32)
    tpg, ids, flat = orc.intersect_tile(m2, r, d, 1, 16, 4, 3, True)
    assert tpg.tolist() == [[4, 0, 1]]
    tile_of = (ids >> 32).tolist()
    assert tile_of == [0, 1, 2, 5, 6] and flat.tolist() == [2, 0, 0, 0, 0]
    assert (ids & 0xFFFFFFFF).tolist()[0] == int(np.float32(0.5).view(np.uint32))
    off = orc.intersect_offset(ids, 1, 4, 3)
    assert off.reshape(-1).tolist() == [0, 1, 2, 3, 3, 3, 4, 5, 5, 5, 5, 5]
    # ties in depth keep ascending index; unsorted emission is row-major per Gaussian
    d2 = np.array([[1.0, 1.0, 1.0]], np.float32)
    _, ids2, flat2 = orc.intersect_tile(m2, np.array([[[10, 8], [3, 3], [6, 6]]], np.int32), d2, 1, 16, 4, 3, True)
    assert flat2.tolist()[:2] == [1, 2]


def test_oracle_rasterizer_single_gaussian(orc):
    """One Gaussian on the axis: centre pixel alpha = opacity * exp(-0.5 dist^2) with dist the ray offset in
    units of sigma; alpha-compositing against a background."""
    vm = np.eye(4, dtype=np.float32); vm[2, 3] = 4.0
    K = np.array([[64, 0, 16], [0, 64, 16], [0, 0, 1]], np.float32)
    s, o = 0.05, 0.6
    P = dict(means=np.zeros((1, 3), np.float32), sh0=np.full((1, 1, 3), 0.5 / 0.2820947917738781, np.float32),
             shN=np.zeros((1, 0, 3), np.float32), scaling_raw=np.full((1, 3), np.log(s), np.float32),
             rotation_raw=np.array([[1, 0, 0, 0]], np.float32), opacity_raw=np.full((1, 1), np.log(o / (1 - o)), np.float32))
    bg = np.array([0.1, 0.2, 0.3], np.float32)
    f = orc.render_fwd(P, vm, K, 32, 32, 0, background=bg)
    # pixel (16,16) has its centre at (16.5,16.5): ray offset 0.5/64 * 4 = 0.03125 in x and y at depth 4
    dist2 = 2 * (0.03125 / s) ** 2 / (1 + 2 * (0.5 / 64) ** 2)
    a = o * np.exp(-0.5 * dist2)
    assert abs(f["alpha"][16, 16, 0] - a) < 2e-4
    assert np.allclose(f["render"][16, 16], a * 1.0 + (1 - a) * bg, atol=3e-4)
    assert np.allclose(f["render"][0, 0], bg) and f["alpha"][0, 0, 0] == 0


def _loss_of(orc, P, vm, K, W, H, deg, target, bg):
    f = orc.render_fwd(P, vm, K, W, H, deg, background=bg)
    return orc.photometric_loss(f["render"], target, 0.2, want_grad=False)[0], f


def test_oracle_gradients_finite_difference(orc, synth):
    """Backward of the whole chain (rasterizer VJPs, SH, activations, L1+SSIM) against central differences of
    the oracle's own forward. Float32 forward => loose tolerance, but any wrong term is off by O(1)."""
    cfg, P, vm, K = make_scene(synth, 60, 48, 40, 2, seed=4, fx=60.0)
    P["scaling_raw"] += 1.6  # big enough to overlap many pixels
    bg = np.array([0.3, 0.1, 0.2], np.float32)
    _, P2, _, _ = make_scene(synth, 60, 48, 40, 2, seed=77, fx=60.0)
    P2["scaling_raw"] += 1.6
    target = np.ascontiguousarray(np.clip(orc.render_fwd(P2, vm, K, 48, 40, 2, background=bg)["render"], 0, 1).transpose(2, 0, 1))
    loss, f = _loss_of(orc, P, vm, K, 48, 40, 2, target, bg)
    _, g, _, _ = orc.photometric_loss(f["render"], target, 0.2)
    bwd = orc.render_bwd(P, f, vm, K, 48, 40, 2, g, background=bg)
    rng = np.random.default_rng(0)
    checked = 0
    for name, eps in (("means", 2e-3), ("scaling_raw", 5e-3), ("rotation_raw", 5e-3), ("opacity_raw", 1e-2), ("sh0", 1e-2), ("shN", 2e-2)):
        gflat = bwd[name].reshape(-1)
        order = np.argsort(-np.abs(gflat))[:6]
        for idx in order:
            if abs(gflat[idx]) < 1e-6:
                continue
            vals = []
            for sgn in (+1, -1):
                Q = {k: v.copy() for k, v in P.items()}
                Q[name].reshape(-1)[idx] += sgn * eps
                vals.append(_loss_of(orc, Q, vm, K, 48, 40, 2, target, bg)[0])
            fd = (vals[0] - vals[1]) / (2 * eps)
            assert abs(fd - gflat[idx]) < 0.15 * abs(gflat[idx]) + 2e-5, (name, idx, fd, gflat[idx])
            checked += 1
    assert checked >= 20


def test_oracle_ssim_properties(orc):
    rng = np.random.default_rng(1)
    a = rng.random((3, 40, 50)).astype(np.float32)
    m, d1, d2, d3 = orc.fusedssim(a, a)
    assert np.abs(m - 1).max() < 1e-5  # identical images
    b = rng.random((3, 40, 50)).astype(np.float32)
    loss, g, l1, ss = orc.photometric_loss(np.ascontiguousarray(a.transpose(1, 2, 0)), b, 0.2)
    assert abs(l1 - np.abs(a - b).mean()) < 1e-6 and abs(loss - (0.8 * l1 + 0.2 * (1 - ss))) < 1e-6
    # gradient of the loss w.r.t. the render by central differences on a few pixels
    r = np.ascontiguousarray(a.transpose(1, 2, 0))
    for (y, x, c) in ((20, 25, 0), (7, 44, 2), (0, 0, 1)):
        vals = []
        for sgn in (1, -1):
            q = r.copy(); q[y, x, c] += sgn * 1e-2
            vals.append(orc.photometric_loss(q, b, 0.2, want_grad=False)[0])
        assert abs((vals[0] - vals[1]) / 2e-2 - g[y, x, c]) < 0.05 * abs(g[y, x, c]) + 1e-6


def test_oracle_adam_and_relocation(orc):
    p = np.array([1.0, -2.0], np.float32); m = np.zeros(2, np.float32); v = np.zeros(2, np.float32)
    orc.adam_step(p, m, v, np.array([0.5, -0.25], np.float32), 0.1, 0.9, 0.999, 1e-15, 1)
    assert np.allclose(p, [0.9, -1.9], atol=1e-6) and np.allclose(m, [0.05, -0.025]) and np.allclose(v, [2.5e-4, 6.25e-5], rtol=1e-4)
    b = orc.binoms_table(51)
    assert b[4, 2] == 6 and b[10, 3] == 120 and b[0, 0] == 1 and b[3, 5] == 0
    # ratio 1 keeps the Gaussian unchanged; ratio n keeps total opacity: 1 - (1 - o')^n = o
    no, ns = orc.relocation(np.array([0.7, 0.7], np.float32), np.ones((2, 3), np.float32), np.array([1, 4], np.int32), b, 51)
    assert abs(no[0] - 0.7) < 1e-6 and np.allclose(ns[0], 1, atol=1e-5)
    assert abs(1 - (1 - no[1]) ** 4 - 0.7) < 1e-5 and (ns[1] < 1).all()


def test_splat_data_layout_and_strategy_schedule(pkg):
    import torch
    tr, st = pkg.trainer, pkg.strategy
    sd = tr.SplatData(10, 16, "cpu", capacity=13)
    assert sd.capacity == 16 and sd.row_floats == 59 and sd.flat.numel() == 16 * 59
    assert sd.tensor("shN").shape == (10, 15, 3) and sd.tensor("sh0").shape == (10, 1, 3) and sd.tensor("opacity_raw").shape == (10, 1)
    sd.tensor("means").fill_(1.0)
    assert sd.flat[:30].eq(1).all() and sd.flat[30:].eq(0).all()
    for name in tr.PARAM_NAMES:  # every group starts 16-byte aligned
        assert (sd._full[name].data_ptr() - sd.flat.data_ptr()) % 16 == 0
    assert np.array_equal(st.binoms_table(51), __import__("oracle.oracle", fromlist=["x"]).binoms_table(51))
    p = st.OptimizationParameters()
    assert (p.iterations, p.min_opacity, p.refine_every, p.start_refine, p.stop_refine, p.max_cap) == (30000, 0.005, 100, 500, 25000, 1000000)


def test_remove_gaussians_compacts_all_buffers(pkg):
    """Host-side row surgery of MCMC::remove_gaussians (mcmc.cpp:406-444) on CPU tensors."""
    import torch
    tr, st = pkg.trainer, pkg.strategy
    sd = tr.SplatData(12, 4, "cpu", capacity=20)
    sd.flat.copy_(torch.arange(sd.flat.numel(), dtype=torch.float32))
    s = st.MCMC(sd)
    s.initialize(st.OptimizationParameters(max_cap=20, sh_degree=1))
    s._optimizer.exp_avg.flat.copy_(sd.flat + 1000)
    s._optimizer.exp_avg_sq.flat.copy_(sd.flat + 2000)
    before = {n: sd.tensor(n).clone() for n in tr.PARAM_NAMES}
    mask = torch.zeros(12, dtype=torch.bool)
    mask[[0, 5, 11]] = True
    s.remove_gaussians(mask)
    assert sd.size == 9 and s._optimizer.exp_avg.size == 9 and s._optimizer.exp_avg_sq.size == 9 and s.grads.size == 9
    for n in tr.PARAM_NAMES:
        assert torch.equal(sd.tensor(n), before[n][~mask])
        assert torch.equal(s._optimizer.exp_avg.tensor(n), before[n][~mask] + 1000)
        assert torch.equal(s._optimizer.exp_avg_sq.tensor(n), before[n][~mask] + 2000)
    with pytest.raises(RuntimeError, match="mask must have"):
        s.remove_gaussians(torch.zeros(12, dtype=torch.bool))
    s.remove_gaussians(torch.zeros(9, dtype=torch.bool))  # nothing to remove
    assert sd.size == 9


def test_library_fails_loudly_without_gpu(pkg):
    """No CPU fallback: on a machine without a GPU the calls must raise, not silently compute elsewhere."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        pkg.ops.quats_to_rotmats(torch.zeros(4, 4))
    with pytest.raises(pkg.LfsError):
        pkg._capi.call("lfs_quats_to_rotmats", 4, ctypes.c_void_p(256), ctypes.c_void_p(512), None)


def test_default_strategy_adc_on_cpu_tensors(pkg):
    """DefaultStrategy (src/training/strategies/default_strategy.cpp) duplicate / prune / reset on CPU tensors:
    row order, appended rows, zeroed moments, size bookkeeping. split() needs the CUDA quats_to_rotmats."""
    import torch
    tr, st = pkg.trainer, pkg.strategy
    n = 10
    sd = tr.SplatData(n, 4, "cpu", capacity=40)
    g = torch.Generator().manual_seed(0)
    for name in tr.PARAM_NAMES:
        sd.tensor(name).copy_(torch.randn(sd.tensor(name).shape, generator=g))
    sd.tensor("scaling_raw").fill_(-6.0)           # small: exp(-6) = 0.0025 <= 0.01
    sd.tensor("opacity_raw").fill_(2.0)
    s = st.DefaultStrategy(sd)
    p = st.DefaultStrategy.Parameters(sh_degree=1)
    s.initialize(p)
    assert s.is_refining(600) and not s.is_refining(500) and not s.is_refining(650)
    s._optimizer.exp_avg.flat.fill_(1.0); s._optimizer.exp_avg_sq.flat.fill_(2.0)
    before = {k: sd.tensor(k).clone() for k in tr.PARAM_NAMES}
    s.densification_info = torch.zeros(2, n)
    s.densification_info[0] = 4.0
    s.densification_info[1, [1, 7]] = 4.0 * 0.001   # mean gradient 0.001 > 0.0002 for rows 1 and 7
    s.grow_gs(600)
    assert sd.size == 12 and s._optimizer.exp_avg.size == 12 and s.grads.size == 12
    for k in tr.PARAM_NAMES:
        assert torch.equal(sd.tensor(k)[:10], before[k]) and torch.equal(sd.tensor(k)[10:], before[k][[1, 7]])
        assert s._optimizer.exp_avg.tensor(k)[:10].eq(1).all() and s._optimizer.exp_avg.tensor(k)[10:].eq(0).all()
        assert s._optimizer.exp_avg_sq.tensor(k)[10:].eq(0).all()
    # prune: transparent rows, zero quaternions and (after the first reset) huge Gaussians
    sd.tensor("opacity_raw")[3] = -8.0
    sd.tensor("rotation_raw")[5] = 0.0
    sd.tensor("scaling_raw")[8] = 0.0            # exp(0) = 1 > 0.1
    keep_means = sd.tensor("means").clone()
    s.prune_gs(600)
    assert sd.size == 10 and torch.equal(sd.tensor("means"), keep_means[[0, 1, 2, 4, 6, 7, 8, 9, 10, 11]])
    s.prune_gs(3100)
    assert sd.size == 9
    s.reset_opacity()
    lim = float(torch.logit(torch.tensor(0.01)))
    assert float(sd.tensor("opacity_raw").max()) <= lim + 1e-6 and s._optimizer.exp_avg.tensor("opacity_raw").eq(0).all()
    m = s._optimizer.exp_avg.tensor("means")   # the two duplicated rows keep their zero moments
    assert m[:7].eq(1).all() and m[7:].eq(0).all()
    mask = torch.zeros(9, dtype=torch.bool); mask[0] = True
    s.remove_gaussians(mask)
    assert sd.size == 8
    s.post_backward(25000)
    assert s.densification_info.numel() == 0


def test_ply_header_reader_and_checkpoint_roundtrip(pkg, tmp_path):
    """Header text of SplatData::save_ply (src/core/splat_data.cpp:113-169, :402-418), the reader on a file made with
    numpy in a shuffled property order, and the checkpoint format on CPU tensors."""
    import torch
    fm, tr, st = pkg.formats, pkg.trainer, pkg.strategy
    K = 4
    names = fm.ply_attribute_names(K)
    assert names[:9] == ["x", "y", "z", "nx", "ny", "nz", "f_dc_0", "f_dc_1", "f_dc_2"]
    assert names[9] == "f_rest_0" and names[17] == "f_rest_8" and names[18:] == ["opacity", "scale_0", "scale_1", "scale_2", "rot_0", "rot_1", "rot_2", "rot_3"]
    assert len(names) == 14 + 3 * K
    hdr = fm.ply_header(5, K).decode()
    assert hdr.startswith("ply\nformat binary_little_endian 1.0\nelement vertex 5\nproperty float x\n") and hdr.endswith("end_header\n")
    rng = np.random.default_rng(0)
    rows = rng.normal(size=(5, len(names))).astype(np.float32)
    p = tmp_path / "a.ply"
    p.write_bytes(fm.ply_header(5, K) + rows.tobytes())
    n2, r2 = fm.read_ply(str(p))
    assert n2 == names and np.array_equal(r2, rows)
    with pytest.raises(RuntimeError):
        (tmp_path / "bad.ply").write_bytes(b"plx\n")
        fm.read_ply(str(tmp_path / "bad.ply"))

    # checkpoint: parameters, moments, optimizer counters; restoring into a fresh strategy reproduces every buffer
    def fresh(seed):
        sd = tr.SplatData(9, K, "cpu", capacity=16)
        g = torch.Generator().manual_seed(seed)
        for name in tr.PARAM_NAMES:
            sd.tensor(name).copy_(torch.randn(sd.tensor(name).shape, generator=g))
        s = st.DefaultStrategy(sd)
        s.initialize(st.DefaultStrategy.Parameters(sh_degree=1))
        return s
    a = fresh(1)
    a._optimizer.exp_avg.flat.normal_(generator=torch.Generator().manual_seed(5))
    a._optimizer.exp_avg_sq.flat.uniform_(generator=torch.Generator().manual_seed(6))
    a._optimizer.step_count, a._optimizer.lr[0], a.active_sh_degree = 1234, 1.23e-4, 1
    path = fm.save_checkpoint(a, str(tmp_path / "c.ckpt"), 777)
    b = fresh(2)
    b.get_model().size = 3   # a different size before the restore
    assert fm.load_checkpoint(b, path) == 777
    assert b.get_model().size == 9 and b._optimizer.step_count == 1234 and b._optimizer.lr == a._optimizer.lr and b.active_sh_degree == 1
    for x, y in ((a.get_model(), b.get_model()), (a._optimizer.exp_avg, b._optimizer.exp_avg), (a._optimizer.exp_avg_sq, b._optimizer.exp_avg_sq)):
        for name in tr.PARAM_NAMES:
            assert torch.equal(x.tensor(name), y.tensor(name)), name
    small = tr.SplatData(2, K, "cpu", capacity=4)
    s2 = st.DefaultStrategy(small); s2.initialize(st.DefaultStrategy.Parameters(sh_degree=1))
    with pytest.raises(RuntimeError):
        fm.load_checkpoint(s2, path)


def test_oracle_opencv_distortion_closed_form_and_roundtrip(orc):
    """Pins the oracle's OpenCV pinhole model (gsplat/Cameras.cuh:504-597, :635-754): the forward map against the
    published OpenCV formula evaluated in float64, and pixel -> ray -> pixel through the Newton inversion."""
    K = np.array([[210.0, 0, 162.0], [0, 205.0, 118.0], [0, 0, 1]], np.float32)
    W, H = 320, 240
    k = np.array([-0.22, 0.06, -0.004, 0.01, 0.002, 0.0]); p = np.array([0.0015, -0.002]); s = np.array([0.0008, 0.0, -0.0005, 0.0002])
    dist = orc.pack_distortion(k, p, s)
    rng = np.random.default_rng(0)
    n_ok = 0
    for _ in range(300):
        pt = np.array([rng.uniform(-0.6, 0.6), rng.uniform(-0.45, 0.45), 1.0]) * rng.uniform(0.5, 5.0)
        x, y = pt[0] / pt[2], pt[1] / pt[2]
        r2 = x * x + y * y
        icd = (1 + k[0] * r2 + k[1] * r2 ** 2 + k[2] * r2 ** 3) / (1 + k[3] * r2 + k[4] * r2 ** 2 + k[5] * r2 ** 3)
        xd = x * icd + 2 * p[0] * x * y + p[1] * (r2 + 2 * x * x) + s[0] * r2 + s[1] * r2 * r2
        yd = y * icd + p[0] * (r2 + 2 * y * y) + 2 * p[1] * x * y + s[2] * r2 + s[3] * r2 * r2
        u, v = 210.0 * xd + 162.0, 205.0 * yd + 118.0
        got, ok = orc.cam_point_to_image(0, K, W, H, dist, pt.astype(np.float32))
        assert abs(got[0] - u) < 2e-3 and abs(got[1] - v) < 2e-3
        inside = (-0.1 * W <= u < 1.1 * W) and (-0.1 * H <= v < 1.1 * H) and icd > 0.8
        assert ok == inside
        if ok:
            ray, conv = orc.image_to_cam_ray(0, K, W, H, dist, float(got[0]), float(got[1]))
            d = pt / np.linalg.norm(pt)
            assert conv and np.abs(ray - d).max() < 2e-5
            n_ok += 1
    assert n_ok > 200
    # behind the camera: invalid, projects to the origin; no distortion block: the plain pinhole
    out, ok = orc.cam_point_to_image(0, K, W, H, dist, np.array([0.1, 0.1, -1.0], np.float32))
    assert not ok and (out == 0).all()
    out, ok = orc.cam_point_to_image(0, K, W, H, None, np.array([0.2, -0.1, 2.0], np.float32))
    assert ok and abs(out[0] - (210 * 0.1 + 162)) < 1e-4 and abs(out[1] - (205 * -0.05 + 118)) < 1e-4


def _golden():
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiny_step.npz"))


def test_oracle_reproduces_golden_step(orc):
    """tests/golden/tiny_step.npz (written by tests/golden/make_golden.py from this oracle) anchors the oracle against
    drift: integer results must match exactly, floats to a few ulp (libm's float exp may differ between hosts)."""
    g = _golden()
    P = {k: g[f"in_{k}"] for k in ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")}
    W, H, deg = (int(x) for x in g["in_size"])
    assert g["flatten_ids"].size > 2000
    fwd = orc.render_fwd(P, g["in_viewmat"], g["in_K"], W, H, deg, background=g["in_bg"])
    for k in ("radii", "tiles_per_gauss", "flatten_ids", "tile_offsets", "last_ids"):
        assert np.array_equal(fwd[k], g[k]), k
    vis = g["visible"]
    assert np.array_equal(fwd["means2d"][vis].view(np.uint32), g["means2d"][vis].view(np.uint32))
    assert np.abs(fwd["render"] - g["render"]).max() < 2e-6 and np.abs(fwd["alpha"] - g["alpha"]).max() < 2e-6
    loss, gr, l1, ssim = orc.photometric_loss(fwd["render"], g["in_target"], 0.2)
    assert np.allclose([loss, l1, ssim], g["loss"], atol=2e-6)
    bwd = orc.render_bwd(P, fwd, g["in_viewmat"], g["in_K"], W, H, deg, g["v_render"], background=g["in_bg"])
    for k in P:
        assert np.allclose(bwd[k], g[f"grad_{k}"], rtol=1e-4, atol=1e-9), k
    fd = orc.render_fwd(P, g["in_viewmat"], g["in_K"], W, H, deg, background=np.append(g["in_bg"], 0).astype(np.float32),
                        radial=g["in_dist"], render_mode=4)
    assert np.array_equal(fd["radii"], g["dist_radii"]) and np.array_equal(fd["flatten_ids"], g["dist_flatten_ids"])
    assert np.abs(fd["render"] - g["dist_render"]).max() < 1e-5 and np.abs(fd["depth"] - g["dist_depth"]).max() < 1e-4
    no, ns = orc.relocation(g["in_reloc_opacity"], g["in_reloc_scale"], g["in_reloc_ratios"], orc.binoms_table(51), 51)
    assert np.allclose(no, g["reloc_opacity"], rtol=1e-6) and np.allclose(ns, g["reloc_scale"], rtol=1e-6)
    p, m, v = g["in_adam_p"].copy(), g["in_adam_m"].copy(), g["in_adam_v"].copy()
    orc.adam_step(p, m, v, g["in_adam_g"], 1e-3, 0.9, 0.999, 1e-15, 5)
    assert np.allclose(p, g["adam_p"], rtol=1e-6) and np.array_equal(m, g["adam_m"]) and np.array_equal(v, g["adam_v"])


def test_oracle_matches_reference_cuda_golden(orc):
    """PINS THE ORACLE TO THE REFERENCE: tests/golden/reference_step.npz holds what the reference's own, unmodified CUDA
    kernels (oracle/_ref, built by oracle/ref_build.py, run on a B200 by tests/golden/make_reference_golden.py) produce
    for the inputs of tiny_step.npz. Integer work on identical inputs must agree bit for bit; from raw parameters the
    reference's --use_fast_math arithmetic may move a radius by one for a handful of Gaussians; images 1e-4 (a few
    pixels may flip at the 1/255 alpha cut), gradients 1e-3 relative L2, loss 1e-6."""
    import os
    g, r = _golden(), np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_step.npz"))
    names = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")
    P = {k: g[f"in_{k}"] for k in names}
    W, H, deg = (int(x) for x in g["in_size"])
    vm, K, bg = g["in_viewmat"], g["in_K"], g["in_bg"]
    n = P["means"].shape[0]
    # projection from the activated parameters
    q, _ = orc.act_quat(P["rotation_raw"])
    pr = orc.projection_ut_3dgs_fused(P["means"], q, orc.act_scale(P["scaling_raw"]), orc.act_opacity(P["opacity_raw"]), vm[None], K[None],
                                      W, H, calc_compensations=True)
    vis_ref, vis = r["visible"], (pr[0][0] > 0).all(-1)
    assert vis_ref.sum() > 300
    assert (vis != vis_ref).sum() <= 1 and (pr[0][0] != r["radii"]).any(-1).sum() <= 2
    both = vis & vis_ref
    assert np.abs(pr[1][0][both] - r["means2d"][both]).max() < 0.02
    assert np.array_equal(pr[2][0][both].view(np.uint32), r["depths"][both].view(np.uint32))
    assert rel_l2(pr[3][0][both], r["conics"][both]) < 1e-3 and np.abs(pr[4][0][both] - r["compensations"][both]).max() < 1e-3
    # tile lists from the REFERENCE's projection outputs: bit-exact
    tw, th = (W + 15) // 16, (H + 15) // 16
    tpg, ids, flat = orc.intersect_tile(r["means2d"][None], r["radii"][None], r["depths"][None], 1, 16, tw, th, True)
    assert np.array_equal(tpg[0], r["tiles_per_gauss"]) and np.array_equal(ids, r["isect_ids"]) and np.array_equal(flat, r["flatten_ids"])
    assert np.array_equal(orc.intersect_offset(ids, 1, tw, th)[0], r["tile_offsets"])
    # the training step
    fwd = orc.render_fwd(P, vm, K, W, H, deg, background=bg)
    d = np.abs(np.clip(fwd["render"].transpose(2, 0, 1), 0, 1) - r["image"]).max(0)
    assert (d > 1e-4).sum() <= 4 and np.quantile(d, 0.998) < 1e-4, d.max()
    assert (np.abs(fwd["alpha"][..., 0] - r["alpha"][0]) > 1e-4).sum() <= 4
    loss, gr, l1, ssim = orc.photometric_loss(fwd["render"], g["in_target"], 0.2)
    assert abs(loss - float(r["loss"])) < 1e-6
    bwd = orc.render_bwd(P, fwd, vm, K, W, H, deg, gr, background=bg)
    for k in names:
        assert rel_l2(bwd[k], r[f"grad_{k}"]) < 1e-3, k
    # SSIM map of the reference's own image
    m, dm1, _, _ = orc.fusedssim(np.clip(r["image"], 0, 1), g["in_target"], 1e-4, 9e-4)
    assert np.abs(m - r["ssim_map"]).max() < 3e-5 and rel_l2(dm1, r["ssim_dm_dmu1"]) < 1e-5
    # the default (EWA) path
    K_ = K
    ef = orc.ewa_forward(P, vm, orc.campos(vm), W, H, K_[0, 0], K_[1, 1], K_[0, 2], K_[1, 2], (deg + 1) ** 2, background=bg)
    d = np.abs(ef["image"] - r["ewa_image"]).max(0)
    assert (d > 1e-4).sum() <= 4 and np.quantile(d, 0.998) < 1e-4, d.max()
    # its loss, backward (FastGSRasterize::backward) and camera-pose gradient (kernels_backward.cuh:160-173)
    eloss, egr, _, _ = orc.photometric_loss(np.ascontiguousarray(ef["image"].transpose(1, 2, 0)), g["in_target"], 0.2)
    assert abs(eloss - float(r["ewa_loss"])) < 1e-6
    eb = orc.ewa_backward(P, ef, np.ascontiguousarray(egr.transpose(2, 0, 1)))
    for k in names:
        assert rel_l2(eb[k], r[f"ewa_grad_{k}"]) < 1e-3, k          # measured: 6e-5 .. 1e-4
    assert (r["ewa_grad_w2c"][3] == 0).all() and rel_l2(eb["grad_w2c"][:3], r["ewa_grad_w2c"][:3]) < 1e-3     # measured: 3.4e-5
    # relocation (the reference's pow is fast-math), Adam, noise, rotation matrices
    no, ns = orc.relocation(g["in_reloc_opacity"], g["in_reloc_scale"], g["in_reloc_ratios"], orc.binoms_table(51), 51)
    assert np.allclose(no, r["reloc_opacity"], rtol=1e-3) and np.allclose(ns, r["reloc_scale"], rtol=1e-3)
    p, mo, v = g["in_adam_p"].copy(), g["in_adam_m"].copy(), g["in_adam_v"].copy()
    orc.adam_step(p, mo, v, g["in_adam_g"], 1e-3, 0.9, 0.999, 1e-15, 5)
    assert np.allclose(p, r["adam_p"], rtol=1e-5, atol=1e-7) and np.allclose(mo, r["adam_m"], rtol=1e-6) and np.allclose(v, r["adam_v"], rtol=1e-6)
    moved = P["means"].copy()
    orc.add_noise(P["opacity_raw"], P["scaling_raw"], P["rotation_raw"], r["in_noise"], moved, 80.0)
    assert rel_l2(moved - P["means"], r["noise_means"] - P["means"]) < 1e-4
    assert np.abs(orc.quats_to_rotmats(P["rotation_raw"]) - r["rotmats"]).max() < 1e-6


def _ewa_scene(synth, n, W, H, deg, seed, fx):
    cfg, P, vm, K = make_scene(synth, n, W, H, deg, seed=seed, fx=fx)
    return P, vm, K


def test_oracle_ewa_analytic_single_gaussian(orc):
    """Pins the EWA restatement (src/training/fastgs/rasterization/include/kernels_forward.cuh:19-192, :336-459) with a
    closed form: an isotropic Gaussian on the optical axis projects to a circular 2-D Gaussian with variance
    (f s / z)^2 + 0.3, and a pixel's alpha is opacity * exp(-r^2 / (2 var))."""
    W = H = 64
    f_, z, s, op_raw = 50.0, 4.0, 0.2, 1.5
    P = dict(means=np.array([[0, 0, 0]], np.float32), sh0=np.array([[[0.7, -0.2, 3.0]]], np.float32), shN=np.zeros((1, 0, 3), np.float32),
             scaling_raw=np.full((1, 3), np.log(s), np.float32), rotation_raw=np.array([[0.3, -0.5, 0.2, 0.7]], np.float32),
             opacity_raw=np.array([[op_raw]], np.float32))
    w2c = np.eye(4, dtype=np.float32); w2c[2, 3] = z
    out = orc.ewa_forward(P, w2c, np.array([0, 0, -z], np.float32), W, H, f_, f_, 32.0, 32.0, 1)
    var = (f_ * s / z) ** 2 + 0.3
    op = 1 / (1 + np.exp(-op_raw))
    assert np.allclose(out["mean2d"][0], [32.0, 32.0]) and np.allclose(out["conic_opacity"][0], [1 / var, 0, 1 / var, op], rtol=1e-5, atol=1e-7)
    ys, xs = np.mgrid[0:H, 0:W] + 0.5
    r2 = (xs - 32.0) ** 2 + (ys - 32.0) ** 2
    a = np.minimum(op * np.exp(-r2 / (2 * var)), 0.999)
    a[a < 1 / 255] = 0
    assert np.abs(out["alpha"] - a).max() < 1e-5
    col = np.maximum(0.5 + 0.28209479177387814 * P["sh0"][0, 0], 0)
    assert np.abs(out["image"] - col[:, None, None] * a[None]).max() < 1e-5
    # bounds: the tiles reached by sqrt(2 ln(255 op)) standard deviations, and exactly those are in the lists
    ext = np.sqrt(2 * np.log(255 * op)) * np.sqrt(var) - 0.5
    assert list(out["bounds"][0]) == [int(np.floor((32 - ext) / 16)), int(np.ceil((32 + ext) / 16))] * 2
    assert out["n_touched"][0] == out["instance_ids"].size == 4


def test_oracle_ewa_gradients_finite_difference(orc, synth):
    """Backward of the EWA chain (blend, conic inverse, J W Sigma W^T J^T, quaternion / scale / sigmoid, SH incl. the
    view-direction term) against central differences of the oracle's own forward."""
    W, H, deg = 48, 40, 2
    P, vm, K = _ewa_scene(synth, 50, W, H, deg, 4, 60.0)
    P["scaling_raw"] += 1.4
    campos = orc.campos(vm)
    bg = np.array([0.3, 0.1, 0.2], np.float32)
    rng = np.random.default_rng(1)
    wi = rng.normal(size=(3, H, W)).astype(np.float32)
    wa = rng.normal(size=(H, W)).astype(np.float32)

    def fwd(Q):
        f = orc.ewa_forward(Q, vm, campos, W, H, K[0, 0], K[1, 1], K[0, 2], K[1, 2], (deg + 1) ** 2, background=bg)
        return float((f["image"].astype(np.float64) * wi).sum() + (f["alpha"].astype(np.float64) * wa).sum()), f

    _, f = fwd(P)
    dens = np.zeros((2, 50), np.float32)
    bwd = orc.ewa_backward(P, f, wi, wa, dens)
    vis = f["n_touched"] > 0
    assert np.array_equal(dens[0], vis.astype(np.float32)) and (dens[1][vis] > 0).all()
    assert np.allclose(dens[1], np.hypot(bwd["grad_mean2d"][:, 0] * W / 2, bwd["grad_mean2d"][:, 1] * H / 2) * vis, rtol=1e-5)
    # the forward has jumps (1/255 alpha cut, tile membership), so a single step size can straddle one: a term counts
    # as confirmed when any of three step sizes reproduces it to 4 % (most agree to 1e-4)
    checked = 0
    for name in ("means", "scaling_raw", "rotation_raw", "opacity_raw", "sh0", "shN"):
        gflat = bwd[name].reshape(-1)
        for idx in np.argsort(-np.abs(gflat))[:6]:
            if abs(gflat[idx]) < 1e-6:
                continue
            errs = []
            for eps in (1e-2, 3e-3, 1e-3):
                vals = []
                for sgn in (+1, -1):
                    Q = {k: v.copy() for k, v in P.items()}
                    Q[name].reshape(-1)[idx] += sgn * eps
                    vals.append(fwd(Q)[0])
                errs.append(abs((vals[0] - vals[1]) / (2 * eps) - gflat[idx]))
            assert min(errs) < 0.04 * abs(gflat[idx]) + 1e-3, (name, idx, errs, gflat[idx])
            checked += 1
    assert checked >= 30


def test_oracle_rolling_shutter_rows_equal_global_renders_at_the_row_pose(orc, synth):
    """Pins the rolling-shutter restatement (gsplat/Cameras.cuh:253-413): with a top-to-bottom shutter every image row
    is seen from the pose interpolated at that row's frame time, so row y of the rolling render equals row y of a
    global-shutter render from that pose (up to Gaussians whose tile lists differ by the iterative projection)."""
    n, W, H, deg = 1500, 64, 48, 1
    cfg, P, vm0, K = make_scene(synth, n, W, H, deg, seed=7, fx=70.0)
    P["scaling_raw"] += 1.0
    vm1 = vm0.copy()
    vm1[0, 3] += 0.30          # the camera translates during the exposure (slerp of equal rotations stays put)
    vm1[1, 3] -= 0.10
    with orc.shutter(vm0, 0):
        same = orc.render_fwd(P, vm0, K, W, H, deg)
    ref0 = orc.render_fwd(P, vm0, K, W, H, deg)
    assert np.array_equal(same["flatten_ids"], ref0["flatten_ids"]) and np.abs(same["render"] - ref0["render"]).max() == 0.0
    with orc.shutter(vm1, 0):
        roll = orc.render_fwd(P, vm0, K, W, H, deg)
    assert np.abs(roll["render"] - ref0["render"]).max() > 0.05        # the motion is visible
    for y in (0, 17, 30, 47):
        t = np.float32(np.floor(y + 0.5) / (H - 1))
        vmy = vm0.copy()
        vmy[:3, 3] = (np.float32(1) - t) * vm0[:3, 3] + t * vm1[:3, 3]
        glob = orc.render_fwd(P, vmy, K, W, H, deg)
        diff = np.abs(roll["render"][y] - glob["render"][y]).max(-1)
        assert np.quantile(diff, 0.9) < 2e-3 and diff.max() < 0.1, (y, diff.max())
    # left-to-right: columns instead of rows
    with orc.shutter(vm1, 1):
        roll_x = orc.render_fwd(P, vm0, K, W, H, deg)
    x = 40
    t = np.float32(np.floor(x + 0.5) / (W - 1))
    vmx = vm0.copy(); vmx[:3, 3] = (np.float32(1) - t) * vm0[:3, 3] + t * vm1[:3, 3]
    diff = np.abs(roll_x["render"][:, x] - orc.render_fwd(P, vmx, K, W, H, deg)["render"][:, x]).max(-1)
    assert np.quantile(diff, 0.9) < 2e-3


def test_oracle_equirectangular_pixels_equal_pinhole_renders_along_the_pixel_ray(orc, synth):
    """Pins the oracle's EQUIRECTANGULAR model (gsplat/Cameras.cuh:1003-1039) to its pinhole model, which the reference's
    golden vectors pin: pixel (x, y) of an equirectangular render looks along (cos E sin A, sin E, cos A cos E) with
    A = 2 pi ((x + 0.5) / W - 0.5), E = pi ((y + 0.5) / H - 0.5); a pinhole camera at the same position, rotated so that its
    optical axis is that direction, sees the same colour at its principal point (the rasterizer evaluates the Gaussians
    along the world-space ray; only culling and the depth order, which is by camera z in both, can differ)."""
    n, W, H, deg = 3000, 129, 65, 2
    P = synth.make_gaussians(n, 6, "cube", deg)
    vm = np.eye(4, dtype=np.float32)
    vm[:3, 3] = [0.0, 0.0, 4.0]
    K = synth.intrinsics(40.0, 40.0, W / 2, H / 2)
    bg = np.array([0.1, 0.2, 0.3], np.float32)
    e = orc.render_fwd(P, vm, K, W, H, deg, background=bg, camera_model=orc.EQUIRECTANGULAR)
    assert (e["radii"] > 0).all(-1).sum() > 0.8 * n          # no frustum: (nearly) everything is kept

    def rot_y(a):
        c, s = np.cos(a), np.sin(a)
        return np.array([[c, 0, s, 0], [0, 1, 0, 0], [-s, 0, c, 0], [0, 0, 0, 1]], np.float64)

    def rot_x(a):
        c, s = np.cos(a), np.sin(a)
        return np.array([[1, 0, 0, 0], [0, c, -s, 0], [0, s, c, 0], [0, 0, 0, 1]], np.float64)

    errs, covered = [], 0
    for x, y in [(64, 32), (60, 32), (70, 32), (64, 28), (64, 36), (58, 27), (72, 38), (62, 30), (67, 34)]:
        A, E = 2 * np.pi * ((x + 0.5) / W - 0.5), np.pi * ((y + 0.5) / H - 0.5)
        d = np.array([np.cos(E) * np.sin(A), np.sin(E), np.cos(A) * np.cos(E)])
        Cm = rot_x(E) @ rot_y(-A)                      # camera rotation that takes d to the optical axis
        assert np.allclose(Cm[:3, :3] @ d, [0, 0, 1], atol=1e-12)
        p = orc.render_fwd(P, (Cm @ vm.astype(np.float64)).astype(np.float32), K, W, H, deg, background=bg, camera_model=orc.PINHOLE)
        errs.append(float(np.abs(e["render"][y, x] - p["render"][H // 2, W // 2]).max()))
        assert abs(float(e["alpha"][y, x, 0]) - float(p["alpha"][H // 2, W // 2, 0])) < 3e-2
        covered += float(e["alpha"][y, x, 0]) > 0.05
    assert covered >= 6                                       # the probes do look at the Gaussians
    # a Gaussian that one model culls (sub-pixel radius, image margin) or a depth-order swap shows in a probe or two; the rest
    # agree to rounding
    assert max(errs) < 3e-2 and np.median(errs) < 1e-5 and sum(v < 1e-5 for v in errs) >= 6, errs


def test_oracle_equirectangular_matches_reference_cuda_golden(orc):
    """The oracle's EQUIRECTANGULAR model against the reference's own CUDA build (eq_* of tests/golden/reference_step.npz,
    written on a B200 by tests/golden/make_reference_golden.py): rasterize() of the 512 Gaussians of tiny_step.npz from a camera
    inside the scene, 64x32, so 224 of them lie behind the camera. atan2f / asinf differ in the last bit between the device
    and the host's libm, hence bounds on means2d instead of bit equality; radii and depths are exact."""
    gold = np.load(Path(__file__).parent / "golden" / "reference_step.npz")
    g = np.load(Path(__file__).parent / "golden" / "tiny_step.npz")
    names = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")
    P = {k: g[f"in_{k}"] for k in names}
    W, H = (int(x) for x in gold["eq_size"])
    deg = int(g["in_size"][2])
    f = orc.render_fwd(P, gold["eq_viewmat"], g["in_K"], W, H, deg, background=g["in_bg"], camera_model=orc.EQUIRECTANGULAR)
    vis = (gold["eq_radii"] > 0).all(-1)
    assert np.array_equal(f["masks"], vis) and (gold["eq_depths"][vis] < 0).sum() > 100
    assert np.array_equal(f["radii"][vis], gold["eq_radii"][vis])
    assert np.array_equal(f["depths"][vis].view(np.uint32), gold["eq_depths"][vis].view(np.uint32))
    assert np.abs(f["means2d"][vis] - gold["eq_means2d"][vis]).max() < 5e-3
    img = np.clip(f["render"], 0, 1).transpose(2, 0, 1)
    assert np.abs(img - gold["eq_image"]).max() < 1e-5
    assert np.abs(f["alpha"].reshape(H, W) - gold["eq_alpha"].reshape(H, W)).max() < 1e-5


def test_oracle_camera_features_match_reference_cuda_golden(orc):
    """The oracle against the reference's own CUDA build for what the training-step golden does not exercise
    (tests/golden/reference_cameras.npz, written on a B200 by tests/golden/make_reference_camera_golden.py from the outputs of
    gsplat::rasterize_from_world_with_sh_fwd): OpenCV distortion (radial + tangential + thin prism), fisheye with radial
    coefficients, two rolling shutters, the render modes D / ED / RGB_D / RGB_ED, the antialiased compensation and the scaling
    modifier, on the 512 Gaussians and the 64x48 camera of tiny_step.npz, and for seven of the cases the operator's backward.
    The reference is built with fast-math, the oracle is IEEE: colours within 1e-5, the depth channel within 1e-5 of its
    range, one radius of 512 may differ, gradients within 2e-4 relative L2."""
    import contextlib
    import importlib.util
    here = Path(__file__).parent / "golden"
    spec = importlib.util.spec_from_file_location("make_reference_camera_golden", here / "make_reference_camera_golden.py")
    G = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(G)                          # the case table and the coefficient values of the generator
    gold, g = np.load(here / "reference_cameras.npz"), np.load(here / "tiny_step.npz")
    P = {k: g[f"in_{k}"] for k in G.NAMES}
    W, H, deg = (int(x) for x in g["in_size"])
    vm, K, vm1 = g["in_viewmat"], g["in_K"], gold["viewmat_end"]
    assert np.array_equal(vm1, G.end_pose(vm)) and np.array_equal(gold["radial"], G.RADIAL)
    for name, c in G.CASES.items():
        radial = None
        if c["dist"]:
            radial = orc.pack_distortion(radial=G.RADIAL, tangential=G.TANGENTIAL, thin_prism=G.THIN_PRISM)
        if c["fish"]:
            radial = G.FISHEYE_RADIAL
        with (orc.shutter(vm1, c["rs"]) if c["rs"] != 4 else contextlib.nullcontext()):
            f = orc.render_fwd(P, vm, K, W, H, deg, background=G.background(c["mode"]), camera_model=c["model"], radial=radial,
                               render_mode=c["mode"], calc_compensations=c["aa"], scaling_modifier=c["smod"])
        ref_render, ref_alpha, ref_radii = gold[name + "_render"], gold[name + "_alpha"], gold[name + "_radii"]
        assert f["render"].shape == ref_render.shape, name
        scale = np.maximum(np.abs(ref_render).reshape(H * W, -1).max(0), 1.0)      # depth channels are a few units wide
        assert (np.abs(f["render"] - ref_render).reshape(H * W, -1) / scale).max() < 1e-5, name
        assert np.abs(f["alpha"] - ref_alpha).max() < 1e-5, name
        assert (f["radii"] != ref_radii).any(-1).sum() <= 1 and (ref_radii > 0).all(-1).sum() > 400, name
        if name in G.BACKWARD_CASES:
            # gsplat::rasterize_from_world_with_sh_bwd for seeded output gradients: gradients w.r.t. the ACTIVATED parameters
            v_r, v_a = G.output_gradients(name, H, W, G.channels(c["mode"]))
            with (orc.shutter(vm1, c["rs"]) if c["rs"] != 4 else contextlib.nullcontext()):
                b = orc.render_bwd(P, f, vm, K, W, H, deg, v_r, v_a, background=G.background(c["mode"]), camera_model=c["model"],
                                   radial=radial)
            pairs = (("v_means", b["means"]), ("v_quats", b["v_quats"]), ("v_scales", b["v_scales"]),
                     ("v_opacities", b["v_opacities"].reshape(-1)), ("v_sh_coeffs", np.concatenate([b["sh0"], b["shN"]], 1)))
            for key, mine in pairs:
                theirs = gold[f"{name}_{key}"].reshape(mine.shape)
                if np.abs(theirs).max() > 0:
                    assert rel_l2(mine, theirs) < 2e-4, (name, key)      # measured: at most 3.3e-5
                else:
                    assert np.abs(mine).max() == 0, (name, key)         # depth-only mode: no colour gradient
    # the features do change the picture: each case differs from the plain pinhole RGB render where it should
    plain = orc.render_fwd(P, vm, K, W, H, deg, background=G.background(0))["render"]
    for name in ("dist_full", "fisheye", "rolling_tb", "antialiased_smod"):
        assert np.abs(gold[name + "_render"] - plain).max() > 1e-2, name
