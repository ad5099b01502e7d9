"""PLY export / import rows on the device against a numpy restatement of SplatData::to_point_cloud
(src/core/splat_data.cpp:483-503), a file round trip, and resume-from-checkpoint equality."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAMES = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")


def expected_rows(P, K):
    n = P["means"].shape[0]
    sh0 = P["sh0"].reshape(n, 1, 3).transpose(0, 2, 1).reshape(n, -1)
    shN = P["shN"].reshape(n, K - 1, 3).transpose(0, 2, 1).reshape(n, -1)
    q = P["rotation_raw"].astype(np.float32)
    n2 = ((q[:, 0] * q[:, 0] + q[:, 1] * q[:, 1]) + q[:, 2] * q[:, 2]) + q[:, 3] * q[:, 3]
    nrm = np.maximum(np.sqrt(n2, dtype=np.float32), np.float32(1e-12))
    return np.concatenate([P["means"], np.zeros((n, 3), np.float32), sh0, shN, P["opacity_raw"].reshape(n, 1), P["scaling_raw"],
                           (q / nrm[:, None]).astype(np.float32)], axis=1).astype(np.float32)


@pytest.mark.parametrize("n,deg", [(1, 0), (1001, 3), (4096, 1)])
def test_rows_bit_exact_and_file_roundtrip(pkg, synth, tmp_path, n, deg):
    tr, fm = pkg.trainer, pkg.formats
    K = (deg + 1) ** 2
    P = synth.make_gaussians(n, 21, "cube", deg)
    model = tr.SplatData(n, K, DEV, capacity=n + 7).load(P)
    rows = fm.pack_rows(model).cpu().numpy()
    exp = expected_rows(P, K)
    assert rows.shape == exp.shape and np.array_equal(rows.view(np.uint32), exp.view(np.uint32))
    path = fm.save_ply(model, str(tmp_path), 30000)
    assert path.endswith("splat_30000.ply")
    names, body = fm.read_ply(path)
    assert names == fm.ply_attribute_names(K) and np.array_equal(body, exp)
    back = fm.load_ply(path, DEV)
    assert back.size == n and back.K == K
    for name in NAMES:
        a = back.tensor(name).cpu().numpy()
        ref = P[name].reshape(a.shape) if name != "rotation_raw" else exp[:, -4:]
        assert np.array_equal(a, ref), name


def test_resume_from_checkpoint_continues_identically(pkg, synth, tmp_path):
    """Four MCMC-strategy Adam steps in one go vs two steps, save, restore into a fresh process state, two more."""
    tr, st, fm = pkg.trainer, pkg.strategy, pkg.formats
    n, deg = 5000, 2
    K = (deg + 1) ** 2
    P = synth.make_gaussians(n, 3, "cube", deg)
    rng = np.random.default_rng(0)
    G = [{k: rng.normal(size=v.shape).astype(np.float32) * 1e-2 for k, v in P.items()} for _ in range(4)]

    def make():
        s = st.MCMC(tr.SplatData(n, K, DEV).load(P))
        s.initialize(st.OptimizationParameters(max_cap=n, sh_degree=deg, iterations=100))
        return s

    def run(s, its):
        for it in its:
            s.grads.load(G[it - 1])
            s.step(it)

    a = make(); run(a, [1, 2, 3, 4])
    b = make(); run(b, [1, 2])
    path = fm.save_checkpoint(b, str(tmp_path / "x.ckpt"), 2)
    c = make()
    assert fm.load_checkpoint(c, path) == 2
    run(c, [3, 4])
    for name in NAMES:
        assert torch.equal(a.get_model().tensor(name), c.get_model().tensor(name)), name
        assert torch.equal(a._optimizer.exp_avg.tensor(name), c._optimizer.exp_avg.tensor(name)), name
    assert a._optimizer.lr == c._optimizer.lr and a._optimizer.step_count == c._optimizer.step_count
