"""MCMC densification (relocate / add / noise) and the strategy interface against a numpy restatement of
src/training/strategies/mcmc.cpp:112-367. Index-valued results (dead / alive lists, ratios, which rows are
copied where, which moments are reset) must be bit-exact; float results within float32 rounding."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAMES = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")


def sig32(x):
    x = x.astype(np.float32)
    return (np.float32(1) / (np.float32(1) + np.exp(-x, dtype=np.float32))).astype(np.float32)


def ref_apply(orc, P, M, V, sampled, dst, min_opacity, zero_at_dst):
    """numpy restatement of the post-draw part of relocate_gs / add_new_gs."""
    N = P["means"].shape[0]
    op = sig32(P["opacity_raw"].reshape(-1))
    sc = np.exp(P["scaling_raw"].astype(np.float32), dtype=np.float32)
    counts = np.bincount(sampled, minlength=N)
    ratios = np.clip(1 + counts[sampled], 1, 51).astype(np.int32)
    no, ns = orc.relocation(op[sampled], sc[sampled], ratios, orc.binoms_table(51), 51)
    no = np.clip(no, np.float32(min_opacity), np.float32(1.0 - 1e-7)).astype(np.float32)
    P["opacity_raw"][sampled, 0] = np.log(no / (np.float32(1) - no))
    P["scaling_raw"][sampled] = np.log(ns)
    for n in NAMES:
        P[n][dst] = P[n][sampled]
        z = dst if zero_at_dst else sampled
        M[n][z] = 0
        V[n][z] = 0
    return ratios


def build(pkg, synth, n, deg, cap=None, seed=5):
    st, tr = pkg.strategy, pkg.trainer
    P = synth.make_gaussians(n, seed, "clusters", deg)
    P["opacity_raw"][np.arange(n) % 20 == 7] = -6.0  # dead: sigmoid(-6) = 0.0025 < 0.005
    P["rotation_raw"][13] = 0.0                     # dead: zero quaternion
    model = tr.SplatData(n, (deg + 1) ** 2, DEV, capacity=cap or n).load(P)
    s = st.MCMC(model)
    s.initialize(st.OptimizationParameters(max_cap=cap or n, sh_degree=deg))
    rng = np.random.default_rng(1)
    M = {k: rng.normal(size=v.shape).astype(np.float32) for k, v in P.items()}
    V = {k: rng.random(size=v.shape).astype(np.float32) for k, v in P.items()}
    s._optimizer.exp_avg.load(M)
    s._optimizer.exp_avg_sq.load(V)
    return s, P, M, V


def compare(s, P, M, V, n):
    sd, opt = s._splat_data, s._optimizer
    assert sd.size == n and opt.exp_avg.size == n and opt.exp_avg_sq.size == n
    for k in NAMES:
        a = sd.tensor(k).cpu().numpy()
        assert np.allclose(a, P[k][:n], rtol=3e-5, atol=1e-6), k
        # rows that were only copied are bit-identical
        assert np.array_equal(opt.exp_avg.tensor(k).cpu().numpy(), M[k][:n]), k
        assert np.array_equal(opt.exp_avg_sq.tensor(k).cpu().numpy(), V[k][:n]), k


@pytest.mark.parametrize("deg", [0, 3])
def test_relocate(pkg, orc, synth, deg):
    n = 20000
    s, P, M, V = build(pkg, synth, n, deg)
    sd = s._splat_data
    op = sig32(P["opacity_raw"].reshape(-1))
    dead_mask = (op <= np.float32(0.005)) | ((P["rotation_raw"] ** 2).sum(-1) < 1e-8)
    dead, alive = np.nonzero(dead_mask)[0], np.nonzero(~dead_mask)[0]
    rng = np.random.default_rng(2)
    local = rng.integers(0, alive.size, size=dead.size)
    local[:50] = local[0]  # force a heavily repeated index (ratio > 1, clamped path for > 51)
    n_dead = s.relocate_gs(torch.from_numpy(local).to(DEV))
    assert n_dead == dead.size
    assert np.array_equal(s._dead[:n_dead].cpu().numpy(), dead)
    assert np.array_equal(s._alive[:alive.size].cpu().numpy(), alive)
    # sampling probabilities are exactly torch.sigmoid of the raw opacities
    assert torch.equal(s._alive_opac[:alive.size], torch.sigmoid(torch.from_numpy(P["opacity_raw"]).to(DEV)).reshape(-1)[torch.from_numpy(alive).to(DEV)])
    sampled = alive[local]
    assert np.array_equal(s._sampled[:n_dead].cpu().numpy(), sampled)
    ratios = ref_apply(orc, P, M, V, sampled, dead, 0.005, zero_at_dst=False)
    assert np.array_equal(s._ratios[:n_dead].cpu().numpy(), ratios)
    assert ratios.max() == 51
    compare(s, P, M, V, n)


def test_add_new_and_noise(pkg, orc, synth):
    n, deg = 8000, 2
    s, P, M, V = build(pkg, synth, n, deg, cap=9000)
    n_new = int(np.float32(1.05) * np.float32(n)) - n
    rng = np.random.default_rng(3)
    sampled = rng.integers(0, n, size=n_new)
    sampled[:5] = sampled[0]
    assert s.add_new_gs(torch.from_numpy(sampled).to(DEV)) == n_new
    for d in (P, M, V):
        for k in NAMES:
            d[k] = np.concatenate([d[k], np.zeros((n_new,) + d[k].shape[1:], np.float32)], 0)
    ref_apply(orc, P, M, V, sampled, np.arange(n, n + n_new), 0.005, zero_at_dst=True)
    compare(s, P, M, V, n + n_new)
    # capacity guard, then noise with an injected sample
    noise = rng.normal(size=(n + n_new, 3)).astype(np.float32)
    s.inject_noise(torch.from_numpy(noise).to(DEV))
    ref_means = P["means"].copy()
    orc.add_noise(P["opacity_raw"], P["scaling_raw"], P["rotation_raw"], noise, ref_means, float(np.float32(s._optimizer.lr[0])) * 5e5)
    assert np.abs(s._splat_data.tensor("means").cpu().numpy() - ref_means).max() < 2e-5
    s._params.max_cap = 10**9
    torch.manual_seed(7)
    with pytest.raises(RuntimeError, match="capacity"):
        for _ in range(5):  # 8400 -> 8820 fits in 9000 rows, the next growth does not
            s.add_new_gs()
    assert s._splat_data.size == 8820


def test_strategy_schedule_and_step(pkg, synth):
    st = pkg.strategy
    s, P, M, V = build(pkg, synth, 2000, 1, cap=4000)
    p = s._params
    assert not s.is_refining(500) and s.is_refining(600) and not s.is_refining(650) and not s.is_refining(25000)
    lr0 = s._optimizer.lr[0]
    s.grads.flat.normal_()
    before = s._splat_data.flat.clone()
    s.step(5)
    assert s._optimizer.step_count == 1 and abs(s._optimizer.lr[0] - lr0 * 0.01 ** (1 / 30000)) < 1e-18
    # shN untouched while iteration <= 1000, updated afterwards
    shn0 = s._splat_data.tensor("shN").clone()
    s.step(7)
    assert torch.equal(s._splat_data.tensor("shN"), shn0)
    s.step(1001)
    assert not torch.equal(s._splat_data.tensor("shN"), shn0)
    # post_backward: degree increments on the interval, refinement grows the model within max_cap, and removal compacts
    torch.manual_seed(1234)
    s.post_backward(1000)
    assert s.active_sh_degree == 1 and s._splat_data.size == min(4000, int(np.float32(1.05) * np.float32(2000)))
    n = s._splat_data.size
    mask = torch.zeros(n, dtype=torch.bool, device=DEV)
    mask[::3] = True
    keep_rows = s._splat_data.tensor("means")[~mask].clone()
    s.remove_gaussians(mask)
    assert s._splat_data.size == n - int(mask.sum()) and torch.equal(s._splat_data.tensor("means"), keep_rows)
    assert s._optimizer.exp_avg.size == s._splat_data.size


def test_rank1_step_is_refused_after_post_backward(pkg, synth):
    """The rank-1 shN update rebuilds its gradient rows from the current means: after post_backward (noise on every mean,
    relocated rows) those are no longer the forward's, so the strategy refuses it; the reference's order with a
    materialised shN gradient goes through."""
    s, P, M, V = build(pkg, synth, 1501, 1, cap=3000)
    s.grads.flat.normal_()
    marker = object()
    s.post_backward(1501)              # no refinement on this iteration: noise only
    with pytest.raises(RuntimeError, match="moved the means"):
        s.step(1501, rasterizer=marker)
    assert s._optimizer.step_count == 0
    s.step(1501)                       # materialised gradients: fine
    assert s._optimizer.step_count == 1
