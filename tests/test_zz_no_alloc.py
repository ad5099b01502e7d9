"""The allocation-free classify entry point against the workspace-based one.

lfs_mcmc_classify_noalloc keeps its scratch in a fixed array inside the library, for hosts that may not
allocate device memory where they refine the model (under a viewer's render lock, or with a memory
budget fixed at start-up). The scratch is shared by all calls and keeps the previous call's contents,
so the check runs two calls in a row with different inputs and sizes: the second must not see
anything of the first. Index outputs and counts must be identical to lfs_mcmc_classify; the sampling
probabilities are the same float32 values bit for bit. This file sorts last on purpose."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _classify(pkg, which, opacity_raw, rotation_raw, min_opacity):
    capi = pkg._capi
    n = opacity_raw.shape[0]
    dead = torch.full((n,), -1, dtype=torch.int64, device=DEV)
    alive = torch.full((n,), -1, dtype=torch.int64, device=DEV)
    probs = torch.full((n,), -1.0, dtype=torch.float32, device=DEV)
    counts = torch.full((2,), -1, dtype=torch.int32, device=DEV)
    st = capi.vp(torch.cuda.current_stream().cuda_stream)
    args = [n, capi.ptr(opacity_raw), capi.ptr(rotation_raw), float(min_opacity), capi.ptr(dead), capi.ptr(alive),
            capi.ptr(probs), capi.ptr(counts)]
    if which == "workspace":
        ws = torch.empty(capi.lib().lfs_mcmc_workspace_bytes(n), dtype=torch.uint8, device=DEV)
        capi.call("lfs_mcmc_classify", *args, capi.ptr(ws), ws.numel(), st)
    else:
        capi.call("lfs_mcmc_classify_noalloc", *args, st)
    torch.cuda.synchronize()
    return dead.cpu().numpy(), alive.cpu().numpy(), probs.cpu().numpy(), counts.cpu().numpy()


def test_noalloc_matches_workspace_entry_point_twice(pkg):
    rng = np.random.default_rng(11)
    # second call is smaller and has a different dead pattern, so stale flags / prefix / count would show
    for n, dead_every in ((200_000, 9), (70_001, 4)):
        op = (rng.normal(size=(n, 1)) - 1).astype(np.float32)
        op[::dead_every] = -7.0
        rot = rng.normal(size=(n, 4)).astype(np.float32)
        rot[5] = 0.0
        t_op, t_rot = torch.from_numpy(op).to(DEV), torch.from_numpy(rot).to(DEV)
        ref = _classify(pkg, "workspace", t_op, t_rot, 0.005)
        out = _classify(pkg, "noalloc", t_op, t_rot, 0.005)
        n_dead, n_alive = ref[3]
        assert n_dead + n_alive == n and n_dead >= n // dead_every
        assert np.array_equal(out[3], ref[3])
        assert np.array_equal(out[0][:n_dead], ref[0][:n_dead]) and np.array_equal(out[1][:n_alive], ref[1][:n_alive])
        assert np.array_equal(out[2][:n_alive].view(np.uint32), ref[2][:n_alive].view(np.uint32))
        # nothing is written past the live part of the outputs
        assert (out[0][n_dead:] == -1).all() and (out[1][n_alive:] == -1).all()


def test_noalloc_at_its_size_limit_and_with_no_gaussians(pkg):
    """N equal to the built-in maximum is served; N = 0 writes the counts {0, 0} and touches nothing else."""
    rng = np.random.default_rng(3)
    n = 262144
    op = (rng.normal(size=(n, 1)) - 1).astype(np.float32)
    op[::7] = -7.0
    rot = rng.normal(size=(n, 4)).astype(np.float32)
    t_op, t_rot = torch.from_numpy(op).to(DEV), torch.from_numpy(rot).to(DEV)
    ref = _classify(pkg, "workspace", t_op, t_rot, 0.005)
    out = _classify(pkg, "noalloc", t_op, t_rot, 0.005)
    n_dead, n_alive = ref[3]
    assert n_dead + n_alive == n and np.array_equal(out[3], ref[3])
    assert np.array_equal(out[0][:n_dead], ref[0][:n_dead]) and np.array_equal(out[1][:n_alive], ref[1][:n_alive])
    empty_op, empty_rot = torch.empty((0, 1), device=DEV), torch.empty((0, 4), device=DEV)
    out = _classify(pkg, "noalloc", empty_op, empty_rot, 0.005)
    assert out[3].tolist() == [0, 0]


def test_noalloc_rejects_sizes_beyond_its_scratch(pkg):
    capi = pkg._capi
    n = 262144 + 1
    z = torch.zeros(8, device=DEV)
    with pytest.raises(pkg.LfsError, match="exceeds the built-in scratch"):
        capi.call("lfs_mcmc_classify_noalloc", n, capi.ptr(z), capi.ptr(z), 0.005, capi.ptr(z), capi.ptr(z), capi.ptr(z),
                  capi.ptr(z), None)
