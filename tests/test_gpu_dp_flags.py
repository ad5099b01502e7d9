"""Ordering and failure detection of the data-parallel exchange (lfs_dp_signal / lfs_dp_wait) on ONE GPU.

The flag arrays of the emulated ranks live on the same device, so the peer pointers are plain local pointers. No kernel here
waits for another kernel: a wait either finds its flags already stored by an earlier launch on the same stream, or waits for
a flag that nothing sets and gives up after its (short) limit, which is the failure the status word reports."""
import ctypes as C
import time

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _arrays(capi, world):
    flags = [torch.zeros(capi.LFS_DP_FLAG_WORDS, dtype=torch.int32, device=DEV) for _ in range(world)]
    peers = (C.c_void_p * world)(*[f.data_ptr() for f in flags])
    return flags, peers


def test_wait_returns_at_once_when_every_rank_signalled(pkg):
    capi = pkg._capi
    world, slot, step = 4, 1, 7
    flags, peers = _arrays(capi, world)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    for r in range(world):
        capi.call("lfs_dp_signal", world, peers, r, slot, step, _stream())
    t0 = time.perf_counter()
    for r in range(world):
        capi.call("lfs_dp_wait", world, capi.vp(flags[r].data_ptr()), slot, step, 2_000_000_000, capi.vp(status.data_ptr()), _stream())
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.5
    assert status.tolist() == [0, 0, 0, 0]
    for r in range(world):                      # rank r's array holds everyone's step in the slot's row, nothing elsewhere
        f = flags[r].view(capi.LFS_DP_FLAG_SLOTS, capi.LFS_DP_MAX_WORLD)
        assert f[slot, :world].tolist() == [step] * world
        assert int(f.abs().sum()) == step * world
    # a later step's flag also satisfies the wait for an earlier one (a fast peer may already be one step ahead)
    capi.call("lfs_dp_wait", world, capi.vp(flags[0].data_ptr()), slot, step - 1, 1_000_000, capi.vp(status.data_ptr()), _stream())
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]


def test_wait_gives_up_and_names_the_missing_ranks(pkg):
    capi = pkg._capi
    world, slot, step = 4, 2, 3
    flags, peers = _arrays(capi, world)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    for r in (0, 2):                            # ranks 1 and 3 never reach the step
        capi.call("lfs_dp_signal", world, peers, r, slot, step, _stream())
    t0 = time.perf_counter()
    capi.call("lfs_dp_wait", world, capi.vp(flags[0].data_ptr()), slot, step, 50_000_000, capi.vp(status.data_ptr()), _stream())
    probe = torch.arange(8, device=DEV) * 2     # the stream carries on after the wait gave up
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert 0.04 < dt < 1.0, dt
    assert status.tolist() == [1, (1 << 1) | (1 << 3), slot, step]
    assert probe.tolist() == [0, 2, 4, 6, 8, 10, 12, 14]
    # the context is intact: a wait that is satisfied still works and leaves the recorded failure in place
    capi.call("lfs_dp_signal", world, peers, 1, slot, step, _stream())
    capi.call("lfs_dp_signal", world, peers, 3, slot, step, _stream())
    status2 = torch.zeros(4, dtype=torch.int32, device=DEV)
    capi.call("lfs_dp_wait", world, capi.vp(flags[0].data_ptr()), slot, step, 50_000_000, capi.vp(status2.data_ptr()), _stream())
    torch.cuda.synchronize()
    assert status2.tolist() == [0, 0, 0, 0]


def test_barrier_is_signal_and_wait_in_one_launch(pkg):
    capi = pkg._capi
    world, slot = 3, 0
    flags, peers = _arrays(capi, world)
    status = [torch.zeros(4, dtype=torch.int32, device=DEV) for _ in range(world)]
    # ranks 0 and 1 have signalled step 1 already; rank 2's barrier then finds everything in place (its own word by itself)
    capi.call("lfs_dp_signal", world, peers, 0, slot, 1, _stream())
    capi.call("lfs_dp_signal", world, peers, 1, slot, 1, _stream())
    capi.call("lfs_dp_barrier", world, peers, 2, slot, 1, 50_000_000, capi.vp(status[2].data_ptr()), _stream())
    torch.cuda.synchronize()
    assert status[2].tolist() == [0, 0, 0, 0]
    for r in range(world):
        assert flags[r].view(capi.LFS_DP_FLAG_SLOTS, capi.LFS_DP_MAX_WORLD)[slot, :world].tolist() == [1, 1, 1]
    # step 2: rank 0 arrives alone; its barrier gives up after the limit and names ranks 1 and 2; a second failure (slot 3)
    # adds to the mask but the first one keeps slot and step
    capi.call("lfs_dp_barrier", world, peers, 0, slot, 2, 30_000_000, capi.vp(status[0].data_ptr()), _stream())
    capi.call("lfs_dp_barrier", world, peers, 0, 3, 2, 30_000_000, capi.vp(status[0].data_ptr()), _stream())
    torch.cuda.synchronize()
    assert status[0].tolist() == [1, 0b110, slot, 2]
    assert flags[1].view(capi.LFS_DP_FLAG_SLOTS, capi.LFS_DP_MAX_WORLD)[slot, :world].tolist() == [2, 1, 1]


def test_arguments_are_checked(pkg):
    capi = pkg._capi
    flags, peers = _arrays(capi, 2)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError):
        capi.call("lfs_dp_wait", 2, capi.vp(flags[0].data_ptr()), 0, 1, 0, capi.vp(status.data_ptr()), _stream())                    # no limit
    with pytest.raises(RuntimeError):
        capi.call("lfs_dp_wait", 2, capi.vp(flags[0].data_ptr()), 0, 1, 61_000_000_000, capi.vp(status.data_ptr()), _stream())       # limit beyond 60 s
    with pytest.raises(RuntimeError):
        capi.call("lfs_dp_wait", 2, capi.vp(flags[0].data_ptr()), capi.LFS_DP_FLAG_SLOTS, 1, 1000, capi.vp(status.data_ptr()), _stream())
    with pytest.raises(RuntimeError):
        capi.call("lfs_dp_signal", capi.LFS_DP_MAX_WORLD + 1, peers, 0, 0, 1, _stream())
    with pytest.raises(RuntimeError):
        capi.call("lfs_dp_signal", 2, peers, 2, 0, 1, _stream())
    torch.cuda.synchronize()
