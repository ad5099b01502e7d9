"""World-size-2 gloo test of the data-parallel exchange logic on CPU: shard bounds, group segments,
reduce-scatter / all-gather with padding, and that the all-reduce and the sharded exchange leave the
same parameters on every rank as a single-process Adam on the summed gradients. The CUDA Adam is replaced
by the oracle's Adam through the adam_fn hook; the collectives and the segment arithmetic are the code
that runs on the GPUs."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
LRS = [1.6e-4, 2.5e-3, 1.25e-4, 5e-3, 1e-3, 5e-2]


def test_shard_bounds_and_segments(pkg):
    dp = pkg.dp
    for total, world in ((59 * 12, 2), (59 * 100, 8), (1000, 3), (7, 4)):
        seen = 0
        for r in range(world):
            lo, n, per = dp.shard_bounds(total, world, r)
            assert lo == min(r * per, total) and per % 4 == 0 and per * world >= total
            seen += n
        assert seen == total
    segs = dp.group_segments(8, 4, 0, 8 * 23, LRS)
    assert [s[0] for s in segs] == [0, 1, 2, 3, 4, 5] and sum(s[2] for s in segs) == 8 * 23
    assert [s[1] for s in segs] == [0, 24, 48, 120, 144, 176]
    segs = dp.group_segments(8, 4, 30, 100, LRS, skip_shN=True)
    assert [(s[0], s[1], s[2]) for s in segs] == [(1, 30, 18), (3, 120, 10)]
    assert dp.group_segments(8, 1, 0, 8 * 14, LRS)[2][0] == 3  # K = 1: the empty shN group is skipped


def _worker(rank, world, port, mode, tmp):
    sys.path.insert(0, str(ROOT))
    import importlib
    pkg = importlib.import_module("lichtfeld-studio_b200")
    from oracle import oracle as orc
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tr, dp = pkg.trainer, pkg.dp
    n, K = 37, 4  # capacity 40 -> 920 floats: not a multiple of 2 * 4 * anything convenient => exercises padding
    model, grads = tr.SplatData(n, K, "cpu"), tr.SplatData(n, K, "cpu")
    g0 = torch.Generator().manual_seed(0)
    model.flat.copy_(torch.randn(model.flat.numel(), generator=g0))

    def adam_fn(p, m, v, g, lr, step, gs):
        pa, ma, va = p.numpy(), m.numpy(), v.numpy()
        orc.adam_step(pa, ma, va, (g.numpy() * np.float32(gs)).astype(np.float32), lr, 0.9, 0.999, 1e-15, step)

    ex = dp.GradExchange(model, grads, LRS, mode=mode)
    for it in (5, 1001):  # first with the shN group skipped, then with it
        gr = torch.Generator().manual_seed(100 * it + rank)
        grads.flat.copy_(torch.randn(grads.flat.numel(), generator=gr))
        ex.step(it, adam_fn=adam_fn)
    torch.save(model.flat.clone(), os.path.join(tmp, f"{mode}_{rank}.pt"))
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["allreduce", "sharded"])
def test_exchange_modes_agree_under_gloo(pkg, orc, tmp_path, mode):
    world = 2
    port = 29600 + (os.getpid() % 200) + (0 if mode == "allreduce" else 1)
    mp.spawn(_worker, args=(world, port, mode, str(tmp_path)), nprocs=world, join=True)
    outs = [torch.load(tmp_path / f"{mode}_{r}.pt") for r in range(world)]
    assert torch.equal(outs[0], outs[1])  # identical parameters on every rank
    # single-process reference: Adam on the summed gradients, mean over the batch of `world` cameras
    tr, dp = pkg.trainer, pkg.dp
    n, K = 37, 4
    model = tr.SplatData(n, K, "cpu")
    model.flat.copy_(torch.randn(model.flat.numel(), generator=torch.Generator().manual_seed(0)))
    m, v = torch.zeros_like(model.flat), torch.zeros_like(model.flat)
    for step, it in enumerate((5, 1001), start=1):
        g = sum(torch.randn(model.flat.numel(), generator=torch.Generator().manual_seed(100 * it + r)) for r in range(world))
        for gi, off, cnt, lr in dp.group_segments(model.capacity, K, 0, model.flat.numel(), LRS, it <= 1000):
            orc.adam_step(model.flat[off:off + cnt].numpy(), m[off:off + cnt].numpy(), v[off:off + cnt].numpy(),
                          (g[off:off + cnt].numpy() * np.float32(0.5)).astype(np.float32), lr, 0.9, 0.999, 1e-15, step)
    assert torch.allclose(outs[0], model.flat, rtol=1e-6, atol=1e-7)


def test_class_segments_partition_each_class_exactly_once(pkg):
    """The split exchange shards the geometry class and the colour class separately: over all ranks every element of
    a class is covered exactly once, offsets and counts stay 4-element aligned, moments offsets are consistent, and
    skipping shN only removes segments."""
    dp, tr = pkg.dp, pkg.trainer
    for capacity, K, world in ((1000, 16, 8), (64, 4, 3), (20, 1, 2), (4096, 25, 5)):
        w = tr.row_widths(K)
        total = capacity * sum(w.values())
        lrs = [1, 2, 3, 4, 5, 6]
        for names in (dp.GEOMETRY_CLASS, dp.COLOR_CLASS):
            cover = np.zeros(total, np.int32)
            for rank in range(world):
                segs, per = dp.class_segments(capacity, K, names, world, rank, lrs)
                segs_skip, per2 = dp.class_segments(capacity, K, names, world, rank, lrs, skip_shN=True)
                assert per == per2 and len(segs) <= 6
                assert [s for s in segs if tr.PARAM_NAMES[s[0]] != "shN"] == segs_skip
                used = 0
                for gi, off, cnt, lr, rel in segs:
                    assert cnt > 0 and off % 4 == 0 and rel % 4 == 0 and lr == lrs[gi] and rel + cnt <= per
                    assert rel == used          # the shard's moments are laid out in segment order
                    used += cnt
                    cover[off:off + cnt] += 1
            off = 0
            for name in tr.PARAM_NAMES:
                size = capacity * w[name]
                assert (cover[off:off + size] == (1 if name in names else 0)).all(), name
                off += size


def test_wait_status_names_the_missing_ranks(pkg):
    """Host side of the bounded waits: the status word of lfs_dp_wait / lfs_dp_barrier as the error the step raises."""
    dp = pkg.dp
    assert dp.describe_wait_status([0, 0, 0, 0], 8, 20.0) is None
    msg = dp.describe_wait_status([1, (1 << 7) | (1 << 2), 1, 41], 8, 0.5)
    assert "ranks [2, 7]" in msg and "step 41" in msg and "slot 1" in msg and "0.5 s" in msg
    assert "ranks [0]" in dp.describe_wait_status([1, 1, 0, 3], 2, 20.0)


def _watch_worker(rank, world, port, tmp, scenario):
    sys.path.insert(0, str(ROOT))
    import importlib
    pkg = importlib.import_module("lichtfeld-studio_b200")
    dp = pkg.dp
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.distributed_c10d._get_default_store()
    watch = dp.PeerWatch(store, rank, world, timeout_s=(1.0 if scenario == "silent" else 20.0))
    x = torch.ones(4)
    done, verdict = 0, "finished"
    try:
        with watch:
            for step in range(1, 6):
                if rank == world - 1 and step == 3:
                    if scenario == "raises":
                        raise ValueError("bad batch")          # the failure, made on the host, between steps
                    if scenario == "silent":
                        store.wait([f"silent_done/{r}" for r in range(world - 1)])   # stops stepping without a word
                        break
                watch.ready(step)                              # nobody enqueues a collective that a peer will not join
                dist.all_reduce(x)
                done = step
    except dp.PeerLeft as e:
        verdict = f"peer_left:{e.ranks}:{e}"
    except ValueError as e:
        verdict = f"raised:{e}"
    with open(os.path.join(tmp, f"watch_{scenario}_{rank}.txt"), "w") as f:
        f.write(f"{done}|{verdict}")
    if scenario == "silent" and rank != world - 1:
        store.set(f"silent_done/{rank}", "1")
    # no destroy_process_group barrier games: every rank reaches this point on its own


@pytest.mark.parametrize("scenario", ["raises", "silent", "healthy"])
def test_peer_watch_reports_a_rank_that_stops_stepping(pkg, tmp_path, scenario):
    """Failure detection on the host, as gloo ranks: a rank that raises between steps (its `with PeerWatch` block publishes the
    reason), a rank that silently stops (the others' ready() gives up after its limit), and a healthy run. In both failures the
    others stop BEFORE the collective of the step the failed rank never launches, with two completed steps."""
    world = 3
    port = 29850 + (os.getpid() % 100) + {"raises": 0, "silent": 1, "healthy": 2}[scenario]
    mp.spawn(_watch_worker, args=(world, port, str(tmp_path), scenario), nprocs=world, join=True)
    res = [open(tmp_path / f"watch_{scenario}_{r}.txt").read().split("|", 1) for r in range(world)]
    if scenario == "healthy":
        assert all(d == "5" and v == "finished" for d, v in res)
        return
    for r in range(world - 1):
        done, verdict = res[r]
        assert done == "2" and verdict.startswith(f"peer_left:[{world - 1}]"), res
        assert ("ValueError: bad batch" in verdict) if scenario == "raises" else ("did not get there within" in verdict), verdict
    assert res[world - 1][0] == "2" and res[world - 1][1] == ("raised:bad batch" if scenario == "raises" else "finished")
