"""Multi-GPU check of the data-parallel training step (run under torchrun, one rank per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 tests/run_dp_check.py

Every rank renders its own camera; the three exchanges (NCCL all-reduce, NCCL reduce-scatter + sharded Adam
+ all-gather, fused peer-memory kernel, also split over two streams and with the shN gradient as rank-1 factors) must
leave the same parameters on every rank, equal to what one GPU gets by rendering all cameras itself and averaging the
gradients. Then: the flag ordering against the NCCL ordering, the multimem.st broadcast (where the box has NVSwitch
multicast), and failure detection: one rank stops stepping between steps (it stays alive, nothing of its own in flight)
and the others' bounded waits report it. Run with NCCL_NVLS_ENABLE=0. Not collected by pytest."""
import datetime
import importlib
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
LRS = [1.6e-4, 2.5e-3, 1.25e-4, 5e-3, 1e-3, 5e-2]
LAST_EXCHANGE = [None]


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=60))
    pkg = importlib.import_module("lichtfeld-studio_b200")
    synth, tr, dp = pkg.synth, pkg.trainer, pkg.dp
    n, W, H, deg, steps = 30000, 320, 208, 3, 3
    K = (deg + 1) ** 2
    P = synth.make_gaussians(n, 0, "clusters", deg)
    poses = synth.hemisphere_poses(16, 5.0)
    Kmat = torch.from_numpy(synth.intrinsics(280.0, 280.0, W / 2, H / 2)).to(dev)
    bg = torch.zeros(3, device=dev)
    targets = [torch.rand(3, H, W, generator=torch.Generator().manual_seed(s)).to(dev) for s in range(steps * world)]

    def cam(i):
        return tr.Camera(torch.from_numpy(poses[i % 16]).to(dev), Kmat, W, H)

    def run(mode):
        cap = (n + 31) // 32 * 32
        numel = cap * tr.SplatData(1, K, "cpu").row_floats
        peer = None
        if mode.startswith("fused_p2p"):
            pf, gf, peer = dp.symmetric_flat_buffers(numel, dev)
            model, grads = tr.SplatData(n, K, dev, cap, flat=pf).load(P), tr.SplatData(n, K, dev, cap, flat=gf)
        else:
            model, grads = tr.SplatData(n, K, dev, cap).load(P), tr.SplatData(n, K, dev, cap)
        rast, lossfn = tr.Rasterizer(model, W, H, deg), tr.PhotometricLoss(W, H, dev)
        if mode == "local":  # one GPU renders the whole batch and averages
            m, v = model.like(), model.like()
            for s in range(steps):
                for r in range(world):
                    out = rast.forward(cam(s * world + r), bg)
                    _, vr = lossfn(out.image, targets[s * world + r])
                    rast.backward(vr, grads, bg, accumulate=(r > 0))
                tr.adam_step_splats(model, m, v, grads, LRS, s + 1, skip_shN=False, grad_scale=1.0 / world)
            return model.flat.clone()
        if mode == "fused_p2p_split_rank1":
            # as fused_p2p_split, with the shN gradient crossing NVLink as its two rank-1 factors
            ex = LAST_EXCHANGE[0] = dp.GradExchange(model, grads, LRS, mode="fused_p2p", peer_ptrs=peer)
            side = torch.cuda.Stream(device=dev)
            for s in range(steps):
                rast.forward_lists(cam(s * world + rank))
                ex.wait_color()
                out = rast.forward_shade(bg)
                _, vr = lossfn(out.image, targets[s * world + rank])
                rast.backward(vr, grads, bg, sh_factors=True)
                ex.step_split(2000 + s, side, rank1_sh=True, sh_degree=deg)
            ex.wait_color()
            torch.cuda.synchronize()
            return model.flat.clone()
        if mode == "fused_p2p_split":
            # geometry groups exchanged on the main stream, colour groups on a side stream under the next step's lists
            ex = LAST_EXCHANGE[0] = dp.GradExchange(model, grads, LRS, mode="fused_p2p", peer_ptrs=peer)
            side = torch.cuda.Stream(device=dev)
            for s in range(steps):
                rast.forward_lists(cam(s * world + rank))
                ex.wait_color()
                out = rast.forward_shade(bg)
                _, vr = lossfn(out.image, targets[s * world + rank])
                rast.backward(vr, grads, bg)
                ex.step_split(2000 + s, side)
            ex.wait_color()
            torch.cuda.synchronize()
            return model.flat.clone()
        ex = LAST_EXCHANGE[0] = dp.GradExchange(model, grads, LRS, mode=mode, peer_ptrs=peer)
        for s in range(steps):
            out = rast.forward(cam(s * world + rank), bg)
            _, vr = lossfn(out.image, targets[s * world + rank])
            rast.backward(vr, grads, bg)
            ex.step(2000 + s)
        torch.cuda.synchronize()
        return model.flat.clone()

    ref = run("local")
    start = tr.SplatData(n, K, dev, (n + 31) // 32 * 32).load(P).flat
    ok = True
    for mode in ("allreduce", "sharded", "fused_p2p", "fused_p2p_split", "fused_p2p_split_rank1"):
        try:
            out = run(mode)
        except Exception as e:  # report and keep the ranks in lock step
            print(f"[rank {rank}] {mode}: FAILED {type(e).__name__}: {e}", flush=True)
            ok = False
            break
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        same = all(torch.equal(gathered[0], g) for g in gathered)
        rel = float((out - ref).norm() / (ref - tr.SplatData(n, K, dev, (n + 31) // 32 * 32).load(P).flat).norm())
        if rank == 0:
            print(f"{mode}: identical on all ranks = {same}; |update - local update| / |local update| = {rel:.2e}", flush=True)
        ok = ok and same and rel < 2e-3
    if rank == 0:
        print("DP CHECK", "OK" if ok else "FAILED", flush=True)
    for ordering in ("flags", "nccl"):          # both orderings give the same parameters, bit for bit
        os.environ["LFS_DP_ORDERING"] = ordering
        res = run("fused_p2p_split_rank1")
        if ordering == "flags":
            first = res
        elif rank == 0:     # the backward sums with atomics, so two runs agree to rounding, not bit for bit
            print(f"orderings flags / nccl: |difference| / |update| = {float((first - res).norm() / (first - start).norm()):.2e}", flush=True)
    os.environ["LFS_DP_ORDERING"] = "flags"
    os.environ["LFS_DP_MULTICAST"] = "1"        # parameters broadcast with multimem.st where the box has NVSwitch multicast
    for mode in ("fused_p2p", "fused_p2p_split_rank1"):
        out = run(mode)
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        same = all(torch.equal(gathered[0], g) for g in gathered)
        rel = float((out - ref).norm() / (ref - start).norm())
        if rank == 0:
            print(f"{mode} + multimem.st: identical on all ranks = {same}; |update - local update| / |local update| = {rel:.2e}"
                  f" (multicast address {'present' if LAST_EXCHANGE[0].mc_params else 'ABSENT: plain stores were used'})", flush=True)
            print("DP MULTICAST CHECK", "OK" if same and rel < 2e-3 else "FAILED", flush=True)
    os.environ["LFS_DP_MULTICAST"] = "0"
    failure_detection(dp, tr, dev, rank, world, n, K, P)
    dist.destroy_process_group()


def failure_detection(dp, tr, dev, rank, world, n, K, P):
    """The last rank stops stepping after step 1, between steps, with nothing of its own in flight; it stays alive (its memory
    stays mapped) and waits on the host. The others run step 2: their bounded wait for its flag gives up, the status word
    names it, raise_if_failed() raises, and their CUDA contexts stay usable. Plain peer loads and stores only (no multimem)."""
    cap = (n + 31) // 32 * 32
    numel = cap * tr.SplatData(1, K, "cpu").row_floats
    pf, gf, peer = dp.symmetric_flat_buffers(numel, dev)
    model, grads = tr.SplatData(n, K, dev, cap, flat=pf).load(P), tr.SplatData(n, K, dev, cap, flat=gf)
    grads.flat.fill_(1e-3)
    ex = dp.GradExchange(model, grads, LRS, mode="fused_p2p", peer_ptrs=peer, wait_timeout_s=0.5, multicast=False)
    ex.step(2000)
    ex.raise_if_failed()                       # step 1: everybody took part
    torch.cuda.synchronize()
    store = dist.distributed_c10d._get_default_store()
    leaver = world - 1
    if rank == leaver:
        store.set("dp_failure/left", "1")      # what a heartbeat would stop saying
        store.wait([f"dp_failure/done{r}" for r in range(world - 1)], datetime.timedelta(seconds=60))
        passed = True
    else:
        store.wait(["dp_failure/left"], datetime.timedelta(seconds=60))
        ex.step(2001)                          # the leaver's flag never arrives
        try:
            ex.raise_if_failed()
            passed = False
        except RuntimeError as e:
            passed = f"ranks [{leaver}]" in str(e)
            if rank == 0:
                print("detected:", e, flush=True)
        alive = float((torch.ones(1024, device=dev) * 2).sum())    # the context still works
        passed = passed and alive == 2048.0
        store.set(f"dp_failure/done{rank}", "1" if passed else "0")
    votes = [store.get(f"dp_failure/done{r}") == b"1" for r in range(world - 1)]
    if rank == 0:
        print("DP FAILURE DETECTION", "OK" if all(votes) and passed else "FAILED", flush=True)


if __name__ == "__main__":
    main()
