"""Benchmark of the Gaussian-splatting training step (forward + L1/SSIM loss + backward + fused Adam).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--batch B]

Workload `train_1m` (default at every N): 1,000,000 Gaussians, SH degree 3, one 1296x840 pinhole camera
per GPU per step out of 200 hemisphere poses, loss 0.8 L1 + 0.2 (1 - SSIM), Adam with the per-group rates
of the reference's MCMC strategy. N > 1 is weak scaling by camera: each rank renders its own camera against
replicated Gaussians, the gradients are summed and Adam applied by --dp-mode (default: one fused kernel over
NVLink peer memory that does reduce-scatter + Adam + all-gather). `--batch B` fixes the camera batch of one
optimizer step (each rank renders B / N cameras and accumulates). `--workload dp_3m` is the 3,000,000
Gaussian / 1600x1064 data-parallel configuration, `mcmc_3m` the densification step, `wide_4k` /
`wide_fisheye` the forward-only renders, `ewa_1m` the default (non --gut) rasterizer on the train_1m scene.
Synthetic seeded inputs stand in for the Mip-NeRF-360 shapes.

Rank 0 prints ONE JSON line. `value` is (camera-)steps/s with every input resident in HBM, from one CUDA-event
bracket around the K timed steps (max over ranks); `step_ms` holds the median / p10 / p90 of the per-step event
intervals. `e2e` is the same step driven from pinned host memory (target image + camera copied in, loss read back
each step).

`--impl reference` times the REFERENCE'S OWN CUDA implementation of the same step on the same GPU: the reference's
unmodified kernels, autograd nodes and FusedAdam, built by oracle/ref_build.py into oracle/_ref (never this
repository's library). Under torchrun only rank 0 runs it, on one GPU, and reports that one GPU's rate (the reference
has no multi-GPU path). Where that build is absent the arm falls back to the CPU oracle on the host cores and says so.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

LRS = [1.6e-4, 2.5e-3, 1.25e-4, 5e-3, 1e-3, 5e-2]  # means, sh0, shN, scaling, rotation, opacity
METRIC = "train steps/s (fwd+loss+bwd+Adam)"
# Profiler counters of ONE raster_bwd_kernel launch on train_1m (ncu, --clock-control none): DRAM bytes read + written,
# share of issue slots used, share of issued warp instructions on the FMA pipe relative to the FP32 peak rate. They are
# reported next to the event-timed figures because a kernel's traffic and pipe utilisation cannot be read outside a profiler.
NCU_RASTER_BWD = {"dram_bytes": 180.7e6, "issue_slots_active": 0.82, "fma_pipe_of_fp32_peak": 0.42, "shared_pipe": 0.77,
                  # 666e6 warp instructions on the FMA pipe x 32 lanes x 2 flop over the 4.25e8 pairs of the captured launch
                  "executed_flop_per_pair": 100.3}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------------- CPU arm
_SCENE_CACHE = {}


def cpu_step_sample(workload: str, n_rows: int = 6, step: int = 0):
    """One training step of the CPU oracle on a bounded sample: projection, SH, tile lists, loss, SH
    backward and Adam in full; rasterizer forward / backward on `n_rows` full rows of tiles spread evenly
    over the image height, their time scaled to the whole image. Returns (seconds for a full step,
    description, threads)."""
    from oracle import oracle as orc
    orc.use_all_cores()
    synth = importlib.import_module("lichtfeld-studio_b200").synth
    cfg = synth.CONFIGS[workload]
    W, H, deg, n = cfg["W"], cfg["H"], cfg["sh_degree"], cfg["n"]
    if workload not in _SCENE_CACHE:
        _SCENE_CACHE[workload] = synth.make_gaussians(n, 0, cfg["layout"], deg)
    P = {k: v.copy() for k, v in _SCENE_CACHE[workload].items()}
    poses, K = synth.make_cameras(cfg)
    vm = poses[synth.pose_index(step, cfg["n_poses"])]
    bg = np.zeros(3, np.float32)
    tw, th = (W + 15) // 16, (H + 15) // 16
    rows = sorted({int((k + 1) * th / (n_rows + 1)) for k in range(n_rows)})
    t_start = time.perf_counter()
    fwd = orc.render_fwd(P, vm, K, W, H, deg, background=bg, tile_range=(0, 0))  # everything but the rasterizer
    t_front = time.perf_counter() - t_start
    a = [P["means"], fwd["quats"], fwd["scales"], fwd["colors"], fwd["opac"]]
    t_rf = 0.0
    for r in rows:
        t0 = time.perf_counter()
        ren, alp, last, _ = orc.rasterize_fwd(*a, bg, W, H, 16, vm, K, fwd["tile_offsets"], fwd["flatten_ids"],
                                              tile_range=(r * tw, (r + 1) * tw))
        t_rf += time.perf_counter() - t0
        y0, y1 = r * 16, min(H, (r + 1) * 16)
        fwd["render"][y0:y1], fwd["alpha"][y0:y1], fwd["last_ids"][y0:y1] = ren[y0:y1], alp[y0:y1], last[y0:y1]
    target = np.ascontiguousarray(np.clip(fwd["render"], 0, 1).transpose(2, 0, 1)) * np.float32(0.9)
    t0 = time.perf_counter()
    loss, g, _, _ = orc.photometric_loss(fwd["render"], target, 0.2)
    t_loss = time.perf_counter() - t0
    t_rb = 0.0
    for r in rows:
        t0 = time.perf_counter()
        orc.rasterize_bwd(*a, bg, W, H, 16, vm, K, fwd["tile_offsets"], fwd["flatten_ids"], fwd["alpha"], fwd["last_ids"], g,
                          np.zeros((H, W, 1), np.float32), tile_range=(r * tw, (r + 1) * tw))
        t_rb += time.perf_counter() - t0
    t0 = time.perf_counter()
    bwd = orc.render_bwd(P, fwd, vm, K, W, H, deg, g, background=bg, tile_range=(0, 0))  # SH + activation backward
    for gi, name in enumerate(("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")):
        p = P[name].reshape(-1)
        orc.adam_step(p, np.zeros_like(p), np.zeros_like(p), bwd[name].reshape(-1), LRS[gi], 0.9, 0.999, 1e-15, 1)
    t_back = time.perf_counter() - t0
    scale = th / len(rows)
    full = t_front + t_loss + t_back + (t_rf + t_rb) * scale
    desc = (f"{workload}: projection+SH+tile lists {t_front:.2f}s, loss {t_loss:.2f}s, SH/activation bwd+Adam {t_back:.2f}s in full; "
            f"rasterizer fwd {t_rf:.2f}s + bwd {t_rb:.2f}s on tile rows {rows} of {th}, scaled by {scale:.1f}; "
            f"sample wall time {time.perf_counter() - t_start:.1f}s")
    return full, desc, orc.num_threads()


def run_reference_cpu(args, why: str):
    """Fallback of the reference arm where the reference's CUDA build is absent: the CPU oracle port on the host cores."""
    workload = args.workload or "train_1m"
    times = []
    for s in range(args.warmup + args.steps):
        full, desc, threads = cpu_step_sample(workload, step=s)
        if s >= args.warmup:
            times.append(full)
    sec = float(np.mean(times))
    val = 1.0 / sec
    out = {"impl": "reference", "reference_class": "CPU oracle port (" + why + ")", "metric": METRIC, "value": val, "unit": "steps/s",
           "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": workload},
           "cpu_baseline": {"value": val, "unit": "steps/s", "cores": threads, "kind": "port", "sample": desc},
           "e2e": {"value": val, "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(_finite(out)), flush=True)


def _reference_line(args, workload, metric, unit, value, ms, higher, config, e2e, sample, extra=None):
    out = {"impl": "reference", "reference_class": "the reference's own CUDA sources (unmodified), built into oracle/_ref",
           "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "gpus_used": 1, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": ms, "higher_is_better": higher, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": config,
           "cpu_baseline": {"value": value, "unit": unit, "cores": 1, "kind": "reference",
                            "sample": sample + " (runs on the GPU: the reference has no CPU implementation of this path; one host thread drives it)"},
           "e2e": e2e}
    if extra:
        out.update(extra)
    print(json.dumps(_finite(out)), flush=True)


def run_reference(args):
    """The reference arm: the reference's own CUDA step (oracle/_ref) on ONE GPU, same workload, same K and W, same per-step
    host-to-device upload and loss read-back in its end-to-end figure. Rank 0 only; one GPU's rate at every --gpus."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    workload = args.workload or "train_1m"
    from oracle import reference as R
    import torch
    if not R.available():
        return run_reference_cpu(args, "oracle/_ref is not built here")
    if not torch.cuda.is_available():
        return run_reference_cpu(args, "no GPU")
    synth = importlib.import_module("lichtfeld-studio_b200").synth
    cfg = synth.CONFIGS["train_1m" if workload == "ewa_1m" else workload]
    if workload == "ewa_1m":
        print(json.dumps({"impl": "reference", "unavailable": "the reference's default (EWA) rasterizer fails on the host from about 200,000 Gaussians "
                          "in this toolchain (garbage bucket count -> `numel: integer multiplication overflow`); by reading, its tile count and "
                          "tile emission evaluate the same float test in two kernels under --use_fast_math, which can disagree and write out "
                          "of range, so it is not run at this size"}), flush=True)
        return
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    W, H, deg, n = cfg["W"], cfg["H"], cfg["sh_degree"], cfg["n"]
    T = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    P = synth.make_gaussians(n, 0, cfg["layout"], deg)
    if workload == "mcmc_3m":
        P["opacity_raw"][np.arange(n) % 20 == 7] = -6.0
        cap = int(np.float32(1.05) * np.float32(n)) + 64
        times, counts = [], None
        for rep in range(args.warmup + args.steps):
            m = R.McmcReference(P, 0.005, cap, dev)
            torch.manual_seed(1234)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            nd = m.relocate_gs()
            na = m.add_new_gs()
            m.inject_noise(1.6e-4 * 5e5)
            e1.record(); torch.cuda.synchronize()
            if rep >= args.warmup:
                times.append(e0.elapsed_time(e1))
            counts = (nd, na)
            del m
        ms = float(np.mean(times))
        return _reference_line(args, workload, "MCMC refine step (relocate + add + noise) ms", "ms", ms, ms, False,
                               {"workload": workload, "gaussians": n, "relocated": counts[0], "added": counts[1]},
                               {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 8},
                               "MCMC::relocate_gs / add_new_gs / inject_noise with the reference's ATen calls and kernels")
    poses, Kmat = synth.make_cameras(cfg)
    Kt, bg = T(Kmat[None]), torch.zeros(3, device=dev)
    if workload in ("wide_4k", "wide_fisheye"):
        t = R.make_trainer(P, LRS, deg, device=dev)
        vms = [T(p[None]) for p in poses]
        for vm in vms[: max(3, args.warmup)]:
            t.render_no_grad(True, vm, Kt, W, H, bg, cfg["model"])
        torch.cuda.synchronize()
        reps = max(1, args.steps // len(vms)) if args.steps > len(vms) else 1
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            for vm in vms:
                t.render_no_grad(True, vm, Kt, W, H, bg, cfg["model"])
        e1.record(); torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (reps * len(vms))
        val = W * H / (ms * 1e-3) / 1e9
        return _reference_line(args, workload, "forward render Gpix/s", "Gpix/s", val, ms, True,
                               {"workload": workload, "gaussians": n, "image": [W, H], "poses": len(vms)},
                               {"value": val, "unit": "Gpix/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                               "rasterize() of the reference (projection, SH, tile lists, blending) over the seeded poses")
    # training step (train_1m / dp_3m scenes): render, loss, backward, loss.item(), FusedAdam step, one camera per step
    t = R.make_trainer(P, LRS, deg, device=dev)
    held = R.make_trainer(synth.make_gaussians(n, 1000, cfg["layout"], deg), LRS, deg, device=dev)
    total = args.warmup + args.steps
    n_e2e = min(args.steps, 50)
    vms, targets = [], []
    for s in range(max(total, n_e2e)):
        vm = T(poses[synth.pose_index(s, cfg["n_poses"])][None])
        vms.append(vm)
        targets.append(held.render_no_grad(True, vm, Kt, W, H, bg, 0).image.contiguous())
    del held
    torch.cuda.empty_cache()
    it0 = 2000   # past the iteration up to which the reference skips the shN group
    for s in range(args.warmup):
        t.train_step(it0 + s, True, vms[s], Kt, W, H, bg, targets[s], 0.2, 0.0, 0.0)
    torch.cuda.synchronize()
    sampler = ClockSampler(dev.index or 0); sampler.start()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    evs[0].record()
    for k, s in enumerate(range(args.warmup, total)):
        t.train_step(it0 + s, True, vms[s], Kt, W, H, bg, targets[s], 0.2, 0.0, 0.0)
        evs[k + 1].record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = evs[0].elapsed_time(evs[-1]) / args.steps
    per = np.array([evs[k].elapsed_time(evs[k + 1]) for k in range(args.steps)])
    # end to end: target image and camera from pinned host memory every step, loss read back every step
    th = [x.cpu().pin_memory() for x in targets[:n_e2e]]
    vh = [x.cpu().pin_memory() for x in vms[:n_e2e]]
    tgt, vmb = torch.empty_like(targets[0]), torch.empty_like(vms[0])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(n_e2e):
        tgt.copy_(th[s], non_blocking=True)
        vmb.copy_(vh[s], non_blocking=True)
        t.train_step(it0 + total + s, True, vmb, Kt, W, H, bg, tgt, 0.2, 0.0, 0.0)
    e1.record(); torch.cuda.synchronize()
    ms_e2e = e0.elapsed_time(e1) / n_e2e
    _reference_line(args, workload, METRIC, "steps/s", 1e3 / ms, ms, True,
                    {"workload": workload, "gaussians": n, "image": [W, H], "sh_degree": deg, "cameras_per_step": 1,
                     "path": "rasterize() -> FusedRasterizationWithSHFunction -> gsplat::rasterize_from_world_with_sh_fwd/_bwd, fused_ssim, FusedAdam"},
                    {"value": 1e3 / ms_e2e, "unit": "steps/s", "h2d_bytes_per_step": th[0].numel() * 4 + 64, "d2h_bytes_per_step": 4, "steps": n_e2e},
                    "Trainer::train_step's render + photometric loss + backward + loss.item() + MCMC::step (FusedAdam, zero_grad, scheduler)",
                    {"clocks": clocks, "step_ms": {"median": float(np.median(per)), "p10": float(np.percentile(per, 10)),
                                                   "p90": float(np.percentile(per, 90))}})


# --------------------------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))
    pkg = importlib.import_module("lichtfeld-studio_b200")
    synth, tr, capi = pkg.synth, pkg.trainer, pkg._capi
    capi.lib()  # fails loudly if the CUDA library is missing

    workload = args.workload or "train_1m"
    cfg = synth.CONFIGS[workload]
    W, H, deg, n = cfg["W"], cfg["H"], cfg["sh_degree"], cfg["n"]
    K_sh = (deg + 1) ** 2
    P = synth.make_gaussians(n, 0, cfg["layout"], deg)
    P_target = synth.make_gaussians(n, 1000, cfg["layout"], deg)
    poses, Kmat = synth.make_cameras(cfg)
    total_steps = args.warmup + args.steps

    # cameras of one optimizer step: `world` by default (one per rank), or a fixed --batch spread over the ranks
    batch = args.batch or world
    if batch % world:
        raise SystemExit(f"--batch {batch} must be a multiple of the number of GPUs ({world})")
    cams_per_rank = batch // world
    dp = pkg.dp
    cap = (n + 31) // 32 * 32
    peer = None
    if world > 1 and args.dp_mode == "fused_p2p":
        numel = cap * tr.SplatData(1, K_sh, "cpu").row_floats
        pf, gf, peer = dp.symmetric_flat_buffers(numel, dev)
        model, grads = tr.SplatData(n, K_sh, dev, cap, flat=pf).load(P), tr.SplatData(n, K_sh, dev, cap, flat=gf)
    else:
        model, grads = tr.SplatData(n, K_sh, dev, cap).load(P), tr.SplatData(n, K_sh, dev, cap)
    held_out = tr.SplatData(n, K_sh, dev).load(P_target)
    if world == 1:
        m, v = model.like(), model.like()
    else:
        exchange = dp.GradExchange(model, grads, LRS, mode=args.dp_mode, peer_ptrs=peer, ordering=args.dp_ordering, multicast=args.dp_multicast)
    rast = tr.Rasterizer(model, W, H, deg, isect_capacity=max(12 * n, 1 << 22))
    rast_t = tr.Rasterizer(held_out, W, H, deg, isect_capacity=max(12 * n, 1 << 22))
    lossfn = tr.PhotometricLoss(W, H, dev)
    bg = torch.zeros(3, device=dev)
    Kt = torch.from_numpy(Kmat).to(dev)

    # the camera of (step, rank) and its target, rendered from the held-out Gaussians with this library
    def pose_of(step, c=0):
        return poses[synth.pose_index((step * cams_per_rank + c) * world + rank, cfg["n_poses"])]

    n_e2e = min(args.steps, 50)
    # per step: [cams_per_rank, 3, H, W] targets and [cams_per_rank, 4, 4] poses
    targets_dev, targets_host, vms_dev, vms_host = [], [], [], []
    n_distinct = max(total_steps, n_e2e) if cams_per_rank == 1 else min(max(total_steps, n_e2e), 8)   # bounded memory for batches
    for s in range(n_distinct):
        tg, vm_l = [], []
        for c in range(cams_per_rank):
            vm = torch.from_numpy(pose_of(s, c)).to(dev)
            out = rast_t.forward(tr.Camera(vm, Kt, W, H), bg)
            tg.append(out.image.clamp(0, 1).permute(2, 0, 1).contiguous())
            vm_l.append(vm)
        targets_dev.append(torch.stack(tg))
        vms_dev.append(torch.stack(vm_l))
        if s < n_e2e:
            targets_host.append(targets_dev[-1].cpu().pin_memory())
            vms_host.append(vms_dev[-1].cpu().pin_memory())
    del rast_t, held_out
    torch.cuda.synchronize()
    pick = lambda lst, s: lst[s % len(lst)]

    flat_len = model.flat.numel()
    shard = (flat_len + world - 1) // world
    pad = shard * world - flat_len

    def exchange_and_adam(step_count):
        if world == 1:
            tr.adam_step_splats(model, m, v, grads, LRS, step_count)
            return
        # gradients summed over cameras, mean over the batch folded into Adam's gradient read
        exchange.step(2000 + step_count)

    # Optional (--overlap), single GPU: the optimizer is split. The geometry groups (means, scales, rotations, opacities: a quarter of the
    # bytes) are updated on the main stream, the colour groups (sh0, shN) on a side stream, and the next step's
    # projection and tile lists (which do not read the colour groups) start right after the geometry update; the SH
    # colours are evaluated once the side stream is done. Every kernel of every step is inside the timed region.
    side = torch.cuda.Stream(device=dev)
    ev_bwd, ev_color = torch.cuda.Event(), torch.cuda.Event()
    ev_projected = torch.cuda.Event()
    ev_projected.record()          # creates the handle that forward_lists(projected_event=...) records
    overlap = world == 1 and args.overlap
    state = {"color_pending": False}

    dp_split = world > 1 and args.dp_mode == "fused_p2p" and not args.no_dp_split
    # the rank-1 form of the shN gradient exists for ONE camera per rank; a sum over cameras is materialised
    rank1_sh = world == 1 and cams_per_rank == 1 and not overlap and not args.materialize_sh_grad
    dp_rank1 = dp_split and cams_per_rank == 1 and not args.materialize_sh_grad
    inv_batch = 1.0 / batch

    def step_batch(s, targets, vms):
        """One optimizer step over cams_per_rank cameras on this rank: gradients accumulate, then exchange + Adam with the
        mean over the whole batch folded into Adam's gradient read."""
        last = None
        for c in range(cams_per_rank):
            out = rast.forward(tr.Camera(vms[c], Kt, W, H), bg)
            last, v_render = lossfn(out.image, targets[c])
            rast.backward(v_render, grads, bg, accumulate=(c > 0))
        if world == 1:
            tr.adam_step_splats(model, m, v, grads, LRS, s + 1, grad_scale=inv_batch)
        else:
            exchange.step(2000 + s + 1, grad_scale=inv_batch)   # all groups in one exchange after the last backward
        return last

    def step(s, target, vm):
        if cams_per_rank > 1:
            return step_batch(s, target, vm)
        target, vm = target[0], vm[0]
        cam = tr.Camera(vm, Kt, W, H)
        if dp_split:
            # N > 1: the geometry groups are exchanged first; the colour groups (three quarters of the bytes) cross
            # NVLink on a side stream while this step's projection and tile lists are built
            if args.dp_color_after_projection:
                # the colour exchange of the previous step starts when this projection kernel is done (event recorded inside
                # forward_lists) and runs next to the sorting kernels
                rast.forward_lists(cam, projected_event=ev_projected)
                exchange.launch_color(after=ev_projected)
            else:
                rast.forward_lists(cam)
            exchange.wait_color()
            out = rast.forward_shade(bg)
            loss, v_render = lossfn(out.image, target)
            # one camera per rank: the shN gradient crosses NVLink as its two rank-1 factors (24 bytes per Gaussian)
            rast.backward(v_render, grads, bg, sh_factors=dp_rank1)
            exchange.step_split(2000 + s + 1, side, rank1_sh=dp_rank1, sh_degree=deg, defer_color=args.dp_color_after_projection)
            return loss
        if not overlap:
            out = rast.forward(cam, bg)
        else:
            main = torch.cuda.current_stream()
            rast.forward_lists(cam)
            if state["color_pending"]:
                main.wait_event(ev_color)      # the colour groups of the previous step are up to date
            out = rast.forward_shade(bg)
        loss, v_render = lossfn(out.image, target)
        if rank1_sh and args.one_call_optimizer:
            # one camera per step on one GPU: backward and optimizer in one call, no gradient tensor at all
            rast.backward_adam(v_render, m, v, LRS, s + 1, bg)
            return loss
        if rank1_sh:
            # the same with the reference's two calls: the shN gradient (three quarters of the gradient bytes) is never
            # written; the optimizer rebuilds its rows from the sh0 gradient and the view direction
            rast.backward(v_render, grads, bg, write_shN=False)
            rast.adam_step_rank1_sh(m, v, grads, LRS, s + 1)
            return loss
        rast.backward(v_render, grads, bg)
        if not overlap:
            exchange_and_adam(s + 1)
            return loss
        ev_bwd.record(main)
        tr.adam_step_groups(model, m, v, grads, LRS, s + 1, tr.GEOMETRY_GROUPS)
        with torch.cuda.stream(side):
            side.wait_event(ev_bwd)
            tr.adam_step_groups(model, m, v, grads, LRS, s + 1, tr.COLOR_GROUPS, ctas_per_sm=args.overlap_ctas)
            ev_color.record(side)
        state["color_pending"] = True
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing -------------------------------------------------------------
    for s in range(args.warmup):
        step(s, pick(targets_dev, s), pick(vms_dev, s))
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # one bracket around the K timed steps (the reported figure) and an event after every step (the series)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    evs[0].record()
    for k, s in enumerate(range(args.warmup, total_steps)):
        step(s, pick(targets_dev, s), pick(vms_dev, s))
        evs[k + 1].record()
    barrier()
    ms_total = evs[0].elapsed_time(evs[-1])
    per_step = torch.tensor([evs[k].elapsed_time(evs[k + 1]) for k in range(args.steps)], device=dev, dtype=torch.float64)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
        dist.all_reduce(per_step, op=dist.ReduceOp.MAX)      # a step takes as long as its slowest rank
    ms_per_step = ms_total / args.steps
    per_step = per_step.cpu().numpy()
    step_ms = {"median": float(np.median(per_step)), "p10": float(np.percentile(per_step, 10)), "p90": float(np.percentile(per_step, 90)),
               "min": float(per_step.min()), "max": float(per_step.max())}
    status = rast.status.cpu().numpy()

    # ---- end to end from pinned host memory ---------------------------------------------------
    # Every step's inputs (target image, camera) come from pinned host memory and every step's loss is read back to
    # the host, all inside the timed region. The copies run on a second stream into double buffers, so the input of
    # step s+1 crosses PCIe while step s computes, and the loss of step s is read on the host one step later
    # (pinned buffer + event) instead of stalling the launch queue.
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream()
    tgt_bufs = [torch.empty_like(targets_dev[0]) for _ in range(2)]
    vm_bufs = [torch.empty_like(vms_dev[0]) for _ in range(2)]
    loss_pinned = [torch.empty(4, dtype=torch.float32).pin_memory() for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    loss_done = [torch.cuda.Event() for _ in range(2)]
    losses_read = []

    def upload(s):
        k = s % 2
        with torch.cuda.stream(copy_stream):
            if s >= 2:
                copy_stream.wait_event(consumed[k])   # step s-2 has finished with this buffer
            tgt_bufs[k].copy_(pick(targets_host, s), non_blocking=True)
            vm_bufs[k].copy_(pick(vms_host, s), non_blocking=True)
            ready[k].record(copy_stream)

    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    upload(0)
    for s in range(n_e2e):
        k = s % 2
        if s + 1 < n_e2e:
            upload(s + 1)
        main_stream.wait_event(ready[k])
        loss = step(total_steps + s, tgt_bufs[k], vm_bufs[k])
        consumed[k].record(main_stream)
        loss_pinned[k].copy_(loss, non_blocking=True)   # device -> host read of the step's result
        loss_done[k].record(main_stream)
        if s >= 1:
            loss_done[1 - k].synchronize()
            losses_read.append(float(loss_pinned[1 - k][0]))
    loss_done[(n_e2e - 1) % 2].synchronize()
    losses_read.append(float(loss_pinned[(n_e2e - 1) % 2][0]))
    loss_host = loss_pinned[0]
    assert len(losses_read) == n_e2e and all(np.isfinite(losses_read))
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item())
    ms_e2e /= n_e2e
    h2d = targets_host[0].numel() * 4 + vms_host[0].numel() * 4
    d2h = loss_host.numel() * 4

    # ---- per-kernel times (CUDA events inside the library), pair counts, rooflines --------------------
    kernels, roofline, extra = {}, None, {}
    n_prof = 3
    capi.profile_enable(True)          # every rank records: the per-rank spread of the backward is part of the report
    if world > 1:
        exchange.timing = []
    for s in range(n_prof):
        step(s, pick(targets_dev, s), pick(vms_dev, s))
    barrier()
    recs = capi.profile_collect()
    capi.profile_enable(False)
    for name, msv in recs:
        kernels.setdefault(name, []).append(msv)
    rendezvous = {}
    if world > 1:
        for name, msv in exchange.collect_timing():
            rendezvous.setdefault(name, []).append(msv)
        exchange.timing = None
    per_rank = None
    if world > 1:
        names = ("raster_bwd", "raster_fwd", "project_pack", "dp_exchange_main", "dp_exchange_side", "dp_exchange_side_sh_rank1")
        rnames = ("rendezvous_gradients_written", "rendezvous_geometry_done", "rendezvous_exchange_done", "rendezvous_color_done_side")
        mine = torch.tensor([float(np.sum(kernels.get(k, [0.0])) / n_prof) for k in names] +
                            [float(np.sum(rendezvous.get(k, [0.0])) / n_prof) for k in rnames], device=dev, dtype=torch.float64)
        allr = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        allr = torch.stack(allr).cpu().numpy()
        per_rank = {k: {"min": float(allr[:, i].min()), "max": float(allr[:, i].max()), "by_rank": [round(float(x), 4) for x in allr[:, i]]}
                    for i, k in enumerate(names + rnames) if allr[:, i].max() > 0}
    # every rank must hold the same parameters after the timed steps: integer checksum of the raw bits
    dp_check = None
    if world > 1:
        bits = model.flat.view(torch.int32).to(torch.int64)
        chk = torch.stack([bits.sum(), (bits * (torch.arange(bits.numel(), device=dev) % 1021 + 1)).sum()])
        allc = [torch.empty_like(chk) for _ in range(world)]
        dist.all_gather(allc, chk)
        same_params = all(bool(torch.equal(allc[0], c)) for c in allc)
        exchange.raise_if_failed()      # no bounded wait of the timed steps ran out
        small = dp_self_check(pkg, dev, rank, world, args.dp_mode, dp_split, dp_rank1, args.dp_ordering, args.dp_multicast, args.dp_color_after_projection)
        dp_check = {"ok": bool(same_params and small["ok"]), "bench_parameters_identical_on_all_ranks": bool(same_params), **small}
    if rank == 0:
        # launches inside one call that are not individually bracketed: scan = 3 kernels, sort = 3 per pass
        per_step_kernels = {"exclusive_scan": 3, "radix_sort_depth": 12, "radix_sort_tile": 6}
        gpu_launches_step = sum(per_step_kernels.get(k, 1) * len(vs) / n_prof for k, vs in kernels.items()) + 4
        st = rast.state()
        last, offs = st["last_ids"].long(), st["tile_offsets"].long()
        tw = (W + 15) // 16
        ys, xs = torch.meshgrid(torch.arange(H, device=dev), torch.arange(W, device=dev), indexing="ij")
        tile = (ys // 16) * tw + xs // 16
        start, end = offs[tile], offs[tile + 1]
        q_b = int(torch.clamp(torch.minimum(last, end - 1) - start + 1, min=0).sum().item())
        q_list = int((end - start).sum().item())
        sm_clock = (clocks or {}).get("sm_mhz") or 1965.0
        n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
        fp32_peak = n_sm * 128 * 2 * sm_clock * 1e6 / 1e12
        calls = cams_per_rank * n_prof
        t_bwd = float(np.sum(kernels.get("raster_bwd", [float("nan")])) / calls)
        t_fwd = float(np.sum(kernels.get("raster_fwd", [float("nan")])) / calls)
        # per step: the split optimizer launches "adam" twice (geometry groups, colour groups); the roofline figure uses
        # the sum of both (each is timed alone on its stream, but they may overlap other kernels)
        t_adam = float(np.sum(kernels["adam"]) / n_prof) if "adam" in kernels else float("nan")
        hbm_peak, peak_kind = load_peaks()
        ach = 370.0 * q_b / (t_bwd * 1e-3) / 1e12
        # DRAM bytes and pipe utilisation of one raster_bwd launch come from an ncu capture of this kernel on this workload
        # (they cannot be read outside a profiler); other workloads report null
        ncu = NCU_RASTER_BWD if workload == "train_1m" else None
        roofline = {"kernel": "raster_bwd_kernel", "bound": "fp32", "achieved": ach, "peak": fp32_peak, "unit": "TFLOP/s",
                    "frac": ach / fp32_peak, "traffic": ncu["dram_bytes"] if ncu else None,
                    "pairs_per_s": q_b / (t_bwd * 1e-3),
                    # what the FP32 pipe really executes: flops per pair counted by the profiler x the pairs of THIS launch / its
                    # event-timed duration, against the same peak; the kernel's actual limit is the issue rate (utilisation_ncu)
                    "achieved_executed": (ncu["executed_flop_per_pair"] * q_b / (t_bwd * 1e-3) / 1e12) if ncu else None,
                    "frac_executed": (ncu["executed_flop_per_pair"] * q_b / (t_bwd * 1e-3) / 1e12 / fp32_peak) if ncu else None,
                    "utilisation_ncu": ncu,
                    "note": f"achieved / frac follow the fixed accounting 370 flop x {q_b} (pixel,Gaussian) pairs / {t_bwd:.3f} ms, i.e. the REFERENCE's "
                            f"arithmetic per pair; this kernel executes fewer flops per pair (per-Gaussian work is hoisted out of the pair loop), so "
                            f"frac can exceed 1 and is NOT pipe utilisation. Utilisation is frac_executed (executed FP32 flops of this launch / peak) and "
                            f"utilisation_ncu (issue slots, FMA pipe, shared-memory pipe) from the profiler capture. peak = {n_sm} SM x 128 lanes x 2 x {sm_clock:.0f} MHz sampled under load (no tensor cores on this path)"}
        adam_bytes = 28.0 * 59 * n if K_sh == 16 else 28.0 * model.row_floats * n
        adam_kernel = "adam_groups_kernel"
        adam_note = f"28 B x {model.row_floats} floats x {n} Gaussians"
        if "adam_sh_rank1" in kernels:
            # the shN update without a gradient tensor: parameters and both moments read and written once (24 B per
            # element), 12 B of means and 12 B of sh0 gradient per Gaussian
            rest = model.row_floats - 14
            t_adam = float(np.sum(kernels["adam_sh_rank1"]) / n_prof)
            adam_bytes = (24.0 * rest + 24.0) * n
            adam_kernel = "adam_sh_rank1_kernel"
            adam_note = f"(24 B x {rest} shN floats + 24 B) x {n} Gaussians"
        adam_gbs = adam_bytes / (t_adam * 1e-3) / 1e9 if np.isfinite(t_adam) else None   # N > 1: Adam runs inside the exchange
        list_keys = ("radix_sort_depth", "exclusive_scan", "emit_instances", "radix_sort_tile", "tile_offsets", "tile_order")
        t_lists = sum(float(np.sum(kernels[k])) / calls for k in list_keys if k in kernels)
        V, I = float(status[2]), float(status[1])
        tiles = ((W + 15) // 16) * ((H + 15) // 16)
        list_bytes = 20 * V + 36 * I + 4 * tiles
        t_pp = float(np.sum(kernels.get("project_pack", [float("nan")])) / calls)
        pp_bytes = 52.0 * n + 216.0 * V
        extra = {"roofline_adam": {"kernel": adam_kernel, "bound": "hbm", "achieved": adam_gbs,
                                   "peak": hbm_peak, "unit": "GB/s", "frac": adam_gbs / hbm_peak if adam_gbs else None,
                                   "traffic": None, "note": f"{adam_note}, of {peak_kind}"},
                 "roofline_raster_fwd": {"kernel": "raster_fwd_kernel", "bound": "fp32",
                                         "achieved": 70.0 * q_list / (t_fwd * 1e-3) / 1e12, "peak": fp32_peak, "unit": "TFLOP/s",
                                         "frac": 70.0 * q_list / (t_fwd * 1e-3) / 1e12 / fp32_peak,
                                         "note": f"70 flop x {q_list} list entries x pixels (upper bound of pairs visited); same caveat as raster_bwd"},
                 "roofline_tile_lists": {"kernel": "depth sort + scan + emit + tile sort + offsets + order", "bound": "hbm",
                                         "achieved": list_bytes / (t_lists * 1e-3) / 1e9 if t_lists else None, "peak": hbm_peak, "unit": "GB/s",
                                         "frac": list_bytes / (t_lists * 1e-3) / 1e9 / hbm_peak if t_lists else None, "ms": t_lists,
                                         "note": f"20 V + 36 I + 4 tiles bytes, of {peak_kind}"},
                 "roofline_project_pack": {"kernel": "project_pack_kernel", "bound": "hbm", "achieved": pp_bytes / (t_pp * 1e-3) / 1e9,
                                           "peak": hbm_peak, "unit": "GB/s", "frac": pp_bytes / (t_pp * 1e-3) / 1e9 / hbm_peak,
                                           "note": f"52 N + 216 V bytes, of {peak_kind}"},
                 "kernel_ms": {k: float(np.sum(vs) / n_prof) for k, vs in kernels.items()},
                 "n_isects": int(status[1]), "n_visible": int(status[2]), "pairs_bwd": q_b, "pairs_list": q_list,
                 "gpix_per_s_fwd": W * H / ((t_pp + t_lists + t_fwd) * 1e-3) / 1e9}
        if world > 1:
            extra["rendezvous_ms"] = {k: float(np.sum(vs) / n_prof) for k, vs in rendezvous.items()}
            extra["per_rank_kernel_ms"] = per_rank
            extra["dp_check"] = dp_check

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu:
            full, desc, threads = cpu_step_sample(workload)
            cpu = {"value": 1.0 / full, "unit": "steps/s", "cores": threads, "kind": "port", "sample": desc}
        unit = "steps/s" if batch == 1 else "camera-steps/s"
        out = {"metric": METRIC, "value": batch * 1e3 / ms_per_step, "unit": unit, "n_gpus": world, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": ms_per_step, "step_ms": step_ms, "optimizer_steps_per_s": 1e3 / ms_per_step,
               "higher_is_better": True, "scaling": "weak" if not args.batch else "strong",
               "vs_baseline": None, "dtype": "f32", "data": "synthetic",
               "config": {"workload": workload, "gaussians": n, "image": [W, H], "sh_degree": deg, "cameras_per_step": batch,
                          "cameras_per_rank": cams_per_rank,
                          "optimizer_overlap": bool(overlap), "optimizer": ("inside lfs_render_backward_adam" if (rank1_sh and args.one_call_optimizer) else "separate call"),
                          "shN_gradient": "rank-1, rebuilt inside Adam" if rank1_sh else ("rank-1 factors over NVLink" if dp_rank1 else "materialised"),
                          "parallelism": (f"dp{world}:{args.dp_mode}" + ("+split" if dp_split and cams_per_rank == 1 else "") + (f"+{exchange.ordering}" + ("+multimem" if exchange.mc_params else "") + ("+colour-after-projection" if dp_split and args.dp_color_after_projection else "") if args.dp_mode == "fused_p2p" else "")) if world > 1 else "single", "l2": "inputs larger than L2 "
                          f"({model.flat.numel() * 4 * 4 / 1e6:.0f} MB of parameters, moments and gradients streamed per step)"},
               "clocks": clocks, "e2e": {"value": batch * 1e3 / ms_e2e, "unit": unit, "h2d_bytes_per_step": h2d,
                                         "d2h_bytes_per_step": d2h, "steps": n_e2e},
               "gpu_launches": int(round(gpu_launches_step * args.steps)), "roofline": roofline, "cpu_baseline": cpu,
               "gpix_per_s_step": batch * W * H / (ms_per_step * 1e-3) / 1e9}
        out.update(extra)
        print(json.dumps(_finite(out)), flush=True)
    if world > 1:
        dist.destroy_process_group()


def dp_self_check(pkg, dev, rank, world, mode, split, rank1, ordering=None, multicast=None, after_projection=False):
    """Cross-rank correctness of the exchange the benchmark just timed, on a small scene: three data-parallel steps with
    the same mode flags must leave bit-identical parameters on every rank, equal (to gradient-summation rounding) to what
    ONE process gets by rendering every camera itself, accumulating the gradients and applying Adam to their mean."""
    import torch
    import torch.distributed as dist
    synth, tr, dp = pkg.synth, pkg.trainer, pkg.dp
    n, W, H, deg, steps = 30000, 320, 208, 3, 3
    K = (deg + 1) ** 2
    P = synth.make_gaussians(n, 0, "clusters", deg)
    poses = synth.hemisphere_poses(16, 5.0)
    Kmat = torch.from_numpy(synth.intrinsics(280.0, 280.0, W / 2, H / 2)).to(dev)
    bg = torch.zeros(3, device=dev)
    targets = [torch.rand(3, H, W, generator=torch.Generator().manual_seed(s)).to(dev) for s in range(steps * world)]
    cam = lambda i: tr.Camera(torch.from_numpy(poses[i % 16]).to(dev), Kmat, W, H)
    cap = (n + 31) // 32 * 32
    # one process, all cameras
    model, grads = tr.SplatData(n, K, dev, cap).load(P), tr.SplatData(n, K, dev, cap)
    rast, lossfn = tr.Rasterizer(model, W, H, deg), tr.PhotometricLoss(W, H, dev)
    m, v = model.like(), model.like()
    for s in range(steps):
        for r in range(world):
            out = rast.forward(cam(s * world + r), bg)
            _, vr = lossfn(out.image, targets[s * world + r])
            rast.backward(vr, grads, bg, accumulate=(r > 0))
        tr.adam_step_splats(model, m, v, grads, LRS, s + 1, skip_shN=False, grad_scale=1.0 / world)
    local = model.flat.clone()
    start = tr.SplatData(n, K, dev, cap).load(P).flat.clone()
    # the exchange under test
    peer = None
    if mode == "fused_p2p":
        numel = cap * tr.SplatData(1, K, "cpu").row_floats
        pf, gf, peer = dp.symmetric_flat_buffers(numel, dev)
        model, grads = tr.SplatData(n, K, dev, cap, flat=pf).load(P), tr.SplatData(n, K, dev, cap, flat=gf)
    else:
        model, grads = tr.SplatData(n, K, dev, cap).load(P), tr.SplatData(n, K, dev, cap)
    rast = tr.Rasterizer(model, W, H, deg)
    ex = dp.GradExchange(model, grads, LRS, mode=mode, peer_ptrs=peer, ordering=ordering, multicast=multicast)
    side = torch.cuda.Stream(device=dev)
    evp = torch.cuda.Event()
    evp.record()
    for s in range(steps):
        if split:
            if after_projection:
                rast.forward_lists(cam(s * world + rank), projected_event=evp)
                ex.launch_color(after=evp)
            else:
                rast.forward_lists(cam(s * world + rank))
            ex.wait_color()
            out = rast.forward_shade(bg)
        else:
            out = rast.forward(cam(s * world + rank), bg)
        _, vr = lossfn(out.image, targets[s * world + rank])
        rast.backward(vr, grads, bg, sh_factors=bool(split and rank1))
        if split:
            ex.step_split(2000 + s, side, rank1_sh=bool(rank1), sh_degree=deg, defer_color=after_projection)
        else:
            ex.step(2000 + s)
    ex.wait_color()
    torch.cuda.synchronize()
    ex.raise_if_failed()
    outp = model.flat.clone()
    gathered = [torch.empty_like(outp) for _ in range(world)]
    dist.all_gather(gathered, outp)
    same = all(bool(torch.equal(gathered[0], g)) for g in gathered)
    rel = float((outp - local).norm() / (local - start).norm())
    return {"small_scene_identical_on_all_ranks": bool(same), "small_scene_update_error_vs_one_process": rel, "ok": bool(same and rel < 2e-3)}


def _finite(x):
    """Strict JSON has no NaN / Infinity: replace non-finite floats by null."""
    if isinstance(x, dict):
        return {k: _finite(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_finite(v) for v in x]
    if isinstance(x, float) and not np.isfinite(x):
        return None
    return x


def _kernel_means(recs):
    agg = {}
    for name, ms in recs:
        agg.setdefault(name, []).append(ms)
    return agg


def run_forward_only(args):
    """Forward-only render of a large scene (workloads wide_4k / wide_fisheye): tile-list length, time of the
    tile-list stage (depth sort + scan + emit + tile sort + offsets) and Gpix/s over the seeded poses."""
    import torch
    pkg = importlib.import_module("lichtfeld-studio_b200")
    synth, tr, capi = pkg.synth, pkg.trainer, pkg._capi
    dev = torch.device("cuda", 0)
    cfg = synth.CONFIGS[args.workload]
    W, H, deg, n = cfg["W"], cfg["H"], cfg["sh_degree"], cfg["n"]
    model = tr.SplatData(n, (deg + 1) ** 2, dev).load(synth.make_gaussians(n, 0, cfg["layout"], deg))
    rast = tr.Rasterizer(model, W, H, deg, camera_model=cfg["model"], isect_capacity=4 * n)
    poses, Kmat = synth.make_cameras(cfg)
    Kt, bg = torch.from_numpy(Kmat).to(dev), torch.zeros(3, device=dev)
    cams = [tr.Camera(torch.from_numpy(p).to(dev), Kt, W, H, camera_model=cfg["model"]) for p in poses]
    for c in cams[: max(3, args.warmup)]:
        rast.forward(c, bg)
    torch.cuda.synchronize()
    sampler = ClockSampler(0); sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(1, args.steps // len(cams)) if args.steps > len(cams) else 1
    e0.record()
    for _ in range(reps):
        for c in cams:
            rast.forward(c, bg)
    e1.record(); torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / (reps * len(cams))
    capi.profile_enable(True)
    n_isects, n_vis = [], []
    for c in cams:
        out = rast.forward(c, bg)
        st = out.status.cpu().numpy()
        assert st[0] == 0, "tile-instance capacity exceeded"
        n_isects.append(int(st[1])); n_vis.append(int(st[2]))
    torch.cuda.synchronize()
    km = {k: float(np.mean(v)) for k, v in _kernel_means(capi.profile_collect()).items()}
    capi.profile_enable(False)
    sort_ms = sum(km.get(k, 0.0) for k in ("radix_sort_depth", "exclusive_scan", "emit_instances", "radix_sort_tile", "tile_offsets"))
    hbm_peak, kind = load_peaks()
    V, I = float(np.mean(n_vis)), float(np.mean(n_isects))
    tiles = ((W + 15) // 16) * ((H + 15) // 16)
    sort_bytes = 20 * V + 36 * I + 4 * tiles
    out = {"metric": "forward render Gpix/s", "value": W * H / (ms * 1e-3) / 1e9, "unit": "Gpix/s", "n_gpus": 1, "steps": reps * len(cams),
           "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
           "data": "synthetic", "config": {"workload": args.workload, "gaussians": n, "image": [W, H], "poses": len(cams),
                                           "camera": "fisheye" if cfg["model"] == 2 else "pinhole"},
           "clocks": clocks, "n_isects_mean": I, "n_isects_max": int(np.max(n_isects)), "n_visible_mean": V, "tile_list_ms": sort_ms,
           "kernel_ms": km, "gpu_launches": int(reps * len(cams) * 30),
           "roofline": {"kernel": "tile-list stage (radix_* + scan_* + emit + offsets)", "bound": "hbm",
                        "achieved": sort_bytes / (sort_ms * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                        "frac": sort_bytes / (sort_ms * 1e-3) / 1e9 / hbm_peak, "traffic": None,
                        "note": f"20 V + 36 I + 4 tiles bytes, of {kind}; 21 launches, launch-latency bound at this size"}}
    print(json.dumps(_finite(out)), flush=True)


def run_ewa(args):
    """Training step of the default (non --gut) path on the train_1m scene (workload ewa_1m): EWA forward, fused
    L1 + SSIM loss, EWA backward with densification statistics, fused Adam. Device-resident inputs; kernel times from
    CUDA events inside the library."""
    import torch
    pkg = importlib.import_module("lichtfeld-studio_b200")
    synth, tr, capi = pkg.synth, pkg.trainer, pkg._capi
    dev = torch.device("cuda", 0)
    cfg = synth.CONFIGS["train_1m"]
    W, H, deg, n = cfg["W"], cfg["H"], cfg["sh_degree"], cfg["n"]
    model = tr.SplatData(n, (deg + 1) ** 2, dev, capacity=(n + 31) // 32 * 32).load(synth.make_gaussians(n, 0, cfg["layout"], deg))
    grads, m, v = model.like(), model.like(), model.like()
    rast = tr.FastRasterizer(model, W, H, deg, instance_capacity=16 * n)
    lossfn = tr.PhotometricLoss(W, H, dev, 0.2)
    poses, Kmat = synth.make_cameras(cfg)
    Kt, bg = torch.from_numpy(Kmat).to(dev), torch.zeros(3, device=dev)
    n_steps = args.warmup + args.steps + 3
    cams = [tr.Camera(torch.from_numpy(poses[synth.pose_index(s, len(poses))]).to(dev), Kt, W, H) for s in range(n_steps)]
    target = torch.rand((3, H, W), generator=torch.Generator().manual_seed(1)).to(dev)
    dens = torch.zeros((2, n), device=dev)
    lrs = [1.6e-4, 2.5e-3, 1.25e-4, 5e-3, 1e-3, 5e-2]
    hwc = torch.empty((H, W, 3), device=dev)
    chw = torch.empty((3, H, W), device=dev)

    def step(s):
        out = rast.forward(cams[s], bg)
        hwc.copy_(out.image.permute(1, 2, 0))        # the loss kernels read HWC; two small layout copies per step
        loss, v_hwc = lossfn(hwc, target)
        chw.copy_(v_hwc.permute(2, 0, 1))
        if args.materialize_sh_grad:
            rast.backward(chw, grads, bg, densification_info=dens)
            tr.adam_step_splats(model, m, v, grads, lrs, s + 1)
        else:
            # one camera per step: the shN gradient rows are rebuilt inside the optimizer kernel
            rast.backward(chw, grads, bg, densification_info=dens, write_shN=False)
            rast.adam_step_rank1_sh(m, v, grads, lrs, s + 1)
        return out

    for s in range(max(3, args.warmup)):
        step(s)
    torch.cuda.synchronize()
    sampler = ClockSampler(0); sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(args.steps):
        out = step(args.warmup + s)
    e1.record(); torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    st = out.status.cpu().numpy()
    assert st[0] == 0, "instance capacity exceeded"
    capi.profile_enable(True)
    for s in range(3):
        step(args.warmup + args.steps + s)
    torch.cuda.synchronize()
    km = {k: float(np.mean(x)) for k, x in _kernel_means(capi.profile_collect()).items()}
    capi.profile_enable(False)
    hbm_peak, kind = load_peaks()
    adam_bytes = 28.0 * model.row_floats * n
    t_adam = km.get("adam", float("nan"))
    out = {"metric": "train steps/s (EWA fwd+loss+bwd+Adam)", "value": 1e3 / ms, "unit": "steps/s", "n_gpus": 1, "steps": args.steps,
           "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "f32", "data": "synthetic",
           "config": {"workload": "ewa_1m", "gaussians": n, "image": [W, H], "sh_degree": deg, "path": "default (non --gut) EWA rasterizer",
                      "l2": "inputs larger than L2 (parameters, moments and gradients streamed per step)"},
           "clocks": clocks, "n_instances": int(st[1]), "n_visible": int(st[2]), "kernel_ms": km, "gpu_launches": int(args.steps * 36),
           "roofline": {"kernel": "adam_groups_kernel", "bound": "hbm", "achieved": adam_bytes / (t_adam * 1e-3) / 1e9, "peak": hbm_peak,
                        "unit": "GB/s", "frac": adam_bytes / (t_adam * 1e-3) / 1e9 / hbm_peak, "traffic": None,
                        "note": f"the blend kernels are instruction-issue bound; the streaming kernel shown is Adam, of {kind}"}}
    print(json.dumps(_finite(out)), flush=True)


def run_mcmc(args):
    """MCMC densification step (workload mcmc_3m): relocate dead Gaussians, add 5 % new ones, inject noise."""
    import torch
    pkg = importlib.import_module("lichtfeld-studio_b200")
    synth, tr, st, capi = pkg.synth, pkg.trainer, pkg.strategy, pkg._capi
    dev = torch.device("cuda", 0)
    cfg = synth.CONFIGS[args.workload]
    n, deg = cfg["n"], cfg["sh_degree"]
    P = synth.make_gaussians(n, 0, cfg["layout"], deg)
    P["opacity_raw"][np.arange(n) % 20 == 7] = -6.0
    cap = int(np.float32(1.05) * np.float32(n)) + 64
    model = tr.SplatData(n, (deg + 1) ** 2, dev, capacity=cap).load(P)
    backup = model.flat.clone()
    s = st.MCMC(model)
    s.initialize(st.OptimizationParameters(max_cap=cap, sh_degree=deg))
    times, counts = [], None
    for rep in range(args.warmup + args.steps):
        model.size = s._optimizer.exp_avg.size = s._optimizer.exp_avg_sq.size = s.grads.size = n
        model.flat.copy_(backup)
        torch.manual_seed(1234)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if rep == args.warmup + args.steps - 1:
            capi.profile_enable(True)
        e0.record()
        n_dead = s.relocate_gs()
        n_new = s.add_new_gs()
        s.inject_noise()
        e1.record(); torch.cuda.synchronize()
        if rep >= args.warmup:
            times.append(e0.elapsed_time(e1))
        counts = (n_dead, n_new)
    km = {k: float(np.sum(v)) for k, v in _kernel_means(capi.profile_collect()).items()}
    capi.profile_enable(False)
    ms = float(np.mean(times))
    hbm_peak, kind = load_peaks()
    M = counts[0] + counts[1]
    bytes_alg = 56.0 * M + 56.0 * (n + counts[1]) + 12.0 * (n + counts[1]) + 2 * 236.0 * M
    out = {"metric": "MCMC refine step (relocate + add + noise) ms", "value": ms, "unit": "ms", "n_gpus": 1, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
           "data": "synthetic", "config": {"workload": args.workload, "gaussians": n, "relocated": counts[0], "added": counts[1],
                                           "rng": "torch CUDA generator seeded 1234 before relocate_gs"},
           "kernel_ms_total": km, "gpu_launches": int(args.steps * 20),
           "roofline": {"kernel": "whole refine step", "bound": "hbm", "achieved": bytes_alg / (ms * 1e-3) / 1e9, "peak": hbm_peak,
                        "unit": "GB/s", "frac": bytes_alg / (ms * 1e-3) / 1e9 / hbm_peak, "traffic": None,
                        "note": f"56 M + 68 N + 472 M bytes with M = {M} sampled rows, of {kind}; includes torch.multinomial / normal_ "
                                "and two host reads of the dead / alive counts"}}
    print(json.dumps(_finite(out)), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--batch", type=int, default=0,
                    help="cameras of one optimizer step, fixed over the number of GPUs (each rank renders batch / gpus cameras and "
                         "accumulates); default: one camera per GPU")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--overlap-ctas", type=int, default=2, help="launch footprint (CTAs per SM) of the overlapped colour-group Adam")
    ap.add_argument("--overlap", action="store_true",
                    help="single GPU: split optimizer, colour groups on a side stream under the next step's projection and tile lists")
    ap.add_argument("--materialize-sh-grad", action="store_true",
                    help="write the shN gradient rows (lfs_adam_step_splats / element-wise exchange) instead of using their rank-1 form")
    ap.add_argument("--one-call-optimizer", action="store_true",
                    help="single GPU: lfs_render_backward_adam (no gradient tensor at all) instead of "
                         "lfs_render_backward + lfs_adam_step_splats_rank1_sh")
    ap.add_argument("--no-dp-split", action="store_true",
                    help="N > 1, fused_p2p: exchange all groups in one kernel after the backward. Default: geometry groups first, "
                         "colour groups on a side stream (one CTA per SM) under the next step's projection and tile lists")
    ap.add_argument("--dp-ordering", default="flags", choices=["flags", "nccl"],
                    help="N > 1, fused_p2p: how the ranks' kernels are ordered around the peer-memory exchange: flag words in peer "
                         "memory with bounded waits (lfs_dp_signal / lfs_dp_wait), or 4-byte NCCL all-reduces")
    ap.add_argument("--dp-color-after-projection", action=argparse.BooleanOptionalAction, default=False,
                    help="N > 1, split exchange: start the colour exchange of a step when the NEXT step's projection kernel has "
                         "finished (event inside lfs_render_forward_lists_event), so that it runs next to the sorting kernels only")
    ap.add_argument("--dp-multicast", action=argparse.BooleanOptionalAction, default=None,
                    help="N > 1, fused_p2p: broadcast the new parameters with multimem.st through the NVSwitch multicast mapping of "
                         "the parameter buffer instead of one peer store per rank (default: environment LFS_DP_MULTICAST, else off)")
    ap.add_argument("--dp-mode", default="fused_p2p", choices=["allreduce", "sharded", "fused_p2p"],
                    help="gradient exchange for N > 1 (see lichtfeld-studio_b200/dp.py)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload in ("wide_4k", "wide_fisheye"):
        run_forward_only(args)
    elif args.workload == "mcmc_3m":
        run_mcmc(args)
    elif args.workload == "ewa_1m":
        run_ewa(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
