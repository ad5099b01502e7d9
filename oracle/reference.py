"""Python face of the reference's own CUDA build (oracle/_ref/lfs_reference.so, made by oracle/ref_build.py).

TEST INFRASTRUCTURE: the checker of the parity tests and the timed comparator of `bench.py --impl reference`.
Nothing here imports or calls the CUDA library of this repository; nothing in the product imports this.

The module runs the reference's unmodified kernels, so it needs a GPU. Inputs are the dictionaries of raw
SplatData tensors that lichtfeld-studio_b200/synth.py makes (numpy, float32)."""
from __future__ import annotations

import numpy as np

from . import ref_build

NAMES = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")


def available() -> bool:
    return ref_build.available()


def load():
    return ref_build.load()


def to_dev(a, device="cuda:0"):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def make_trainer(P: dict, lrs, sh_degree: int, iterations: int = 30000, device="cuda:0"):
    """RefTrainer over copies of the six raw tensors (leaves with requires_grad, FusedAdam with the MCMC strategy's
    group order and options, exponential decay of the means' rate)."""
    m = load()
    return m.RefTrainer(*(to_dev(P[n], device) for n in NAMES), [float(x) for x in lrs], int(iterations), int(sh_degree))


def activated(P: dict, device="cuda:0"):
    """SplatData's activations with torch, as the reference computes them (src/core/splat_data.cpp:267-286):
    means, normalised quaternions, exp(scales), sigmoid(opacity) squeezed, cat(sh0, shN)."""
    import torch
    t = {n: to_dev(P[n], device) for n in NAMES}
    return (t["means"], torch.nn.functional.normalize(t["rotation_raw"], dim=-1), torch.exp(t["scaling_raw"]),
            torch.sigmoid(t["opacity_raw"]).squeeze(-1), torch.cat([t["sh0"], t["shN"]], 1))


def step_outputs(P: dict, viewmat, K, W: int, H: int, sh_degree: int, background, target_chw, lambda_dssim=0.2,
                 gut: bool = True, lrs=None, device="cuda:0") -> dict:
    """One forward + loss + backward (+ one Adam step when `lrs` is given) of the reference; numpy outputs:
    image [3,H,W] (clamped on the gut path), alpha [1,H,W], loss, the six gradients, the updated parameters."""
    import torch
    tr = make_trainer(P, lrs if lrs is not None else [0.0] * 6, sh_degree, device=device)
    vm = to_dev(np.asarray(viewmat, np.float32).reshape(1, 4, 4), device)
    Kt = to_dev(np.asarray(K, np.float32).reshape(1, 3, 3), device)
    bg = to_dev(np.asarray(background if background is not None else np.zeros(3), np.float32), device)
    image, alpha, loss = tr.forward_backward(gut, vm, Kt, W, H, bg, to_dev(target_chw, device), float(lambda_dssim))
    out = dict(image=image.cpu().numpy(), alpha=alpha.cpu().numpy(), loss=float(loss.item()))
    for n, g in zip(NAMES, tr.grads()):
        out["grad_" + n] = g.cpu().numpy()
    if lrs is not None:
        tr.optimizer_step(1)
        for n, p in zip(NAMES, tr.params()):
            out["new_" + n] = p.detach().cpu().numpy()
    torch.cuda.synchronize()
    return out


def binoms_tensor(device="cuda:0"):
    """MCMC::initialize's table (src/training/strategies/mcmc.cpp:459-472), float32 running products."""
    import torch
    n_max = 51
    b = np.zeros((n_max, n_max), np.float32)
    for n in range(n_max):
        for k in range(n + 1):
            v = np.float32(1.0)
            for i in range(k):
                v = np.float32(v * (np.float32(n - i) / np.float32(i + 1)))
            b[n, k] = v
    return torch.from_numpy(b).to(device)


class McmcReference:
    """MCMC::relocate_gs / add_new_gs / inject_noise (src/training/strategies/mcmc.cpp:112-190, :192-347, :349-367) with
    the same ATen calls on plain tensors and the reference's own gsplat::relocation / gsplat::add_noise kernels. The
    parameters `p` and the Adam moments `m`, `v` are dictionaries of the six raw tensors; add_new_gs grows them by
    torch.cat like the reference does. torch.multinomial and randn_like draw from torch's CUDA generator, so a caller
    that seeds it (torch.manual_seed) gets the reference's indices and noise."""

    def __init__(self, P: dict, min_opacity=0.005, max_cap=1_000_000, device="cuda:0"):
        import torch
        self.ref = load()
        self.p = {n: to_dev(P[n], device).clone() for n in NAMES}
        self.m = {n: torch.zeros_like(t) for n, t in self.p.items()}
        self.v = {n: torch.zeros_like(t) for n, t in self.p.items()}
        self.binoms = binoms_tensor(device)
        self.min_opacity, self.max_cap = float(min_opacity), int(max_cap)
        self.last = {}

    def _opacities(self):
        import torch
        return torch.sigmoid(self.p["opacity_raw"]).squeeze(-1)

    @staticmethod
    def multinomial_sample(weights, n):
        import torch
        if weights.shape[0] > (1 << 24):
            raise RuntimeError("more than 2^24 weights: the reference falls back to an unseeded host sampler")
        return torch.multinomial(weights, n, True)

    def relocate_gs(self) -> int:
        import torch
        p, ref = self.p, self.ref
        opacities = self._opacities()
        rot = p["rotation_raw"]
        dead_mask = (opacities <= self.min_opacity) | ((rot * rot).sum(-1) < 1e-8)
        dead_indices = dead_mask.nonzero().squeeze(-1)
        n_dead = dead_indices.numel()
        if n_dead == 0:
            return 0
        alive_indices = (~dead_mask).nonzero().squeeze(-1)
        if alive_indices.numel() == 0:
            return 0
        probs = opacities.index_select(0, alive_indices)
        sampled_local = self.multinomial_sample(probs, n_dead)
        sampled = alive_indices.index_select(0, sampled_local)
        s_opac = opacities.index_select(0, sampled)
        s_scales = torch.exp(p["scaling_raw"]).index_select(0, sampled)
        ratios = torch.ones_like(opacities, dtype=torch.int32)
        ratios.index_add_(0, sampled, torch.ones_like(sampled, dtype=torch.int32))
        ratios = ratios.index_select(0, sampled).contiguous()
        n_max = self.binoms.shape[0]
        ratios = torch.clamp_max_(ratios, n_max)
        new_opac, new_scales = ref.relocation(s_opac, s_scales, ratios, self.binoms, n_max)
        new_opac = torch.clamp_(new_opac, self.min_opacity, 1.0 - 1e-7)
        p["opacity_raw"][sampled, :] = torch.logit(new_opac).unsqueeze(-1)
        p["scaling_raw"].index_put_((sampled,), torch.log(new_scales))
        for n in NAMES:
            p[n].index_put_((dead_indices,), p[n].index_select(0, sampled))
        for n in NAMES:
            self.m[n].index_put_((sampled,), torch.zeros((), device=sampled.device))
            self.v[n].index_put_((sampled,), torch.zeros((), device=sampled.device))
        self.last.update(dead_indices=dead_indices, alive_indices=alive_indices, relocate_sampled=sampled, relocate_ratios=ratios,
                         relocate_sampled_local=sampled_local)
        return int(n_dead)

    def add_new_gs(self) -> int:
        import torch
        p, ref = self.p, self.ref
        current_n = p["means"].shape[0]
        n_target = min(self.max_cap, int(np.float32(1.05) * np.float32(current_n)))
        n_new = max(0, n_target - current_n)
        if n_new == 0:
            return 0
        opacities = self._opacities()
        sampled = self.multinomial_sample(opacities.flatten(), n_new)
        s_opac = opacities.index_select(0, sampled)
        s_scales = torch.exp(p["scaling_raw"]).index_select(0, sampled)
        ratios = torch.zeros(opacities.shape[0], dtype=torch.float32, device=sampled.device)
        ratios.index_add_(0, sampled, torch.ones_like(sampled, dtype=torch.float32))
        ratios = ratios.index_select(0, sampled) + 1
        n_max = self.binoms.shape[0]
        ratios = torch.clamp(ratios, 1, n_max).to(torch.int32).contiguous()
        new_opac, new_scales = ref.relocation(s_opac, s_scales, ratios, self.binoms, n_max)
        new_opac = torch.clamp(new_opac, self.min_opacity, 1.0 - 1e-7)
        p["opacity_raw"][sampled, :] = torch.logit(new_opac).unsqueeze(-1)
        p["scaling_raw"].index_put_((sampled,), torch.log(new_scales))
        for n in NAMES:
            new_rows = p[n].index_select(0, sampled)
            p[n] = torch.cat([p[n], new_rows], 0)
            zeros = torch.zeros_like(new_rows)
            self.m[n] = torch.cat([self.m[n], zeros], 0)
            self.v[n] = torch.cat([self.v[n], zeros], 0)
        self.last.update(add_sampled=sampled, add_ratios=ratios)
        return int(n_new)

    def inject_noise(self, current_lr: float):
        import torch
        p = self.p
        noise = torch.randn_like(p["means"])
        self.ref.add_noise(p["opacity_raw"], p["scaling_raw"], p["rotation_raw"], noise, p["means"], float(current_lr))
        self.last.update(noise=noise)
