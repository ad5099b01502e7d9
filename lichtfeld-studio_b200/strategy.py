"""Training-strategy interface of the reference over the C ABI.

Mirrors src/training/strategies/istrategy.hpp:13-32 (IStrategy), src/training/strategies/mcmc.{hpp,cpp}
(MCMC: relocate / add / noise / Adam step / LR decay), src/training/optimizers/fused_adam.{hpp,cpp}
(FusedAdam) and src/training/optimizers/scheduler.cpp (ExponentialLR) with the same method names,
argument meaning and defaults (include/core/parameters.hpp:16-40).

Differences that follow from the buffer design: parameters, gradients and Adam moments live in
capacity-reserved flat buffers (trainer.SplatData), so add_new_gs appends rows in place instead of
six torch::cat re-allocations and a re-keying of the optimizer state, and gradients are passed to
step() explicitly because there is no autograd .grad slot."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _capi as capi
from ._capi import call, ptr
from .trainer import SplatData, adam_step_splats


def _stream():
    return capi.vp(torch.cuda.current_stream().cuda_stream)


@dataclass
class OptimizationParameters:
    """Subset of gs::param::OptimizationParameters used on this path (include/core/parameters.hpp:16-40)."""
    iterations: int = 30_000
    sh_degree_interval: int = 1_000
    means_lr: float = 0.00016
    shs_lr: float = 0.0025
    opacity_lr: float = 0.05
    scaling_lr: float = 0.005
    rotation_lr: float = 0.001
    lambda_dssim: float = 0.2
    min_opacity: float = 0.005
    refine_every: int = 100
    start_refine: int = 500
    stop_refine: int = 25_000
    max_cap: int = 1_000_000
    sh_degree: int = 3
    scene_scale: float = 1.0


class FusedAdam:
    """torch::optim-style Adam over the six parameter groups with one fused launch per step
    (fused_adam.cpp:22-95). Group order: means, sh0, shN, scaling, rotation, opacity."""

    def __init__(self, model: SplatData, lrs, betas=(0.9, 0.999), eps=1e-15):
        self.model = model
        self.lr = [float(x) for x in lrs]
        self.betas, self.eps = (float(betas[0]), float(betas[1])), float(eps)
        self.exp_avg, self.exp_avg_sq = model.like(), model.like()
        self.step_count = 0

    def step(self, iteration: int, grads: SplatData, grad_scale: float = 1.0, first_row: int = 0, n_rows=None):
        self.step_count += 1  # advances for the skipped shN group as well (fused_adam.cpp:66-70)
        self.exp_avg.size = self.exp_avg_sq.size = grads.size = self.model.size
        adam_step_splats(self.model, self.exp_avg, self.exp_avg_sq, grads, self.lr, self.step_count, self.betas[0], self.betas[1],
                         self.eps, skip_shN=(iteration <= 1000), first_row=first_row, n_rows=n_rows, grad_scale=grad_scale)

    def zero_grad(self, set_to_none=True, iteration=0):
        """No-op: the next backward overwrites every gradient row."""


class ExponentialLR:
    """scheduler.cpp:10 / mcmc.cpp:20: lr *= gamma for one group (or all when index < 0)."""

    def __init__(self, optimizer: FusedAdam, gamma: float, param_group_index: int = -1):
        self.opt, self.gamma, self.idx = optimizer, float(gamma), int(param_group_index)

    def step(self):
        if self.idx >= 0:
            self.opt.lr[self.idx] *= self.gamma
        else:
            self.opt.lr = [x * self.gamma for x in self.opt.lr]


class IStrategy:
    def initialize(self, optim_params): raise NotImplementedError
    def post_backward(self, iter, render_output): raise NotImplementedError
    def step(self, iter): raise NotImplementedError
    def is_refining(self, iter) -> bool: raise NotImplementedError
    def get_model(self): raise NotImplementedError
    def remove_gaussians(self, mask): raise NotImplementedError


def binoms_table(n_max: int = 51) -> np.ndarray:
    """mcmc.cpp:459-472: running float32 product of (n - i) / (i + 1)."""
    b = np.zeros((n_max, n_max), np.float32)
    for n in range(n_max):
        for k in range(n + 1):
            v = np.float32(1.0)
            for i in range(k):
                v = np.float32(v * (np.float32(n - i) / np.float32(i + 1)))
            b[n, k] = v
    return b


class MCMC(IStrategy):
    """"3D Gaussian Splatting as Markov Chain Monte Carlo" strategy (mcmc.cpp)."""

    _noise_lr = 5e5  # mcmc.hpp:79

    def __init__(self, splat_data: SplatData):
        self._splat_data = splat_data
        self._params = None
        self._optimizer = None
        self._scheduler = None
        self.grads = splat_data.like()
        self.active_sh_degree = 0

    # ------------------------------------------------------------------ IStrategy
    def initialize(self, optim_params: OptimizationParameters):
        p = self._params = optim_params
        dev = self._splat_data.device
        self._binoms = torch.from_numpy(binoms_table(51)).to(dev)
        lrs = [p.means_lr * p.scene_scale, p.shs_lr, p.shs_lr / 20.0, p.scaling_lr, p.rotation_lr, p.opacity_lr]  # mcmc.cpp:487-492
        self._optimizer = FusedAdam(self._splat_data, lrs, (0.9, 0.999), 1e-15)
        self._scheduler = ExponentialLR(self._optimizer, 0.01 ** (1.0 / p.iterations), 0)
        cap = self._splat_data.capacity
        i64 = lambda n: torch.empty(n, dtype=torch.int64, device=dev)
        self._dead, self._alive, self._sampled = i64(cap), i64(cap), i64(cap)
        self._alive_opac = torch.empty(cap, dtype=torch.float32, device=dev)
        self._counts2 = torch.zeros(2, dtype=torch.int32, device=dev)
        self._counts = torch.empty(cap, dtype=torch.int32, device=dev)
        self._ratios = torch.empty(cap, dtype=torch.int32, device=dev)
        self._s_opac = torch.empty(cap, dtype=torch.float32, device=dev)
        self._s_scales = torch.empty((cap, 3), dtype=torch.float32, device=dev)
        self._new_opac = torch.empty(cap, dtype=torch.float32, device=dev)
        self._new_scales = torch.empty((cap, 3), dtype=torch.float32, device=dev)
        self._noise = torch.empty((cap, 3), dtype=torch.float32, device=dev)
        self._ws = torch.empty(capi.lib().lfs_mcmc_workspace_bytes(cap), dtype=torch.uint8, device=dev)

    def is_refining(self, iter: int) -> bool:
        p = self._params
        return iter < p.stop_refine and iter > p.start_refine and iter % p.refine_every == 0

    def get_model(self) -> SplatData:
        return self._splat_data

    def post_backward(self, iter: int, render_output=None):
        if iter % self._params.sh_degree_interval == 0:
            self.active_sh_degree = min(self.active_sh_degree + 1, self._params.sh_degree)  # increment_sh_degree
        if self.is_refining(iter):
            self.relocate_gs()
            self.add_new_gs()
        self.inject_noise()

    def step(self, iter: int, grad_scale: float = 1.0):
        if iter < self._params.iterations:
            self._optimizer.step(iter, self.grads, grad_scale)
            self._optimizer.zero_grad(True, iter)
            self._scheduler.step()

    def remove_gaussians(self, mask: torch.Tensor):
        """mcmc.cpp:406-444: keep rows where mask is False (parameters and Adam moments)."""
        old_n = self._splat_data.size
        if mask.numel() != old_n:
            raise RuntimeError(f"mask must have {old_n} elements, got {mask.numel()}")
        keep = (~mask.bool()).nonzero().squeeze(-1)
        new_n = int(keep.numel())
        if new_n == old_n:
            return
        for sd in (self._splat_data, self._optimizer.exp_avg, self._optimizer.exp_avg_sq):
            sd.size = old_n  # every buffer is gathered with indices into the OLD row range
            kept = {n: sd.tensor(n).index_select(0, keep) for n in ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")}
            sd.size = new_n
            for n, t in kept.items():
                sd.tensor(n).copy_(t)
        self.grads.size = new_n

    # ------------------------------------------------------------------ pieces
    @staticmethod
    def multinomial_sample(weights: torch.Tensor, n: int, replacement: bool = True) -> torch.Tensor:
        """mcmc.cpp:43-84. torch.multinomial is the same libtorch call the reference makes, so for the same
        generator state and bit-identical weights the sampled indices are those of the reference."""
        if weights.numel() <= (1 << 24):
            return torch.multinomial(weights, n, replacement)
        w = (weights / weights.sum()).cpu()
        cdf = w.cumsum(0).numpy()
        u = np.random.default_rng().random(n).astype(np.float32)
        return torch.from_numpy(np.minimum(np.searchsorted(cdf, u, side="left"), weights.numel() - 1)).to(weights.device)

    def _relocate_with(self, sampled: torch.Tensor, dst, n: int):
        """Everything after the draw: ratios, eq. (9), write-back, row copies, moment reset."""
        sd, opt = self._splat_data, self._optimizer
        N = sd.size
        st = _stream()
        call("lfs_mcmc_gather_ratios", N, n, ptr(sampled), ptr(sd._full["opacity_raw"]), ptr(sd._full["scaling_raw"]), 51,
             ptr(self._counts), ptr(self._ratios), ptr(self._s_opac), ptr(self._s_scales), st)
        call("lfs_relocation", n, ptr(self._s_opac), ptr(self._s_scales), ptr(self._ratios), ptr(self._binoms), 51,
             ptr(self._new_opac), ptr(self._new_scales), st)
        p, m, v = sd.struct(), opt.exp_avg.struct(), opt.exp_avg_sq.struct()
        call("lfs_mcmc_apply", N, sd.K, n, ptr(sampled), ptr(dst), ptr(self._new_opac), ptr(self._new_scales),
             float(self._params.min_opacity), C.byref(p), C.byref(m), C.byref(v), st)

    def relocate_gs(self, sampled_local: torch.Tensor | None = None) -> int:
        """mcmc.cpp:112-190. `sampled_local` (indices into the alive list) may be injected for tests."""
        sd = self._splat_data
        N = sd.size
        call("lfs_mcmc_classify", N, ptr(sd._full["opacity_raw"]), ptr(sd._full["rotation_raw"]), float(self._params.min_opacity),
             ptr(self._dead), ptr(self._alive), ptr(self._alive_opac), ptr(self._counts2), ptr(self._ws), self._ws.numel(), _stream())
        n_dead, n_alive = (int(x) for x in self._counts2.tolist())  # host read, like dead_indices.numel()
        if n_dead == 0 or n_alive == 0:
            return 0
        if sampled_local is None:
            sampled_local = self.multinomial_sample(self._alive_opac[:n_alive], n_dead, True)
        call("lfs_mcmc_map_indices", n_dead, ptr(sampled_local), ptr(self._alive), ptr(self._sampled), _stream())
        self._relocate_with(self._sampled, self._dead, n_dead)
        return n_dead

    def add_new_gs(self, sampled: torch.Tensor | None = None) -> int:
        """mcmc.cpp:192-347."""
        sd, opt = self._splat_data, self._optimizer
        current_n = sd.size
        n_target = min(self._params.max_cap, int(np.float32(1.05) * np.float32(current_n)))
        n_new = max(0, n_target - current_n)
        if n_new == 0:
            return 0
        if current_n + n_new > sd.capacity:
            raise RuntimeError("SplatData capacity exhausted: reserve max_cap rows")
        if sampled is None:
            probs = torch.sigmoid(sd.tensor("opacity_raw")).flatten()
            sampled = self.multinomial_sample(probs, n_new, True)
        self._relocate_with(sampled, None, n_new)
        for s in (sd, opt.exp_avg, opt.exp_avg_sq, self.grads):
            s.size = current_n + n_new
        return n_new

    def inject_noise(self, noise: torch.Tensor | None = None):
        """mcmc.cpp:349-367."""
        sd = self._splat_data
        current_lr = float(np.float32(self._optimizer.lr[0])) * self._noise_lr
        if noise is None:
            noise = self._noise[: sd.size]
            noise.normal_()  # torch::randn_like
        call("lfs_add_noise", sd.size, ptr(sd._full["opacity_raw"]), ptr(sd._full["scaling_raw"]), ptr(sd._full["rotation_raw"]),
             ptr(noise), ptr(sd._full["means"]), current_lr, _stream())
