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

    def step(self, iteration: int, grads: SplatData, grad_scale: float = 1.0, first_row: int = 0, n_rows=None,
             rasterizer=None):
        """rasterizer: the Rasterizer whose backward(write_shN=False) of ONE camera produced `grads`; the shN rows are then
        updated from gradient rows rebuilt inside the optimizer kernel (lfs_adam_step_splats_rank1_sh)."""
        self.step_count += 1  # advances for the skipped shN group as well (fused_adam.cpp:66-70)
        self.exp_avg.size = self.exp_avg_sq.size = grads.size = self.model.size
        if rasterizer is not None:
            if first_row != 0 or n_rows not in (None, self.model.size):
                raise RuntimeError("the rank-1 shN update covers all rows")
            rasterizer.adam_step_rank1_sh(self.exp_avg, self.exp_avg_sq, grads, self.lr, self.step_count, self.betas[0],
                                          self.betas[1], self.eps, skip_shN=(iteration <= 1000), grad_scale=grad_scale)
            return
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
        # False once a refinement has replaced the parameter rows of this iteration: the reference's new leaf tensors
        # have no .grad, so FusedAdam::step skips them before it counts the step (fused_adam.cpp:46-48)
        self._grads_valid = True

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
        self._means_moved_iter = iter     # the noise moved every mean; relocation rewrote rows

    def step(self, iter: int, grad_scale: float = 1.0, rasterizer=None):
        """mcmc.cpp:395-402. On an iteration whose post_backward appended or removed rows the optimizer does nothing and
        does not count the step (the gradients belong to the old rows); the scheduler still runs. The next backward
        writes every gradient row again.
        rasterizer (FusedAdam.step): the rank-1 shN update rebuilds each gradient row from the CURRENT means and the camera
        of the forward, so it is only equal to the materialised gradient while the means are those the forward saw. It is
        refused after this iteration's post_backward (which moved them); leave rasterizer=None in the reference's order
        backward -> post_backward -> step."""
        if rasterizer is not None and getattr(self, "_means_moved_iter", None) == iter:
            raise RuntimeError("MCMC.step(rasterizer=...): post_backward of this iteration moved the means; the rank-1 shN "
                               "update would rebuild its gradient rows from other view directions than the forward's. "
                               "Call step() without a rasterizer (backward must then write the shN gradient).")
        if iter < self._params.iterations:
            if self._grads_valid:
                self._optimizer.step(iter, self.grads, grad_scale, rasterizer=rasterizer)
            self._grads_valid = True
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
        self._grads_valid = False

    # ------------------------------------------------------------------ pieces
    @staticmethod
    def multinomial_sample(weights: torch.Tensor, n: int, replacement: bool = True) -> torch.Tensor:
        """mcmc.cpp:43-84. torch.multinomial is the same libtorch call the reference makes, so for the same
        generator state and bit-identical weights the sampled indices are those of the reference."""
        if weights.numel() <= (1 << 24):
            return torch.multinomial(weights, n, replacement)
        w = (weights / weights.sum()).cpu()
        cdf = w.cumsum(0).numpy()
        # drawn from torch's generator so that ranks seeded alike stay replicated
        u = torch.rand(n, dtype=torch.float32, device=weights.device).cpu().numpy()
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
        self._grads_valid = False   # the reference concatenates into new leaves without .grad (mcmc.cpp:254-259)
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


def _rewrite_rows(buffers, new_rows: dict, new_n: int):
    """Replace the live rows of several SplatData buffers (parameters, moments) by freshly gathered rows.
    new_rows[i] is a dict name -> tensor for buffers[i]; counterpart of update_param_with_optimizer
    (src/training/strategies/strategy_utils.cpp:57) on capacity-reserved storage."""
    for sd, rows in zip(buffers, new_rows):
        if new_n > sd.capacity:
            raise RuntimeError("SplatData capacity exhausted: reserve more rows")
        sd.size = new_n
        for name, t in rows.items():
            sd.tensor(name).copy_(t.reshape(sd.tensor(name).shape))


class DefaultStrategy(IStrategy):
    """Adaptive density control of the original 3DGS (src/training/strategies/default_strategy.cpp):
    duplicate small / split large Gaussians with a high image-plane gradient, prune transparent or huge
    ones, reset opacities periodically. `densification_info` [2, N] (visibility count, accumulated
    image-plane gradient norm) is an input: the reference's gsplat path does not fill it either; its
    default EWA rasterizer does."""

    def __init__(self, splat_data: SplatData):
        self._splat_data = splat_data
        self._params = None
        self._optimizer = None
        self._scheduler = None
        self.grads = splat_data.like()
        self.active_sh_degree = 0
        self.densification_info = None
        self._grads_valid = True   # see MCMC: row surgery invalidates this iteration's gradients

    @dataclass
    class Parameters(OptimizationParameters):
        grad_threshold: float = 0.0002
        prune_opacity: float = 0.005
        grow_scale3d: float = 0.01
        prune_scale3d: float = 0.1
        reset_every: int = 3_000
        pause_refine_after_reset: int = 0
        revised_opacity: bool = False

    # ------------------------------------------------------------------ IStrategy
    def initialize(self, optim_params):
        p = self._params = optim_params
        sd = self._splat_data
        self.densification_info = torch.zeros((2, sd.size), dtype=torch.float32, device=sd.device)
        lrs = [p.means_lr * p.scene_scale, p.shs_lr, p.shs_lr / 20.0, p.scaling_lr, p.rotation_lr, p.opacity_lr]
        self._optimizer = FusedAdam(sd, lrs, (0.9, 0.999), 1e-15)
        self._scheduler = ExponentialLR(self._optimizer, 0.01 ** (1.0 / p.iterations), 0)

    def is_refining(self, iter: int) -> bool:
        p = self._params
        return iter > p.start_refine and iter % p.refine_every == 0 and iter % p.reset_every >= p.pause_refine_after_reset

    def get_model(self) -> SplatData:
        return self._splat_data

    def remove_gaussians(self, mask: torch.Tensor):
        if int(mask.sum()) == 0:
            return
        self.remove(mask)

    def post_backward(self, iter: int, render_output=None):
        p = self._params
        if iter % p.sh_degree_interval == 0:
            self.active_sh_degree = min(self.active_sh_degree + 1, p.sh_degree)
        if iter == p.stop_refine:
            self.densification_info = torch.empty(0)
        if iter >= p.stop_refine:
            return
        if self.is_refining(iter):
            self.grow_gs(iter)
            self.prune_gs(iter)
            self.densification_info = torch.zeros((2, self._splat_data.size), dtype=torch.float32, device=self._splat_data.device)
        if iter % p.reset_every == 0 and iter > 0:
            self.reset_opacity()

    def step(self, iter: int, grad_scale: float = 1.0):
        """default_strategy.cpp step(): duplicate / split / remove go through update_param_with_optimizer
        (strategy_utils.cpp:57), whose new leaf tensors have no .grad, so on those iterations FusedAdam::step skips every
        group before counting the step; the scheduler still runs."""
        if iter < self._params.iterations:
            if self._grads_valid:
                self._optimizer.step(iter, self.grads, grad_scale)
            self._grads_valid = True
            self._optimizer.zero_grad(True, iter)
            self._scheduler.step()

    # ------------------------------------------------------------------ pieces
    def _buffers(self):
        return (self._splat_data, self._optimizer.exp_avg, self._optimizer.exp_avg_sq)

    def _sync_sizes(self):
        n = self._splat_data.size
        for sd in (self._optimizer.exp_avg, self._optimizer.exp_avg_sq, self.grads):
            sd.size = n

    def _activated(self):
        sd = self._splat_data
        return torch.sigmoid(sd.tensor("opacity_raw")).squeeze(-1), torch.exp(sd.tensor("scaling_raw")), \
            torch.nn.functional.normalize(sd.tensor("rotation_raw"), dim=-1)

    def duplicate(self, is_duplicated: torch.Tensor):
        """default_strategy.cpp:49-87: append copies of the selected rows; their moments start at zero."""
        self._sync_sizes()
        idx = is_duplicated.nonzero().squeeze(-1)
        n, k = self._splat_data.size, int(idx.numel())
        rows = []
        for bi, sd in enumerate(self._buffers()):
            d = {}
            for name in ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw"):
                t = sd.tensor(name)
                extra = t.index_select(0, idx) if bi == 0 else torch.zeros((k,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
                d[name] = torch.cat([t, extra], 0)
            rows.append(d)
        _rewrite_rows(self._buffers(), rows, n + k)
        self._sync_sizes()
        self._grads_valid = False

    def split(self, is_split: torch.Tensor, noise: torch.Tensor | None = None):
        """default_strategy.cpp:89-159: each selected Gaussian is replaced by two samples of itself with scale / 1.6;
        the rest keep their order, the new rows are appended, their moments start at zero."""
        from . import ops
        self._sync_sizes()
        sd = self._splat_data
        idx = is_split.nonzero().squeeze(-1)
        rest = (~is_split.bool()).nonzero().squeeze(-1)
        k = int(idx.numel())
        _, scales, quats = self._activated()
        s_scales, s_quats = scales.index_select(0, idx), quats.index_select(0, idx).contiguous()
        rotmats = ops.quats_to_rotmats(s_quats)  # [k, 3, 3]
        if noise is None:
            noise = torch.randn((2, k, 3), dtype=torch.float32, device=sd.device)
        samples = torch.einsum("nij,nj,bnj->bni", rotmats, s_scales, noise)  # [2, k, 3]
        rows = []
        for bi, buf in enumerate(self._buffers()):
            d = {}
            for gi, name in enumerate(("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")):
                t = buf.tensor(name)
                rest_rows = t.index_select(0, rest)
                if bi > 0:
                    new = torch.zeros((2 * k,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
                else:
                    sel = t.index_select(0, idx)
                    if gi == 0:
                        new = (sel.unsqueeze(0) + samples).reshape(-1, 3)
                    elif gi == 3:
                        new = torch.log(s_scales / 1.6).repeat(2, 1)
                    elif gi == 5 and self._params.revised_opacity:
                        new = torch.logit(1.0 - torch.sqrt(1.0 - torch.sigmoid(sel))).repeat(2, 1)
                    else:
                        new = sel.repeat((2,) + (1,) * (sel.dim() - 1))
                d[name] = torch.cat([rest_rows, new], 0)
            rows.append(d)
        _rewrite_rows(self._buffers(), rows, int(rest.numel()) + 2 * k)
        self._sync_sizes()
        self._grads_valid = False

    def grow_gs(self, iter: int):
        """default_strategy.cpp:161-189."""
        p, sd = self._params, self._splat_data
        info = self.densification_info
        grads = info[1] / torch.clamp_min(info[0], 1.0)
        _, scales, _ = self._activated()
        is_grad_high = grads > p.grad_threshold
        is_small = scales.max(-1).values <= p.grow_scale3d * p.scene_scale
        is_duplicated = is_grad_high & is_small
        num_dup = int(is_duplicated.sum())
        is_split = is_grad_high & ~is_small
        num_split = int(is_split.sum())
        if num_dup > 0:
            self.duplicate(is_duplicated)
        is_split = torch.cat([is_split, torch.zeros(num_dup, dtype=torch.bool, device=sd.device)])
        if num_split > 0:
            self.split(is_split)

    def remove(self, is_prune: torch.Tensor):
        """default_strategy.cpp:191-219."""
        self._sync_sizes()
        keep = (~is_prune.bool()).nonzero().squeeze(-1)
        rows = [{name: sd.tensor(name).index_select(0, keep) for name in ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")}
                for sd in self._buffers()]
        _rewrite_rows(self._buffers(), rows, int(keep.numel()))
        self._sync_sizes()
        self._grads_valid = False

    def prune_gs(self, iter: int):
        """default_strategy.cpp:221-241."""
        p, sd = self._params, self._splat_data
        opac, scales, _ = self._activated()
        is_prune = opac < p.prune_opacity
        rot = sd.tensor("rotation_raw")
        is_prune |= (rot * rot).sum(-1) < 1e-8
        if iter > p.reset_every:
            is_prune |= scales.max(-1).values > p.prune_scale3d * p.scene_scale
        if int(is_prune.sum()) > 0:
            self.remove(is_prune)

    def reset_opacity(self):
        """default_strategy.cpp:243-282: clamp the logits at logit(2 prune_opacity), zero the opacity moments."""
        thr = torch.logit(torch.tensor(2.0 * self._params.prune_opacity)).item()
        self._sync_sizes()
        self._splat_data.tensor("opacity_raw").clamp_(max=thr)
        self._optimizer.exp_avg.tensor("opacity_raw").zero_()
        self._optimizer.exp_avg_sq.tensor("opacity_raw").zero_()
