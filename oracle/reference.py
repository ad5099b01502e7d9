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
