"""Fused training-step path over the C ABI: the call sequence of Trainer::train_step
(src/training/trainer.cpp:599-875) for the gsplat / 3DGUT rasterizer — rasterize()
(src/training/rasterization/rasterizer.cpp:15), compute_photometric_loss (trainer.cpp:107-134),
backward (rasterizer_autograd.cpp:105) and strategy->step — without autograd or ATen glue.

All buffers (parameters, gradients, forward state, loss scratch) are allocated once and reused;
every step is a fixed sequence of asynchronous launches on the current stream with no host
synchronisation. torch provides device memory and streams only."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import torch

from . import _capi as capi
from ._capi import RenderConfig, UTParams, call, ptr, splats_struct

PARAM_NAMES = ("means", "sh0", "shN", "scaling_raw", "rotation_raw", "opacity_raw")


def _stream():
    return capi.vp(torch.cuda.current_stream().cuda_stream)


def row_widths(K: int):
    return dict(means=3, sh0=3, shN=(K - 1) * 3, scaling_raw=3, rotation_raw=4, opacity_raw=1)


class SplatData:
    """The six raw parameter tensors of src/core/splat_data.hpp:104-109 as views into ONE flat
    buffer, group-major ([means | sh0 | shN | scaling | rotation | opacity], each with room for
    `capacity` rows) so that gradients / moments of all groups can be reduced or updated as one
    range. `size` rows are live; densification appends rows in place instead of torch.cat."""

    def __init__(self, n: int, sh_coeffs: int, device, capacity: int | None = None, flat: torch.Tensor | None = None):
        self.K = int(sh_coeffs)
        # a multiple of 4 rows keeps every group's start (and each quaternion row) 16-byte aligned
        self.capacity = (int(capacity or n) + 3) // 4 * 4
        self.size = int(n)
        self.device = device
        w = row_widths(self.K)
        self.row_floats = sum(w.values())
        numel = self.capacity * self.row_floats
        if flat is None:
            flat = torch.zeros(numel, dtype=torch.float32, device=device)
        elif flat.numel() != numel or flat.dtype != torch.float32 or not flat.is_contiguous():
            raise RuntimeError(f"flat buffer must be a contiguous float32 tensor of {numel} elements")
        self.flat = flat  # may be peer-mapped (symmetric) memory for the fused multi-GPU exchange
        self._full = {}
        off = 0
        for name in PARAM_NAMES:
            cnt = self.capacity * w[name]
            self._full[name] = self.flat[off:off + cnt]
            off += cnt
        self._w = w

    def tensor(self, name: str) -> torch.Tensor:
        """Live rows of one group in the reference's shape."""
        w = self._w[name]
        t = self._full[name][: self.size * w]
        if name == "sh0":
            return t.view(self.size, 1, 3)
        if name == "shN":
            return t.view(self.size, self.K - 1, 3)
        return t.view(self.size, w)

    def tensors(self) -> dict:
        return {n: self.tensor(n) for n in PARAM_NAMES}

    def load(self, params: dict):
        for n in PARAM_NAMES:
            self.tensor(n).copy_(torch.as_tensor(params[n]).to(self.device).reshape(self.tensor(n).shape))
        return self

    def struct(self) -> capi.Splats:
        return capi.Splats(*(self._full[n].data_ptr() for n in PARAM_NAMES))

    def like(self) -> "SplatData":
        return SplatData(self.size, self.K, self.device, self.capacity)


@dataclass
class Camera:
    """What the step needs of gs::Camera: world-to-camera [R|t] (world_view_transform), K, size, model."""
    viewmat: torch.Tensor  # [4,4] float32 on device
    K: torch.Tensor        # [3,3]
    width: int
    height: int
    camera_model: int = capi.PINHOLE
    radial: torch.Tensor | None = None      # fisheye: [4] coefficients; pinhole: [6] radial distortion (k1..k6)
    tangential: torch.Tensor | None = None  # pinhole: [2]
    thin_prism: torch.Tensor | None = None  # pinhole: [4]
    shutter: int = 0                        # 0 global, 1 top-to-bottom, 2 left-to-right, 3 bottom-to-top, 4 right-to-left
    viewmat_end: torch.Tensor | None = None  # [4,4] end-of-frame pose of a rolling shutter (None = the start pose)

    def coefficient_pointers(self):
        """Device pointers in the widths the C ABI reads (pinhole radial 6, tangential 2, thin prism 4; fisheye radial 4);
        shorter tensors are zero-padded once and cached, like rasterize() pads the loader's coefficient vectors
        (src/training/rasterization/rasterizer.cpp:96-121)."""
        if not hasattr(self, "_padded"):
            def widen(t, n):
                if t is None:
                    return None
                t = t.reshape(-1).float()
                if t.numel() > n:
                    raise RuntimeError(f"at most {n} distortion coefficients, got {t.numel()}")
                return torch.nn.functional.pad(t, (0, n - t.numel())).contiguous()
            fisheye = self.camera_model == capi.FISHEYE
            if fisheye and (self.tangential is not None or self.thin_prism is not None):
                raise RuntimeError("tangential / thin-prism coefficients belong to the pinhole model")
            self._padded = (widen(self.radial, 4 if fisheye else 6), widen(self.tangential, 2), widen(self.thin_prism, 4))
        return tuple(None if t is None else t.data_ptr() for t in self._padded)


@dataclass
class RenderOutput:
    """src/training/rasterization/rasterizer.hpp RenderOutput (fields the trainer uses)."""
    image: torch.Tensor   # [H,W,3] unclamped render; the clamp / permute is folded into the loss kernel (None in D / ED)
    alpha: torch.Tensor   # [H,W,1]
    width: int
    height: int
    status: torch.Tensor  # int32[4] on device: overflow flag, n_isects, n_visible
    depth: torch.Tensor | None = None   # [H,W,1] accumulated (D, RGB_D) or expected (ED, RGB_ED) depth
    render: torch.Tensor | None = None  # [H,W,channels] as the kernel wrote it; v_render of backward() has this shape


RENDER_RGB, RENDER_D, RENDER_ED, RENDER_RGB_D, RENDER_RGB_ED = 0, 1, 2, 3, 4  # RenderMode, rasterizer.hpp


class Rasterizer:
    """rasterize() + FusedRasterizationWithSHFunction for a fixed (N capacity, image size): owns the
    workspace that carries the forward state to the backward."""

    def __init__(self, model: SplatData, width: int, height: int, sh_degree: int, camera_model=capi.PINHOLE,
                 isect_capacity: int | None = None, eps2d=0.3, near_plane=0.01, far_plane=10000.0, radius_clip=0.0,
                 render_mode: int = RENDER_RGB, antialiased: bool = False, scaling_modifier: float = 1.0):
        self.model = model
        self.W, self.H = int(width), int(height)
        cap = int(isect_capacity) if isect_capacity is not None else max(8 * model.capacity, 1 << 20)
        self.cfg = RenderConfig(model.size, model.K, int(sh_degree), self.W, self.H, 16, int(camera_model),
                                eps2d, near_plane, far_plane, radius_clip, UTParams(), cap, int(render_mode),
                                1 if antialiased else 0, float(scaling_modifier), None)
        self.channels = {RENDER_RGB: 3, RENDER_D: 1, RENDER_ED: 1, RENDER_RGB_D: 4, RENDER_RGB_ED: 4}[int(render_mode)]
        self._masks = None
        self._alloc()
        dev = model.device
        self.render = torch.empty((self.H, self.W, self.channels), dtype=torch.float32, device=dev)
        self.alpha = torch.empty((self.H, self.W, 1), dtype=torch.float32, device=dev)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)

    def _alloc(self):
        cfg = RenderConfig.from_buffer_copy(self.cfg)
        cfg.N = self.model.capacity
        nbytes = capi.lib().lfs_render_workspace_bytes(C.byref(cfg))
        if nbytes == 0:
            raise capi.LfsError("lfs_render_workspace_bytes: " + capi.lib().lfs_last_error().decode())
        self.ws = torch.empty(nbytes, dtype=torch.uint8, device=self.model.device)

    def set_sh_degree(self, d: int):
        self.cfg.sh_degree = int(d)

    def set_tile_masks(self, masks: torch.Tensor | None):
        """[tile_h, tile_w] bool on the device, or None: tiles labelled False show the background and get no gradient
        (the `masks` argument of gsplat/Ops.h:97-160)."""
        if masks is None:
            self._masks, self.cfg.tile_masks = None, None
            return
        tw, th = (self.W + 15) // 16, (self.H + 15) // 16
        if masks.numel() != tw * th or masks.dtype != torch.bool or masks.device != self.render.device:
            raise RuntimeError(f"tile masks must be a bool tensor [{th}, {tw}] on {self.model.device}")
        self._masks = masks.contiguous().view(torch.uint8)
        self.cfg.tile_masks = self._masks.data_ptr()

    def forward(self, cam: Camera, background: torch.Tensor | None) -> RenderOutput:
        if cam.width != self.W or cam.height != self.H:
            raise RuntimeError("camera size does not match the rasterizer")
        self.cfg.N = self.model.size
        self.cfg.camera_model = int(cam.camera_model)
        self.cfg.radial_coeffs, self.cfg.tangential_coeffs, self.cfg.thin_prism_coeffs = cam.coefficient_pointers()
        self.cfg.shutter = int(cam.shutter)
        self.cfg.viewmat_end = None if cam.viewmat_end is None else cam.viewmat_end.data_ptr()
        p = self.model.struct()
        call("lfs_render_forward", C.byref(self.cfg), C.byref(p), ptr(cam.viewmat), ptr(cam.K),
             ptr(background), ptr(self.render), ptr(self.alpha), ptr(self.status), ptr(self.ws), self.ws.numel(), _stream())
        image = self.render if self.channels == 3 else (self.render[..., :3].contiguous() if self.channels == 4 else None)
        depth = None if self.channels == 3 else self.render[..., self.channels - 1:]
        return RenderOutput(image, self.alpha, self.W, self.H, self.status, depth, self.render)

    def forward_lists(self, cam: Camera, projected_event: torch.cuda.Event | None = None):
        """First half of forward(): per-Gaussian stage without colours and the tile lists. Needs only means, scales,
        rotations and opacities, so it can run while the SH tensors are still being updated on another stream.
        projected_event: recorded on the current stream between the projection kernel and the sorting kernels (an event
        that was recorded at least once before, so that its handle exists)."""
        if cam.width != self.W or cam.height != self.H:
            raise RuntimeError("camera size does not match the rasterizer")
        self.cfg.N = self.model.size
        self.cfg.camera_model = int(cam.camera_model)
        self.cfg.radial_coeffs, self.cfg.tangential_coeffs, self.cfg.thin_prism_coeffs = cam.coefficient_pointers()
        self.cfg.shutter = int(cam.shutter)
        self.cfg.viewmat_end = None if cam.viewmat_end is None else cam.viewmat_end.data_ptr()
        p = self.model.struct()
        ev = None
        if projected_event is not None:
            ev = int(projected_event.cuda_event)
            if not ev:
                raise RuntimeError("projected_event has no handle yet: record it once before the first use")
        call("lfs_render_forward_lists_event", C.byref(self.cfg), C.byref(p), ptr(cam.viewmat), ptr(cam.K), C.c_void_p(ev), ptr(self.ws),
             self.ws.numel(), _stream())

    def forward_shade(self, background: torch.Tensor | None) -> RenderOutput:
        """Second half: SH colours of the visible Gaussians, then blending. forward_lists + forward_shade == forward."""
        p = self.model.struct()
        call("lfs_render_forward_shade", C.byref(self.cfg), C.byref(p), ptr(background), ptr(self.render), ptr(self.alpha),
             ptr(self.status), ptr(self.ws), self.ws.numel(), _stream())
        image = self.render if self.channels == 3 else (self.render[..., :3].contiguous() if self.channels == 4 else None)
        depth = None if self.channels == 3 else self.render[..., self.channels - 1:]
        return RenderOutput(image, self.alpha, self.W, self.H, self.status, depth, self.render)

    def backward(self, v_render: torch.Tensor, grads: SplatData, background: torch.Tensor | None = None,
                 v_alpha: torch.Tensor | None = None, accumulate: bool = False, write_shN: bool = True,
                 sh_factors: bool = False):
        """write_shN=False leaves grads' shN tensor untouched (one-camera steps that update shN with adam_step_rank1_sh).
        sh_factors=True writes the two factors of the rank-1 shN rows, [N,6], at the start of grads' shN tensor instead
        of the rows (data-parallel steps of one camera per rank, GradExchange.step_split(rank1_sh=True))."""
        p, g = self.model.struct(), grads.struct()
        if not write_shN:
            g.shN = None
        flags = (1 if accumulate else 0) | (2 if sh_factors else 0)
        call("lfs_render_backward", C.byref(self.cfg), C.byref(p), ptr(background), ptr(self.alpha), ptr(v_render), ptr(v_alpha),
             C.byref(g), flags, ptr(self.ws), self.ws.numel(), _stream())

    def background_gradient(self, v_render: torch.Tensor) -> torch.Tensor:
        """v_bg_color of the autograd node (rasterizer_autograd.cpp:206-209): sum over pixels of v_render (1 - alpha) per
        channel, for trainers whose background colour is a parameter. Uses the alpha of the last forward."""
        if not hasattr(self, "_bg_ws"):
            self._bg_ws = torch.empty(4, dtype=torch.float64, device=self.render.device)
        out = torch.empty(self.channels, dtype=torch.float32, device=self.render.device)
        call("lfs_background_gradient", self.H, self.W, self.channels, ptr(v_render), ptr(self.alpha), ptr(out), ptr(self._bg_ws),
             self._bg_ws.numel() * 8, _stream())
        return out

    def backward_adam(self, v_render: torch.Tensor, exp_avg: SplatData, exp_avg_sq: SplatData, lrs, step_count: int,
                      background: torch.Tensor | None = None, v_alpha: torch.Tensor | None = None, beta1=0.9, beta2=0.999,
                      eps=1e-15, skip_shN=False, grad_scale=1.0):
        """backward() and FusedAdam::step in one call for steps of ONE camera: the gradients never go to memory (the small
        groups are updated inside the per-Gaussian gradient stage, shN from its rank-1 factors)."""
        p, m, v = self.model.struct(), exp_avg.struct(), exp_avg_sq.struct()
        lr = (C.c_float * 6)(*[float(x) for x in lrs])
        call("lfs_render_backward_adam", C.byref(self.cfg), C.byref(p), ptr(background), ptr(self.alpha), ptr(v_render),
             ptr(v_alpha), C.byref(m), C.byref(v), lr, float(beta1), float(beta2), float(eps), int(step_count),
             1 if skip_shN else 0, float(grad_scale), ptr(self.ws), self.ws.numel(), _stream())

    def adam_step_rank1_sh(self, exp_avg: SplatData, exp_avg_sq: SplatData, grads: SplatData, lrs, step_count: int,
                           beta1=0.9, beta2=0.999, eps=1e-15, skip_shN=False, grad_scale=1.0):
        """FusedAdam::step after backward(write_shN=False) of ONE camera: the shN rows are updated from gradient rows
        rebuilt on the fly as (SH basis of the view direction) x (sh0 gradient / Y_0); the other groups as usual."""
        p, m, v, g = self.model.struct(), exp_avg.struct(), exp_avg_sq.struct(), grads.struct()
        lr = (C.c_float * 6)(*[float(x) for x in lrs])
        call("lfs_adam_step_splats_rank1_sh", C.byref(self.cfg), C.byref(p), C.byref(m), C.byref(v), C.byref(g), lr, float(beta1),
             float(beta2), float(eps), int(step_count), 1 if skip_shN else 0, float(grad_scale), ptr(self.ws), self.ws.numel(),
             _stream())


    def state(self) -> dict:
        """Copies of the forward state in the workspace (per-Gaussian projection outputs and tile lists);
        synchronises. For inspection, tests and strategies that need radii / means2d."""
        view = capi.RenderView()
        cfg = RenderConfig.from_buffer_copy(self.cfg)   # the layout of the last forward: its N, not the capacity
        call("lfs_render_workspace_view", C.byref(cfg), ptr(self.ws), self.ws.numel(), C.byref(view))
        torch.cuda.synchronize()
        n_isects = int(self.status[1].item())
        n, tiles = int(self.cfg.N), ((self.W + 15) // 16) * ((self.H + 15) // 16)
        base = self.ws.data_ptr()

        def grab(p, count, dtype):
            nbytes = count * torch.empty(0, dtype=dtype).element_size()
            off = p - base
            return self.ws[off:off + nbytes].view(dtype).clone()

        return dict(radii=grab(view.radii, n * 2, torch.int32).view(n, 2),
                    means2d=grab(view.means2d, n * 2, torch.float32).view(n, 2),
                    depths=grab(view.depths, n, torch.float32),
                    tiles_per_gauss=grab(view.tiles_per_gauss, n, torch.int32),
                    tile_offsets=grab(view.tile_offsets, tiles + 1, torch.int32),
                    flatten_ids=grab(view.flatten_ids, n_isects, torch.int32),
                    last_ids=grab(view.last_ids, self.W * self.H, torch.int32).view(self.H, self.W),
                    records=grab(view.records, n * 16, torch.float32).view(n, 16), n_isects=n_isects)


class FastRasterizer:
    """fast_rasterize() + FastGSRasterize (src/training/rasterization/fast_rasterizer.cpp:13-71,
    fast_rasterizer_autograd.cpp): the default, non --gut path. EWA splatting with exact per-tile culling on the raw
    SplatData tensors; owns the workspace that carries the forward state to the backward. Image output is CHW like
    the reference's; `world_view_transform` is the camera's viewmat, `cam_position` is derived from it once per
    camera when not given."""

    def __init__(self, model: SplatData, width: int, height: int, sh_degree: int, instance_capacity: int | None = None,
                 near_plane: float = 0.01, far_plane: float = 1e10):
        self.model = model
        self.W, self.H = int(width), int(height)
        cap = int(instance_capacity) if instance_capacity is not None else max(8 * model.capacity, 1 << 20)
        self.cfg = capi.EwaConfig(model.size, model.K, (int(sh_degree) + 1) ** 2, self.W, self.H, 0.0, 0.0, 0.0, 0.0,
                                  float(near_plane), float(far_plane), cap)
        cfg = capi.EwaConfig.from_buffer_copy(self.cfg)
        cfg.N, cfg.focal_x, cfg.focal_y = model.capacity, 1.0, 1.0
        nbytes = capi.lib().lfs_ewa_workspace_bytes(C.byref(cfg))
        if nbytes == 0:
            raise capi.LfsError("lfs_ewa_workspace_bytes: " + capi.lib().lfs_last_error().decode())
        dev = model.device
        self.ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        self.image = torch.empty((3, self.H, self.W), dtype=torch.float32, device=dev)
        self.alpha = torch.empty((1, self.H, self.W), dtype=torch.float32, device=dev)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        self._cam = None

    def set_sh_degree(self, d: int):
        self.cfg.active_sh_bases = (int(d) + 1) ** 2

    @staticmethod
    def cam_position(viewmat: torch.Tensor) -> torch.Tensor:
        """-R^T t of the world-to-camera matrix (what Camera::cam_position holds)."""
        Rm, t = viewmat[:3, :3].double(), viewmat[:3, 3].double()
        return (-(Rm.T @ t)).float().contiguous()

    def forward(self, cam: Camera, background: torch.Tensor | None, cam_position: torch.Tensor | None = None) -> RenderOutput:
        if cam.width != self.W or cam.height != self.H:
            raise RuntimeError("camera size does not match the rasterizer")
        K = cam.K
        if not hasattr(cam, "_intrinsics"):
            cam._intrinsics = tuple(float(v) for v in (K[0, 0], K[1, 1], K[0, 2], K[1, 2]))  # one host read per camera
            cam._campos = self.cam_position(cam.viewmat) if cam_position is None else cam_position
        self.cfg.N = self.model.size
        self.cfg.focal_x, self.cfg.focal_y, self.cfg.center_x, self.cfg.center_y = cam._intrinsics
        self._cam = cam
        p = self.model.struct()
        call("lfs_ewa_forward", C.byref(self.cfg), C.byref(p), ptr(cam.viewmat), ptr(cam._campos), ptr(background), ptr(self.image),
             ptr(self.alpha), ptr(self.status), ptr(self.ws), self.ws.numel(), _stream())
        return RenderOutput(self.image, self.alpha, self.W, self.H, self.status)

    def backward(self, grad_image: torch.Tensor, grads: SplatData, background: torch.Tensor | None = None,
                 grad_alpha: torch.Tensor | None = None, accumulate: bool = False, densification_info: torch.Tensor | None = None,
                 write_shN: bool = True, grad_w2c: torch.Tensor | None = None):
        """grad_image [3,H,W] w.r.t. the final (background-blended) image; densification_info [2,N] is updated in place.
        write_shN=False leaves grads' shN tensor untouched (one-camera steps that update shN with adam_step_rank1_sh).
        grad_w2c: float32 [4,4] on the device, receives the camera-pose gradient (kernels_backward.cuh:160-173)."""
        if grad_w2c is not None and (grad_w2c.dtype != torch.float32 or grad_w2c.numel() != 16 or not grad_w2c.is_contiguous()):
            raise ValueError("grad_w2c must be a contiguous float32 [4,4] tensor")
        cam = self._cam
        p, g = self.model.struct(), grads.struct()
        if not write_shN:
            g.shN = None
        call("lfs_ewa_backward", C.byref(self.cfg), C.byref(p), ptr(cam.viewmat), ptr(cam._campos), ptr(background), ptr(self.alpha),
             ptr(grad_image), ptr(grad_alpha), C.byref(g), 1 if accumulate else 0, ptr(densification_info), ptr(grad_w2c), ptr(self.ws),
             self.ws.numel(), _stream())

    def adam_step_rank1_sh(self, exp_avg: SplatData, exp_avg_sq: SplatData, grads: SplatData, lrs, step_count: int,
                           beta1=0.9, beta2=0.999, eps=1e-15, skip_shN=False, grad_scale=1.0):
        """FusedAdam::step after backward(write_shN=False) of ONE camera (see Rasterizer.adam_step_rank1_sh)."""
        p, m, v, g = self.model.struct(), exp_avg.struct(), exp_avg_sq.struct(), grads.struct()
        lr = (C.c_float * 6)(*[float(x) for x in lrs])
        call("lfs_ewa_adam_step_rank1_sh", C.byref(self.cfg), C.byref(p), ptr(self._cam._campos), C.byref(m), C.byref(v), C.byref(g),
             lr, float(beta1), float(beta2), float(eps), int(step_count), 1 if skip_shN else 0, float(grad_scale), _stream())

    def state(self) -> dict:
        """Copies of the forward state (synchronises): per-Gaussian records, bounds, tile lists."""
        view = capi.EwaView()
        cfg = capi.EwaConfig.from_buffer_copy(self.cfg)   # the layout of the last forward: its N, not the capacity
        call("lfs_ewa_workspace_view", C.byref(cfg), ptr(self.ws), self.ws.numel(), C.byref(view))
        torch.cuda.synchronize()
        n, tiles = int(self.cfg.N), ((self.W + 15) // 16) * ((self.H + 15) // 16)
        n_inst = int(self.status[1].item())
        base = self.ws.data_ptr()

        def grab(p, count, dtype):
            nbytes = count * torch.empty(0, dtype=dtype).element_size()
            return self.ws[p - base:p - base + nbytes].view(dtype).clone()

        rec = grab(view.records, n * 12, torch.float32).view(n, 12)
        return dict(n_touched=grab(view.n_touched, n, torch.int32), bounds=grab(view.bounds, n * 4, torch.int16).view(n, 4),
                    mean2d=rec[:, 0:2], conic_opacity=torch.stack([rec[:, 2], rec[:, 3], rec[:, 4], rec[:, 5]], 1),
                    color=rec[:, 6:9], instance_ids=grab(view.instance_ids, n_inst, torch.int32),
                    tile_offsets=grab(view.tile_offsets, tiles + 1, torch.int32),
                    n_contrib=grab(view.n_contrib, self.W * self.H, torch.int32).view(self.H, self.W), n_instances=n_inst)


class PhotometricLoss:
    """Trainer::compute_photometric_loss and its backward in two kernels."""

    def __init__(self, width: int, height: int, device, lambda_dssim: float = 0.2):
        self.W, self.H, self.lam = int(width), int(height), float(lambda_dssim)
        self.ws = torch.empty(capi.lib().lfs_photometric_loss_workspace_bytes(self.H, self.W), dtype=torch.uint8, device=device)
        self.v_render = torch.empty((self.H, self.W, 3), dtype=torch.float32, device=device)
        self.loss = torch.zeros(4, dtype=torch.float32, device=device)

    def __call__(self, render_hwc: torch.Tensor, target_chw: torch.Tensor, grad_scale: float = 1.0, want_grad: bool = True):
        call("lfs_photometric_loss", self.H, self.W, self.lam, float(grad_scale), ptr(render_hwc), ptr(target_chw),
             ptr(self.v_render) if want_grad else None, ptr(self.loss), ptr(self.ws), self.ws.numel(), _stream())
        return self.loss, self.v_render


GEOMETRY_GROUPS = ("means", "scaling_raw", "rotation_raw", "opacity_raw")   # what the tile lists depend on
COLOR_GROUPS = ("sh0", "shN")


def adam_step_groups(model: SplatData, exp_avg: SplatData, exp_avg_sq: SplatData, grads: SplatData, lrs, step_count: int,
                     groups, beta1=0.9, beta2=0.999, eps=1e-15, grad_scale=1.0, ctas_per_sm=0):
    """The fused Adam on a subset of the six parameter groups (one launch). Splitting FusedAdam::step into the geometry
    groups and the colour groups lets the colour update (three quarters of the bytes) run on a second stream while the
    next step's projection and tile lists are built from the geometry groups."""
    segs = []
    for name in groups:
        gi = PARAM_NAMES.index(name)
        n = model.size * model._w[name]
        if n == 0:
            continue
        segs.append(capi.AdamSegment(model._full[name].data_ptr(), exp_avg._full[name].data_ptr(), exp_avg_sq._full[name].data_ptr(),
                                     grads._full[name].data_ptr(), n, float(lrs[gi])))
    if not segs:
        return
    arr = (capi.AdamSegment * len(segs))(*segs)
    call("lfs_adam_step_segments", len(segs), arr, float(beta1), float(beta2), float(eps), int(step_count), float(grad_scale),
         int(ctas_per_sm), _stream())


def regularization(model: SplatData, grads: SplatData, scale_reg: float, opacity_reg: float, out: torch.Tensor | None = None):
    """Trainer::compute_scale_reg_loss / compute_opacity_reg_loss (src/training/trainer.cpp:136-174) in one launch:
    adds the regularisers' gradients to `grads` and returns a device float[2] = (scale loss, opacity loss). Unlike the
    reference there is no host read; call .tolist() on the result if the values are needed on the host."""
    if out is None:
        out = torch.zeros(2, dtype=torch.float32, device=model.device)
    call("lfs_regularization", model.size, ptr(model._full["scaling_raw"]), ptr(model._full["opacity_raw"]), float(scale_reg),
         float(opacity_reg), ptr(grads._full["scaling_raw"]), ptr(grads._full["opacity_raw"]), ptr(out), _stream())
    return out


def adam_step_splats(model: SplatData, exp_avg: SplatData, exp_avg_sq: SplatData, grads: SplatData, lrs, step_count: int,
                     beta1=0.9, beta2=0.999, eps=1e-15, skip_shN=False, first_row=0, n_rows=None, grad_scale=1.0):
    """One launch of the fused Adam over all six groups (FusedAdam::step)."""
    n_rows = model.size - first_row if n_rows is None else n_rows
    lr = (C.c_float * 6)(*[float(x) for x in lrs])
    p, m, v, g = model.struct(), exp_avg.struct(), exp_avg_sq.struct(), grads.struct()
    call("lfs_adam_step_splats", model.size, model.K, C.byref(p), C.byref(m), C.byref(v), C.byref(g), lr, float(beta1),
         float(beta2), float(eps), int(step_count), 1 if skip_shN else 0, int(first_row), int(n_rows), float(grad_scale), _stream())
