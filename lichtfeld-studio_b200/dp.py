"""Camera-parallel data parallelism for the training step: each rank renders its own camera(s) against
replicated Gaussians; the only exchange is the sum of the flat gradient buffer, followed by Adam.
The reference is single-GPU (no collectives anywhere in its tree); this is the multi-GPU design of the
training path, one process per GPU over torch.distributed.

Three interchangeable exchanges (all leave bit-identical parameters on every rank):
  "allreduce" : all_reduce(grads)              -> full fused Adam on every rank
  "sharded"   : reduce_scatter(grads)          -> Adam on this rank's flat shard -> all_gather(params)
  "fused_p2p" : one CUDA kernel per rank that reads every rank's gradient shard through NVLink peer
                pointers, sums in a fixed order, applies Adam and writes the new parameters into every
                rank's buffer (lfs_dp_reduce_adam_broadcast); needs symmetric (peer-mapped) buffers.
The flat buffers are group-major [means | sh0 | shN | scaling | rotation | opacity] x capacity rows, so a
contiguous shard intersects at most six groups, each with its own learning rate.
"""
from __future__ import annotations

import ctypes as C
import os

import torch
import torch.distributed as dist

from . import _capi as capi
from .trainer import PARAM_NAMES, SplatData, row_widths


def shard_bounds(total: int, world: int, rank: int, align: int = 4):
    """Equal shards of ceil(total / world) rounded up to `align` elements; the last shards may be short or
    empty. Returns (first, count, shard_len)."""
    per = -(-total // world)
    per = -(-per // align) * align
    lo = min(rank * per, total)
    hi = min(lo + per, total)
    return lo, hi - lo, per


def group_segments(capacity: int, K: int, lo: int, n: int, lrs, skip_shN: bool = False):
    """Intersect the flat element range [lo, lo + n) with the six parameter groups.
    Returns [(group index, flat offset, count, lr)]; the shN group is dropped when skip_shN."""
    w = row_widths(K)
    out, off = [], 0
    for gi, name in enumerate(PARAM_NAMES):
        size = capacity * w[name]
        a, b = max(lo, off), min(lo + n, off + size)
        if b > a and not (skip_shN and name == "shN"):
            out.append((gi, a, b - a, float(lrs[gi])))
        off += size
    return out


GEOMETRY_CLASS = ("means", "scaling_raw", "rotation_raw", "opacity_raw")   # what projection and tile lists read
COLOR_CLASS = ("sh0", "shN")


def class_segments(capacity: int, K: int, names, world: int, rank: int, lrs, skip_shN: bool = False, align: int = 4):
    """Shard the groups `names` (a class of parameter groups) over `world` ranks: the class's flat ranges are laid end
    to end, cut into equal shards (rounded up to `align` elements) and mapped back to the flat buffer.
    Returns (segments [(group index, flat offset, count, lr, offset inside this rank's class shard)], shard length).
    Every element of the class belongs to exactly one rank. The partition does not depend on skip_shN (the moments
    keep their place); a skipped shN group only drops its segments."""
    w = row_widths(K)
    ranges, off = [], 0
    for gi, name in enumerate(PARAM_NAMES):
        size = capacity * w[name]
        if name in names and size > 0:
            ranges.append((gi, off, size))
        off += size
    total = sum(r[2] for r in ranges)
    lo, n, per = shard_bounds(total, world, rank, align)
    out, pos = [], 0
    for gi, goff, size in ranges:
        a, b = max(lo, pos), min(lo + n, pos + size)
        if b > a and not (skip_shN and PARAM_NAMES[gi] == "shN"):
            out.append((gi, goff + (a - pos), b - a, float(lrs[gi]), a - lo))
        pos += size
    return out, per


class GradExchange:
    """Owns the sharded optimizer state and performs exchange + Adam for one rank."""

    # slots of the flag array (lfs_dp_signal / lfs_dp_wait)
    SLOT_GRADS, SLOT_EXCHANGED, SLOT_COLOR = 0, 1, 2

    def __init__(self, model: SplatData, grads: SplatData, lrs, mode: str = "sharded", betas=(0.9, 0.999), eps=1e-15,
                 group=None, peer_ptrs=None, ordering: str | None = None, wait_timeout_s: float = 20.0,
                 multicast: bool | None = None):
        """ordering (fused_p2p only; default: environment LFS_DP_ORDERING, else "flags"): how the ranks' kernels are ordered
        around the peer-memory exchange. "flags": every rank stores its step number into a flag word of every peer
        (lfs_dp_signal) and waits, for at most `wait_timeout_s` (<= 60), until all its own words show the step
        (lfs_dp_wait); a wait that runs out sets a status word that raise_if_failed() reports, and the stream carries on.
        "nccl": stream-ordered 4-byte all-reduces.
        multicast (fused_p2p; default: environment LFS_DP_MULTICAST, else off): send the new parameters with multimem.st through
        the NVSwitch multicast mapping of the parameter buffer (peer_ptrs[2], from symmetric_flat_buffers) when there is one."""
        self.model, self.grads, self.lrs, self.mode = model, grads, [float(x) for x in lrs], mode
        self.betas, self.eps, self.group = betas, eps, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        total = model.flat.numel()
        self.lo, self.n, self.per = shard_bounds(total, self.world, self.rank)
        dev = model.flat.device
        if mode == "allreduce":
            self.m, self.v = model.like(), model.like()
        else:
            # moments only for this rank's shard (optimizer-state sharding)
            self.m = torch.zeros(self.per, dtype=torch.float32, device=dev)
            self.v = torch.zeros(self.per, dtype=torch.float32, device=dev)
            self.g_shard = torch.zeros(self.per, dtype=torch.float32, device=dev)
            self.padded = self.per * self.world
        self.mc_params = 0
        if mode == "fused_p2p":
            if peer_ptrs is None:
                raise RuntimeError("fused_p2p needs the peer-mapped addresses of every rank's parameter and gradient buffers")
            self.peer_grads, self.peer_params = peer_ptrs[0], peer_ptrs[1]
            want_mc = (os.environ.get("LFS_DP_MULTICAST", "0") not in ("", "0")) if multicast is None else bool(multicast)
            self.mc_params = int(peer_ptrs[2]) if (want_mc and len(peer_ptrs) > 2 and self.world > 1) else 0
        ordering = ordering or os.environ.get("LFS_DP_ORDERING", "flags")
        if ordering not in ("flags", "nccl"):
            raise ValueError(f"ordering {ordering!r}: expected 'flags' or 'nccl'")
        self.flags, self.peer_flags = None, None
        if mode == "fused_p2p" and self.world > 1 and ordering == "flags":
            self.flags, self.peer_flags = symmetric_flags(dev, group)
        self.ordering = ordering if self.flags is not None else "nccl"
        self.wait_timeout_ns = int(wait_timeout_s * 1e9)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev) if self.flags is not None else None
        self.step_count = 0
        self._split = None   # lazily built state of step_split()
        self.timing = None   # set to a list to collect (name, start event, end event) of every rendezvous
        self.color_ctas_per_sm = int(os.environ.get("LFS_DP_COLOR_CTAS", "1"))   # launch footprint of the overlapped part
        # when the colour exchange may start: 0 = with the geometry exchange (every rank's gradients are written), 1 = after this
        # rank's geometry kernel, 2 = after every rank's geometry kernel (the exchange on the critical path then has NVLink to itself)
        # Measured on B200s (train_1m): with 8 ranks 2 is fastest (3.16 against 3.20 ms: the exchange on the critical path takes
        # 0.15 instead of 0.5 ms), with 4 ranks 2 and 0 are level (3.045 / 3.054 ms), with 2 ranks 0 is fastest (2.89 against
        # 2.95 ms: there is little traffic to compete with).
        default_after = "2" if self.world >= 4 else "0"
        self.color_after_geometry = int(os.environ.get("LFS_DP_COLOR_AFTER_GEOMETRY", default_after) or 0)

    # -- helpers --------------------------------------------------------------------------------
    def _stream(self):
        return capi.vp(torch.cuda.current_stream().cuda_stream)

    def _rendezvous(self, token, group, name, slot=None):
        """No rank's later kernels start before every rank's earlier ones (on the current stream) finished. With flags:
        lfs_dp_barrier (signal + bounded wait) on slot `slot` with this step's number (bounded wait, see raise_if_failed); else a
        stream-ordered 4-byte all-reduce. When `timing` is a list the wait (which includes waiting for the slowest rank) is
        bracketed by events."""
        if self.timing is not None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        if self.flags is not None and slot is not None:
            pf = (C.c_void_p * self.world)(*self.peer_flags)
            capi.call("lfs_dp_barrier", self.world, pf, self.rank, int(slot), int(self.step_count), self.wait_timeout_ns,
                      capi.vp(self.status.data_ptr()), self._stream())
        else:
            dist.all_reduce(token, group=group)
        if self.timing is not None:
            e1.record()
            self.timing.append((name, e0, e1))

    def raise_if_failed(self):
        """Reads the status word of the bounded waits (synchronises). Raises when a wait ran out, naming the ranks whose
        flag never arrived: they stopped stepping (crashed, hung on the host, or left the job)."""
        if self.status is None:
            return
        msg = describe_wait_status(self.status.tolist(), self.world, self.wait_timeout_ns / 1e9)
        if msg:
            raise RuntimeError(msg)

    def collect_timing(self):
        """[(name, ms)] of the recorded rendezvous; synchronises."""
        torch.cuda.synchronize()
        out = [(n, a.elapsed_time(b)) for n, a, b in (self.timing or [])]
        if self.timing is not None:
            self.timing = []
        return out

    def _adam_shard(self, iteration: int, grad_shard: torch.Tensor, grad_scale: float):
        segs = group_segments(self.model.capacity, self.model.K, self.lo, self.n, self.lrs, skip_shN=(iteration <= 1000))
        arr = (capi.AdamSegment * max(len(segs), 1))()
        base = self.model.flat.data_ptr()
        for i, (gi, off, cnt, lr) in enumerate(segs):
            rel = off - self.lo
            arr[i] = capi.AdamSegment(base + 4 * off, self.m.data_ptr() + 4 * rel, self.v.data_ptr() + 4 * rel,
                                      grad_shard.data_ptr() + 4 * rel, cnt, lr)
        capi.call("lfs_adam_step_segments", len(segs), arr, self.betas[0], self.betas[1], self.eps, self.step_count,
                  float(grad_scale), 0, self._stream())

    # -- the exchange ---------------------------------------------------------------------------
    def step(self, iteration: int, grad_scale: float | None = None, adam_fn=None):
        """Sum gradients over ranks and apply Adam. grad_scale defaults to 1 / world (mean over the camera
        batch). adam_fn(param_view, m_view, v_view, grad_view, lr, step_count, grad_scale) replaces the CUDA
        Adam for host-only testing of the exchange logic."""
        self.step_count += 1
        gs = 1.0 / self.world if grad_scale is None else grad_scale
        model, grads = self.model, self.grads
        if self.mode == "allreduce":
            if self.world > 1:
                dist.all_reduce(grads.flat, group=self.group)
            if adam_fn is None:
                from .trainer import adam_step_splats
                self.m.size = self.v.size = grads.size = model.size
                adam_step_splats(model, self.m, self.v, grads, self.lrs, self.step_count, self.betas[0], self.betas[1], self.eps,
                                 skip_shN=(iteration <= 1000), grad_scale=gs)
            else:
                for gi, off, cnt, lr in group_segments(model.capacity, model.K, 0, model.flat.numel(), self.lrs, iteration <= 1000):
                    adam_fn(model.flat[off:off + cnt], self.m.flat[off:off + cnt], self.v.flat[off:off + cnt],
                            grads.flat[off:off + cnt], lr, self.step_count, gs)
            return
        if self.mode == "sharded":
            total = model.flat.numel()
            if self.world > 1:
                if self.padded != total:
                    src = torch.zeros(self.padded, dtype=torch.float32, device=grads.flat.device)
                    src[:total].copy_(grads.flat)
                else:
                    src = grads.flat
                dist.reduce_scatter_tensor(self.g_shard, src, group=self.group)
            else:
                self.g_shard[: self.n].copy_(grads.flat[self.lo:self.lo + self.n])
            if adam_fn is None:
                self._adam_shard(iteration, self.g_shard, gs)
            else:
                for gi, off, cnt, lr in group_segments(model.capacity, model.K, self.lo, self.n, self.lrs, iteration <= 1000):
                    rel = off - self.lo
                    adam_fn(model.flat[off:off + cnt], self.m[rel:rel + cnt], self.v[rel:rel + cnt], self.g_shard[rel:rel + cnt],
                            lr, self.step_count, gs)
            if self.world > 1:
                if self.padded != total:
                    out = torch.empty(self.padded, dtype=torch.float32, device=model.flat.device)
                    mine = torch.zeros(self.per, dtype=torch.float32, device=model.flat.device)
                    mine[: self.n].copy_(model.flat[self.lo:self.lo + self.n])
                    dist.all_gather_into_tensor(out, mine, group=self.group)
                    model.flat.copy_(out[:total])
                else:
                    dist.all_gather_into_tensor(model.flat, model.flat[self.lo:self.lo + self.n].clone(), group=self.group)
            return
        if self.mode == "fused_p2p":
            # stream-ordered rendezvous: every rank's backward has written its gradients
            token = torch.zeros(1, device=model.flat.device)
            self._rendezvous(token, self.group, "rendezvous_gradients_written", self.SLOT_GRADS)
            segs = group_segments(model.capacity, model.K, self.lo, self.n, self.lrs, skip_shN=(iteration <= 1000))
            arr = (capi.DpSegment * max(len(segs), 1))()
            for i, (gi, off, cnt, lr) in enumerate(segs):
                rel = off - self.lo
                arr[i] = capi.DpSegment(off, cnt, self.m.data_ptr() + 4 * rel, self.v.data_ptr() + 4 * rel, lr)
            order = [(self.rank + i) % self.world for i in range(self.world)]
            pg = (C.c_void_p * self.world)(*[self.peer_grads[r] for r in order])
            pp = (C.c_void_p * self.world)(*[self.peer_params[r] for r in order])
            capi.call("lfs_dp_reduce_adam_broadcast", self.world, pg, pp, capi.vp(self.mc_params or None), len(segs), arr, self.betas[0],
                      self.betas[1], self.eps, self.step_count, float(gs), 0, self._stream())
            # nobody may read parameters or overwrite gradients before every rank's kernel has finished
            self._rendezvous(token, self.group, "rendezvous_exchange_done", self.SLOT_EXCHANGED)
            return
        raise ValueError(self.mode)

    # -- split exchange: geometry groups now, colour groups under the next step's projection and sorting -------
    def _split_state(self, side_stream):
        if self._split is None:
            dev = self.model.flat.device
            st = {"side": side_stream, "group_b": dist.new_group() if (self.world > 1 and self.flags is None) else None,   # second communicator: NCCL ordering only
                  "ev_grads": torch.cuda.Event(), "ev_geo": torch.cuda.Event(), "ev_color": torch.cuda.Event(), "pending": False, "color_args": None}
            for cls, names in (("geo", GEOMETRY_CLASS), ("col", COLOR_CLASS)):
                _, per = class_segments(self.model.capacity, self.model.K, names, self.world, self.rank, self.lrs)
                st[cls + "_m"] = torch.zeros(max(per, 4), dtype=torch.float32, device=dev)
                st[cls + "_v"] = torch.zeros(max(per, 4), dtype=torch.float32, device=dev)
            st["token_a"] = torch.zeros(1, device=dev)
            st["token_b"] = torch.zeros(1, device=dev)
            self._split = st
        return self._split

    def _fused_call(self, segs, m, v, gs, ctas_per_sm=0):
        arr = (capi.DpSegment * max(len(segs), 1))()
        for i, (gi, off, cnt, lr, rel) in enumerate(segs):
            arr[i] = capi.DpSegment(off, cnt, m.data_ptr() + 4 * rel, v.data_ptr() + 4 * rel, lr)
        order = [(self.rank + i) % self.world for i in range(self.world)]
        pg = (C.c_void_p * self.world)(*[self.peer_grads[r] for r in order])
        pp = (C.c_void_p * self.world)(*[self.peer_params[r] for r in order])
        capi.call("lfs_dp_reduce_adam_broadcast", self.world, pg, pp, capi.vp(self.mc_params or None), len(segs), arr, self.betas[0],
                  self.betas[1], self.eps, self.step_count, float(gs), int(ctas_per_sm), self._stream())

    def _rank1_call(self, seg, m, v, gs, sh_degree, ctas_per_sm=0):
        """The shN part of this rank's colour shard from every rank's factor buffer (see Rasterizer.backward(sh_factors=True))."""
        gi, off, cnt, lr, rel = seg
        w = row_widths(self.model.K)
        shn_off = self.model.capacity * (w["means"] + w["sh0"])      # flat offset of the shN tensor (group-major layout)
        order = [(self.rank + i) % self.world for i in range(self.world)]
        pf = (C.c_void_p * self.world)(*[self.peer_grads[r] + 4 * shn_off for r in order])
        ps = (C.c_void_p * self.world)(*[self.peer_params[r] + 4 * shn_off for r in order])
        mc = capi.vp(self.mc_params + 4 * shn_off) if self.mc_params else capi.vp(None)
        capi.call("lfs_dp_sh_rank1_adam_broadcast", self.world, pf, ps, mc, self.model.size, self.model.K, int(sh_degree),
                  off - shn_off, cnt, capi.vp(m.data_ptr() + 4 * rel), capi.vp(v.data_ptr() + 4 * rel), float(lr), self.betas[0],
                  self.betas[1], self.eps, self.step_count, float(gs), int(ctas_per_sm), self._stream())

    def step_split(self, iteration: int, side_stream, grad_scale: float | None = None, rank1_sh: bool = False,
                   sh_degree: int | None = None, defer_color: bool = False):
        """fused_p2p in two parts. On the current stream: rendezvous, reduce + Adam + broadcast of the geometry groups
        (means, scales, rotations, opacities), rendezvous. On `side_stream`: the same for the colour groups (sh0, shN:
        three quarters of the bytes), finishing with its own rendezvous on a second communicator. The caller may start
        the next step's projection and tile lists right away and must call wait_color() before anything reads the
        colour groups or overwrites the gradients. defer_color: the colour kernels are not enqueued here but by
        launch_color(after=event), which the caller invokes once the next step's forward_lists(projected_event=event) is
        enqueued: the colour exchange then starts when the projection kernel has finished and runs next to the sorting
        kernels (next to the projection, its queued peer stores slowed that kernel threefold). rank1_sh: every rank
        rendered ONE camera and ran backward(sh_factors=True); the shN gradient then crosses NVLink as 24 bytes per Gaussian and rank (sh_degree = the
        degree the forward used)."""
        if self.mode != "fused_p2p":
            raise RuntimeError("step_split needs mode fused_p2p")
        if rank1_sh and sh_degree is None:
            raise RuntimeError("rank1_sh needs the SH degree of the forward")
        st = self._split_state(side_stream)
        self.step_count += 1
        gs = 1.0 / self.world if grad_scale is None else grad_scale
        model = self.model
        skip = iteration <= 1000
        main = torch.cuda.current_stream()
        # every rank's backward has written its gradients
        self._rendezvous(st["token_a"], self.group, "rendezvous_gradients_written", self.SLOT_GRADS)
        st["ev_grads"].record(main)
        segs, _ = class_segments(model.capacity, model.K, GEOMETRY_CLASS, self.world, self.rank, self.lrs)
        self._fused_call(segs, st["geo_m"], st["geo_v"], gs)
        if self.color_after_geometry == 1:
            st["ev_geo"].record(main)
        self._rendezvous(st["token_a"], self.group, "rendezvous_geometry_done", self.SLOT_EXCHANGED)   # every rank's geometry kernel has finished
        if self.color_after_geometry == 2:
            st["ev_geo"].record(main)
        st["pending"] = True
        st["color_args"] = (skip, rank1_sh, sh_degree, gs)
        if not defer_color:
            self.launch_color()

    def launch_color(self, after: torch.cuda.Event | None = None):
        """Enqueue the colour part of the last step_split() on the side stream; `after`: an event (already recorded on some
        stream) that it additionally waits for. A no-op when it is already enqueued."""
        st = self._split
        if st is None or st.get("color_args") is None:
            return
        skip, rank1_sh, sh_degree, gs = st["color_args"]
        st["color_args"] = None
        model = self.model
        with torch.cuda.stream(st["side"]):
            # the colour exchange starts once every rank's gradients are written; optionally only after this rank's geometry
            # kernel or every rank's, so that the exchange on the critical path has the NVLink ports to itself
            st["side"].wait_event(st["ev_geo"] if self.color_after_geometry else st["ev_grads"])
            if after is not None:
                st["side"].wait_event(after)
            segs, _ = class_segments(model.capacity, model.K, COLOR_CLASS, self.world, self.rank, self.lrs, skip_shN=skip)
            # small footprint: this kernel shares the SMs with the next step's projection and sorting
            if rank1_sh:
                # every rank's backward wrote the factors of its rank-1 shN rows instead of the rows: sh0 goes through the
                # element-wise kernel, shN through the kernel that sums the outer products
                plain = [sg for sg in segs if PARAM_NAMES[sg[0]] != "shN"]
                if plain:
                    self._fused_call(plain, st["col_m"], st["col_v"], gs, ctas_per_sm=self.color_ctas_per_sm)
                for sg in segs:
                    if PARAM_NAMES[sg[0]] == "shN":
                        self._rank1_call(sg, st["col_m"], st["col_v"], gs, sh_degree, ctas_per_sm=self.color_ctas_per_sm)
            else:
                self._fused_call(segs, st["col_m"], st["col_v"], gs, ctas_per_sm=self.color_ctas_per_sm)
            self._rendezvous(st["token_b"], st["group_b"], "rendezvous_color_done_side", self.SLOT_COLOR)  # every rank's colour kernel has finished
            st["ev_color"].record(st["side"])

    def wait_color(self):
        """Make the current stream wait for the colour part of the last step_split()."""
        if self._split is not None and self._split["pending"]:
            self.launch_color()
            torch.cuda.current_stream().wait_event(self._split["ev_color"])


class PeerLeft(RuntimeError):
    """A peer rank stopped stepping (it raised, exited, or did not reach the step in time)."""

    def __init__(self, message: str, ranks):
        super().__init__(message)
        self.ranks = list(ranks)


class PeerWatch:
    """Host side of failure detection, over the job's key-value store (torch.distributed's TCPStore / FileStore): what the
    ranks tell each other BEFORE they launch a step, so that nobody enqueues an exchange a peer will never join.

    Every rank publishes the number of the step it is about to launch (ready) and, when it stops for good (an exception
    leaves the `with` block, or leave() is called), a mark with the reason. ready(step) returns once every peer has
    published that step or a later one; it raises PeerLeft naming the ranks that left, or that did not get there within
    `timeout_s`. The device-side counterpart, for a rank that dies without saying so, are the bounded waits of
    lfs_dp_barrier (GradExchange.raise_if_failed). A store round trip costs tens of microseconds per peer: call ready() every
    `interval` steps (it returns at once on the others)."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, interval: int = 1, prefix: str = "lfs_dp_watch",
                 poll_s: float = 0.002):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.timeout_s, self.interval, self.prefix, self.poll_s = float(timeout_s), max(1, int(interval)), prefix, float(poll_s)

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def leave(self, reason: str = "left"):
        self.store.set(self._key("left", self.rank), reason or "left")

    def left(self) -> dict:
        """{rank: reason} of the peers that have left."""
        out = {}
        for r in range(self.world):
            if r != self.rank and self.store.check([self._key("left", r)]):
                out[r] = self.store.get(self._key("left", r)).decode()
        return out

    def ready(self, step: int):
        if step % self.interval:
            return
        import time
        self.store.set(self._key("step", self.rank), str(int(step)))
        deadline = time.monotonic() + self.timeout_s
        waiting = [r for r in range(self.world) if r != self.rank]
        while True:
            gone = self.left()
            if gone:
                raise PeerLeft(f"data-parallel step {step}: ranks {sorted(gone)} left the job ({gone})", sorted(gone))
            waiting = [r for r in waiting
                       if not (self.store.check([self._key("step", r)]) and int(self.store.get(self._key("step", r))) >= step)]
            if not waiting:
                return
            if time.monotonic() > deadline:
                raise PeerLeft(f"data-parallel step {step}: ranks {waiting} did not get there within {self.timeout_s:.1f} s", waiting)
            time.sleep(self.poll_s)

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        if exc_type is not None and not issubclass(exc_type, PeerLeft):
            self.leave(f"{exc_type.__name__}: {exc}")
        return False


def describe_wait_status(status, world: int, timeout_s: float) -> str | None:
    """The status word of lfs_dp_wait / lfs_dp_barrier ({failed, bit mask of the missing ranks, slot, step}) as a message,
    or None when no wait ran out."""
    failed, mask, slot, step = (int(x) for x in status[:4])
    if not failed:
        return None
    missing = [r for r in range(world) if mask >> r & 1]
    return (f"data-parallel step: ranks {missing} did not reach step {step} (flag slot {slot}) within {timeout_s:.1f} s; "
            f"the parameters of this step are not valid")


def symmetric_flat_buffers(numel: int, device, group=None):
    """Two peer-mapped float32 buffers (parameters, gradients) of `numel` elements and the device addresses
    of every rank's copies, via torch's symmetric memory (CUDA VMM over NVLink). Returns
    (param_flat, grad_flat, (peer_grad_ptrs, peer_param_ptrs, multicast address of the parameter buffer or 0))."""
    import torch.distributed._symmetric_memory as symm_mem
    name = (group or dist.group.WORLD).group_name
    if hasattr(symm_mem, "enable_symm_mem_for_group"):
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")   # deprecated (a no-op) in newer torch, required by older ones
            try:
                symm_mem.enable_symm_mem_for_group(name)
            except Exception:
                pass
    p = symm_mem.empty(numel, dtype=torch.float32, device=device)
    g = symm_mem.empty(numel, dtype=torch.float32, device=device)
    hp = symm_mem.rendezvous(p, name)
    hg = symm_mem.rendezvous(g, name)
    p.zero_(); g.zero_()
    mc = int(getattr(hp, "multicast_ptr", 0) or 0)     # 0 where the GPUs / the driver offer no NVSwitch multicast
    return p, g, ([int(x) for x in hg.buffer_ptrs], [int(x) for x in hp.buffer_ptrs], mc)


def symmetric_flags(device, group=None):
    """One zeroed, peer-mapped int32 flag array per rank for lfs_dp_signal / lfs_dp_wait. Returns (local tensor,
    [device address of every rank's array, indexed by rank])."""
    import torch.distributed._symmetric_memory as symm_mem
    name = (group or dist.group.WORLD).group_name
    f = symm_mem.empty(capi.LFS_DP_FLAG_WORDS, dtype=torch.int32, device=device)
    h = symm_mem.rendezvous(f, name)
    f.zero_()
    torch.cuda.synchronize()
    dist.barrier(group=group)      # nobody signals before every array is zeroed
    return f, [int(x) for x in h.buffer_ptrs]
