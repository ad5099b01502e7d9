"""On-disk formats either side of the training step.

* PLY export / import compatible with the reference (`SplatData::save_ply`, src/core/splat_data.cpp:113-169,
  :402-418, :483-503; read back by src/loader/formats/ply.cpp): binary little-endian, one `vertex` element of
  float32 properties  x y z nx ny nz f_dc_* f_rest_* opacity scale_* rot_*,  SH written channel-major, raw
  logit opacity / log scale, normalised quaternions. The interleaved rows are built on the device by one kernel
  (`lfs_ply_pack_rows`) and cross PCIe once through a pinned buffer.
* Checkpoint (no counterpart file format in the reference, which resumes from PLY only): parameters, both Adam
  moments, the step count, learning rates and strategy counters in one flat binary file:
      magic "LFSCKPT1" | uint64 header length | JSON header | float32 payload (params, exp_avg, exp_avg_sq rows)
  Each payload section is the six groups [means | sh0 | shN | scaling | rotation | opacity] of the LIVE rows."""
from __future__ import annotations

import ctypes as C
import json
import os
import struct

import numpy as np
import torch

from . import _capi as capi
from ._capi import call, ptr
from .trainer import PARAM_NAMES, SplatData

_MAGIC = b"LFSCKPT1"


def ply_attribute_names(K: int) -> list[str]:
    """SplatData::get_attribute_names (splat_data.cpp:402-418) for K SH bases per channel."""
    a = ["x", "y", "z", "nx", "ny", "nz"]
    a += [f"f_dc_{i}" for i in range(3)]
    a += [f"f_rest_{i}" for i in range(3 * (K - 1))]
    a += ["opacity"] + [f"scale_{i}" for i in range(3)] + [f"rot_{i}" for i in range(4)]
    return a


def ply_header(n: int, K: int) -> bytes:
    lines = ["ply", "format binary_little_endian 1.0", f"element vertex {n}"]
    lines += [f"property float {name}" for name in ply_attribute_names(K)]
    lines.append("end_header")
    return ("\n".join(lines) + "\n").encode("ascii")


def _stream():
    return capi.vp(torch.cuda.current_stream().cuda_stream)


def pack_rows(model: SplatData) -> torch.Tensor:
    """[N, 14 + 3K] float32 vertex rows on the model's device (CUDA only: there is no host fallback)."""
    rows = torch.empty((model.size, 14 + 3 * model.K), dtype=torch.float32, device=model.device)
    p = model.struct()
    call("lfs_ply_pack_rows", model.size, model.K, C.byref(p), ptr(rows), _stream())
    return rows


def save_ply(model: SplatData, root: str, iteration: int = 0, stem: str = "") -> str:
    """SplatData::save_ply: writes root/splat_<iteration>.ply (or root/<stem>.ply) and returns the path."""
    os.makedirs(root, exist_ok=True)
    path = os.path.join(root, f"{stem}.ply" if stem else f"splat_{iteration}.ply")
    rows = pack_rows(model)
    host = torch.empty(rows.shape, dtype=torch.float32, pin_memory=True)
    host.copy_(rows, non_blocking=True)
    torch.cuda.current_stream().synchronize()
    with open(path, "wb") as f:
        f.write(ply_header(model.size, model.K))
        f.write(host.numpy().tobytes())
    return path


def read_ply(path: str):
    """Parse a binary little-endian PLY whose vertex properties are all float32 (what save_ply writes and what the
    reference's loader accepts). Returns (names, rows [N, len(names)] float32)."""
    with open(path, "rb") as f:
        data = f.read()
    end = data.find(b"end_header\n")
    if not data.startswith(b"ply") or end < 0:
        raise RuntimeError(f"{path}: not a PLY file")
    header = data[:end].decode("ascii").split("\n")
    if "format binary_little_endian 1.0" not in header:
        raise RuntimeError(f"{path}: only binary_little_endian 1.0 is supported")
    n, names, in_vertex = None, [], False
    for line in header:
        tok = line.split()
        if not tok:
            continue
        if tok[0] == "element":
            in_vertex = tok[1] == "vertex"
            if in_vertex:
                n = int(tok[2])
        elif tok[0] == "property" and in_vertex:
            if tok[1] not in ("float", "float32"):
                raise RuntimeError(f"{path}: vertex property {tok[-1]} is {tok[1]}, expected float")
            names.append(tok[-1])
    if n is None:
        raise RuntimeError(f"{path}: no vertex element")
    body = np.frombuffer(data, dtype="<f4", count=n * len(names), offset=end + len(b"end_header\n"))
    return names, body.reshape(n, len(names))


def load_ply(path: str, device, capacity: int | None = None) -> SplatData:
    """Read a Gaussian-splat PLY into a SplatData (properties may come in any order; SH degree from the f_rest count)."""
    names, rows = read_ply(path)
    n_rest = sum(1 for x in names if x.startswith("f_rest_"))
    if n_rest % 3:
        raise RuntimeError(f"{path}: f_rest count {n_rest} is not a multiple of 3")
    K = n_rest // 3 + 1
    want = ply_attribute_names(K)
    missing = [x for x in want if x not in names and x not in ("nx", "ny", "nz")]
    if missing:
        raise RuntimeError(f"{path}: missing properties {missing[:4]}")
    n = rows.shape[0]
    if names != want:  # reorder columns into the canonical layout (absent normals become zeros)
        idx = {x: i for i, x in enumerate(names)}
        canon = np.zeros((n, len(want)), np.float32)
        for j, x in enumerate(want):
            if x in idx:
                canon[:, j] = rows[:, idx[x]]
        rows = canon
    model = SplatData(n, K, device, capacity)
    dev_rows = torch.from_numpy(np.array(rows, dtype=np.float32, order="C")).to(device)  # a writable copy
    p = model.struct()
    call("lfs_ply_unpack_rows", n, K, ptr(dev_rows), C.byref(p), _stream())
    return model


# ---------------------------------------------------------------------------------------------- checkpoint
def _sections(strategy):
    opt = strategy._optimizer
    return [("params", strategy.get_model()), ("exp_avg", opt.exp_avg), ("exp_avg_sq", opt.exp_avg_sq)]


def save_checkpoint(strategy, path: str, iteration: int) -> str:
    """Everything needed to continue training bit-identically: live rows of the parameters and both Adam moments,
    optimizer step count, per-group learning rates (after decay), active SH degree and the iteration."""
    model, opt = strategy.get_model(), strategy._optimizer
    n = model.size
    header = dict(version=1, iteration=int(iteration), n=n, sh_coeffs=model.K, step_count=int(opt.step_count), lr=list(opt.lr),
                  betas=list(opt.betas), eps=opt.eps, active_sh_degree=int(getattr(strategy, "active_sh_degree", 0)),
                  strategy=type(strategy).__name__, sections=[s for s, _ in _sections(strategy)], groups=list(PARAM_NAMES))
    hj = json.dumps(header).encode("utf-8")
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(_MAGIC)
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for _, sd in _sections(strategy):
            sd.size = n
            for name in PARAM_NAMES:
                f.write(sd.tensor(name).detach().cpu().numpy().astype("<f4", copy=False).tobytes())
    os.replace(tmp, path)  # a crash while writing never leaves a truncated checkpoint under the final name
    return path


def load_checkpoint(strategy, path: str) -> int:
    """Restore a strategy (already initialize()d, with enough capacity) from save_checkpoint; returns the iteration."""
    with open(path, "rb") as f:
        if f.read(8) != _MAGIC:
            raise RuntimeError(f"{path}: not a checkpoint of this library")
        (hl,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hl).decode("utf-8"))
        model, opt = strategy.get_model(), strategy._optimizer
        n, K = int(header["n"]), int(header["sh_coeffs"])
        if K != model.K:
            raise RuntimeError(f"{path}: checkpoint has {K} SH bases, the model {model.K}")
        if n > model.capacity:
            raise RuntimeError(f"{path}: {n} Gaussians exceed the model's capacity {model.capacity}")
        if header.get("groups") != list(PARAM_NAMES):
            raise RuntimeError(f"{path}: unexpected group order")
        for _, sd in _sections(strategy):
            sd.size = n
            for name in PARAM_NAMES:
                t = sd.tensor(name)
                raw = f.read(t.numel() * 4)
                if len(raw) != t.numel() * 4:
                    raise RuntimeError(f"{path}: truncated payload")
                t.copy_(torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy()).reshape(t.shape))
    if hasattr(strategy, "grads"):
        strategy.grads.size = n
    opt.step_count = int(header["step_count"])
    opt.lr = [float(x) for x in header["lr"]]
    if hasattr(strategy, "active_sh_degree"):
        strategy.active_sh_degree = int(header["active_sh_degree"])
    return int(header["iteration"])
