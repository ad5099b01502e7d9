"""lichtfeld-studio_b200: the Gaussian-splatting training step of LichtFeld Studio's gsplat / 3DGUT
path as hand-written sm_100a CUDA behind a C ABI (include/lfs_b200.h), plus the host-side mirror
of the reference's operator and strategy interfaces.

The directory name contains a hyphen, so import it with importlib:
    lfs = importlib.import_module("lichtfeld-studio_b200")
"""
from . import _capi, dp, formats, ops, strategy, synth, trainer  # noqa: F401
from ._capi import LfsError, UTParams  # noqa: F401

__all__ = ["ops", "trainer", "strategy", "synth", "formats", "dp", "LfsError", "UTParams"]
