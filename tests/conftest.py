import importlib
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    return importlib.import_module("lichtfeld-studio_b200")


@pytest.fixture(scope="session")
def orc():
    from oracle import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def synth(pkg):
    return pkg.synth


def make_scene(synth, n, W, H, sh_degree, seed=0, layout="cube", fx=300.0, radius=4.0, model=0):
    cfg = dict(n=n, layout=layout, sh_degree=sh_degree, W=W, H=H, fx=fx, n_poses=1, radius=radius, model=model)
    P = synth.make_gaussians(n, seed, layout, sh_degree)
    poses, K = synth.make_cameras(cfg)
    return cfg, P, poses[0], K


def rel_l2(a, b):
    a = np.asarray(a, np.float64).reshape(-1)
    b = np.asarray(b, np.float64).reshape(-1)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
