"""Builds the reference's own CUDA implementation of the training-step path into oracle/_ref/.

TEST INFRASTRUCTURE. The recipe compiles the reference's UNMODIFIED sources where they lie in the reference
checkout (nothing is copied into this repository), together with oracle/ref_harness.cpp (bindings and the
step driver) and oracle/glm_standin/ (the only third-party headers the sources need that are not installed),
into one Python extension module, oracle/_ref/lfs_reference.so. The flags are the reference's own
(gsplat/CMakeLists.txt:80, src/training/fastgs/CMakeLists.txt:62, src/training/CMakeLists.txt:82):
-O3 --use_fast_math --expt-relaxed-constexpr, relocatable device code, CUDA C++20 / host C++23, and the
architecture its `native` setting resolves to on a B200 (sm_100).

The module is the checker of the parity tests and the timed comparator of `bench.py --impl reference`. The
output directory is git-ignored; the built module travels with the working tree to the GPU machine, where the
reference checkout does not exist and load() only imports what was built.

    python oracle/ref_build.py            # build (skips what is up to date)
    python oracle/ref_build.py --force
"""
from __future__ import annotations

import importlib.util
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
OBJ_DIR = OUT_DIR / "obj"
MODULE = "lfs_reference"
OUT = OUT_DIR / f"{MODULE}.so"

CUDA_SOURCES = [
    "gsplat/IntersectTile.cu",
    "gsplat/ProjectionUT3DGSFused.cu",
    "gsplat/QuatToRotmatCUDA.cu",
    "gsplat/RasterizeToPixelsFromWorld3DGSBwd.cu",
    "gsplat/RasterizeToPixelsFromWorld3DGSFwd.cu",
    "gsplat/RelocationCUDA.cu",
    "gsplat/SphericalHarmonicsCUDA.cu",
    "src/training/kernels/ssim.cu",
    "src/training/kernels/regularization.cu",
    "src/training/fastgs/rasterization/src/rasterization_api.cu",
    "src/training/fastgs/rasterization/src/forward.cu",
    "src/training/fastgs/rasterization/src/backward.cu",
    "src/training/fastgs/optimizer/src/adam_api.cu",
    "src/training/fastgs/optimizer/src/adam.cu",
]
HOST_SOURCES = [
    "gsplat/Intersect.cpp",
    "gsplat/Projection.cpp",
    "gsplat/QuatToRotmat.cpp",
    "gsplat/Rasterization.cpp",
    "gsplat/Relocation.cpp",
    "gsplat/SphericalHarmonics.cpp",
    "src/training/rasterization/rasterizer_autograd.cpp",
    "src/training/rasterization/fast_rasterizer_autograd.cpp",
    "src/training/optimizers/fused_adam.cpp",
    "src/training/optimizers/scheduler.cpp",
]
INCLUDE_DIRS = [
    "gsplat",
    "include",
    "src/training",
    "src/training/fastgs/rasterization/include",
    "src/training/fastgs/optimizer/include",
    "src/training/fastgs/utils",
]
ARCH = ["-gencode", "arch=compute_100,code=sm_100"]
NVCC_FLAGS = ["-O3", "-DNDEBUG", "-DRELEASE_BUILD", "--use_fast_math", "--expt-relaxed-constexpr",
              "--diag-suppress=20012,186,221,3189", "-std=c++20", "-rdc=true", "-Xcompiler", "-fPIC",
              "-Wno-deprecated-gpu-targets"]
CXX_FLAGS = ["-std=c++23", "-O3", "-DNDEBUG", "-DRELEASE_BUILD", "-fPIC", "-w"]


def reference_root() -> Path | None:
    root = Path(os.environ.get("LFS_REFERENCE_ROOT", "/root/reference"))
    return root if (root / "gsplat" / "Ops.h").exists() else None


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    return "nvcc"


def _includes(root: Path) -> list[str]:
    from torch.utils import cpp_extension as ce
    inc = [str(HERE / "glm_standin")] + [str(root / d) for d in INCLUDE_DIRS] + ce.include_paths()
    inc += [str(HERE.parent / "lichtfeld-studio_b200" / "csrc")]   # gsplat_ops_pybind.inc, the bindings shared with the operator shim
    inc += [sysconfig.get_paths()["include"], "/usr/local/cuda/include"]
    return [f"-I{p}" for p in inc]


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path | None:
    """Compiles what is out of date. Returns the module path, or None when there is no reference checkout
    and nothing was built earlier."""
    root = reference_root()
    if root is None:
        return OUT if OUT.exists() else None
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    inc = _includes(root)
    defs = [f"-DTORCH_EXTENSION_NAME={MODULE}", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    standin_headers = list((HERE / "glm_standin").rglob("*.hpp"))

    def standin(rel: str):  # only these translation units see the glm stand-in
        return standin_headers if (rel.startswith("gsplat/") or "rasterizer_autograd" in rel) else []
    jobs = []
    objs = []
    for rel in CUDA_SOURCES:
        src = root / rel
        obj = OBJ_DIR / (rel.replace("/", "_") + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + standin(rel)):
            jobs.append([_nvcc()] + ARCH + NVCC_FLAGS + inc + ["-c", str(src), "-o", str(obj)])
    for rel in HOST_SOURCES:
        src = root / rel
        obj = OBJ_DIR / (rel.replace("/", "_") + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + standin(rel)):
            jobs.append(["g++"] + CXX_FLAGS + inc + ["-c", str(src), "-o", str(obj)])
    harness = HERE / "ref_harness.cpp"
    obj = OBJ_DIR / "ref_harness.o"
    objs.append(obj)
    shared_bindings = HERE.parent / "lichtfeld-studio_b200" / "csrc" / "gsplat_ops_pybind.inc"
    if force or _stale(obj, [harness, shared_bindings] + standin_headers):
        jobs.append(["g++"] + CXX_FLAGS + defs + inc + ["-c", str(harness), "-o", str(obj)])
    if jobs:
        workers = max(1, min(len(jobs), (os.cpu_count() or 4)))
        with ThreadPoolExecutor(max_workers=workers) as ex:
            for res in ex.map(lambda c: subprocess.run(c, capture_output=True, text=True), jobs):
                if verbose and res.stderr:
                    sys.stderr.write(res.stderr[-4000:])
                if res.returncode != 0:
                    raise RuntimeError("reference build failed:\n" + " ".join(res.args) + "\n" + res.stderr[-8000:])
    if force or jobs or _stale(OUT, objs):
        from torch.utils import cpp_extension as ce
        libs = [f"-L{p}" for p in ce.library_paths()] + ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
                                                          "-ltorch_python", "-lcudart"]
        cmd = [_nvcc()] + ARCH + ["-shared", "-Wno-deprecated-gpu-targets", "-o", str(OUT)] + [str(o) for o in objs] + libs
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("reference link failed:\n" + res.stderr[-8000:])
    return OUT


def available() -> bool:
    return OUT.exists()


def load():
    """Imports the built module (torch must be importable; its libraries are resolved through it)."""
    import torch  # noqa: F401  (loads libtorch before the extension)
    if not OUT.exists():
        raise RuntimeError("the reference build is missing: run `python oracle/ref_build.py` where the reference checkout is")
    if MODULE in sys.modules:
        return sys.modules[MODULE]
    spec = importlib.util.spec_from_file_location(MODULE, OUT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[MODULE] = mod
    return mod


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
