"""Builds liblfs_b200.so (sm_100a) in-tree with nvcc. No torch involved: the library is plain CUDA
behind a C ABI. build_shim() then compiles the C++ operator shim (namespace gsplat of gsplat/Ops.h over that C ABI,
csrc/ops_shim.cpp) with its Python module against libtorch into lfs_ops_shim.so. Run as a script or call build()."""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "liblfs_b200.so"
OBJ = HERE / "build"

# (source, extra flags). The per-Gaussian projection and the tile-list code are built without FMA
# contraction: their float results feed integer tile lists and sort keys.
SOURCES = [
    ("projection.cu", ["--fmad=false"]),
    ("sort.cu", ["--fmad=false"]),
    ("ewa.cu", ["--fmad=false"]),
    ("ewa_raster.cu", []),
    ("raster.cu", []),
    ("loss.cu", []),
    ("elementwise.cu", []),
    ("api.cu", []),
    ("noalloc.cu", []),
    ("error.cu", []),
]
COMMON = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
          "-Xcompiler", "-fPIC", "-Wno-deprecated-gpu-targets"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (cand == "nvcc" or Path(cand).exists()):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "lfs_b200.h"]
    nvcc = _nvcc()
    jobs = []
    for src, extra in SOURCES:
        obj = OBJ / (src + ".o")
        if force or _stale(obj, [CSRC / src] + headers):
            cmd = [nvcc] + COMMON + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", str(CSRC / src), "-o", str(obj)]
            jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for res in ex.map(lambda c: subprocess.run(c, capture_output=True, text=True), jobs):
                if verbose and res.stderr:
                    sys.stderr.write(res.stderr)
                if res.returncode != 0:
                    raise RuntimeError("nvcc failed:\n" + " ".join(res.args) + "\n" + res.stderr)
    objs = [str(OBJ / (s + ".o")) for s, _ in SOURCES]
    if force or jobs or _stale(OUT, objs):
        subprocess.check_call([nvcc, "-shared", "-Wno-deprecated-gpu-targets", "-o", str(OUT)] + objs + ["-lcudart", "-ldl"])
    return OUT


SHIM_OUT = HERE / "lfs_ops_shim.so"
SHIM_SOURCES = ["ops_shim.cpp", "ops_shim_module.cpp"]


def build_shim(force: bool = False) -> Path:
    """g++ against libtorch (host code only); links liblfs_b200.so from the same directory ($ORIGIN)."""
    import sysconfig
    from torch.utils import cpp_extension as ce
    build()
    OBJ.mkdir(exist_ok=True)
    inc = [f"-I{p}" for p in ce.include_paths() + [str(HERE.parent / "include"), str(CSRC), sysconfig.get_paths()["include"],
                                                   "/usr/local/cuda/include"]]
    deps = [HERE.parent / "include" / "lfs_gsplat_ops.h", HERE.parent / "include" / "lfs_b200.h", CSRC / "gsplat_ops_pybind.inc"]
    jobs, objs = [], []
    for src in SHIM_SOURCES:
        obj = OBJ / (src + ".o")
        objs.append(str(obj))
        if force or _stale(obj, [CSRC / src] + deps):
            jobs.append(["g++", "-std=c++17", "-O2", "-fPIC", "-w", "-DTORCH_EXTENSION_NAME=lfs_ops_shim", "-DTORCH_API_INCLUDE_EXTENSION_H"]
                        + inc + ["-c", str(CSRC / src), "-o", str(obj)])
    if jobs:
        with ThreadPoolExecutor(max_workers=len(jobs)) as ex:
            for res in ex.map(lambda c: subprocess.run(c, capture_output=True, text=True), jobs):
                if res.returncode != 0:
                    raise RuntimeError("operator shim: g++ failed:\n" + " ".join(res.args) + "\n" + res.stderr[-6000:])
    if force or jobs or _stale(SHIM_OUT, objs + [OUT]):
        libs = [f"-L{p}" for p in ce.library_paths()] + ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python"]
        subprocess.check_call(["g++", "-shared", "-o", str(SHIM_OUT)] + objs + [f"-L{HERE}", "-llfs_b200", "-Wl,-rpath,$ORIGIN"] + libs
                              + ["-L/usr/local/cuda/lib64", "-lcudart"])
    return SHIM_OUT


def load_shim():
    """Imports lfs_ops_shim (the operator shim's Python module); builds nothing."""
    import importlib.util
    import torch  # noqa: F401
    if "lfs_ops_shim" in sys.modules:
        return sys.modules["lfs_ops_shim"]
    if not SHIM_OUT.exists():
        raise RuntimeError("lfs_ops_shim.so is missing: run lichtfeld-studio_b200/build.py")
    spec = importlib.util.spec_from_file_location("lfs_ops_shim", SHIM_OUT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules["lfs_ops_shim"] = mod
    return mod


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_shim(force="--force" in sys.argv))
