"""Builds liblfs_b200.so (sm_100a) in-tree with nvcc. No torch involved: the library is plain CUDA
behind a C ABI. Run as a script or call build()."""
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
        subprocess.check_call([nvcc, "-shared", "-Wno-deprecated-gpu-targets", "-o", str(OUT)] + objs + ["-lcudart"])
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
