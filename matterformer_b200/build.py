"""Builds ``libmatterformer_b200.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

Each ``csrc/*.cu`` is compiled to an object file in parallel and the objects are linked into
one shared library next to this file.  Nothing here needs a GPU: nvcc cross-compiles.
Run ``python -m matterformer_b200.build`` or call :func:`build_library`.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libmatterformer_b200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
]
if os.environ.get("MF_DEBUG_BOUNDS", "0") not in ("", "0"):  # index checks in the kernels' table lookups (see common.cuh)
    NVCC_FLAGS.append("-DMF_DEBUG_BOUNDS")


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the C-ABI library cannot be built")
    return exe


def _newest(paths) -> float:
    return max(p.stat().st_mtime for p in paths)


def _compile_one(src: Path, obj: Path, headers, verbose: bool) -> str:
    if obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, _newest(headers)):
        return f"up to date: {obj.name}"
    cmd = [_nvcc(), *NVCC_FLAGS, "-Xptxas", "-v", "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    (obj.with_suffix(".ptxas.log")).write_text(res.stderr)
    if verbose:
        print(res.stderr, file=sys.stderr)
    return f"compiled: {src.name}"


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel source for sm_100a and link the shared library. Returns its path."""
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "matterformer_b200.h"]
    OBJ_DIR.mkdir(exist_ok=True)
    if force:
        for f in OBJ_DIR.glob("*.o"):
            f.unlink()
    objs = [OBJ_DIR / (s.stem + ".o") for s in sources]
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        for msg in pool.map(lambda so: _compile_one(so[0], so[1], headers, verbose), zip(sources, objs)):
            if verbose:
                print(msg)
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < _newest(objs):
        cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objs), "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose=True))
