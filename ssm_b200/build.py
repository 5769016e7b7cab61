"""Builds ``libssm_b200.so`` (the C-ABI library of hand-written sm_100a kernels) in-tree.

``python -m ssm_b200.build`` compiles every ``csrc/*.cu`` with
``nvcc -gencode arch=compute_100a,code=sm_100a`` and links them into
``ssm_b200/lib/libssm_b200.so``.  nvcc cross-compiles, so no GPU is needed to build.
Objects are rebuilt only when a source or header is newer than they are.

It then builds ``ssm_b200/lib/ssm_b200_ext.so``, the thin PyTorch extension
(``csrc/torch_ext/ssm_b200_ext.cpp``, plain C++ compiled with g++ against the torch headers)
that exposes the library under the ten names of upstream's compiled backend.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "lib" / "obj"
LIB = PKG / "lib" / "libssm_b200.so"
EXT_SRC = CSRC / "torch_ext" / "ssm_b200_ext.cpp"
EXT = PKG / "lib" / "ssm_b200_ext.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted((PKG.parent / "include").glob("*.h"))

    def compile_one(src: Path) -> Path:
        obj = OBJ / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            res = subprocess.run(cmd, capture_output=True, text=True)
            (OBJ / (src.stem + ".ptxas.log")).write_text(res.stderr)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stderr[-4000:]}")
            if verbose:
                print(f"compiled {src.name}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, sources()))
    if force or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stderr[-4000:]}")
        if verbose:
            print(f"linked {LIB}")
    return LIB


def build_extension(force: bool = False, verbose: bool = False) -> Path:
    """Compile the pybind / ATen layer over the C ABI.  Needs the library of `build_library` to link against."""
    import sysconfig

    import torch
    from torch.utils.cpp_extension import include_paths, library_paths

    header = PKG.parent / "include" / "ssm_b200.h"
    if not (force or _stale(EXT, [EXT_SRC, header, LIB])):
        return EXT
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    cuda_home = Path(_nvcc()).resolve().parent.parent
    incs = [sysconfig.get_paths()["include"], *include_paths(), str(cuda_home / "include")]
    libdirs = [*library_paths(), str(LIB.parent)]
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=ssm_b200_ext", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-Wno-deprecated-declarations",
           *[f"-isystem{i}" for i in incs], str(EXT_SRC), "-o", str(EXT),
           *[f"-L{d}" for d in libdirs], "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lssm_b200",
           "-Wl,-rpath,$ORIGIN", *[f"-Wl,-rpath,{d}" for d in library_paths()]]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building the torch extension failed:\n{res.stderr[-6000:]}")
    if verbose:
        print(f"built {EXT}")
    return EXT


if __name__ == "__main__":
    build_library(force="--force" in sys.argv, verbose=True)
    build_extension(force="--force" in sys.argv, verbose=True)
