"""Builds the C-ABI kernel library ``torchpairwise_b200/lib/libtpw_b200.so`` for sm_100a.

Plain ``nvcc`` on the ``csrc/*.cu`` files (no torch headers), one object per source compiled in
parallel, linked into one shared object that sits in-tree next to the package.

    python torchpairwise_b200/build.py            # rebuild the objects whose sources changed
    python torchpairwise_b200/build.py --force -v # rebuild everything, print ptxas resource usage

Run it as a file (not with ``-m``): importing the package needs the library this script makes.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
LIB_DIR = PKG_DIR / "lib"
OBJ_DIR = LIB_DIR / "obj"
LIB_PATH = LIB_DIR / "libtpw_b200.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def find_nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _deps() -> list[Path]:
    return _sources() + sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h")) + [Path(__file__)]


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    return any(p.stat().st_mtime > t for p in _deps())


def _obj_stale(src: Path, obj: Path) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    shared = sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h")) + [Path(__file__)]
    return any(p.stat().st_mtime > t for p in [src, *shared])


def _compile_one(nvcc: str, src: Path, verbose: bool, force: bool) -> tuple[Path, str]:
    obj = OBJ_DIR / (src.stem + ".o")
    if not force and not _obj_stale(src, obj):
        return obj, ""
    cmd = [nvcc, *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC,-fvisibility=hidden",
           "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libtpw_b200.so``; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    srcs = _sources()
    objs = []
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        for obj, log in ex.map(lambda s: _compile_one(nvcc, s, verbose, force), srcs):
            objs.append(obj)
            if verbose and log:
                print(log, file=sys.stderr)
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd = [nvcc, *ARCH_FLAGS, "-shared", "-cudart", "shared", "-o", str(tmp), *map(str, objs)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


TORCH_SRC = CSRC / "torch" / "tpw_torch.cpp"
TORCH_LIB_PATH = LIB_DIR / "libtpw_b200_torch.so"


def build_torch_ops(force: bool = False) -> Path:
    """Compile the C++ host layer (``csrc/torch/tpw_torch.cpp``: the ``torchpairwise::`` operator
    registrations on top of the C ABI) with g++ against the installed torch, linked to
    ``libtpw_b200.so``; returns the path of ``libtpw_b200_torch.so``."""
    build_library()
    deps = [TORCH_SRC, *sorted(INCLUDE.glob("*.h")), Path(__file__)]
    if not force and TORCH_LIB_PATH.exists() and all(p.stat().st_mtime <= TORCH_LIB_PATH.stat().st_mtime for p in deps):
        return TORCH_LIB_PATH
    import torch
    from torch.utils import cpp_extension as ce
    tdir = Path(torch.__file__).resolve().parent
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cxx = os.environ.get("CXX", "g++")
    tmp = TORCH_LIB_PATH.with_suffix(".so.tmp")
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-w", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *[f"-I{p}" for p in ce.include_paths()], f"-I{cuda_home}/include", f"-I{INCLUDE}",
           str(TORCH_SRC), "-o", str(tmp),
           f"-L{tdir / 'lib'}", "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
           f"-L{LIB_DIR}", "-ltpw_b200", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tdir / 'lib'}",
           # the shared C++ runtime by name: a toolchain whose own libstdc++.so link is broken would otherwise
           # fall back to libstdc++.a, and a second, private copy of the stream classes inside this library
           # crashes as soon as an error message formats a number
           "-nostdlib++", "-l:libstdc++.so.6"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building the torch host layer failed:\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}")
    os.replace(tmp, TORCH_LIB_PATH)
    return TORCH_LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true", help="print ptxas resource usage")
    a = ap.parse_args()
    print(build_library(force=a.force, verbose=a.verbose))
    print(build_torch_ops(force=a.force))
