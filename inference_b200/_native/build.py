"""In-tree build of the native libraries.

`libswb200_kernels.so` holds every CUDA kernel, compiled by nvcc for sm_100a only; `libswb200_host.so`
holds the C++ host policy (scheduler, paging, prefix index, speculative math, sampler, constraint,
checkpoint readers). Both are plain C-ABI shared objects loaded with ctypes, so they carry no
dependency on the PyTorch headers and rebuild in seconds.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
CSRC = PKG / "csrc"
OUT = Path(__file__).resolve().parent
OBJ = OUT / "build"

NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
CXX = os.environ.get("CXX") or shutil.which("g++") or "g++"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "-I", str(CSRC / "include"), "-I", str(CSRC / "kernels"),
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-I", str(CSRC / "include"), "-I", str(CSRC / "host")]


def _newer(src: Path, dst: Path, deps: list[Path]) -> bool:
    if not dst.exists():
        return True
    t = dst.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *deps])


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    if os.environ.get("SWB_BUILD_VERBOSE") and (r.stdout or r.stderr):
        sys.stderr.write(r.stdout + r.stderr)


def _compile_all(srcs: list[Path], headers: list[Path], compiler: list[str], tag: str, force: bool) -> list[Path]:
    OBJ.mkdir(parents=True, exist_ok=True)
    jobs = []
    objs = []
    for s in srcs:
        o = OBJ / f"{tag}_{s.stem}.o"
        objs.append(o)
        if force or _newer(s, o, headers):
            jobs.append(compiler + ["-c", str(s), "-o", str(o)])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(_run, jobs))
    return objs


def build_kernels(force: bool = False, verbose_ptxas: bool = False) -> Path:
    srcs = sorted((CSRC / "kernels").glob("*.cu"))
    headers = (sorted((CSRC / "kernels").glob("*.cuh")) + sorted((CSRC / "kernels").glob("*.h")) +
               sorted((CSRC / "include").glob("*.h")))
    flags = list(NVCC_FLAGS)
    if verbose_ptxas:
        flags += ["-Xptxas", "-v"]
        os.environ["SWB_BUILD_VERBOSE"] = "1"
    objs = _compile_all(srcs, headers, [NVCC, *flags], "k", force or verbose_ptxas)
    lib = OUT / "libswb200_kernels.so"
    if force or not lib.exists() or any(o.stat().st_mtime > lib.stat().st_mtime for o in objs):
        _run([NVCC, "-shared", "-o", str(lib), *map(str, objs), "-lcudart"])
    return lib


def build_host(force: bool = False) -> Path:
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    headers = sorted((CSRC / "host").glob("*.h")) + sorted((CSRC / "host").glob("*.hpp")) + sorted(
        (CSRC / "include").glob("*.h"))
    lib = OUT / "libswb200_host.so"
    if not srcs:
        return lib
    objs = _compile_all(srcs, headers, [CXX, *CXX_FLAGS], "h", force)
    if force or not lib.exists() or any(o.stat().st_mtime > lib.stat().st_mtime for o in objs):
        _run([CXX, "-shared", "-o", str(lib), *map(str, objs), "-lpthread"])
    return lib


def build_capi(force: bool = False) -> Path:
    """The contracts C ABI (embeds / joins a Python interpreter at run time; links no libpython)."""
    src = CSRC / "capi" / "capi.cpp"
    lib = OUT / "libswb200_capi.so"
    if force or _newer(src, lib, [CSRC / "include" / "swb200_contracts.h"]):
        _run([CXX, *CXX_FLAGS, "-shared", "-o", str(lib), str(src), "-ldl", "-lpthread"])
    return lib


def build_all(force: bool = False) -> dict[str, Path]:
    return {"kernels": build_kernels(force), "host": build_host(force), "capi": build_capi(force)}


if __name__ == "__main__":
    force = "--force" in sys.argv
    if "--ptxas" in sys.argv:
        print(build_kernels(force=True, verbose_ptxas=True))
    else:
        for k, v in build_all(force).items():
            print(k, v)
