"""In-tree build of the native libraries.

``libxorl_b200.so``      -- every ``csrc/*.cu`` kernel, compiled for sm_100a only.
``libxorl_b200_host.so`` -- the C++ host runtime under ``csrc/host`` (no CUDA needed; used by the
                            CPU test-suite as well).

Both are written to ``xorl_b200/lib`` so that a snapshot of the source tree carries them.
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
LIBDIR = PKG / "lib"
OBJDIR = PKG.parent / "build" / "obj"

CUDA_LIB = LIBDIR / "libxorl_b200.so"
HOST_LIB = LIBDIR / "libxorl_b200_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def _newer(src: Path, dst: Path, deps: list[Path]) -> bool:
    if not dst.exists():
        return True
    t = dst.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *deps])


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build libxorl_b200.so")
    OBJDIR.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    jobs = []
    objs = []
    for src in sources:
        obj = OBJDIR / (src.stem + ".o")
        objs.append(obj)
        if force or _newer(src, obj, headers):
            jobs.append([nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)])
    if jobs:
        if verbose:
            print(f"[xorl_b200] compiling {len(jobs)} CUDA sources for sm_100a", file=sys.stderr)
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
    if jobs or not CUDA_LIB.exists():
        _run([nvcc, "-shared", "-o", str(CUDA_LIB), *map(str, objs), "-cudart", "static"])
    return CUDA_LIB


def build_host(force: bool = False, verbose: bool = False) -> Path:
    cxx = shutil.which("g++") or "g++"
    LIBDIR.mkdir(parents=True, exist_ok=True)
    sources = sorted((CSRC / "host").glob("*.cpp"))
    if not sources:
        return HOST_LIB
    headers = sorted((CSRC / "host").glob("*.h"))
    if force or any(_newer(s, HOST_LIB, headers) for s in sources):
        if verbose:
            print(f"[xorl_b200] compiling {len(sources)} host sources", file=sys.stderr)
        _run([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-o", str(HOST_LIB),
              *map(str, sources)])
    return HOST_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_host(force=force, verbose=verbose)
    build_cuda(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print(CUDA_LIB, HOST_LIB)
