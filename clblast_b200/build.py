"""Ahead-of-time build of libclblast.so (sm_100a only) with nvcc.

Run as ``python -m clblast_b200.build`` or call :func:`build_library`. Objects are rebuilt only when a source
or header is newer; translation units compile in parallel. The result is ``clblast_b200/lib/libclblast.so``,
which exports both the C ABI of ``include/b200blas.h`` and the C++ symbols of ``include/clblast_cuda.h``.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "lib" / "libclblast.so"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=default", "-I", str(ROOT / "include"),
          "-I", str(CSRC)]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the library cannot be built")
    return exe


def _sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cpp")) + list(CSRC.glob("*.cu")) + list((CSRC / "kernels").glob("*.cu")))


def _headers() -> list[Path]:
    return (list(CSRC.glob("*.h")) + list((CSRC / "kernels").glob("*.h")) + list((CSRC / "kernels").glob("*.cuh"))
            + list((ROOT / "include").glob("*.h")))


def _compile(src: Path, obj: Path, verbose: bool) -> str:
    cmd = [_nvcc(), *ARCH, *COMMON, "-Xptxas", "-v", "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    (obj.with_suffix(".ptxas.txt")).write_text(res.stderr)
    if verbose:
        print(f"  compiled {src.name}", flush=True)
    return res.stderr


def build_library(force: bool = False, verbose: bool = True) -> Path:
    """Compile every translation unit for sm_100a and link the shared library. Returns its path."""
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB.parent.mkdir(parents=True, exist_ok=True)
    newest_header = max((h.stat().st_mtime for h in _headers()), default=0.0)
    self_mtime = Path(__file__).stat().st_mtime
    todo, objs = [], []
    for src in _sources():
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        stale = (force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, newest_header, self_mtime))
        if stale:
            todo.append((src, obj))
    if todo:
        if verbose:
            print(f"building {len(todo)} translation unit(s) for sm_100a", flush=True)
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
            for fut in [pool.submit(_compile, s, o, verbose) for s, o in todo]:
                fut.result()
    if todo or not LIB.exists():
        cmd = [_nvcc(), *ARCH, "-shared", "-cudart", "static", "-o", str(LIB), *map(str, objs), "-ldl", "-lpthread"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(f"linked {LIB}", flush=True)
    return LIB


if __name__ == "__main__":
    build_library(force="--force" in sys.argv)
