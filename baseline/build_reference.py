"""Builds the reference's own CUDA flavour into baseline/_ref/ so that it can be timed on the same GPU.

The reference's library sources are compiled where they lie in the reference tree (nothing is copied) with g++ and
-DCUDA_API, the flags its own build uses for the CUDA flavour, and linked against the CUDA driver and NVRTC into
baseline/_ref/libclblast_reference.so; baseline/run_reference.cpp (this repository's timing driver, written against
the reference's unmodified include/clblast_cuda.h) is linked against it into baseline/_ref/run_reference. The
directory is git-ignored and travels to the GPU box with the tree. The driver runs in a process of its own: the
reference library exports the same symbols as this repository's library.

    python -m baseline.build_reference      # needs the reference tree; a no-op elsewhere
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
REFERENCE = Path(os.environ.get("CLBLAST_REFERENCE", "/root/reference"))
CUDA = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))

BASE = ["src/database/database.cpp", "src/routines/common.cpp", "src/utilities/compile.cpp",
        "src/utilities/clblast_exceptions.cpp", "src/utilities/timing.cpp", "src/utilities/utilities.cpp",
        "src/api_common.cpp", "src/cache.cpp", "src/kernel_preprocessor.cpp", "src/routine.cpp",
        "src/routines/levelx/xinvert.cpp", "src/tuning/configurations.cpp", "src/clblast_cuda.cpp"]
LEVEL1 = "xswap xscal xcopy xaxpy xdot xdotu xdotc xnrm2 xasum xamax".split()
LEVEL2 = ("xgemv xgbmv xhemv xhbmv xhpmv xsymv xsbmv xspmv xtrmv xtbmv xtpmv xtrsv xger xgeru xgerc xher xhpr xher2 "
          "xhpr2 xsyr xspr xsyr2 xspr2").split()
LEVEL3 = "xgemm xsymm xhemm xsyrk xherk xsyr2k xher2k xtrmm xtrsm".split()
LEVELX = "xhad xomatcopy xim2col xcol2im xconvgemm xaxpybatched xgemmbatched xgemmstridedbatched".split()
DATABASES = ("copy pad padtranspose transpose xaxpy xdot xgemm xgemm_direct xgemv xgemv_fast xgemv_fast_rot xger invert "
             "gemm_routine trsv_routine xconvgemm").split()


def sources() -> list[str]:
    out = list(BASE)
    out += [f"src/routines/level1/{r}.cpp" for r in LEVEL1]
    out += [f"src/routines/level2/{r}.cpp" for r in LEVEL2]
    out += [f"src/routines/level3/{r}.cpp" for r in LEVEL3]
    out += [f"src/routines/levelx/{r}.cpp" for r in LEVELX]
    out += [f"src/database/kernels/{d}/{d}.cpp" for d in DATABASES]
    return out


def reference_available() -> bool:
    return all((REFERENCE / f).exists() for f in sources())


def _compile(src: Path, obj: Path):
    cmd = ["g++", "-std=c++11", "-O2", "-w", "-fPIC", "-DCUDA_API", f"-I{REFERENCE / 'include'}", f"-I{REFERENCE / 'src'}",
           f"-I{CUDA / 'include'}", "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compiling {src} failed:\n{res.stderr[-3000:]}")


def build(force: bool = False):
    """Returns the path of run_reference, or None when the reference tree is absent."""
    if not reference_available():
        return None
    OUT.mkdir(parents=True, exist_ok=True)
    objdir = OUT / "obj"
    objdir.mkdir(exist_ok=True)
    jobs, objs = [], []
    for rel in sources():
        src = REFERENCE / rel
        obj = objdir / (rel.replace("/", "_").rsplit(".", 1)[0] + ".o")
        objs.append(str(obj))
        if force or not obj.exists() or obj.stat().st_mtime < src.stat().st_mtime:
            jobs.append((src, obj))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        for fut in [pool.submit(_compile, s, o) for s, o in jobs]:
            fut.result()
    lib = OUT / "libclblast_reference.so"
    exe = OUT / "run_reference"
    driver = HERE / "run_reference.cpp"
    if jobs or not lib.exists():
        # libcuda is only present on the GPU box: link against the toolkit's stub here
        cmd = ["g++", "-shared", "-o", str(lib), *objs, f"-L{CUDA / 'lib64' / 'stubs'}", f"-L{CUDA / 'lib64'}", "-lcuda",
               "-lnvrtc"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"linking the reference library failed:\n{res.stderr[-3000:]}")
    if jobs or not exe.exists() or exe.stat().st_mtime < driver.stat().st_mtime:
        cmd = ["g++", "-std=c++11", "-O2", f"-I{REFERENCE / 'include'}", f"-I{CUDA / 'include'}", str(driver), "-o", str(exe),
               str(lib), f"-L{CUDA / 'lib64' / 'stubs'}", f"-L{CUDA / 'lib64'}", "-lcuda", "-lnvrtc",
               "-ldl", "-rdynamic", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{CUDA / 'lib64'}", "-Wl,--allow-shlib-undefined"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"linking run_reference failed:\n{res.stderr[-3000:]}")
    return exe


if __name__ == "__main__":
    out = build(force="--force" in sys.argv)
    print(out if out else "reference tree not found: nothing built")
