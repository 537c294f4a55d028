"""Builds the reference's OWN correctness programs against this library (acceptance harness).

The reference's test sources are compiled unmodified from where they lie in the reference tree (nothing is copied):
its hand-rolled harness (test/correctness/tester.cpp, testblas.cpp, test/test_utilities.cpp), one main per routine
(the GEMM family, the level-3 routines built on it, Omatcopy, Im2col, Col2im, override_parameters,
retrieve_parameters) and the two helper
translation units its tests need (src/utilities/utilities.cpp, clblast_exceptions.cpp). They are compiled with
-DCUDA_API against the reference's unmodified include/clblast_cuda.h and linked against THIS repository's
libclblast.so, so they exercise the drop-in boundary exactly as a user program would. Two stand-ins make that possible:
shim/clblast.h (one line: the tests include the OpenCL header name unconditionally) and
shadow/test/wrapper_cblas.hpp (the CBLAS comparison library is replaced by this repository's CPU oracle).

Outputs go to tests/ref_harness/_build/ (git-ignored; they travel to the GPU box with the tree).
    python -m tests.ref_harness.build
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
OUT = HERE / "_build"
REFERENCE = Path(os.environ.get("CLBLAST_REFERENCE", "/root/reference"))
CUDA = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))

COMMON = ["test/correctness/tester.cpp", "test/correctness/testblas.cpp", "test/test_utilities.cpp",
          "src/utilities/utilities.cpp", "src/utilities/clblast_exceptions.cpp"]
PROGRAMS = {
    "xgemm": "test/correctness/routines/level3/xgemm.cpp",
    "xgemmbatched": "test/correctness/routines/levelx/xgemmbatched.cpp",
    "xgemmstridedbatched": "test/correctness/routines/levelx/xgemmstridedbatched.cpp",
    "xconvgemm": "test/correctness/routines/levelx/xconvgemm.cpp",
    "xsymm": "test/correctness/routines/level3/xsymm.cpp",
    "xhemm": "test/correctness/routines/level3/xhemm.cpp",
    "xsyrk": "test/correctness/routines/level3/xsyrk.cpp",
    "xherk": "test/correctness/routines/level3/xherk.cpp",
    "xsyr2k": "test/correctness/routines/level3/xsyr2k.cpp",
    "xher2k": "test/correctness/routines/level3/xher2k.cpp",
    "xtrmm": "test/correctness/routines/level3/xtrmm.cpp",
    "xtrsm": "test/correctness/routines/level3/xtrsm.cpp",
    "xomatcopy": "test/correctness/routines/levelx/xomatcopy.cpp",
    "xim2col": "test/correctness/routines/levelx/xim2col.cpp",
    "xcol2im": "test/correctness/routines/levelx/xcol2im.cpp",
    "override_parameters": "test/correctness/misc/override_parameters.cpp",
    "retrieve_parameters": "test/correctness/misc/retrieve_parameters.cpp",
}


def reference_available() -> bool:
    return all((REFERENCE / f).exists() for f in COMMON + list(PROGRAMS.values()))


def _flags():
    return ["-std=c++11", "-O1", "-w", "-DCUDA_API", "-DCLBLAST_REF_CBLAS", f"-I{HERE / 'shim'}", f"-I{HERE / 'shadow'}",
            f"-I{REFERENCE}", f"-I{REFERENCE / 'src'}", f"-I{REFERENCE / 'include'}", f"-I{CUDA / 'include'}"]


def _compile(src: Path, obj: Path):
    res = subprocess.run(["g++", *_flags(), "-c", str(src), "-o", str(obj)], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compiling {src} failed:\n{res.stderr[-3000:]}")


def build(force: bool = False):
    """Returns {program name: path} or None when the reference tree is absent."""
    if not reference_available():
        return None
    lib = ROOT / "clblast_b200" / "lib" / "libclblast.so"
    oracle = ROOT / "oracle" / "liboracle.so"
    if not lib.exists() or not oracle.exists():
        raise RuntimeError("build libclblast.so and oracle/liboracle.so first")
    OUT.mkdir(parents=True, exist_ok=True)
    jobs = []
    for rel in COMMON + list(PROGRAMS.values()):
        src = REFERENCE / rel
        obj = OUT / (rel.replace("/", "_").rsplit(".", 1)[0] + ".o")
        stale = force or not obj.exists() or obj.stat().st_mtime < max(
            src.stat().st_mtime, (HERE / "shadow/test/wrapper_cblas.hpp").stat().st_mtime, Path(__file__).stat().st_mtime)
        if stale:
            jobs.append((src, obj))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        for fut in [pool.submit(_compile, s, o) for s, o in jobs]:
            fut.result()
    common_objs = [str(OUT / (rel.replace("/", "_").rsplit(".", 1)[0] + ".o")) for rel in COMMON]
    built = {}
    for name, rel in PROGRAMS.items():
        exe = OUT / f"clblast_test_{name}"
        obj = OUT / (rel.replace("/", "_").rsplit(".", 1)[0] + ".o")
        # libcuda is only needed at run time on the GPU box: link against the toolkit's stub here
        cmd = ["g++", "-o", str(exe), str(obj), *common_objs, str(lib), str(oracle), f"-L{CUDA / 'lib64' / 'stubs'}", "-lcuda",
               "-fopenmp", "-Wl,-rpath,$ORIGIN/../../../clblast_b200/lib", "-Wl,-rpath,$ORIGIN/../../../oracle",
               "-Wl,--allow-shlib-undefined"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"linking {name} failed:\n{res.stderr[-3000:]}")
        built[name] = exe
    return built


if __name__ == "__main__":
    out = build(force="--force" in sys.argv)
    print("\n".join(f"{k}: {v}" for k, v in out.items()) if out else "reference tree not found: nothing built")
