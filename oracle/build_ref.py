"""Builds oracle/_ref/libclblast_ref_kernels.so: the reference's own GEMM kernel source, executed on the CPU.

TEST INFRASTRUCTURE ONLY. The reference's device kernels are OpenCL-C kept as C++ raw strings. This script reads
the files of the direct GEMM, convolution, triangle-conversion, im2col and col2im kernels where they lie in the reference tree, takes the text between
the raw-string markers, and compiles it as C (OpenCL C is a C99 dialect) against oracle/ref_shim.h (work-item ids, barrier, vector types)
and oracle/ref_driver.inc (launch logic), once per precision; every symbol but the two entry points of each
precision is made local with objcopy so the five objects link into one shared object. Nothing from the reference is written into the
repository: the generated translation units live in a temporary directory and only the shared object is kept, under
the git-ignored oracle/_ref/. Tests use it to pin the C oracle to the reference's real arithmetic.

    python -m oracle.build_ref            # needs the reference tree; a no-op elsewhere
"""
from __future__ import annotations

import os
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
LIB_PATH = OUT_DIR / "libclblast_ref_kernels.so"
REFERENCE = Path(os.environ.get("CLBLAST_REFERENCE", "/root/reference"))

KERNEL_FILES = [
    "src/kernels/common.opencl",
    "src/kernels/level3/level3.opencl",
    "src/kernels/level3/xgemm_direct_part1.opencl",
    "src/kernels/level3/xgemm_direct_part2.opencl",
    "src/kernels/level3/xgemm_direct_part3.opencl",
    "src/kernels/levelx/xconvgemm_part1.opencl",
    "src/kernels/levelx/xconvgemm_part2.opencl",
    "src/kernels/level3/convert_symmetric.opencl",
    "src/kernels/level3/convert_hermitian.opencl",
    "src/kernels/level3/convert_triangular.opencl",
    "src/kernels/levelx/im2col.opencl",
    "src/kernels/levelx/col2im.opencl",
]
PRECISIONS = {16: "p16", 32: "p32", 64: "p64", 3232: "p3232", 6464: "p6464"}


def reference_available() -> bool:
    return all((REFERENCE / f).exists() for f in KERNEL_FILES)


def raw_string_body(path: Path) -> str:
    text = path.read_text()
    start = text.index('R"(') + 3
    end = text.rindex(')"')
    return text[start:end]


def build(force: bool = False) -> Path | None:
    if not reference_available():
        return None
    newest = max((REFERENCE / f).stat().st_mtime for f in KERNEL_FILES)
    newest = max(newest, (HERE / "ref_shim.h").stat().st_mtime, (HERE / "ref_driver.inc").stat().st_mtime,
                 Path(__file__).stat().st_mtime)
    if LIB_PATH.exists() and LIB_PATH.stat().st_mtime >= newest and not force:
        return LIB_PATH
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        objs = []
        for precision, tag in PRECISIONS.items():
            parts = [f'#include "{HERE / "ref_shim.h"}"', f"#define PRECISION {precision}",
                     f"#define REF_PRECISION_TAG {tag}", "#define ROUTINE_CONVGEMM", "#define ROUTINE_SYMM",
                     "#define ROUTINE_HEMM", "#define ROUTINE_TRMM"]
            for f in KERNEL_FILES:
                if "xconvgemm" in f and precision > 100:
                    continue  # Convgemm has no complex instantiations
                parts.append(f'#line 1 "{REFERENCE / f}"')
                parts.append(raw_string_body(REFERENCE / f))
            parts.append(f'#include "{HERE / "ref_driver.inc"}"')
            src = Path(tmp) / f"ref_{tag}.c"
            src.write_text("\n".join(parts) + "\n")
            obj = Path(tmp) / f"ref_{tag}.o"
            # -ffp-contract=fast: like the device compilers the reference targets, fuse a*b+c where possible
            cmd = ["gcc", "-std=gnu11", "-O2", "-march=x86-64-v3", "-ffp-contract=fast", "-fPIC", "-w", "-c", str(src),
                   "-o", str(obj)]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"compiling the reference kernels for precision {precision} failed:\n{res.stderr[-4000:]}")
            keep = ["-G", f"ref_gemm_direct_{tag}"] + (["-G", f"ref_convgemm_{tag}"] if precision < 100 else [])
            for entry in ("ref_expand_triangle", "ref_im2col", "ref_col2im"):
                keep += ["-G", f"{entry}_{tag}"]
            res = subprocess.run(["objcopy", *keep, str(obj)], capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"objcopy failed:\n{res.stderr[-2000:]}")
            objs.append(str(obj))
        res = subprocess.run(["gcc", "-shared", "-o", str(LIB_PATH), *objs], capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"linking failed:\n{res.stderr[-4000:]}")
    return LIB_PATH


if __name__ == "__main__":
    out = build(force="--force" in sys.argv)
    print(out if out else "reference tree not found: nothing built")
