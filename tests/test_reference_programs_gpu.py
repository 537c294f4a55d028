"""Runs the reference's own correctness programs (its tester, descriptors and mains, compiled unmodified against the
reference's include/clblast_cuda.h by tests/ref_harness/build.py) against this library on the GPU.

Each program walks the reference's full case grid for its routine and all precisions it supports (including half,
which the reference's own CUDA backend cannot compile, and the complex types), checks results with the reference's
margins against the CPU oracle, checks the 127-element canary regions, and exits with the number of failures."""
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
BUILD = Path(__file__).resolve().parent / "ref_harness" / "_build"
PROGRAMS = ("xgemm", "xgemmbatched", "xgemmstridedbatched", "xconvgemm", "xsymm", "xhemm", "xsyrk", "xherk", "xsyr2k",
            "xher2k", "xtrmm", "xtrsm", "xomatcopy", "xim2col", "xcol2im", "override_parameters", "retrieve_parameters")


@pytest.mark.parametrize("name", PROGRAMS)
def test_reference_program_passes(cuda, name):
    exe = BUILD / f"clblast_test_{name}"
    if not exe.exists():
        pytest.skip("reference test programs were not built (the reference tree is only present in the build container)")
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=900)
    tail = "\n".join(res.stdout.splitlines()[-25:])
    assert res.returncode == 0, f"{name} reported failures (exit {res.returncode})\n{tail}\n{res.stderr[-2000:]}"
    assert "failed" not in tail or " 0 test(s) failed" in tail or "0 tests failed" in tail, tail
