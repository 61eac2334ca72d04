"""Builds the test infrastructure: the CPU checker under oracle/ (its own Makefile), the
reference-compiled libraries and programs under oracle/_ref/ when a reference checkout is
named, and the C++ test program that drives the kuiper-style adapters.

The reference checkout is the directory the environment variable KPX_REFERENCE names, else a
directory called `reference` beside this repository; where neither exists only the plain-C
checker is built and what is already under oracle/_ref/ is used as it is.
"""
from __future__ import annotations

import os
from pathlib import Path

from orinmllm_b200 import build as b

ROOT = Path(__file__).resolve().parent.parent


def reference_checkout(reference=None) -> Path | None:
    for ref in (reference, os.environ.get("KPX_REFERENCE"), ROOT.parent / "reference"):
        if ref and Path(ref, "kuiper/include/base/radix_tree.h").exists():
            return Path(ref)
    return None


def build_oracle(verbose=False, reference=None) -> Path:
    odir = ROOT / "oracle"
    b._run(["make", "-C", odir, "all"], verbose)
    ref = reference_checkout(reference)
    if ref is not None:
        b._run(["make", "-C", odir, "ref", f"REF={ref}"], verbose)
    return odir / "liborinkv_oracle.so"


def build_cpp_tests(force=False, verbose=False) -> Path:
    """tests/cpp/test_kuiper_api.cu (layer API against the CPU checker; the only binary that
    links the checker) -> orinmllm_b200/lib/test_kuiper_api."""
    src = ROOT / "tests" / "cpp" / "test_kuiper_api.cu"
    exe = b.LIB / "test_kuiper_api"
    oracle_so = build_oracle(verbose)
    if force or b._newer(exe, [src, b.LIB / "libkpx.so", oracle_so] + b._headers()):
        b._run([b._nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17",
                "-I", b.INCLUDE, "-I", b.INCLUDE / "kuiper", "-o", exe, src, f"-L{b.LIB}", "-lkpx",
                f"-L{ROOT / 'oracle'}", "-lorinkv_oracle",
                "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN",
                "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../oracle"], verbose)
    return exe
