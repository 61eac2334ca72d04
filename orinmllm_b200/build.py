"""In-tree build of the native libraries (nvcc, sm_100a only).

    python -m orinmllm_b200.build            # build what is out of date
    python -m orinmllm_b200.build --force

Produces, next to this file under ``lib/``:
  libkpx.so          CUDA kernels + the C ABI declared in include/kpx.h
  libkuiper_b200.so  C++ host layer (kuiper-style op::Layer adapters, kernel registry,
                     block pool manager, radix tree / prefix cache) on top of libkpx
The CPU checker under ``oracle/`` and the C++ test program are test infrastructure and are
built by tests/buildtools.py, not from here.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"
INCLUDE = ROOT / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
    "--expt-relaxed-constexpr",
    "-I", str(INCLUDE), "-I", str(INCLUDE / "kuiper"), "-I", str(CSRC),
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the CUDA extension cannot be built")


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"build step failed: {' '.join(str(c) for c in cmd[:4])} ...")
    if verbose and (res.stdout or res.stderr):
        print(res.stdout + res.stderr)


def _headers():
    return list(INCLUDE.rglob("*.h")) + list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h"))


def build_kpx(force=False, verbose=False, ptxas_info=False) -> Path:
    """Compile every .cu under csrc/ into lib/libkpx.so."""
    LIB.mkdir(exist_ok=True)
    objdir = LIB / "obj"
    objdir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    cus = sorted(CSRC.glob("*.cu"))
    hdrs = _headers()
    objs = []
    procs = []
    for cu in cus:
        obj = objdir / (cu.stem + ".o")
        objs.append(obj)
        if force or _newer(obj, [cu] + hdrs):
            cmd = [nvcc, *NVCC_FLAGS, "-c", cu, "-o", obj]
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
            if verbose:
                print(" ".join(str(c) for c in cmd), flush=True)
            procs.append((cmd, subprocess.Popen([str(c) for c in cmd], stdout=subprocess.PIPE,
                                                stderr=subprocess.STDOUT, text=True)))
    for cmd, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError(f"nvcc failed on {cmd[-3]}")
        if (verbose or ptxas_info) and out:
            print(out)
    so = LIB / "libkpx.so"
    if force or procs or _newer(so, objs):
        _run([nvcc, "-shared", "-o", so, *objs, "-Xcompiler", "-fPIC", "-cudart", "shared"], verbose)
    return so


def build_host(force=False, verbose=False) -> Path | None:
    """Compile the C++ host layer (csrc/host/*.cpp) into lib/libkuiper_b200.so."""
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    if not srcs:
        return None
    so = LIB / "libkuiper_b200.so"
    if force or _newer(so, srcs + _headers() + [LIB / "libkpx.so"]):
        nvcc = _nvcc()
        cuda_inc = Path(nvcc).resolve().parent.parent / "include"
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-pthread",
               "-I", INCLUDE, "-I", INCLUDE / "kuiper", "-I", cuda_inc, "-o", so, *srcs,
               f"-L{LIB}", "-lkpx", "-Wl,-rpath,$ORIGIN",
               f"-L{Path(nvcc).resolve().parent.parent / 'lib64'}", "-lcudart"]
        _run(cmd, verbose)
    return so


def _nccl_dirs():
    """(include dir, library file) of the NCCL this process would load: the one packaged with the
    Python environment if there is one (torch loads that), else the system's."""
    try:
        import importlib.util
        spec = importlib.util.find_spec("nvidia.nccl")
        if spec and spec.submodule_search_locations:
            base = Path(list(spec.submodule_search_locations)[0])
            lib = base / "lib" / "libnccl.so.2"
            if (base / "include" / "nccl.h").exists() and lib.exists():
                return base / "include", lib
    except Exception:
        pass
    for inc, lib in ((Path("/usr/include"), Path("/usr/lib/x86_64-linux-gnu/libnccl.so.2")),):
        if (inc / "nccl.h").exists() and lib.exists():
            return inc, lib
    return None


def build_comm(force=False, verbose=False) -> Path | None:
    """csrc/comm/*.cpp (the NCCL all-gather of the KV-head-sharded mode) -> lib/libkpx_comm.so.
    Skipped (None) where no NCCL is installed: only the multi-GPU sharded mode needs it."""
    srcs = sorted((CSRC / "comm").glob("*.cpp"))
    found = _nccl_dirs()
    if not srcs or found is None:
        return None
    inc, lib = found
    so = LIB / "libkpx_comm.so"
    if force or _newer(so, srcs + _headers()):
        nvcc = _nvcc()
        cuda_root = Path(nvcc).resolve().parent.parent
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-fvisibility=hidden",
               "-I", INCLUDE, "-I", inc, "-I", cuda_root / "include", "-o", so, *srcs,
               str(lib), f"-Wl,-rpath,{lib.parent}", f"-L{cuda_root / 'lib64'}", "-lcudart"]
        _run(cmd, verbose)
    return so


def build_all(force=False, verbose=False, ptxas_info=False):
    build_kpx(force, verbose, ptxas_info)
    build_host(force, verbose)
    build_comm(force, verbose)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("--ptxas", action="store_true", help="print registers / spills / smem per kernel")
    a = ap.parse_args()
    build_all(a.force, a.verbose, a.ptxas)
    print("built:", ", ".join(p.name for p in sorted(LIB.glob("*.so"))))
