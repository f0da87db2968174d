"""Builds lib/libfkb.so (the CUDA kernels and the C ABI) for sm_100a with nvcc.

Run as ``python -m fusedkernellibrary_b200.build``.  nvcc cross-compiles, so no GPU is needed.  Flags that are
part of the arithmetic contract: ``--fmad=false`` (no FMA contraction; the kernels also use explicit
round-to-nearest intrinsics), default ``-prec-div=true -prec-sqrt=true -ftz=false``.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "lib")
OUT = os.path.join(OUT_DIR, "libfkb.so")
SOURCES = ["fkb_kernels.cu", "fkb_host.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--fmad=false",
    "-Xcompiler", "-fPIC", "-shared", "-Xptxas", "-v", "-ldl",
]


def needs_build() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(ROOT, "include", "fkb", "fkb.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("FKB_NVCC_EXTRA", "").split(), "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-o", os.environ.get("FKB_BUILD_OUT", OUT),
           *[os.path.join(CSRC, s) for s in SOURCES]]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libfkb.so")
    return OUT


def build_debug(force: bool = False) -> str:
    """The self-checking build, lib/libfkb_debug.so: the same sources with -DFKB_DEBUG, which makes every bulk copy and
    every gathered tap test its addresses against the buffer its plane record describes, record FKB_ERR_DEVICE_CHECK and
    skip the access on a miss (it stands in for a memory checker; nothing traps).  The tests run the parity cases on it."""
    out = os.path.join(OUT_DIR, "libfkb_debug.so")
    if not force and os.path.exists(out) and not needs_build() and os.path.getmtime(out) >= os.path.getmtime(OUT):
        return out
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-DFKB_DEBUG", "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-o", out,
           *[os.path.join(CSRC, s) for s in SOURCES]]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libfkb_debug.so")
    return out


def build_phase_clocks() -> str:
    """The phase-clock build, lib/libfkb_phase.so: the same sources with -DFKB_PHASE_CLOCKS, in which the warps of
    staged_kernel add up the cycles they spend in each phase of a resize row (``profile_case.py --phase-clocks`` prints
    them).  A measuring aid, built on request only; it runs slower than the product."""
    out = os.path.join(OUT_DIR, "libfkb_phase.so")
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-DFKB_PHASE_CLOCKS", "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-o", out,
           *[os.path.join(CSRC, s) for s in SOURCES]]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libfkb_phase.so")
    return out


def build_frontend_bench(force: bool = False) -> str:
    """Compiles bench_frontend.cpp (the host-cost measurement bench.py runs: a program written against the fk:: front
    end, linked to libfkb.so and the CUDA runtime only) into lib/bench_frontend."""
    src = os.path.join(ROOT, "bench_frontend.cpp")
    out = os.path.join(OUT_DIR, "bench_frontend")
    if not force and os.path.exists(out) and os.path.getmtime(out) > max(os.path.getmtime(src), os.path.getmtime(OUT)):
        return out
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-std=c++20", "-O2", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"), src, "-o", out,
           "-L", OUT_DIR, "-lfkb", "-L", os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(cuda, "lib64")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("g++ failed building bench_frontend")
    return out


if __name__ == "__main__":
    build(force=True, verbose=True)
    print(OUT)
    print(build_debug(force=True))
    print(build_frontend_bench(force=True))
