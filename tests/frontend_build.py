"""Compiles tests/cpp/frontend_test.cpp — a program written against the fk:: front end (include/fused_kernel/) — with
g++ (C++20) and links it to lib/libfkb.so, the CUDA runtime and the CPU checker (test infrastructure: the checker is
linked into this test program only).  It doubles as the build check of the header-only front end.  Run as
``python tests/frontend_build.py``; no GPU is needed to build.
"""
from __future__ import annotations

import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "frontend_test.cpp")
OUT = os.path.join(ROOT, "tests", "cpp", "frontend_test")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def needs_build() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [SRC, os.path.join(ROOT, "include", "fkb", "fkb.h")]
    fe = os.path.join(ROOT, "include", "fused_kernel", "fkb")
    deps += [os.path.join(fe, f) for f in os.listdir(fe)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return OUT
    lib_dir, oracle_dir = os.path.join(ROOT, "fusedkernellibrary_b200", "lib"), os.path.join(ROOT, "oracle")
    cmd = ["g++", "-std=c++20", "-O1", "-Wall", "-Wno-unused-function", "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(CUDA, "include"), SRC, "-o", OUT,
           "-L", lib_dir, "-lfkb", "-L", oracle_dir, "-loracle", "-L", os.path.join(CUDA, "lib64"), "-lcudart",
           # run-time search paths relative to the binary, so that the snapshot can be moved
           "-Wl,-rpath,$ORIGIN/../../fusedkernellibrary_b200/lib", "-Wl,-rpath,$ORIGIN/../../oracle",
           "-Wl,-rpath," + os.path.join(CUDA, "lib64")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("g++ failed building the front-end test program")
    return OUT


if __name__ == "__main__":
    build(force=True, verbose=True)
    print(OUT)
