"""Build recipe for the C-ABI shared library (``libswa2d.so``) next to this file.

``python dl_templates_b200/build.py`` compiles every ``.cu`` under ``csrc/`` for
sm_100a with nvcc (cross-compiles without a GPU) and links one shared object that
depends only on the CUDA runtime -- no libtorch, no libcuda link (the driver entry
point for tensor-map encoding is fetched at run time).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libswa2d.so")
# source -> extra flags.  The tensor-core kernels are built with fast math (ex2.approx / ftz in their softmax loops:
# their outputs are 16-bit); the C ABI file holds the SIMT kernels, whose fp32 path must hold 1e-4 against the
# oracle, and is built with IEEE division and exp2.
SOURCES = {"swa_abi.cu": [], "swa_tc.cu": ["--use_fast_math"]}
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]


def nvcc_path() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the library is built for sm_100a with the CUDA 12.9 toolkit")
    return cand


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "swa2d.h")]
    return any(os.path.getmtime(d) > t for d in deps if os.path.isfile(d))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    nvcc = nvcc_path()
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    jobs = []
    for src, extra in SOURCES.items():       # the translation units compile side by side
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *extra, *(["-Xptxas", "-v"] if verbose else []), "-c", os.path.join(CSRC, src), "-o", obj]
        jobs.append((obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for obj, proc in jobs:
        out, _ = proc.communicate()
        if verbose or proc.returncode != 0:
            sys.stderr.write(out)
        failed = failed or proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed building libswa2d.so")
    r = subprocess.run([nvcc, "-shared", "-cudart", "shared", *[o for o, _ in jobs], "-o", LIB], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("linking libswa2d.so failed")
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
