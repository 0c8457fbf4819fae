"""Builds libcombskv.so (the C-ABI library) in-tree with nvcc for sm_100a."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcombskv.so")
LIB_MEASURE = os.path.join(HERE, "libcombskv_measure.so")  # -DCBKV_MEASURE: per-role timers, switches read from CBKV_DEBUG
SOURCES = ["manager.cpp", "sessions.cpp", "kernels.cu", "prefill_tc.cu", "rope.cu", "kvquant.cu", "api.cu", "noalloc.cu"]
HEADERS = ["manager.hpp", "kernels.hpp", os.path.join("..", "..", "include", "combs_kv.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared", "-cudart", "static", "-ldl",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def needs_build(lib: str = LIB) -> bool:
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, measure: bool = False) -> str:
    """The product library, or (measure=True) the measurement flavour: the same sources with
    -DCBKV_MEASURE, which adds timers and phase switches the product build does not contain."""
    lib = LIB_MEASURE if measure else LIB
    if not force and not needs_build(lib):
        return lib
    cmd = [_nvcc(), *NVCC_FLAGS, *( ["-DCBKV_MEASURE"] if measure else []), "-ccbin", "/usr/bin/g++",
           *[os.path.join(CSRC, f) for f in SOURCES], "-o", lib]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
    if verbose:
        sys.stderr.write(r.stderr)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, measure="--measure" in sys.argv))
