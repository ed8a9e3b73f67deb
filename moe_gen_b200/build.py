"""Builds libmoegen_b200.so in-tree with nvcc.

The library is sm_100a only; there is no other target and no fallback."""
from __future__ import annotations

import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libmoegen_b200.so")
LIB_CHECKED = os.path.join(PKG, "libmoegen_b200_checked.so")     # the same sources with -DMG_BOUNDS_CHECK
LIB_SANITIZED = os.path.join(PKG, "libmoegen_b200_asan.so")      # host code under ASan + UBSan (tests only)
SOURCES = ["api.cu", "route.cu", "pack.cu", "gemm.cu", "ep.cu"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC", "-shared", "-cudart", "static", "-ldl"]


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_sanitized_library(force: bool = False) -> str:
    """The same sources with the host side compiled under AddressSanitizer and UndefinedBehaviorSanitizer
    (-O1 -g).  It is loaded only by the host-side tests, in a process that preloads the sanitizer
    runtimes (select it with MOEGEN_B200_LIB); device code is not instrumented."""
    srcs = [os.path.join(CSRC, s) for s in SOURCES]
    deps = srcs + [os.path.join(CSRC, "common.cuh"), os.path.join(ROOT, "include", "moegen_b200.h")]
    if force or _stale(LIB_SANITIZED, deps):
        nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
        cmd = [nvcc, "-std=c++17", "-O1", "-g", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler",
               "-fPIC,-fsanitize=address,-fsanitize=undefined,-fno-omit-frame-pointer", "-shared", "-cudart",
               "static", "-ldl"] + srcs + ["-o", LIB_SANITIZED]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
    return LIB_SANITIZED


def build_library(force: bool = False, verbose: bool = False, checked: bool = False) -> str:
    """checked=True builds libmoegen_b200_checked.so: every row index the scatter, combine, duplicate-fill
    and return kernels read from a table is compared with the buffer's declared rows; a violation is
    recorded in the device status word and the access skipped (select it with MOEGEN_B200_LIB)."""
    srcs = [os.path.join(CSRC, s) for s in SOURCES]
    deps = srcs + [os.path.join(CSRC, "common.cuh"), os.path.join(ROOT, "include", "moegen_b200.h")]
    target = LIB_CHECKED if checked else LIB
    if force or _stale(target, deps):
        nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
        cmd = ([nvcc] + NVCC_FLAGS + (["-DMG_BOUNDS_CHECK"] if checked else []) + (["-Xptxas", "-v"] if verbose else [])
               + srcs + ["-o", target])
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
        if verbose:
            sys.stderr.write(r.stderr)
    return target


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv, checked="--checked" in sys.argv))
