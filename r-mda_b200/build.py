"""Builds libmoe_cuda.so (sm_100a only) and the C host-side mirror, in-tree."""
from __future__ import annotations

import glob
import os
import subprocess

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libmoe_cuda.so")
HOST_LIB = os.path.join(PKG, "libmoe_host.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_cuda(force: bool = False, verbose: bool = False) -> str:
    srcs = sorted(glob.glob(os.path.join(PKG, "csrc", "*.cu")))
    deps = srcs + glob.glob(os.path.join(PKG, "csrc", "*.cuh")) + [os.path.join(ROOT, "include", "moe_cuda.h")]
    if force or _stale(LIB, deps):
        cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB] + srcs + ["-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
        if verbose:
            print(r.stderr)
    return LIB


def build_host(force: bool = False) -> str:
    """The C mirror of the reference's call sites and of its weight path, compiled as the reference is (gnu17)."""
    srcs = [os.path.join(PKG, "host", "moe_host.c"), os.path.join(PKG, "host", "moe_weights.c"),
            os.path.join(PKG, "host", "moe_head.c")]
    deps = srcs + [os.path.join(PKG, "host", "moe_host.h"), os.path.join(PKG, "host", "moe_weights.h"),
                   os.path.join(PKG, "host", "moe_head.h"),
                   os.path.join(ROOT, "include", "moe_cuda.h")]
    if force or _stale(HOST_LIB, deps) or _stale(HOST_LIB, [LIB]):
        cmd = ["gcc", "-std=gnu17", "-O2", "-Wall", "-Wextra", "-shared", "-fPIC", "-I", os.path.join(ROOT, "include"),
               "-o", HOST_LIB] + srcs + ["-L", PKG, "-lmoe_cuda", "-lpthread", "-Wl,-rpath,$ORIGIN"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("gcc failed:\n" + r.stdout + r.stderr)
    return HOST_LIB


def build_all(force: bool = False) -> None:
    build_cuda(force)
    build_host(force)


if __name__ == "__main__":
    build_all(force=True)
    print(LIB)
    print(HOST_LIB)
