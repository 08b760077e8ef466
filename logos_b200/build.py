"""Builds the engine's shared library in-tree with nvcc for sm_100a.

    python -m logos_b200.build [--force] [--verbose]

Outputs: logos_b200/liblogos_attn.so (C ABI of include/logos_attn.h) and
logos_b200/liblogos_attn_shim.so (the reference's C++ symbol cuda_flash_attention_fwd on top of it).
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "liblogos_attn.so")
SHIM = os.path.join(PKG, "liblogos_attn_shim.so")
SHIM_SRC = os.path.join(PKG, "shim", "logos_attn_shim.cu")

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "--cudart", "static",
]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def stale() -> bool:
    if not os.path.exists(LIB) or not os.path.exists(SHIM):
        return True
    t = min(os.path.getmtime(LIB), os.path.getmtime(SHIM))
    deps = sources() + [SHIM_SRC] + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(PKG, "..", "include", "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not stale():
        return LIB
    objs = []
    objdir = os.path.join(PKG, "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        cmd = ["nvcc", *NVCC_FLAGS, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                            text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(out)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call(["nvcc", "-shared", "--cudart", "static", "-gencode",
                           "arch=compute_100a,code=sm_100a", "-o", LIB, *objs, "-lcuda"])
    # the drop-in C++ symbol; finds liblogos_attn.so beside itself
    subprocess.check_call(["nvcc", "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "--cudart", "static",
                           "-gencode", "arch=compute_100a,code=sm_100a", "-o", SHIM, SHIM_SRC, "-L" + PKG, "-llogos_attn", "-Xlinker", "-rpath=$ORIGIN"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
