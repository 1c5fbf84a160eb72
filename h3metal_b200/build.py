"""Builds libh3b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m h3metal_b200.build            # build if sources are newer than the library
    python -m h3metal_b200.build --force

The library is written next to this file so that it travels with the source tree; nothing is installed.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libh3b200.so")
SOURCES = ("capi.cu", "rot_q8.cu", "rot_q8_tma.cu", "norm_mod_q8.cu", "gemm_w8a8.cu", "gemm_w8a8_pair.cu", "dequant.cu", "peer.cu", "mma_probe.cu")
HEADERS = ("kernels.h", "ptx.cuh", "rot_common.cuh", "gemm_common.cuh", os.path.join("..", "..", "include", "h3b200.h"))
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
# -fmad=false: the rotate+quantise arithmetic and the dequantising epilogue are defined operation by operation;
# no multiply and add may be fused behind the source's back.
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-fmad=false", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC", ""), shutil.which("nvcc") or "", "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise FileNotFoundError("nvcc not found (set NVCC)")


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles the translation units and links the shared library; returns its path."""
    if not force and not _stale():
        return LIB
    nvcc = _nvcc()
    objs = []
    procs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    for src in SOURCES:
        obj = os.path.join(HERE, "build", src.replace(".cu", ".o"))
        cmd = [nvcc, *ARCH, *COMMON, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd))
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            print(f"--- {src}\n{out}", file=sys.stderr if p.returncode else sys.stdout)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    tmp = LIB + ".tmp"
    link = [nvcc, *ARCH, "-shared", "-o", tmp, *objs, "-Xcompiler", "-fvisibility=hidden"]
    subprocess.run(link, check=True)
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
