"""Compiles the oracle's C witness (oracle/rotq8_witness.c) with gcc into oracle/_build/. Test infrastructure."""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "rotq8_witness.c")
LIB = os.path.join(HERE, "_build", "librotq8_witness.so")


def build(force: bool = False) -> str:
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(SRC):
        os.makedirs(os.path.dirname(LIB), exist_ok=True)
        # -ffp-contract=off: the witness states every fp32 operation separately, as the kernel does
        subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", SRC, "-o", LIB, "-lm"], check=True)
    return LIB


def witness_rot_q8(x_f32: np.ndarray, D: int, block: int, swiglu: bool):
    """(codes int8 [M][D], scales fp32 [M], rotated fp32 [M][D]) from the C witness; x_f32 is [M][D or 2D] fp32."""
    lib = ctypes.CDLL(build())
    lib.rotq8_witness.restype = ctypes.c_int
    lib.rotq8_witness.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_long, ctypes.c_int,
                                  ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    M = x.shape[0]
    codes = np.empty((M, D), np.int8)
    scales = np.empty(M, np.float32)
    rotated = np.empty((M, D), np.float32)
    rc = lib.rotq8_witness(x.ctypes.data, M, D, x.shape[1], block, 1 if swiglu else 0, codes.ctypes.data,
                           scales.ctypes.data, rotated.ctypes.data)
    if rc:
        raise ValueError("rotq8_witness rejected the sizes")
    return codes, scales, rotated
