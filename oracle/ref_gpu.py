"""A CPU stand-in for the reference's `Gpu` object whose dispatches execute the oracle's kernel restatements.

Test infrastructure (see oracle/__init__.py). The reference's host code (h3metal/ops.py: gemm, rot_q8, low_rank,
LowRank.table) only calls Gpu.upload / empty / kernel / launch / wait and Tensor.numpy / view; given this object it
runs unmodified on the CPU, so its padding, strides, two-step LoRA sequence and parameter packing come from the
reference itself and only the two kernels' arithmetic comes from this package. It is used when the reference tree
is importable (fixture generation, and CPU tests that skip otherwise).

Interfaces mirrored: Gpu h3metal/gpu.py:179-265, Tensor :121-157; buffer indices of the two kernels
kernels/gemm.metal:117-128 and kernels/ops.metal:274-277; parameter blocks kernels/params.h:7-16,25-29.
"""

from __future__ import annotations

import math
import struct

import numpy as np

from . import gemm_ref, rotq8_ref

_NP = {"f32": np.float32, "f16": np.float16, "bf16": np.uint16, "i8": np.int8, "u8": np.uint8, "i32": np.int32,
       "u32": np.uint32, "i16": np.int16, "u16": np.uint16}
_FROM_NP = {np.dtype(np.float32): "f32", np.dtype(np.float16): "f16", np.dtype(np.int8): "i8",
            np.dtype(np.uint8): "u8", np.dtype(np.int32): "i32", np.dtype(np.uint32): "u32",
            np.dtype(np.uint16): "bf16", np.dtype(np.int16): "i16"}
_METAL_T = {"half": "f16", "bfloat": "bf16", "float": "f32"}


class HostTensor:
    """Typed view of a byte array: the fields and methods of the reference's Tensor that ops.py touches."""

    def __init__(self, raw: np.ndarray, offset: int, shape, dtype: str):
        self.raw, self.offset, self.shape, self.dtype = raw, int(offset), tuple(int(s) for s in shape), dtype

    @property
    def itemsize(self) -> int:
        return np.dtype(_NP[self.dtype]).itemsize

    @property
    def nbytes(self) -> int:
        return math.prod(self.shape) * self.itemsize

    def numpy(self) -> np.ndarray:
        n = math.prod(self.shape)
        return self.raw[self.offset:self.offset + n * self.itemsize].view(_NP[self.dtype]).reshape(self.shape)

    def flat_from_here(self, dtype: str | None = None) -> np.ndarray:
        """Everything from this view's first byte to the end of its buffer, as a flat array."""
        dt = np.dtype(_NP[dtype or self.dtype])
        usable = (len(self.raw) - self.offset) // dt.itemsize * dt.itemsize
        return self.raw[self.offset:self.offset + usable].view(dt)

    def view(self, shape, dtype=None, offset_elems=0):
        return HostTensor(self.raw, self.offset + int(offset_elems * self.itemsize), shape, dtype or self.dtype)

    def row(self, start: int, count: int):
        per = math.prod(self.shape[1:])
        return HostTensor(self.raw, self.offset + start * per * self.itemsize, (count,) + self.shape[1:],
                          self.dtype)


class OracleGpu:
    """Records nothing and defers nothing: every launch runs at once on the CPU."""

    device = "cpu-oracle"

    def __init__(self, block: int = 256):
        self.block = block       # rotation block of the rot_q8 restatement (the reference's kernel has 256)
        self.launches = []       # (file, fn, macros, grid, threads, params) of every dispatch, for inspection

    def empty(self, shape, dtype="f32"):
        shape = tuple(int(s) for s in shape)
        n = math.prod(shape) * np.dtype(_NP[dtype]).itemsize
        return HostTensor(np.zeros(max(1, n), np.uint8), 0, shape, dtype)

    def upload(self, arr, dtype=None):
        arr = np.ascontiguousarray(arr)
        dtype = dtype or _FROM_NP[arr.dtype]
        t = self.empty(arr.shape, dtype)
        t.numpy()[...] = arr.view(_NP[dtype]).reshape(t.shape)
        return t

    def kernel(self, file, fn, **macros):
        return (file, fn, dict(macros))

    def launch(self, k, grid, threads, args, params=b"", params_index=None, tg_mem=0):
        file, fn, macros = k
        self.launches.append((file, fn, dict(macros), tuple(grid), tuple(threads), bytes(params)))
        if (file, fn) == ("ops.metal", "rot_q8"):
            self._rot_q8(macros, args, params)
        elif (file, fn) == ("gemm.metal", "gemm"):
            self._gemm(macros, args, params)
        else:
            raise NotImplementedError(f"{file}:{fn} is outside the quantised-linear path")

    def commit(self):
        pass

    def wait(self) -> float:
        return 0.0

    # kernels/ops.metal:274-334; buffers 0 in, 1 out, 2 sa; RotQParams M, D, x_stride, mode
    def _rot_q8(self, macros, args, params):
        M, D, x_stride, mode = struct.unpack("<4i", params)
        x, out, sa = args[0], args[1], args[2]
        in_dtype = _METAL_T[macros.get("IN_T", "bfloat")]
        rows = x.flat_from_here(in_dtype)[:(M - 1) * x_stride + (2 * D if mode == 1 else D)]
        mat = np.lib.stride_tricks.as_strided(rows, (M, 2 * D if mode == 1 else D),
                                              (x_stride * rows.itemsize, rows.itemsize))
        if int(macros.get("OUT_HR", 0)):
            out.flat_from_here("f16")[:M * D] = rotq8_ref.rot_q8_rows(
                mat, D, block=self.block, dtype=in_dtype, swiglu=mode == 1, out_hr=True).reshape(-1)
            return
        q, s = rotq8_ref.rot_q8_rows(mat, D, block=self.block, dtype=in_dtype, swiglu=mode == 1)
        out.flat_from_here("i8")[:M * D] = q.reshape(-1)
        sa.flat_from_here("f32")[:M] = s

    # kernels/gemm.metal:117-261, WFMT 1 / EPI 0; buffers 0 a, 1 w, 2 sw, 3 sa, 4 out, 5 bias, 9 lt, 10 lb, 11 lr
    def _gemm(self, macros, args, params):
        if int(macros["WFMT"]) != 1 or int(macros["EPI"]) != 0:
            raise NotImplementedError("only the int8 format with the storing epilogue is on the path")
        M, N, K, a_stride, c_stride, w_stride, _groups, _g_stride = struct.unpack("<8i", params)
        a, w, sw, sa, out, bias = args[:6]

        def strided(t, rows, cols, stride, dtype):
            flat = t.flat_from_here(dtype)[:(rows - 1) * stride + cols]
            return np.lib.stride_tricks.as_strided(flat, (rows, cols), (stride * flat.itemsize, flat.itemsize))

        A = strided(a, M, K, a_stride, "i8")
        W = strided(w, N, K, w_stride, "i8")
        acc = gemm_ref.int32_product(A, W)
        low = None
        if int(macros.get("LORA", 0)):
            lt, lb, lr = args[9], args[10], args[11].numpy()
            tn = int(macros["TN"])
            T = strided(lt, M, int(lr[0]), int(lr[0]), "f16").astype(np.float64)
            B = strided(lb, N, int(lr[1]), int(lr[1]), "f16").astype(np.float64)
            low = np.zeros((M, N), np.float32)
            for t in range(N // tn):
                k0, k1 = int(lr[2 + 2 * t]), int(lr[3 + 2 * t])
                if k1 > k0:
                    low[:, t * tn:(t + 1) * tn] = T[:, k0:k1] @ B[t * tn:(t + 1) * tn, k0:k1].T
        v = gemm_ref.epilogue_q8(acc, sa.flat_from_here("f32")[:M], sw.flat_from_here("f32")[:N],
                                 bias.flat_from_here("f32")[:N] if int(macros.get("HAS_BIAS", 0)) else None, low)
        out_dtype = _METAL_T[macros["OUT_T"]]
        strided(out, M, N, c_stride, out_dtype)[...] = gemm_ref.store_as(v, out_dtype)
