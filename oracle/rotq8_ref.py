"""The run-time rotate+quantise row kernel, restated in fp32 in the kernel's own operation order.

Test infrastructure (see oracle/__init__.py). Follows kernels/ops.metal:19-47 (butterflies), :270 (silu) and
:274-334 (rot_q8) of the reference. The contract for the int8 codes is the sequence of fp32 operations, not a
matrix product: each value goes through log2(B) butterfly stages of increasing stride, every stage replacing
the pair (a, b) = (v[i], v[i + s]) by (a + b, a - b); the whole block is then multiplied once by the
normaliser; amax is the row's largest magnitude; scale = amax / 127 (1 when amax is 0); rs = 1 / scale;
code = rint(v * rs) with ties to even and no clamp.
"""

from __future__ import annotations

import numpy as np

from .quant_ref import bf16_bits_to_f32, hadamard


def _as_f32_input(x: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "bf16":
        return bf16_bits_to_f32(x)
    if dtype == "f16":
        return np.asarray(x, dtype=np.float16).astype(np.float32)
    if dtype == "f32":
        return np.asarray(x, dtype=np.float32)
    raise ValueError(dtype)


def normaliser(block: int) -> np.float32:
    """1/sqrt(block) in fp32: 0.0625 for 256 (kernels/ops.metal:46), 0.125 for 64, and fp32(1/sqrt(128)) for
    128, the value the reference's 128-point transform multiplies by (kernels/ops.metal:444)."""
    return np.float32(1.0 / np.sqrt(np.float64(block)))


def silu_f32(g: np.ndarray) -> np.ndarray:
    """x / (1 + exp(-x)) in fp32 (kernels/ops.metal:270)."""
    g = g.astype(np.float32)
    return (g / (np.float32(1.0) + np.exp(-g).astype(np.float32))).astype(np.float32)


def fwht_blocks_f32(v: np.ndarray, block: int) -> np.ndarray:
    """Unnormalised block Walsh-Hadamard transform along the last axis, fp32, stages by increasing stride.

    kernels/ops.metal:19-31 does strides 1, 2, 4 inside a lane's eight values and :34-44 strides 8..128 across
    lanes (low lane v + o, high lane o - v): position i (bit s clear) receives a + b, position i + s receives
    a - b, a being the value at the lower index."""
    m, d = v.shape
    cur = np.ascontiguousarray(v, dtype=np.float32).reshape(m, d // block, block)
    s = 1
    while s < block:
        pairs = cur.reshape(m, d // block, block // (2 * s), 2, s)
        a = pairs[:, :, :, 0, :]
        b = pairs[:, :, :, 1, :]
        nxt = np.empty_like(pairs)
        nxt[:, :, :, 0, :] = a + b
        nxt[:, :, :, 1, :] = a - b
        cur = nxt.reshape(m, d // block, block)
        s *= 2
    return cur.reshape(m, d)


def rot_q8_rows(x: np.ndarray, D: int, *, block: int = 256, dtype: str = "bf16", swiglu: bool = False,
                out_hr: bool = False):
    """x [M][>= D (2D with swiglu)] -> (int8 codes [M][D], fp32 scales [M]); with out_hr the rotated rows as
    fp16 instead (kernels/ops.metal:303-314).

    Reference: kernels/ops.metal:274-334; launcher h3metal/ops.py:214-222."""
    xf = _as_f32_input(x, dtype)
    val = xf[:, :D]
    if swiglu:
        val = (val * silu_f32(xf[:, D:2 * D])).astype(np.float32)
    v = (fwht_blocks_f32(val, block) * normaliser(block)).astype(np.float32)
    if out_hr:
        return v.astype(np.float16)
    amax = np.abs(v).max(axis=1)
    scale = np.where(amax > 0, amax / np.float32(127.0), np.float32(1.0)).astype(np.float32)
    rs = (np.float32(1.0) / scale).astype(np.float32)
    q = np.rint((v * rs[:, None]).astype(np.float32))
    return q.astype(np.int32).astype(np.int8), scale


def rotate_rows_matmul(x_f32: np.ndarray, block: int) -> np.ndarray:
    """The same rotation written as the reference's tests write it: x.reshape(M, D/B, B) @ H in fp64
    (tests/test_ops.py:15-18). Used for the reference's own 0.6/127 bound, not for bit-exactness."""
    m, d = x_f32.shape
    h = hadamard(block).astype(np.float64)
    return (x_f32.astype(np.float64).reshape(m, d // block, block) @ h.T).reshape(m, d)
