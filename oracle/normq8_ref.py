"""The norm + modulation kernel in front of the rotate+quantise tail, restated on the CPU.

Test infrastructure (see oracle/__init__.py). Follows kernels/ops.metal:111-268 of the reference (launcher
h3metal/ops.py:200-211): RMSNorm of the fp32 row (LayerNorm without affine with LN: the mean is subtracted first;
with POST the row is first updated in place by post * rmsnorm(y)), then v * inv * scale'[type] + shift[type] with
separate fp32 multiplies and add, then the rot_q8 tail. The row statistics (sum of squares, mean) are sums of fp32
terms whose ORDER the reference leaves to its SIMD-group reductions; here the fp32 terms are added in float64 and
rounded once, the order-free answer any fp32 summation order approximates to within a few ulp.
"""

from __future__ import annotations

import numpy as np

from .rotq8_ref import rot_q8_rows


def _rsqrt_f32(v: np.ndarray) -> np.ndarray:
    return (1.0 / np.sqrt(v.astype(np.float64))).astype(np.float32)


def _mean_sq(v: np.ndarray, D: int) -> np.ndarray:
    sq = (v * v).astype(np.float32)
    total = sq.sum(axis=1, dtype=np.float64).astype(np.float32)
    return (total / np.float32(D)).astype(np.float32)


def norm_mod_rows(x: np.ndarray, mod: np.ndarray, rtype: np.ndarray, D: int, *, eps: float, block: int = 256,
                  ln: bool = False, y: np.ndarray | None = None, post: np.ndarray | None = None, out: str = "q8"):
    """x fp32 [M][>= D]; mod fp32 [types][2][D]; rtype uint8 [M].

    out: "q8" -> (int8 codes [M][D], fp32 scales [M]); "f" / "h" -> modulated rows as fp32 / fp16; "hr" -> rotated
    rows as fp16. With y and post also returns the updated x rows as a last element."""
    eps = np.float32(eps)
    v = np.ascontiguousarray(x[:, :D], dtype=np.float32).copy()
    if ln:
        mean = (v.sum(axis=1, dtype=np.float64).astype(np.float32) / np.float32(D)).astype(np.float32)
        v = (v - mean[:, None]).astype(np.float32)
    updated = None
    if post is not None:
        yv = np.ascontiguousarray(y[:, :D], dtype=np.float32)
        iy = _rsqrt_f32((_mean_sq(yv, D) + eps).astype(np.float32))
        term = ((post.astype(np.float32)[None, :] * yv).astype(np.float32) * iy[:, None]).astype(np.float32)
        v = (v + term).astype(np.float32)
        updated = v.copy()
    inv = _rsqrt_f32((_mean_sq(v, D) + eps).astype(np.float32))
    scale = mod[rtype, 0].astype(np.float32)
    shift = mod[rtype, 1].astype(np.float32)
    m = (((v * inv[:, None]).astype(np.float32) * scale).astype(np.float32) + shift).astype(np.float32)
    if out == "f":
        res = m
    elif out == "h":
        res = m.astype(np.float16)
    elif out == "hr":
        res = rot_q8_rows(m, D, block=block, dtype="f32", out_hr=True)
    else:
        res = rot_q8_rows(m, D, block=block, dtype="f32")
    if updated is not None:
        return (*res, updated) if isinstance(res, tuple) else (res, updated)
    return res
