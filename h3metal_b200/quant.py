"""Offline weight rotation and int8 quantisation (NumPy, CPU), with the reference's names and meanings.

Drop-in for the int8 part of the reference's h3metal/quant.py (hadamard :16-20, random_signs :26-28, rotate_in
:31-44, quant_q8 :77-82, dequant :103-115, quantize :118-131). This is the conversion-time side of the path: it
runs once per weight on the host, as it does in the reference; the run-time side (activations) is the CUDA
kernel behind ops.rot_q8. The rotation block is a parameter here (the reference fixes it at 256).

The input dimension of a weight is multiplied by R = diag(signs) * blockdiag(H_B / sqrt(B)); activations are
rotated by the same R before their per-token quantisation, so x W^T = (x R)(W R)^T.
"""

from __future__ import annotations

import functools

import numpy as np

RB = 256  # the reference's rotation block; every function below takes `block=` to override it


@functools.lru_cache(maxsize=8)
def _hadamard_cached(n: int) -> np.ndarray:
    if n < 1 or n & (n - 1):
        raise ValueError(f"Hadamard order {n} is not a power of two")
    h = np.ones((1, 1), dtype=np.float64)
    for _ in range(n.bit_length() - 1):
        h = np.kron(np.array([[1.0, 1.0], [1.0, -1.0]]), h)
    h = (h / np.sqrt(n)).astype(np.float32)
    h.setflags(write=False)
    return h


def hadamard(n: int = RB) -> np.ndarray:
    """Orthonormal Sylvester Hadamard matrix H_n / sqrt(n) in fp32 (built in fp64)."""
    return _hadamard_cached(int(n)).copy()


def random_signs(n: int, seed: int) -> np.ndarray:
    """A +-1 vector of length n; element i is -1 where the i-th uniform draw of default_rng(seed) is below 0.5."""
    return np.where(np.random.default_rng(seed).random(n) < 0.5, np.float32(-1.0), np.float32(1.0))


def rotate_in(w: np.ndarray, signs: np.ndarray | None = None, block: int = RB) -> np.ndarray:
    """W [N][K] -> W diag(signs) blockdiag(H_block), fp32. K must be a multiple of `block`."""
    rows, k = w.shape
    if k % block:
        raise ValueError(f"input dimension {k} is not a multiple of {block}")
    h = _hadamard_cached(int(block))
    src = w.astype(np.float32, copy=False)
    if signs is not None:
        src = src * signs[None, :]
    dst = np.empty((rows, k), dtype=np.float32)
    chunk = max(1, (1 << 24) // k)  # rows per matmul, bounds the temporaries
    for lo in range(0, rows, chunk):
        piece = src[lo:lo + chunk]
        np.matmul(piece.reshape(len(piece), k // block, block), h,  # H is symmetric
                  out=dst[lo:lo + chunk].reshape(len(piece), k // block, block))
    return dst


def _clip_search(w: np.ndarray, amax: np.ndarray, qmax: int, factors) -> np.ndarray:
    """Per row, the scale amax*c/qmax (c from `factors`, first best wins) with the least squared rounding error."""
    least = np.full(amax.shape, np.inf, dtype=np.float64)
    chosen = np.zeros_like(amax)
    for c in factors:
        s = np.maximum(amax * c / qmax, 1e-12)
        back = np.clip(np.rint(w / s[:, None]), -qmax, qmax) * s[:, None]
        err = np.square(back - w).sum(axis=-1, dtype=np.float64)
        win = err < least
        least[win] = err[win]
        chosen[win] = s[win]
    return chosen


def quant_q8(w: np.ndarray, search: bool = True):
    """Per-row symmetric int8: (codes [N][K] int8, scales [N] fp32). With `search` the scale is clipped to the
    best of amax * (1, .97, .94, .9, .85) / 127; without, it is max(amax / 127, 1e-12)."""
    amax = np.abs(w).max(axis=1)
    s = _clip_search(w, amax, 127, (1.0, .97, .94, .9, .85)) if search else np.maximum(amax / 127, 1e-12)
    codes = np.clip(np.rint(w / s[:, None]), -127, 127).astype(np.int8)
    return codes, s.astype(np.float32)


_INT8_FORMATS = ("q8", "h8")


def dequant(fmt: str, w: np.ndarray, sw: np.ndarray | None, N: int, K: int, G: int = 128) -> np.ndarray:
    """The fp32 matrix [N][K] stored codes stand for (in the rotated input space). int8 and bf16/f16 only."""
    if fmt in _INT8_FORMATS:
        return w.astype(np.float32) * sw[:, None]
    if fmt == "f16":
        return w.astype(np.float32)
    if fmt == "bf16":
        return (w.astype(np.uint32) << 16).view(np.float32)
    raise ValueError(f"format {fmt!r} is not part of the int8 linear path")


def quantize(fmt: str, w: np.ndarray, G: int = 128):
    """-> (stored codes, scales or None) for the formats this package carries (q8/h8, f16, bf16)."""
    if fmt in _INT8_FORMATS:
        return quant_q8(w)
    if fmt == "f16":
        return w.astype(np.float16), None
    if fmt == "bf16":
        return bf16_bits(w), None
    raise ValueError(f"format {fmt!r} is not part of the int8 linear path")


def bf16_bits(a: np.ndarray) -> np.ndarray:
    """fp32 -> bfloat16 bit patterns (uint16), round to nearest even (the reference's h3metal/weights.py:41-44)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_to_f32(u: np.ndarray) -> np.ndarray:
    """bfloat16 bit patterns -> fp32 (h3metal/weights.py:47-48)."""
    return (np.asarray(u, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
