"""Offline side of the path, restated: Hadamard matrix, sign vectors, input rotation, int8 quantiser.

Test infrastructure (see oracle/__init__.py). Follows h3metal/quant.py and h3metal/weights.py of the reference.
"""

from __future__ import annotations

import numpy as np


def bf16_round_bits(a) -> np.ndarray:
    """fp32 -> bfloat16 bit patterns (uint16), round to nearest, ties to even.

    Reference: h3metal/weights.py:41-44 (adds 0x7FFF plus the lowest kept bit, then drops 16 bits)."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    keep_lsb = (bits >> np.uint32(16)) & np.uint32(1)
    return ((bits + np.uint32(0x7FFF) + keep_lsb) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(u) -> np.ndarray:
    """bfloat16 bit patterns -> fp32 (exact). Reference: h3metal/weights.py:47-48."""
    return (np.asarray(u, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def hadamard(n: int) -> np.ndarray:
    """Sylvester Hadamard matrix of order n divided by sqrt(n), computed in fp64 and cast to fp32.

    Reference: h3metal/quant.py:16-20. Entry (i, j) of the Sylvester matrix is (-1)^popcount(i & j); the
    reference builds the same matrix by repeated [[h, h], [h, -h]] blocks."""
    if n < 1 or n & (n - 1):
        raise ValueError(f"Hadamard order {n} is not a power of two")
    idx = np.arange(n, dtype=np.int64)
    parity = np.zeros((n, n), dtype=np.int64)
    both = idx[:, None] & idx[None, :]
    while both.any():
        parity ^= both & 1
        both >>= 1
    h = np.where(parity == 1, -1.0, 1.0)
    return (h / np.sqrt(n)).astype(np.float32)


def random_signs(n: int, seed: int) -> np.ndarray:
    """+-1 vector: -1 where default_rng(seed).random(n) < 0.5. Reference: h3metal/quant.py:26-28."""
    draw = np.random.default_rng(seed).random(n)
    s = np.ones(n, dtype=np.float32)
    s[draw < 0.5] = -1.0
    return s


def rotate_in(w: np.ndarray, signs: np.ndarray | None = None, block: int = 256) -> np.ndarray:
    """W [N][K] -> W diag(signs) blockdiag(H_block): rotation of the input dimension, in fp32.

    Reference: h3metal/quant.py:31-44 (block fixed at 256 there; same reshape-and-matmul per block, fp32 BLAS,
    rows processed in batches of max(1, 2^24 // K))."""
    n_rows, k = w.shape
    if k % block:
        raise ValueError(f"input dimension {k} is not a multiple of {block}")
    h = hadamard(block)
    x = np.asarray(w, dtype=np.float32)
    if signs is not None:
        x = x * signs[None, :]
    res = np.empty((n_rows, k), dtype=np.float32)
    batch = max(1, (1 << 24) // k)
    for r0 in range(0, n_rows, batch):
        part = x[r0:r0 + batch]
        res[r0:r0 + batch] = (part.reshape(part.shape[0], k // block, block) @ h).reshape(part.shape[0], k)
    return res


_Q8_GRID = (1.0, 0.97, 0.94, 0.9, 0.85)


def quant_q8(w: np.ndarray, search: bool = True):
    """Per-row symmetric int8 codes and fp32 scales.

    Reference: h3metal/quant.py:77-82 with the clip search of :63-74: for each factor c of the grid the scale is
    max(amax*c/127, 1e-12); the factor with the smallest squared round-to-nearest error (fp64 sum, strict '<', so
    the first best wins) is kept. Without search the scale is max(amax/127, 1e-12). Codes are
    clip(rint(w / s), -127, 127)."""
    amax = np.abs(w).max(axis=1)
    if search:
        best_err = np.full(amax.shape, np.inf, dtype=np.float64)
        scale = np.zeros_like(amax)
        for c in _Q8_GRID:
            s = np.maximum(amax * c / 127, 1e-12)
            q = np.clip(np.rint(w / s[:, None]), -127, 127)
            err = ((q * s[:, None] - w) ** 2).sum(axis=-1, dtype=np.float64)
            better = err < best_err
            best_err = np.where(better, err, best_err)
            scale = np.where(better, s, scale)
    else:
        scale = np.maximum(amax / 127, 1e-12)
    codes = np.clip(np.rint(w / scale[:, None]), -127, 127).astype(np.int8)
    return codes, scale.astype(np.float32)


def dequant_q8(codes: np.ndarray, sw: np.ndarray) -> np.ndarray:
    """The fp32 matrix the codes stand for. Reference: h3metal/quant.py:103-106."""
    return codes.astype(np.float32) * sw[:, None]
