"""The numeric core of LoRA adapters on the int8 linear path: scaling, input-side rotation and rank stacking.

The reference's h3metal/lora.py parses adapter files and maps their modules onto converted (fused, permuted) layers;
that bookkeeping is model- and file-format specific and not part of this library. What the product kernels depend
on is what happens to the two factors once a layer is resolved (h3metal/lora.py:291-310): A is scaled by
strength * alpha / r, its input dimension is rotated exactly like the layer's weight (so the term applies to the
rotated, quantised activations), B's rows are placed at the layer's output rows, and several adapters on one layer
are stacked rank by rank, ordered by their first output row so that each column tile touches a narrow rank range.
The result feeds `ops.low_rank()`.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .quant import RB, rotate_in


@dataclass
class Term:
    """One adapter on one converted layer: A [r][K] in the layer's rotated input space, B [N][r] on its output rows."""
    A: np.ndarray
    B: np.ndarray


def term(A: np.ndarray, B: np.ndarray, *, strength: float = 1.0, scale: float = 1.0, signs: np.ndarray | None = None,
         rotate: bool = True, rows: np.ndarray | None = None, n_out: int | None = None, block: int = RB) -> Term:
    """A [r][K], B [out][r] of the original layer -> the Term of the converted layer.

    strength * scale (scale = alpha / r of the adapter file) moves into A; with `rotate` the input dimension goes
    through the layer's rotation (signs, then block Hadamard); `rows` places B's rows at output rows of a fused layer
    of n_out rows (default: B as is)."""
    a = (np.asarray(A, np.float32) * np.float32(strength * scale)).astype(np.float32)
    if rotate:
        a = rotate_in(a, signs, block)
    b = np.asarray(B, np.float32)
    if rows is not None:
        placed = np.zeros((n_out if n_out is not None else int(np.max(rows)) + 1, b.shape[1]), np.float32)
        placed[np.asarray(rows)] = b
        b = placed
    return Term(a, b)


def order(terms: list) -> list:
    """Terms of one layer sorted by the first output row they touch (h3metal/lora.py:304-305)."""
    return sorted(terms, key=lambda t: int(np.argmax(np.abs(t.B).sum(1) > 0)))


def stack(terms: list) -> tuple:
    """Terms of one layer -> one low-rank pair (A [R][K], B [N][R]) with the ranks side by side
    (h3metal/lora.py:308-310)."""
    return np.concatenate([t.A for t in terms]), np.concatenate([t.B for t in terms], axis=1)
