"""The int8 product, its dequantising epilogue and the low-rank (LoRA) term, restated on the CPU.

Test infrastructure (see oracle/__init__.py). Follows kernels/gemm.metal:117-261 (format 1 = Q8, epilogue 0) and
h3metal/ops.py:54-112,124-174 of the reference.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .quant_ref import bf16_round_bits, quant_q8

RANK_TILE = 32   # the input-side product's tile width: R is a multiple of it (h3metal/ops.py:50)
RANK_STEP = 16   # rank ranges start and end on multiples of it (h3metal/ops.py:51)


def int32_product(a: np.ndarray, w: np.ndarray) -> np.ndarray:
    """acc[m][n] = sum_k a[m][k] * w[n][k], exact, returned as int32 (kernels/gemm.metal:201-208).

    Done in fp64 BLAS, which is exact because K * 127^2 < 2^53 (the reference's tests do the same,
    tests/test_gemm.py:31); |acc| <= K * 127^2 fits int32 for every K of the path."""
    acc = a.astype(np.float64) @ w.astype(np.float64).T
    return np.rint(acc).astype(np.int64).astype(np.int32)


def epilogue_q8(acc: np.ndarray, sa: np.ndarray, sw: np.ndarray, bias: np.ndarray | None = None,
                low: np.ndarray | None = None) -> np.ndarray:
    """fp32 value the kernel stores: float(acc) * sa[m] * sw[n], + bias[n], + low (kernels/gemm.metal:238-253).

    int32 -> fp32 conversion rounds to nearest even above 2^24, as the kernel's float(acc) does; the two
    multiplies and the adds are separate fp32 operations, left to right."""
    v = acc.astype(np.float32)
    v = (v * sa.astype(np.float32)[:, None]).astype(np.float32)
    v = (v * sw.astype(np.float32)[None, :]).astype(np.float32)
    if bias is not None:
        v = (v + bias.astype(np.float32)[None, :]).astype(np.float32)
    if low is not None:
        v = (v + low.astype(np.float32)).astype(np.float32)
    return v


def accumulate_gated(x: np.ndarray, v: np.ndarray, gate: np.ndarray, rtype: np.ndarray) -> np.ndarray:
    """Epilogue 1: X[m][n] += gate[type[m]][n] * v (kernels/gemm.metal:18-20,256-259), fp32 multiply then fp32 add;
    v already holds the bias and the low-rank term. Returns the new X."""
    t = (gate.astype(np.float32)[rtype] * v.astype(np.float32)).astype(np.float32)
    return (x.astype(np.float32) + t).astype(np.float32)


def store_as(v: np.ndarray, dtype: str) -> np.ndarray:
    """OUT_T(v) (kernels/gemm.metal:254-255): bf16 bit patterns (uint16), fp16 or fp32."""
    if dtype == "bf16":
        return bf16_round_bits(v)
    if dtype == "f16":
        return v.astype(np.float16)
    if dtype == "f32":
        return v.astype(np.float32)
    raise ValueError(dtype)


@dataclass
class LowRankRef:
    """What h3metal/ops.py:85-112 keeps of an adapter: int8 input side with scales, fp16 output side, and the
    rank range each output column touches."""
    a_codes: np.ndarray   # int8 [R][K]
    a_scales: np.ndarray  # fp32 [R]
    b: np.ndarray         # fp16 [N][R]
    lo: np.ndarray        # int64 [N]
    hi: np.ndarray        # int64 [N]

    @property
    def R(self) -> int:
        return self.a_codes.shape[0]


def low_rank_ref(A: np.ndarray, B: np.ndarray) -> LowRankRef:
    """Adapter A [r][K], B [N][r] (float, A in the rotated input space) -> stored term.

    Reference: h3metal/ops.py:85-112. R = r rounded up to 32; c_j = max_n |B[n][j]| (1 where that is 0) moves
    from B to A; A' = fp32(fp64(A) * c) zero-padded to R rows and quantised by quant_q8 (clip search on);
    B' = fp16(fp64(B) / c) zero-padded; lo/hi = first and one-past-last non-zero rank of each row of B'."""
    r, k = A.shape
    n = B.shape[0]
    if B.shape[1] != r:
        raise ValueError(f"low rank: A {A.shape} and B {B.shape} disagree")
    R = (r + RANK_TILE - 1) // RANK_TILE * RANK_TILE
    col_max = np.abs(B).max(axis=0)
    col_max = np.where(col_max > 0, col_max, 1.0).astype(np.float64)
    a_scaled = np.zeros((R, k), dtype=np.float32)
    a_scaled[:r] = A.astype(np.float64) * col_max[:, None]
    b_half = np.zeros((n, R), dtype=np.float16)
    b_half[:, :r] = (B.astype(np.float64) / col_max[None, :]).astype(np.float16)
    codes, scales = quant_q8(a_scaled)
    nonzero = b_half != 0
    touched = nonzero.any(axis=1)
    lo = np.where(touched, nonzero.argmax(axis=1), 0).astype(np.int64)
    hi = np.where(touched, R - nonzero[:, ::-1].argmax(axis=1), 0).astype(np.int64)
    return LowRankRef(codes, scales, b_half, lo, hi)


def lora_table(term: LowRankRef, tn: int) -> np.ndarray:
    """int32 [2 + 2 * N/tn]: T's row stride, B's row stride, then (k0, k1) per column tile of width tn.

    Reference: LowRank.table, h3metal/ops.py:71-82: the tile's range is the union of its columns' ranges, k0
    floored and k1 ceiled to multiples of 16, (0, 0) for a tile no rank touches."""
    tiles = len(term.lo) // tn
    lo = term.lo.reshape(tiles, tn).min(axis=1)
    hi = term.hi.reshape(tiles, tn).max(axis=1)
    lo = np.where(hi > lo, lo // RANK_STEP * RANK_STEP, 0)
    hi = np.where(hi > lo, -(-hi // RANK_STEP) * RANK_STEP, 0)
    return np.concatenate([[term.R, term.R], np.stack([lo, hi], axis=1).reshape(-1)]).astype(np.int32)


def lora_T(a: np.ndarray, sa: np.ndarray, term: LowRankRef) -> np.ndarray:
    """T[m][j] = fp16(float(acc_T) * sa[m] * sw_A[j]): the adapter's input-side product through the same Q8
    kernel with fp16 output (h3metal/ops.py:134-142; kernels/gemm.metal:238,254)."""
    acc = int32_product(a, term.a_codes)
    return epilogue_q8(acc, sa, term.a_scales).astype(np.float16)


def lora_low(T: np.ndarray, term: LowRankRef, tn: int | None = None) -> np.ndarray:
    """low[m][n] = sum_j T[m][j] * B'[n][j] (kernels/gemm.metal:211-229), fp16 inputs, wide accumulation.

    The reference's test builds the expected term in fp64 from the fp16 T and B' (tests/test_gemm.py:215-220);
    ranks outside a column tile's [k0, k1) hold zeros of B', so restricting the sum changes nothing."""
    return (T.astype(np.float64) @ term.b.astype(np.float64).T).astype(np.float32)


def gemm_q8(a: np.ndarray, w: np.ndarray, sa: np.ndarray, sw: np.ndarray, bias: np.ndarray | None = None,
            term: LowRankRef | None = None, out_dtype: str = "bf16"):
    """Whole product as ops.gemm runs it (h3metal/ops.py:124-174): optional T product, main product, epilogue.

    Returns (stored output in out_dtype, fp32 value before the store, int32 accumulators)."""
    acc = int32_product(a, w)
    low = lora_low(lora_T(a, sa, term), term) if term is not None else None
    v = epilogue_q8(acc, sa, sw, bias, low)
    return store_as(v, out_dtype), v, acc
