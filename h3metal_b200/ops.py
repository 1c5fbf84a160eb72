"""Launchers of the quantised-linear path, with the signatures of the reference's h3metal/ops.py.

`gemm` (:124-174), `rot_q8` (:214-222), `low_rank` (:85-112), `pad_rows` (:120), the dataclasses `QWeight` (:19-34)
and `LowRank` (:54-82) and the class `Scratch` (:37-47) keep their names, arguments and error behaviour. Each
function enqueues its kernels on `gpu`; results are available after `gpu.wait()`.

In scope: weight format "q8" with the storing epilogue (epi 0; outputs bf16 / f16 / f32) and the gated-residual
epilogue (epi 1, with ksplit), with bias and with a low-rank (LoRA) term; `norm_mod_q8` (:200-211), the other producer of int8 activations. Other weight formats raise. `rot_q8` takes one argument the
reference does not have, `block=` (the rotation block; the reference's kernel fixes it at 256).
"""

from __future__ import annotations

from dataclasses import dataclass, field, replace

import numpy as np

from .gpu import Gpu, Tensor, pack  # noqa: F401  (pack is re-exported like in the reference)
from .quant import RB

FMT_ID = {"q8": 1, "q4": 2, "q4g": 3, "f16": 4, "bf16": 5, "h8": 6, "h4": 7, "h4g": 8}
OUT_DT = {"f16": "half", "bf16": "bfloat", "f32": "float"}


@dataclass
class QWeight:
    """A linear layer's weight on the GPU: W[N][K], int8 codes with one fp32 scale per output row."""
    fmt: str           # "q8" (the other formats of the reference are not part of this library)
    w: Tensor          # codes, [N][K] row-major
    sw: Tensor | None  # fp32 scales [N]
    N: int
    K: int
    G: int = 128
    bias: Tensor | None = None
    ws: int | None = None  # row stride of the codes in elements, when it differs from K (a slice of K)
    low: "LowRank | None" = None  # a low-rank term added to the product (LoRA adapters)

    @property
    def w_stride(self) -> int:
        return self.ws or self.K


class Scratch:
    """A growable fp16 buffer for the low-rank terms' T (one per model: launches run in order)."""

    def __init__(self, gpu: Gpu):
        self.gpu, self.t, self.n = gpu, None, 0
        self.t32, self.n32 = None, 0

    def get(self, rows: int, cols: int) -> Tensor:
        if rows * cols > self.n:
            self.n = max(rows * cols, 2 * self.n)
            self.t = self.gpu.empty((self.n,), "f16")
        return self.t.view((rows, cols))

    def get_i32(self, rows: int, cols: int) -> Tensor:
        """A second, int32 buffer: partial accumulators of T when its product is split along K."""
        if rows * cols > self.n32:
            self.n32 = rows * cols
            self.t32 = self.gpu.empty((self.n32,), "i32")
        return self.t32.view((rows, cols))


LOW_TILE = (64, 32, 2)  # the input-side product's tile in the reference: R is a multiple of 32
RANK_STEP = 16          # rank ranges start and end on multiples of this (the fp16 MMA's K granularity)


@dataclass
class LowRank:
    """out += T B^T with T = A' x^T: the low-rank term of the product.

    a: the input side, a product of R outputs on the same int8 activations as the main product; b: [N][R] fp16;
    lo, hi: per output column, the rank range B touches."""
    a: QWeight
    b: Tensor
    lo: np.ndarray
    hi: np.ndarray
    scratch: Scratch
    tables: dict = field(default_factory=dict)
    codes: np.ndarray | None = None  # host copy of a's int8 codes [R][K], for the K-split layout
    splits: dict = field(default_factory=dict)

    @property
    def R(self) -> int:
        return self.a.N

    def split_major(self, gpu: Gpu, S: int) -> Tensor:
        """a's codes laid out [S][R][K / S]: slice s of every rank's K, contiguous, so that one product of the
        activations seen as [M * S][K / S] with this as [S * R][K / S] yields all S partial sums of T at once."""
        t = self.splits.get(S)
        if t is None:
            R, K = self.codes.shape
            t = gpu.upload(np.ascontiguousarray(self.codes.reshape(R, S, K // S).transpose(1, 0, 2)))
            self.splits[S] = t
        return t

    def table(self, gpu: Gpu, tn: int) -> Tensor:
        """int32 [T's row stride, B's row stride, then (k0, k1) per column tile of width tn]. A last, partial tile
        (N not a multiple of tn) gets the range of the columns it has."""
        t = self.tables.get(tn)
        if t is None:
            n = len(self.lo)
            n_t = -(-n // tn)
            lo = np.zeros(n_t * tn, np.int64)
            hi = np.zeros(n_t * tn, np.int64)
            lo[:n], hi[:n] = self.lo, self.hi  # columns past N (a partial last tile) touch no rank
            lo = lo.reshape(n_t, tn).min(1)
            hi = hi.reshape(n_t, tn).max(1)
            lo = np.where(hi > lo, lo // RANK_STEP * RANK_STEP, 0)
            hi = np.where(hi > lo, -(-hi // RANK_STEP) * RANK_STEP, 0)
            t = gpu.upload(np.concatenate([[self.R, self.R], np.stack([lo, hi], 1).reshape(-1)]).astype(np.int32))
            t.host_head = (self.R, self.R)  # the two leading strides, for callers that would otherwise read them back
            self.tables[tn] = t
        return t


def low_rank(gpu: Gpu, A: np.ndarray, B: np.ndarray, scratch: Scratch, act: str = "q8", rows=None) -> LowRank:
    """The low-rank term out += x A^T B^T for x the product's input (in the stored, rotated input space).

    A [r][K] and B [N][r] in float. Each rank's magnitude moves from B to A (B's columns are normalised to a maximum
    of 1) so that T and B fit fp16; A is then stored as int8 with per-rank scales and applied to the same int8
    activations as the main product. Host-side preparation, as in the reference.

    rows (not in the reference): a list of [start, stop) output ranges; the term is prepared from the WHOLE B - so
    that the normalisation and A's codes are those of the unsharded layer - and only those rows of B' are kept, in
    order (a GPU that holds a slice of the layer's outputs)."""
    from .quant import quant_q8
    if act != "q8":
        raise NotImplementedError("low_rank: only int8 activations (act='q8') are part of this library")
    r, K = A.shape
    N = B.shape[0]
    if B.shape[1] != r:
        raise ValueError(f"low rank: A {A.shape} and B {B.shape} disagree")
    R = -(-r // LOW_TILE[1]) * LOW_TILE[1]
    peak = np.abs(B).max(0)
    peak = np.where(peak > 0, peak, 1.0).astype(np.float64)
    a = np.zeros((R, K), np.float32)
    a[:r] = A.astype(np.float64) * peak[:, None]
    b = np.zeros((N, R), np.float16)
    b[:, :r] = (B.astype(np.float64) / peak[None, :]).astype(np.float16)
    codes, sw = quant_q8(a)
    aw = QWeight("q8", gpu.upload(codes), gpu.upload(sw), R, K)
    if rows is not None:
        b = np.ascontiguousarray(np.concatenate([b[r0:r1] for r0, r1 in rows], axis=0))
    used = b != 0
    any_used = used.any(1)
    lo = np.where(any_used, used.argmax(1), 0).astype(np.int64)
    hi = np.where(any_used, R - used[:, ::-1].argmax(1), 0).astype(np.int64)
    return LowRank(aw, gpu.upload(b), lo, hi, scratch, codes=codes)


def _t_split(gpu, lo: LowRank, m_rows: int, K: int, a_stride) -> int:
    """How many ways to split K in T's product: 1 unless the GPU asks for it (`gpu.lora_t_split`, the real Gpu's
    default), the activations are contiguous and the unsplit product would use at most half of the SMs."""
    want = getattr(gpu, "lora_t_split", 0)
    if not want or lo.codes is None or (a_stride not in (None, K)):
        return 1
    tiles = m_rows // 128
    for S in (4, 2):
        if S <= want and tiles * S <= 2 * getattr(gpu, "sm_count", 148) and tiles * 2 <= getattr(gpu, "sm_count", 148) \
                and K % (S * 128) == 0 and K // S >= 2048:  # measured: no gain from shorter slices (two launches)
            return S
    return 1


def pad_rows(m: int, tile: int = 128) -> int:
    return (m + tile - 1) // tile * tile


def gemm(gpu: Gpu, a: Tensor, wt: QWeight, out: Tensor, M: int, *, sa: Tensor | None = None, epi: int = 0,
         rtype: Tensor | None = None, gate: Tensor | None = None, g_stride: int = 0, c_stride: int | None = None,
         a_stride: int | None = None, tile=(64, 128, 4), swz: int = 1, ksplit: int = 1, _low=None):
    """out = A x W^T (epi 0), or out += gate[rtype] * (A x W^T) (epi 1, out the fp32 residual stream): int8 x int8
    with int32 accumulation, then acc * sa[m] * sw[n] + bias[n] + low.

    ksplit: accumulate the product in that many calls over consecutive slices of K (epi 1 only; the bias and the
    low-rank term join the first slice), exactly the sequence the reference runs. A weight with a low-rank term
    (wt.low) first computes the term's input side T from the same activations, then adds T B^T inside the main
    product's epilogue. `tile` keeps its checking role (its width must divide N, and rows are padded to its height,
    all of which are written); the kernel picks its own tile shape. `swz` is accepted and ignored (the kernel has
    its own L2-friendly tile order).
    """
    if wt.fmt != "q8":
        raise NotImplementedError(f"gemm: weight format {wt.fmt!r} is outside this library (int8 'q8' only)")
    if epi not in (0, 1):
        raise NotImplementedError(f"gemm: epilogue {epi}")
    if sa is None:
        raise ValueError("gemm: int8 activations need their row scales (sa)")
    if epi == 1 and (rtype is None or gate is None):
        raise ValueError("gemm: the gated-residual epilogue needs rtype and gate")
    if wt.low is not None:
        lo = wt.low
        # T covers the rows of the whole 128-row tiles the activations are allocated in
        m_rows = (M + 127) // 128 * 128
        t = lo.scratch.get(m_rows, lo.R)
        S = _t_split(gpu, lo, m_rows, wt.K, a_stride)
        if S > 1:
            # Few row tiles and a long K leave most SMs idle in T's product: split K S ways in ONE launch. The
            # activations seen as [M * S][K / S] times a's codes as [S * R][K / S] give, in the diagonal blocks of an
            # int32 [M * S][S * R] result, the S exact partial sums; the owner-side reduction kernel of the
            # row-parallel layers adds them and applies T's epilogue. Same bits as the unsplit product.
            R, kp = lo.R, wt.K // S
            part = lo.scratch.get_i32(m_rows * S, S * R)
            gpu.gemm_native(a.view((m_rows * S, kp)), kp, lo.split_major(gpu, S), kp, None, None, None, part, "i32", S * R,
                            m_rows * S, S * R, kp, name=f"gemm(q8,{wt.K}->{R},T split {S})")
            gpu.reduce_dequant_native(part.ptr, S * R + R, S * S * R, "i32", S, sa.ptr, lo.a.sw, None, [t.ptr], "f16", R,
                                      m_rows, R)
        else:
            gemm(gpu, a, lo.a, t, m_rows, sa=sa, a_stride=a_stride, tile=LOW_TILE)
        _low = (t, lo)
        wt = replace(wt, low=None)
    if ksplit > 1:
        if epi != 1 or wt.K % (ksplit * 256):
            raise ValueError(f"cannot split K of a {wt.fmt} product (epi {epi}, K {wt.K}) {ksplit} ways")
        kp = wt.K // ksplit
        for i in range(ksplit):
            part = replace(wt, w=wt.w.view((wt.N, kp), offset_elems=i * kp), K=kp, ws=wt.w_stride,
                           bias=wt.bias if i == 0 else None)
            gemm(gpu, a.view((a.shape[0], kp), offset_elems=i * kp), part, out, M, sa=sa, epi=1, rtype=rtype, gate=gate,
                 g_stride=g_stride, c_stride=c_stride, a_stride=a_stride or wt.K, tile=tile, swz=swz,
                 _low=_low if i == 0 else None)
        return
    tm, tn, _nsg = tile
    if wt.N % tn:
        raise ValueError(f"gemm tile {tile}: {tn} columns do not divide the product's {wt.N}")
    if epi == 1 and out.dtype != "f32":
        raise ValueError("gemm: the gated-residual epilogue accumulates into an fp32 tensor")
    if out.dtype not in OUT_DT and out.dtype != "i32":
        raise ValueError(f"gemm: output type {out.dtype}")
    m_pad = (M + tm - 1) // tm * tm
    lt = lb = None
    R = t_stride = b_stride = 0
    ranges_ptr = None
    if _low is not None:
        lt, lo = _low
        if lo.b.shape[0] != wt.N:
            raise ValueError(f"low-rank term for {lo.b.shape[0]} outputs on a product of {wt.N}")
        lb = lo.b
        R = t_stride = b_stride = lo.R
        ranges_ptr = lo.table(gpu, gpu.gemm_tile_n(wt.N, True)).ptr + 8  # skip the table's two leading strides
    tag = f"gemm(q8,{wt.K}->{wt.N}{',lora' if _low is not None else ''}{',epi1' if epi else ''})"
    if epi == 1:
        gpu.gemm_gated_native(a, a_stride or wt.K, wt.w, wt.w_stride, wt.sw, sa, wt.bias, out, c_stride or wt.N, m_pad,
                              wt.N, wt.K, rtype, gate, g_stride or wt.N, lt, t_stride, lb, b_stride, R, ranges_ptr,
                              name=tag)
        return
    gpu.gemm_native(a, a_stride or wt.K, wt.w, wt.w_stride, wt.sw, sa, wt.bias, out, out.dtype, c_stride or wt.N,
                    m_pad, wt.N, wt.K, lt, t_stride, lb, b_stride, R, ranges_ptr, name=tag)


def norm_mod_q8(gpu: Gpu, x: Tensor, mod: Tensor, rtype: Tensor, out: Tensor, sa: Tensor | None, M: int, D: int,
                *, eps: float, mod_stride: int | None = None, x_stride: int | None = None, out_f: bool = False,
                out_h: bool = False, out_hr: bool = False, y: Tensor | None = None, post: Tensor | None = None,
                ln: bool = False, block: int = RB):
    """out = int8(rot(rmsnorm(x) * mod[type][0] + mod[type][1])) and its row scales (or the plain modulated row as
    float with out_f, as half with out_h, the rotated row as half with out_hr). With y and post, first
    x += post * rmsnorm(y) (same eps), written back. ln: LayerNorm without affine (mean subtracted) instead of
    RMSNorm. Same signature as the reference's h3metal/ops.py:200-211 plus block=."""
    if D % block:
        raise ValueError(f"norm_mod_q8: {D} channels are not a multiple of the rotation block {block}")
    if (y is None) != (post is None):
        raise ValueError("norm_mod_q8: y and post go together")
    kind = 1 if out_f else 2 if out_h else 3 if out_hr else 0
    gpu.norm_mod_q8_native(x, x_stride or D, mod, mod_stride or 2 * D, rtype, out, sa, M, D, block, eps, ln, kind, y,
                           post, name=f"norm_mod_q8({D},b{block}{',ln' if ln else ''}{',post' if post is not None else ''})")


def rot_q8(gpu: Gpu, x: Tensor, out: Tensor, sa: Tensor | None, M: int, D: int, *, swiglu: bool = False,
           x_stride: int | None = None, out_hr: bool = False, block: int = RB):
    """out = int8(rot(x)) (or of value * silu(gate) with the gates in columns D..2D-1) and its row scales;
    with out_hr the rotated rows in half precision instead. block: channels per rotation block (64, 128, 256)."""
    if D % block:
        raise ValueError(f"rot_q8: {D} channels are not a multiple of the rotation block {block}")
    gpu.rot_q8_native(x, x_stride or (2 * D if swiglu else D), out, sa, M, D, block, 1 if swiglu else 0, out_hr,
                      name=f"rot_q8({D},b{block}{',swiglu' if swiglu else ''})")
