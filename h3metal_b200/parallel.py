"""Sharding the quantised linears of a transformer block over the GPUs of one node.

The reference is single-GPU; this module is new design on top of its operator API. One process per GPU
(`torch.distributed`, NCCL over NVLink; gloo on CPU for the tests), three strategies:

token-sharded   Rows are independent (per-token scales, per-row products), so each rank runs the whole layer on
                M / p rows with replicated weights. No communication; bit-identical to one GPU.
column-parallel W's rows (outputs) are split; activations are replicated; each rank produces its N / p columns.
                Fused outputs are split PER SEGMENT (q | k | v, value | gate) so that a rank holds matching slices:
                its value and gate columns line up for the swiglu rotate+quantise that feeds the next, row-parallel
                layer. No communication; bit-identical per column.
row-parallel    W's columns (K) are split; the input arrives already sharded on K (it is the previous
                column-parallel layer's output). The reference quantises a token with ONE scale over the whole row
                (kernels/ops.metal:315-317), so: (1) every rank rotates its shard and reports the row maxima,
                (2) MAX all-reduce of M floats, (3) every rank quantises with the reduced maximum, (4) int8 product
                into raw int32 accumulators, (5) SUM all-reduce of the int32 partials - integer addition is exact in
                any order - (6) one epilogue (h3b_dequant_i32). Result: bit-identical to one GPU at any p. With
                `scatter=True` step (5) is a reduce-scatter and every rank finishes only its M / p rows (what a
                following per-token operation needs; half the traffic). A faster, approximate variant all-reduces
                dequantised fp32 or bf16 partials instead (`reduce="f32" | "bf16"`).
                `reduce="push"` (exact) and `reduce="push_bf16"` take the communication library off the data path
                (the row maxima are exchanged the same way, by peer stores into per-rank slots):
                the product kernel stores every finished tile of its partial accumulators straight into the staging
                memory of the GPU that owns those rows (peer stores over NVLink, overlapping the rest of the
                product), a bounded device-side rendezvous follows, and each owner sums its M / p rows, applies the
                epilogue and - unless `scatter=True` - stores the finished bf16 rows into every GPU's output. Exact
                int32 partials cross NVLink once (reduce-scatter) and the all-gather moves 2-byte outputs, a quarter
                less traffic than an int32 all-reduce; `push_bf16` halves the first leg again.
                K / p must be a multiple of the rotation block.
                A LoRA term on a row-parallel layer (`lora=`, push variants with int32 staging): the term's input-side
                product T = A' x is a product over K like the main one, so every rank multiplies its K shard of A'
                (prepared from the whole A, hence the unsharded layer's codes and scales) and pushes the int32
                partial sums [M][R] to the rows' owners next to the main partials; after the same rendezvous the
                owner adds them exactly, stores T for its rows in fp16, forms T B'^T for its rows with the product
                kernel's low-rank path (on an all-zero int8 product, whose epilogue stores 0 + low) and adds it after
                the bias in the reduction. T is bit-identical to one GPU's at any p.
                Failure behaviour of the push variants: the device-side rendezvous polls for about a second; when a
                rank is late or absent the waiting rank's kernel records the give-up and returns, the reduction
                queued behind it stores nothing (no sum over staging that was never filled reaches an output), and
                `gpu.wait()` raises on that rank. `RowParallelLinear.recover()` on every rank re-aligns the layer.

Collectives run on torch's current stream, which is also the stream the kernels are launched on, so a layer is
one ordered sequence of kernels and collectives without host synchronisation.
"""

from __future__ import annotations

import numpy as np

from . import ops
from .gpu import Gpu, Tensor
from .linear import HostStaged


def _dist():
    import torch.distributed as dist
    return dist


def shard_bounds(n: int, rank: int, world: int, multiple: int = 1):
    """[start, stop) of rank's share of n items when n splits evenly into `world` pieces of a multiple of `multiple`."""
    if n % (world * multiple):
        raise ValueError(f"{n} does not split into {world} shards that are multiples of {multiple}")
    per = n // world
    return rank * per, (rank + 1) * per


def column_slices(N: int, splits, rank: int, world: int, multiple: int = 32):
    """Row ranges of W [N][K] a rank owns under column parallelism: its 1/world share of every segment of `splits`
    (default one segment = all of N), in segment order."""
    splits = list(splits) if splits else [N]
    if sum(splits) != N:
        raise ValueError(f"segments {splits} do not add up to {N}")
    out, base = [], 0
    for seg in splits:
        lo, hi = shard_bounds(seg, rank, world, multiple)
        out.append((base + lo, base + hi))
        base += seg
    return out


def take_rows(arr, slices):
    """Concatenation of the row ranges `slices` of a NumPy array or torch tensor."""
    if isinstance(arr, np.ndarray):
        return np.ascontiguousarray(np.concatenate([arr[a:b] for a, b in slices], axis=0))
    import torch
    return torch.cat([arr[a:b] for a, b in slices], dim=0).contiguous()


def _put(gpu, t):
    if t is None:
        return None
    return gpu.upload(t) if isinstance(t, np.ndarray) else gpu.wrap(t)


def push_layout(m_pad: int, N: int, world: int, stage_dtype: str, out_dtype: str | None):
    """Byte layout of a rank's peer block for the push variants, after the flag words: two staging buffers (calls
    alternate between them) of `world` slots [rows][N] each, then, if out_dtype is given, the full output [m_pad][N].
    Returns (rows, slot_bytes, stage_bytes, out_offset, total_bytes)."""
    if m_pad % (128 * world):
        raise ValueError(f"{m_pad} rows do not split into {world} shards of whole 128-row tiles")
    if N % 32:
        raise ValueError(f"N = {N} is not a multiple of 32")
    rows = m_pad // world
    slot = rows * N * {"i32": 4, "bf16": 2}[stage_dtype]
    stage = world * slot
    out = m_pad * N * {"bf16": 2, "f16": 2, "f32": 4}[out_dtype] if out_dtype else 0
    return rows, slot, stage, 2 * stage, 2 * stage + out


class PeerBlock:
    """One block of shareable device memory per rank of `group`, with every other rank's block mapped into this
    process (CUDA IPC; peer access over NVLink). The first 256 bytes of a block are its rendezvous flag words."""

    FLAG_BYTES = 256

    def __init__(self, gpu: Gpu, group, nbytes: int):
        dist = _dist()
        self.gpu, self.group = gpu, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.local = gpu.peer_alloc(self.FLAG_BYTES + int(nbytes))
        self.nbytes = self.FLAG_BYTES + int(nbytes)
        self.base = [self.local.ptr] * self.world
        self.epoch = 0
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, gpu.peer_export(self.local.ptr), group=group)
            self.base = [self.local.ptr if q == self.rank else gpu.peer_import(handles[q]) for q in range(self.world)]
            dist.barrier(group=group)  # every block exists, is zeroed and is mapped everywhere before anyone writes

    def addr(self, q: int, offset: int) -> int:
        """Address, in this process, of byte `offset` of rank q's data area."""
        return self.base[q] + self.FLAG_BYTES + offset

    def view(self, offset: int, shape, dtype: str) -> Tensor:
        """Typed view of this rank's own data area."""
        return type(self.local)(self.local.buf, self.FLAG_BYTES + offset, tuple(shape), dtype)

    def sync(self, mode: int = 0):
        """Rendezvous of all ranks on the device (bounded wait; a rank that never arrives surfaces at wait())."""
        self.epoch += 1
        self.gpu.peer_sync_native(self.base, self.rank, self.world, self.epoch, mode)

    def resync(self):
        """Host-side recovery after a rendezvous ran out on some rank (the error surfaced at that rank's wait()):
        every rank of the group calls this; they agree on the largest epoch any of them reached, so that the next
        rendezvous waits for a value nobody has signalled yet. Collective over the process group, no kernel."""
        if self.world > 1:
            dist = _dist()
            seen = [None] * self.world
            dist.all_gather_object(seen, self.epoch, group=self.group)
            self.epoch = max(seen)

    def close(self):
        if self.base is None:
            return
        self.gpu.wait()
        if self.world > 1:
            _dist().barrier(group=self.group)  # nobody unmaps or frees while a peer may still store into it
        for q, ptr in enumerate(self.base):
            if q != self.rank:
                self.gpu.peer_unmap(ptr)
        self.gpu.peer_free(self.local.ptr)
        self.base = None


class TokenShardedLinear:
    """The whole layer on this rank's rows [m0, m0 + rows) of M."""

    def __init__(self, gpu: Gpu, group, wt: ops.QWeight, M: int, *, block: int = 128, swiglu_in: bool = False,
                 out_dtype: str = "bf16"):
        dist = _dist()
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.m0, m1 = shard_bounds(M, self.rank, self.world, 128)
        self.rows = m1 - self.m0
        self.gpu, self.wt, self.block, self.swiglu_in = gpu, wt, block, swiglu_in
        self.a8 = gpu.empty((self.rows, wt.K), "i8")
        self.sa = gpu.empty((self.rows,), "f32")
        self.out = gpu.empty((self.rows, wt.N), out_dtype)

    def __call__(self, x_local: Tensor) -> Tensor:
        ops.rot_q8(self.gpu, x_local, self.a8, self.sa, self.rows, self.wt.K, swiglu=self.swiglu_in, block=self.block)
        ops.gemm(self.gpu, self.a8, self.wt, self.out, self.rows, sa=self.sa, tile=(128, 32, 4))
        return self.out


class ColumnParallelLinear:
    """This rank's N / p outputs of the layer; x is the full (replicated) activation."""

    def __init__(self, gpu: Gpu, group, codes, scales, bias, M: int, *, block: int = 128, splits=None,
                 swiglu_in: bool = False, out_dtype: str = "bf16", lora=None, scratch: ops.Scratch | None = None,
                 n_total: int | None = None):
        """codes int8 [N][K], scales and bias fp32 [N] of the WHOLE layer, of which this rank keeps its rows - or,
        with n_total given, already only this rank's rows of a layer of n_total outputs (a caller that draws or
        loads per rank need not materialise the whole weight). lora = (A [r][K], B [N][r]) is always the whole term."""
        dist = _dist()
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        N, K = codes.shape
        self.slices = column_slices(int(n_total or N), splits, self.rank, self.world)
        if n_total is not None:
            if sum(b - a for a, b in self.slices) != int(N):
                raise ValueError(f"{N} local rows are not this rank's share of {n_total}")
            local = [(0, int(N))]
        else:
            local = self.slices
        low = None
        if lora is not None:
            # (A [r][K] in the rotated input space, B [N][r]): the term is prepared from the whole B, so that its
            # normalisation and A's codes are the unsharded layer's, and this rank keeps the rows of B' it owns
            A_l, B_l = lora
            low = ops.low_rank(gpu, A_l, B_l, scratch or ops.Scratch(gpu), rows=self.slices)
        self.wt = ops.QWeight("q8", _put(gpu, take_rows(codes, local)), _put(gpu, take_rows(scales, local)),
                              sum(b - a for a, b in local), int(K),
                              bias=_put(gpu, take_rows(bias, local)) if bias is not None else None, low=low)
        self.gpu, self.M, self.block, self.swiglu_in = gpu, M, block, swiglu_in
        self.m_pad = ops.pad_rows(M)
        self.a8 = gpu.empty((self.m_pad, int(K)), "i8")
        self.sa = gpu.empty((self.m_pad,), "f32")
        self.out = gpu.empty((self.m_pad, self.wt.N), out_dtype)

    def __call__(self, x: Tensor, x_stride: int | None = None) -> Tensor:
        ops.rot_q8(self.gpu, x, self.a8, self.sa, self.M, self.wt.K, swiglu=self.swiglu_in, x_stride=x_stride,
                   block=self.block)
        ops.gemm(self.gpu, self.a8, self.wt, self.out, self.M, sa=self.sa, tile=(128, 32, 4))
        return self.out


class RowParallelLinear:
    """The layer with K split over the ranks; x_local is this rank's K / p channels (2K / p holding value | gate with
    swiglu_in). The output [M][N] is complete on every rank after the reduction."""

    def __init__(self, gpu: Gpu, group, codes, scales, bias, M: int, *, block: int = 128, swiglu_in: bool = False,
                 out_dtype: str = "bf16", reduce: str = "int32", scatter: bool = False, lora=None,
                 scratch: ops.Scratch | None = None):
        """lora = (A [r][K], B [N][r]) of the WHOLE layer, A in the rotated input space (reduce="push" only)."""
        dist = _dist()
        if reduce not in ("int32", "f32", "bf16", "push", "push_bf16"):
            raise ValueError(f"reduce={reduce!r}")
        if scatter and reduce not in ("int32", "push", "push_bf16"):
            raise ValueError("scatter=True is implemented for the int32 reduction and the push variants")
        if lora is not None and reduce != "push":
            raise ValueError("a low-rank term on a row-parallel layer needs reduce='push' (exact int32 partial sums of T)")
        self.group, self.reduce, self.scatter = group, reduce, scatter
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        N, K = codes.shape
        k0, k1 = shard_bounds(int(K), self.rank, self.world, block)
        local = codes[:, k0:k1]
        local = np.ascontiguousarray(local) if isinstance(local, np.ndarray) else local.contiguous()
        self.wt = ops.QWeight("q8", _put(gpu, local), _put(gpu, scales), int(N), k1 - k0)
        self.bias = _put(gpu, bias)
        self.gpu, self.M, self.block, self.swiglu_in = gpu, M, block, swiglu_in
        self.m_pad = ops.pad_rows(M)
        self.a8 = gpu.empty((self.m_pad, k1 - k0), "i8")
        self.sa = gpu.empty((self.m_pad,), "f32")
        self.push = reduce.startswith("push")
        if self.push:
            self.stage_dtype = "i32" if reduce == "push" else "bf16"
            self.rows, self.slot_bytes, self.stage_bytes, out_off, total = push_layout(
                self.m_pad, int(N), self.world, self.stage_dtype, None if scatter else out_dtype)
            self.r0 = self.rank * self.rows
            # behind the staging and the output: a table of `world` slots of row maxima, for the whole-row scale
            self.amax_offset = total
            total += self.world * self.m_pad * 4
            self.low = None
            if lora is not None:
                # The term is prepared from the whole A and B; this rank keeps its K shard of A's codes. Behind the
                # maxima: two staging buffers of `world` slots [rows][R] int32 for T's partial sums.
                A_l, B_l = lora
                self.low = ops.low_rank(gpu, A_l, B_l, scratch or ops.Scratch(gpu))
                R = self.low.R
                self.low_a = ops.QWeight("q8", gpu.upload(np.ascontiguousarray(self.low.codes[:, k0:k1])), self.low.a.sw, R,
                                         k1 - k0)
                self.t_slot_bytes = self.rows * R * 4
                self.t_offset = total
                total += 2 * self.world * self.t_slot_bytes
                self.t_rows = gpu.empty((self.rows, R), "f16")        # T of this rank's rows
                self.low_rows = gpu.empty((self.rows, int(N)), "f32")  # T B'^T of this rank's rows
                # an all-zero int8 product of the output's shape: its epilogue stores 0 * sa * sw + low = low
                zero_w = ops.QWeight("q8", gpu.empty((int(N), 128), "i8"), gpu.empty((int(N),), "f32"), int(N), 128)
                self.zero = (gpu.empty((self.rows, 128), "i8"), gpu.empty((self.rows,), "f32"), zero_w)
            self.block_mem = PeerBlock(gpu, group, total)
            self.out_offset, self.calls = out_off, 0
            self.out = (gpu.empty((self.rows, int(N)), out_dtype) if scatter
                        else self.block_mem.view(out_off, (self.m_pad, int(N)), out_dtype))
            return
        self.low = None
        self.out = gpu.empty((self.m_pad, int(N)), out_dtype)
        self.partial = gpu.empty((self.m_pad, int(N)), {"int32": "i32", "f32": "f32", "bf16": "bf16"}[reduce])
        if scatter:  # every rank keeps only its M / p rows of the result: half the traffic of an all-reduce
            self.r0, r1 = shard_bounds(self.m_pad, self.rank, self.world, 1)
            self.rows = r1 - self.r0
            self.part_rows = gpu.empty((self.rows, int(N)), "i32")
            self.out = gpu.empty((self.rows, int(N)), out_dtype)

    def __call__(self, x_local: Tensor, x_stride: int | None = None) -> Tensor:
        dist = _dist()
        gpu, wt, M = self.gpu, self.wt, self.M
        # (1)-(3): one scale per token over the WHOLE row
        self._quantise(x_local, x_stride)
        # (4)-(6)
        if self.push:
            return self._push(gpu, wt)
        if self.reduce == "int32":
            ops.gemm(gpu, self.a8, wt, self.partial, M, sa=self.sa, tile=(128, 32, 4))  # i32 output: raw accumulators
            if self.scatter:
                if self.world > 1:
                    dist.reduce_scatter_tensor(self.part_rows.torch(), self.partial.torch(), op=dist.ReduceOp.SUM,
                                               group=self.group)
                    acc = self.part_rows
                else:
                    acc = self.partial
                gpu.dequant_native(acc, wt.N, self.sa.view((self.rows,), offset_elems=self.r0), wt.sw, self.bias, self.out,
                                   wt.N, self.rows, wt.N)
                return self.out  # rows [r0, r0 + rows) of the layer's output
            if self.world > 1:
                dist.all_reduce(self.partial.torch(), op=dist.ReduceOp.SUM, group=self.group)
            gpu.dequant_native(self.partial, wt.N, self.sa, wt.sw, self.bias, self.out, wt.N, self.m_pad, wt.N)
            return self.out
        # approximate variants: dequantised partials are summed; the bias joins on rank 0 only
        part_wt = ops.QWeight("q8", wt.w, wt.sw, wt.N, wt.K, bias=self.bias if self.rank == 0 else None)
        ops.gemm(gpu, self.a8, part_wt, self.partial, M, sa=self.sa, tile=(128, 32, 4))
        if self.world > 1:
            dist.all_reduce(self.partial.torch(), op=dist.ReduceOp.SUM, group=self.group)
        if self.partial.dtype == self.out.dtype:
            return self.partial
        self.out.torch().copy_(self.partial.torch())
        return self.out


    def accumulate_gated(self, x_local: Tensor, X: Tensor, rtype: Tensor, gate: Tensor, g_stride: int,
                         x_stride: int | None = None) -> Tensor:
        """The layer with the reference's second epilogue (ops.gemm(..., epi=1), h3metal/ops.py:124-174): instead of
        returning the output, X[m][n] += gate[rtype[m]][n] * y[m][n] on THIS rank's M / p rows of the fp32 residual
        stream. X fp32 [rows][N] and rtype u8 [rows] hold the rank's own rows; gate fp32 [types][g_stride]. Push
        variants only (every rank finishes its own rows)."""
        if not self.push:
            raise ValueError("accumulate_gated needs reduce='push' or 'push_bf16'")
        return self._push(self.gpu, self.wt, x_local, x_stride, gated=(X, rtype, gate, g_stride))

    def _quantise(self, x_local: Tensor, x_stride: int | None):
        dist = _dist()
        gpu, D = self.gpu, self.wt.K
        stride = x_stride or (2 * D if self.swiglu_in else D)
        mode = 1 if self.swiglu_in else 0
        if self.push and self.world > 1 and x_local.dtype in ("bf16", "f16") and D % 64 == 0 and D <= 16384:
            # the maxima travel like the partial products: every rank stores its shard's maxima into its slot of
            # every rank's table, a rendezvous, then each rank takes the largest over the slots of its own table
            mem = self.block_mem
            slot = self.amax_offset + self.rank * self.m_pad * 4
            gpu.rot_amax_push_native(x_local, stride, [mem.addr(q, slot) for q in range(self.world)], self.M, D,
                                     self.block, mode)
            mem.sync()
            gpu.rot_q8_given_amax_slots_native(x_local, stride, self.a8, mem.addr(self.rank, self.amax_offset), self.m_pad,
                                               self.world, self.sa, self.M, D, self.block, mode)
            return
        gpu.rot_amax_native(x_local, stride, self.sa, self.M, D, self.block, mode)
        if self.world > 1:
            dist.all_reduce(self.sa.torch(), op=dist.ReduceOp.MAX, group=self.group)
        gpu.rot_q8_given_amax_native(x_local, stride, self.a8, self.sa, self.M, D, self.block, mode)

    def _push(self, gpu: Gpu, wt: ops.QWeight, x_local: Tensor | None = None, x_stride: int | None = None,
              gated=None) -> Tensor:
        if x_local is not None:
            self._quantise(x_local, x_stride)
        mem, N = self.block_mem, wt.N
        buf = (self.calls % 2) * self.stage_bytes  # calls alternate between the two staging buffers
        self.calls += 1
        # this rank's slot in every owner's staging buffer
        slots = [mem.addr(o, buf + self.rank * self.slot_bytes) for o in range(self.world)]
        low = self.low
        if low is not None:
            # the K shard's partial sums of T = A' x, pushed to the rows' owners like the main partials (before them,
            # so that the one rendezvous below covers both)
            t_buf = self.t_offset + ((self.calls - 1) % 2) * self.world * self.t_slot_bytes
            t_slots = [mem.addr(o, t_buf + self.rank * self.t_slot_bytes) for o in range(self.world)]
            gpu.gemm_push_native(self.a8, wt.K, self.low_a.w, self.low_a.w_stride, None, None, t_slots, self.rows, "i32",
                                 low.R, self.m_pad, low.R, wt.K)
        gpu.gemm_push_native(self.a8, wt.K, wt.w, wt.w_stride, wt.sw, self.sa, slots, self.rows, self.stage_dtype, N,
                             self.m_pad, N, wt.K)
        mem.sync()  # every rank's partials of my rows have landed
        esize = 4 if self.stage_dtype == "i32" else 2
        sa_rows = self.sa.ptr + 4 * self.r0
        if low is not None:
            # T of my rows: the exact sum of the shards' partial sums, then T's own epilogue (fp16 store); the term of
            # my rows from the product kernel's low-rank path on an all-zero product
            gpu.reduce_dequant_native(mem.addr(self.rank, t_buf), self.t_slot_bytes // 4, low.R, "i32", self.world, sa_rows,
                                      low.a.sw, None, [self.t_rows.ptr], "f16", low.R, self.rows, low.R)
            a0, sa0, w0 = self.zero
            gpu.gemm_native(a0, 128, w0.w, 128, w0.sw, sa0, None, self.low_rows, "f32", N, self.rows, N, 128,
                            self.t_rows, low.R, low.b, low.R, low.R, low.table(gpu, gpu.gemm_tile_n(N, True)).ptr + 8,
                            name="gemm(low-rank term of my rows)")
        if gated is not None:
            X, rtype, gate, g_stride = gated
            if low is not None:
                gpu.reduce_dequant_low_native(mem.addr(self.rank, buf), self.slot_bytes // esize, N, self.stage_dtype,
                                              self.world, sa_rows, wt.sw, self.bias, self.low_rows, N, [X.ptr], "f32", N,
                                              self.rows, N, 0, rtype.ptr, gate, g_stride)
                return X
            gpu.reduce_dequant_gated_native(mem.addr(self.rank, buf), self.slot_bytes // esize, N, self.stage_dtype,
                                            self.world, sa_rows, wt.sw, self.bias, X, N, self.rows, N, 0,
                                            rtype.ptr, gate, g_stride)
            return X
        outs = [self.out.ptr] if self.scatter else [mem.addr(q, self.out_offset) for q in range(self.world)]
        if low is not None:
            gpu.reduce_dequant_low_native(mem.addr(self.rank, buf), self.slot_bytes // esize, N, self.stage_dtype,
                                          self.world, sa_rows, wt.sw, self.bias, self.low_rows, N, outs, self.out.dtype, N,
                                          self.rows, N, row0=0 if self.scatter else self.r0)
        else:
            gpu.reduce_dequant_native(mem.addr(self.rank, buf), self.slot_bytes // esize, N, self.stage_dtype, self.world,
                                      sa_rows, wt.sw, self.bias, outs, self.out.dtype, N, self.rows, N,
                                      row0=0 if self.scatter else self.r0)
        if not self.scatter:
            mem.sync()  # every rank's finished rows have landed in my output
        return self.out

    def recover(self):
        """After a rendezvous of a push variant ran out (a rank was late or absent; `gpu.wait()` raised on the ranks
        that waited in vain, and their owner-side reductions stored nothing): brings the ranks' rendezvous counters
        and staging-buffer turns back in step. Every rank of the group calls it, between steps, with no kernel of
        the layer in flight. The next call then runs normally."""
        if self.push:
            self.block_mem.resync()
            if self.world > 1:
                dist = _dist()
                seen = [None] * self.world
                dist.all_gather_object(seen, self.calls, group=self.group)
                self.calls = max(seen)

    def close(self):
        if self.push:
            self.block_mem.close()


class TensorParallelBlock(HostStaged):
    """The four linears of a DiT block (QKV, attention-out, w1|w3, w2) sharded as column / row / column / row, with
    synthetic weights drawn per rank on the device (timing only). Inputs that the model's attention and norm kernels
    would produce (outside this path) are synthetic buffers of the right, sharded shapes. With `all_column` every
    linear is column-parallel (N-sharded) and reads its own full-width input: no exchange at all."""

    def __init__(self, gpu: Gpu, group, cfg, seed: int = 0, reduce: str = "int32", scatter: bool = False,
                 all_column: bool = False):
        import torch
        from . import workloads
        dist = _dist()
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        gen = torch.Generator(device=gpu.torch_device)
        gen.manual_seed(seed * 1000 + rank)
        rng = np.random.default_rng(seed)  # the same on every rank: low-rank terms are prepared from the whole B
        dev = gpu.torch_device
        M, m_pad = cfg.M, ops.pad_rows(cfg.M)
        self.gpu, self.cfg, self.layers, self.inputs = gpu, cfg, [], []
        self.rank, self.world = rank, world
        self.scratch = ops.Scratch(gpu)
        for i, spec in enumerate(cfg.layers):
            feeds_swiglu = i + 1 < len(cfg.layers) and cfg.layers[i + 1].swiglu_in  # its output is value | gate
            bias = torch.randn(spec.N, generator=gen, device=dev) * 0.01 if cfg.bias else None
            lora = workloads.lora_np(rng, cfg.lora_rank, spec.K, spec.N, cfg.block) if cfg.lora_rank else None
            if spec.parallel == "column" or all_column:
                # a rank only needs its own rows: draw them directly (N / world rows)
                n_local = spec.N // world
                codes, scales = workloads.weight_torch(gen, n_local, spec.K, dev)
                splits = [spec.N // 2, spec.N // 2] if (not all_column and feeds_swiglu) else None
                layer = ColumnParallelLinear(gpu, group, codes, scales, bias[:n_local].contiguous() if bias is not None else None,
                                             M, block=cfg.block, splits=splits, swiglu_in=spec.swiglu_in and not all_column,
                                             lora=lora, scratch=self.scratch, n_total=spec.N)
                # with all_column a layer fed by swiglu reads its own (already activated) full-width input instead
                x = workloads.activations_torch(gen, m_pad, spec.K, cfg.n_outliers(spec.K), dev)
                self.inputs.append(gpu.wrap(x))
            else:
                codes, scales = workloads.weight_torch(gen, spec.N, spec.K, dev)
                layer = RowParallelLinear(gpu, group, codes, scales, bias, M, block=cfg.block,
                                          swiglu_in=spec.swiglu_in, reduce=reduce, scatter=scatter, lora=lora,
                                          scratch=self.scratch)
                if spec.swiglu_in:
                    self.inputs.append(None)  # the previous (column-parallel) layer's local value | gate output
                else:
                    x = workloads.activations_torch(gen, m_pad, spec.K // world, cfg.n_outliers(spec.K // world), dev)
                    self.inputs.append(gpu.wrap(x))
            self.layers.append(layer)

    def _result(self, i: int):
        """What this rank hands back to the host: its N / p columns of a column-parallel layer; its own M / p rows of
        a row-parallel layer (every rank holds the whole reduced output; together the ranks return it once)."""
        layer = self.layers[i]
        out = layer.out.torch()
        if isinstance(layer, RowParallelLinear) and not layer.scatter and self.world > 1:
            rows = layer.m_pad // self.world
            return out[self.rank * rows:(self.rank + 1) * rows]
        return out

    def step(self):
        prev = None
        for layer, x in zip(self.layers, self.inputs):
            prev = layer(prev if x is None else x)
        return prev

    def link_bytes(self):
        """Bytes this rank sends over NVLink per step, per layer (0 for layers without an exchange). Push variants:
        (p-1)/p of the partials (4 or 2 bytes an element) to the rows' owners plus, unless scatter, the owner's finished
        rows (2 bytes) to the p-1 peers; NCCL all-reduce of int32: 2 (p-1)/p of 4 bytes an element (ring or tree on
        the wire; the in-switch reduction sends every byte once)."""
        out, p = [], self.world
        for layer in self.layers:
            if not isinstance(layer, RowParallelLinear) or p == 1:
                out.append(0)
                continue
            mn = layer.m_pad * layer.wt.N
            if layer.push:
                b = (4 if layer.stage_dtype == "i32" else 2) * mn * (p - 1) // p
                if not layer.scatter:
                    b += 2 * mn * (p - 1) // p
            else:
                esize = {"int32": 4, "f32": 4, "bf16": 2}[layer.reduce]
                b = esize * mn * (p - 1) // p * (1 if layer.scatter else 2)
            out.append(b)
        return out

    def close(self):
        for layer in self.layers:
            if hasattr(layer, "close"):
                layer.close()


def check_sharded_chain(gpu: Gpu, group, reduce: str = "push", seed: int = 5) -> dict:
    """A small column-parallel -> row-parallel chain (value | gate up-projection, swiglu quantiser, down-projection)
    on this group against the SAME chain computed by this rank alone, bit for bit: the column-parallel outputs, the
    whole-row scales, this rank's K-shard of the int8 codes, and the reduced output. Every rank draws the same seeded
    data. Returns {"exact": bool, "failed": [names]}; collective, call on every rank."""
    dist = _dist()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    M, D, F, B = 1024, 1024, 2048, 128
    rng = np.random.default_rng(seed)
    from . import quant
    x = quant.bf16_bits((rng.standard_normal((M, D)) * 2).astype(np.float32))
    w_up = rng.integers(-127, 128, size=(2 * F, D), dtype=np.int8)
    s_up = rng.uniform(1e-3, 2e-3, size=2 * F).astype(np.float32)
    b_up = (rng.standard_normal(2 * F) * 0.01).astype(np.float32)
    w_dn = rng.integers(-127, 128, size=(D, F), dtype=np.int8)
    s_dn = rng.uniform(1e-3, 2e-3, size=D).astype(np.float32)
    b_dn = (rng.standard_normal(D) * 0.01).astype(np.float32)
    up = ColumnParallelLinear(gpu, group, w_up, s_up, b_up, M, block=B, splits=[F, F])
    down = RowParallelLinear(gpu, group, w_dn, s_dn, b_dn, M, block=B, swiglu_in=True, reduce=reduce)
    xs = gpu.upload(x, "bf16")
    h_local = up(xs)
    y = down(h_local)
    gpu.wait()
    full_up = ops.QWeight("q8", gpu.upload(w_up), gpu.upload(s_up), 2 * F, D, bias=gpu.upload(b_up))
    full_dn = ops.QWeight("q8", gpu.upload(w_dn), gpu.upload(s_dn), D, F, bias=gpu.upload(b_dn))
    a8, sa, h = gpu.empty((M, D), "i8"), gpu.empty((M,), "f32"), gpu.empty((M, 2 * F), "bf16")
    ops.rot_q8(gpu, xs, a8, sa, M, D, block=B)
    ops.gemm(gpu, a8, full_up, h, M, sa=sa, tile=(128, 32, 4))
    a8b, sab, y1 = gpu.empty((M, F), "i8"), gpu.empty((M,), "f32"), gpu.empty((M, D), "bf16")
    ops.rot_q8(gpu, h, a8b, sab, M, F, swiglu=True, block=B)
    ops.gemm(gpu, a8b, full_dn, y1, M, sa=sab, tile=(128, 32, 4))
    gpu.wait()
    hh = h.numpy()
    half = F // world
    checks = {
        "column-parallel output": np.array_equal(h_local.numpy(), np.concatenate([hh[:, a:b] for a, b in up.slices], axis=1)),
        "whole-row scales": np.array_equal(down.sa.numpy(), sab.numpy()),
        "K-shard codes": np.array_equal(down.a8.numpy(), a8b.numpy()[:, rank * half:(rank + 1) * half]),
        "row-parallel output": np.array_equal(y.numpy(), y1.numpy()),
    }
    down.close()
    failed = [k for k, ok in checks.items() if not ok]
    return {"exact": not failed, "failed": failed}
