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
                K / p must be a multiple of the rotation block. A LoRA term on a row-parallel layer is not supported.

Collectives run on torch's current stream, which is also the stream the kernels are launched on, so a layer is
one ordered sequence of kernels and collectives without host synchronisation.
"""

from __future__ import annotations

import numpy as np

from . import ops
from .gpu import Gpu, Tensor


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
                 swiglu_in: bool = False, out_dtype: str = "bf16", lora=None, scratch: ops.Scratch | None = None):
        dist = _dist()
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        N, K = codes.shape
        self.slices = column_slices(int(N), splits, self.rank, self.world)
        low = None
        if lora is not None:
            # (A [r][K] in the rotated input space, B [N][r]): the term is prepared from the whole B, so that its
            # normalisation and A's codes are the unsharded layer's, and this rank keeps the rows of B' it owns
            A_l, B_l = lora
            low = ops.low_rank(gpu, A_l, B_l, scratch or ops.Scratch(gpu), rows=self.slices)
        self.wt = ops.QWeight("q8", _put(gpu, take_rows(codes, self.slices)), _put(gpu, take_rows(scales, self.slices)),
                              sum(b - a for a, b in self.slices), int(K),
                              bias=_put(gpu, take_rows(bias, self.slices)) if bias is not None else None, low=low)
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
                 out_dtype: str = "bf16", reduce: str = "int32", scatter: bool = False):
        dist = _dist()
        if reduce not in ("int32", "f32", "bf16", "push", "push_bf16"):
            raise ValueError(f"reduce={reduce!r}")
        if scatter and reduce not in ("int32", "push", "push_bf16"):
            raise ValueError("scatter=True is implemented for the int32 reduction and the push variants")
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
            self.block_mem = PeerBlock(gpu, group, total + self.world * self.m_pad * 4)
            self.out_offset, self.calls = out_off, 0
            self.out = (gpu.empty((self.rows, int(N)), out_dtype) if scatter
                        else self.block_mem.view(out_off, (self.m_pad, int(N)), out_dtype))
            return
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
        gpu.gemm_push_native(self.a8, wt.K, wt.w, wt.w_stride, wt.sw, self.sa, slots, self.rows, self.stage_dtype, N,
                             self.m_pad, N, wt.K)
        mem.sync()  # every rank's partials of my rows have landed
        esize = 4 if self.stage_dtype == "i32" else 2
        if gated is not None:
            X, rtype, gate, g_stride = gated
            gpu.reduce_dequant_gated_native(mem.addr(self.rank, buf), self.slot_bytes // esize, N, self.stage_dtype,
                                            self.world, self.sa.ptr + 4 * self.r0, wt.sw, self.bias, X, N, self.rows, N, 0,
                                            rtype.ptr, gate, g_stride)
            return X
        outs = [self.out.ptr] if self.scatter else [mem.addr(q, self.out_offset) for q in range(self.world)]
        gpu.reduce_dequant_native(mem.addr(self.rank, buf), self.slot_bytes // esize, N, self.stage_dtype, self.world,
                                  self.sa.ptr + 4 * self.r0, wt.sw, self.bias, outs, self.out.dtype, N, self.rows, N,
                                  row0=0 if self.scatter else self.r0)
        if not self.scatter:
            mem.sync()  # every rank's finished rows have landed in my output
        return self.out

    def close(self):
        if self.push:
            self.block_mem.close()


class TensorParallelBlock:
    """The four linears of a DiT block (QKV, attention-out, w1|w3, w2) sharded as column / row / column / row, with
    synthetic weights drawn per rank on the device (timing only). Inputs that the model's attention and norm kernels
    would produce (outside this path) are synthetic buffers of the right, sharded shapes."""

    def __init__(self, gpu: Gpu, group, cfg, seed: int = 0, reduce: str = "int32", scatter: bool = False):
        import torch
        from . import workloads
        dist = _dist()
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        gen = torch.Generator(device=gpu.torch_device)
        gen.manual_seed(seed * 1000 + rank)
        dev = gpu.torch_device
        M, m_pad = cfg.M, ops.pad_rows(cfg.M)
        self.gpu, self.cfg, self.layers, self.inputs = gpu, cfg, [], []
        for spec in cfg.layers:
            bias = torch.randn(spec.N, generator=gen, device=dev) * 0.01 if cfg.bias else None
            if spec.parallel == "column":
                # a rank only needs its own rows: draw them directly (N / world rows)
                codes, scales = workloads.weight_torch(gen, spec.N // world, spec.K, dev)
                layer = ColumnParallelLinear.__new__(ColumnParallelLinear)
                layer.rank, layer.world, layer.slices = rank, world, [(0, spec.N // world)]
                layer.wt = ops.QWeight("q8", gpu.wrap(codes), gpu.wrap(scales), spec.N // world, spec.K,
                                       bias=gpu.wrap(bias[:spec.N // world].contiguous()) if bias is not None else None)
                layer.gpu, layer.M, layer.block, layer.swiglu_in, layer.m_pad = gpu, M, cfg.block, spec.swiglu_in, m_pad
                layer.a8, layer.sa = gpu.empty((m_pad, spec.K), "i8"), gpu.empty((m_pad,), "f32")
                layer.out = gpu.empty((m_pad, spec.N // world), "bf16")
                x = workloads.activations_torch(gen, m_pad, spec.K, cfg.n_outliers(spec.K), dev)
                self.inputs.append(gpu.wrap(x))
            else:
                codes, scales = workloads.weight_torch(gen, spec.N, spec.K, dev)
                layer = RowParallelLinear(gpu, group, codes, scales, bias, M, block=cfg.block,
                                          swiglu_in=spec.swiglu_in, reduce=reduce, scatter=scatter)
                if spec.swiglu_in:
                    self.inputs.append(None)  # the previous (column-parallel) layer's local value | gate output
                else:
                    x = workloads.activations_torch(gen, m_pad, spec.K // world, cfg.n_outliers(spec.K // world), dev)
                    self.inputs.append(gpu.wrap(x))
            self.layers.append(layer)

    def step(self):
        prev = None
        for layer, x in zip(self.layers, self.inputs):
            prev = layer(prev if x is None else x)
        return prev
