"""A quantised linear layer as the reference's transformer blocks run it: rotate + quantise the activations, then
the int8 product with its epilogue (h3metal/dit.py:209-217, h3metal/zimage.py:328-345: `ops.rot_q8` followed by
`ops.gemm`). `QuantLinear` owns the layer's device buffers so that a step launches kernels and nothing else;
`BlockLinears` strings the linears of one transformer block together for the benchmark and the smoke test.
"""

from __future__ import annotations

import numpy as np

from . import ops, workloads
from .gpu import Gpu, Tensor


class QuantLinear:
    """y = W8A8(x): x bf16 [M][K] (or [M][2K] holding value | gate with swiglu_in) -> y [M][N] of out_dtype."""

    def __init__(self, gpu: Gpu, wt: ops.QWeight, M: int, *, block: int = 128, swiglu_in: bool = False,
                 out_dtype: str = "bf16"):
        self.gpu, self.wt, self.M, self.block, self.swiglu_in = gpu, wt, M, block, swiglu_in
        self.m_pad = ops.pad_rows(M)
        self.a8 = gpu.empty((self.m_pad, wt.K), "i8")
        self.sa = gpu.empty((self.m_pad,), "f32")
        self.out = gpu.empty((self.m_pad, wt.N), out_dtype)

    def __call__(self, x: Tensor, x_stride: int | None = None) -> Tensor:
        ops.rot_q8(self.gpu, x, self.a8, self.sa, self.M, self.wt.K, swiglu=self.swiglu_in, x_stride=x_stride,
                   block=self.block)
        ops.gemm(self.gpu, self.a8, self.wt, self.out, self.M, sa=self.sa, tile=(128, 32, 4))
        return self.out

    @property
    def launches_per_call(self) -> int:
        return 3 if self.wt.low is not None else 2


def upload_weight(gpu: Gpu, codes, scales, bias=None, low=None) -> ops.QWeight:
    """QWeight from NumPy arrays or torch device tensors (int8 codes [N][K], fp32 scales [N], fp32 bias [N])."""
    def put(t):
        if t is None:
            return None
        return gpu.upload(t) if isinstance(t, np.ndarray) else gpu.wrap(t)
    N, K = codes.shape
    return ops.QWeight("q8", put(codes), put(scales), int(N), int(K), bias=put(bias), low=low)


class HostStaged:
    """The step of a chain of layers for a caller whose activations live in HOST memory. The class that mixes this in
    provides `gpu`, `layers` (callables: layer(src) -> output Tensor) and `inputs` (per layer its own device input,
    or None when it consumes the previous layer's output)."""

    def _result(self, i: int):
        """torch view of what layer i hands back to the host."""
        return self.layers[i].out.torch()

    def host_buffers(self):
        """Pinned host tensors for step_host(): one input per layer that reads its own input, one output per layer
        whose result leaves the block (a layer that only feeds the next linear on the device has none)."""
        import torch
        ins, outs = [], []
        for i, x in enumerate(self.inputs):
            ins.append(None if x is None else torch.empty(x.shape, dtype=torch.bfloat16).pin_memory())
            feeds_next = i + 1 < len(self.layers) and self.inputs[i + 1] is None
            outs.append(None if feeds_next else torch.empty(self._result(i).shape, dtype=torch.bfloat16).pin_memory())
        return ins, outs

    def step_host(self, host_in, host_out):
        """One pass with host inputs and outputs. Uploads run on one copy stream, kernels on the context's stream,
        downloads on a second copy stream, chained per layer by events: the upload of layer i+1 and the download of
        layer i-1 overlap the kernels of layer i, and (PCIe being full duplex) each other. Buffers are guarded per
        layer, so consecutive calls overlap too. Results are in host_out after `sync_host()`."""
        import torch
        if not hasattr(self, "_up"):
            dev = self.gpu.torch_device
            self._up, self._down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
            n = len(self.layers)
            self._in_ready = [torch.cuda.Event() for _ in range(n)]
            self._in_free = [torch.cuda.Event() for _ in range(n)]
            self._out_ready = [torch.cuda.Event() for _ in range(n)]
            self._out_free = [torch.cuda.Event() for _ in range(n)]
            self._primed = False
        compute = self.gpu.stream
        prev = None
        for i, (layer, x) in enumerate(zip(self.layers, self.inputs)):
            if x is not None:
                if self._primed:
                    self._up.wait_event(self._in_free[i])     # the previous call's kernels have read this input
                with torch.cuda.stream(self._up):
                    x.torch().copy_(host_in[i], non_blocking=True)
                    self._in_ready[i].record(self._up)
                compute.wait_event(self._in_ready[i])
            if self._primed and host_out[i] is not None:
                compute.wait_event(self._out_free[i])         # the previous call's download of this output is done
            prev = layer(prev if x is None else x)
            if x is not None:
                self._in_free[i].record(compute)
            if host_out[i] is not None:
                self._out_ready[i].record(compute)
                self._down.wait_event(self._out_ready[i])
                with torch.cuda.stream(self._down):
                    host_out[i].copy_(self._result(i), non_blocking=True)
                    self._out_free[i].record(self._down)
        self._primed = True

    def finish_host(self):
        """Makes the context's stream wait for every copy step_host() has issued (so that an event recorded on it
        afterwards marks the moment the last download landed)."""
        if hasattr(self, "_down"):
            self._down.wait_stream(self._up)
            self.gpu.stream.wait_stream(self._down)

    def sync_host(self):
        """Blocks until every upload, kernel and download issued by step_host() has finished."""
        if hasattr(self, "_down"):
            self._down.synchronize()
            self._up.synchronize()
        self.gpu.stream.synchronize()


class BlockLinears(HostStaged):
    """The linears of one transformer block of `cfg` on one GPU, with synthetic weights drawn on the device.

    Layers whose input is the previous layer's output (swiglu_in) consume it; the others read their own input
    buffer (in the model these come from the norm / attention kernels, which are not part of this path)."""

    def __init__(self, gpu: Gpu, cfg: workloads.Config, seed: int = 0, M: int | None = None, layers=None):
        import torch
        self.gpu, self.cfg = gpu, cfg
        self.M = M or cfg.M
        gen = torch.Generator(device=gpu.torch_device)
        gen.manual_seed(seed)
        self.scratch = ops.Scratch(gpu)
        self.layers, self.inputs = [], []
        rng = np.random.default_rng(seed)
        for spec in (layers or cfg.layers):
            codes, scales = workloads.weight_torch(gen, spec.N, spec.K, gpu.torch_device)
            bias = (torch.randn(spec.N, generator=gen, device=gpu.torch_device) * 0.01) if cfg.bias else None
            low = None
            if cfg.lora_rank:
                A, B = workloads.lora_np(rng, cfg.lora_rank, spec.K, spec.N, cfg.block)
                low = ops.low_rank(gpu, A, B, self.scratch)
            wt = upload_weight(gpu, codes, scales, bias, low)
            self.layers.append(QuantLinear(gpu, wt, self.M, block=cfg.block, swiglu_in=spec.swiglu_in))
            if spec.swiglu_in:
                self.inputs.append(None)
            else:
                x = workloads.activations_torch(gen, ops.pad_rows(self.M), spec.K, cfg.n_outliers(spec.K),
                                                gpu.torch_device)
                self.inputs.append(gpu.wrap(x))

    def step(self):
        """One pass over the block's linears: 2 launches per layer (3 with a LoRA term)."""
        prev = None
        for layer, x in zip(self.layers, self.inputs):
            prev = layer(prev if x is None else x)
        return prev

    def rot_only(self):
        """Only the rotate+quantise launches of a step (each on the input the step gives it)."""
        prev = None
        for layer, x in zip(self.layers, self.inputs):
            src = prev if x is None else x
            ops.rot_q8(self.gpu, src, layer.a8, layer.sa, layer.M, layer.wt.K, swiglu=layer.swiglu_in, block=layer.block)
            prev = layer.out

    def gemm_only(self):
        """Only the product launches of a step (on the codes the last rotate+quantise left in each layer's buffers)."""
        for layer in self.layers:
            ops.gemm(self.gpu, layer.a8, layer.wt, layer.out, layer.M, sa=layer.sa, tile=(128, 32, 4))

    @property
    def launches_per_step(self) -> int:
        return sum(l.launches_per_call for l in self.layers)

    @property
    def ops_per_step(self) -> int:
        return sum(2 * self.M * l.wt.K * l.wt.N for l in self.layers)
