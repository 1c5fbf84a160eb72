"""One Z-Image-Turbo-shaped transformer block on the quantised-linear path, for block-level checks and timing.

The sequence of operators is the reference's ZImageDiT._block (h3metal/zimage.py:313-346):

    norm_mod_q8(x, pre_attn [, y, post])  ->  gemm qkv (bf16)  ->  per-head q/k RMSNorm + rotary  ->  attention
    ->  rot_q8  ->  gemm out (fp32 y)  ->  norm_mod_q8(x, pre_mlp, y, post_attn)   [x += post_attn * rmsnorm(y)]
    ->  gemm fc1 (bf16, value | gate)  ->  rot_q8(swiglu)  ->  gemm fc2 (fp32 y)   [x += post_mlp * rmsnorm(y) is left
    pending for the next block's first norm, as in the reference]

Every linear and both activation-quantising kernels run through this library. The per-head norm + rotary and the
attention itself are NOT part of the path (the reference has its own kernels for them, kernels/ops.metal:365-468 and
kernels/attention.metal); here they are PyTorch calls (scaled_dot_product_attention), present only so that a
whole block can be timed and compared. `reference_forward` is the same block in plain fp32 PyTorch on the
dequantised weights, the yardstick the reference's mini-model tests use (tests/test_zimage_mini.py:43: < 2 %).
"""

from __future__ import annotations

from . import ops, quant, workloads
from .gpu import Gpu
from .linear import upload_weight


class ZImageBlock:
    def __init__(self, gpu: Gpu, M: int, D: int = 3840, heads: int = 30, F: int = 10240, *, block: int = 128,
                 eps: float = 1e-5, seed: int = 0):
        import torch
        if D % heads or (D // heads) % 2:
            raise ValueError("hidden size must split into heads of even size")
        self.gpu, self.M, self.D, self.H, self.hd, self.F, self.block, self.eps = gpu, M, D, heads, D // heads, F, block, eps
        dev = gpu.torch_device
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed)
        self.m_pad = ops.pad_rows(M)

        def linear(n, k):
            codes, scales = workloads.weight_torch(gen, n, k, dev)
            return upload_weight(gpu, codes, scales), codes, scales
        self.qkv, self.out, self.fc1, self.fc2 = linear(3 * D, D), linear(D, D), linear(2 * F, D), linear(D, F)
        rnd = lambda *shape: torch.randn(*shape, generator=gen, device=dev)  # noqa: E731
        # modulation tables: one row type; scale' = norm weight * (1 + scale), shift
        self.pre_attn = torch.stack([1 + 0.1 * rnd(D), 0.1 * rnd(D)]).reshape(1, 2, D).contiguous()
        self.pre_mlp = torch.stack([1 + 0.1 * rnd(D), 0.1 * rnd(D)]).reshape(1, 2, D).contiguous()
        self.post_attn, self.post_mlp = 0.5 + 0.1 * rnd(D), 0.5 + 0.1 * rnd(D)
        self.q_norm, self.k_norm = 1 + 0.1 * rnd(self.hd), 1 + 0.1 * rnd(self.hd)
        ang = torch.rand(self.m_pad, self.hd // 2, generator=gen, device=dev) * 6.28
        self.cos, self.sin = ang.cos(), ang.sin()
        self.rt = gpu.empty((self.m_pad,), "u8")
        # activations
        self.a8 = gpu.empty((self.m_pad, max(F, D)), "i8")
        self.sa = gpu.empty((self.m_pad,), "f32")
        self.wide = gpu.empty((self.m_pad, max(3 * D, 2 * F)), "bf16")
        self.o = gpu.empty((self.m_pad, D), "bf16")
        self.y = gpu.empty((self.m_pad, D), "f32")
        self._w = {k: gpu.wrap(v) for k, v in (("pre_attn", self.pre_attn), ("pre_mlp", self.pre_mlp),
                                               ("post_attn", self.post_attn), ("post_mlp", self.post_mlp))}

    # -- the parts that are not on the path: PyTorch ---------------------------------------------------------------
    def _rope(self, t):  # t [M][H][hd]; pairs (i, i + hd/2), as the reference's rotary
        half = self.hd // 2
        c, s = self.cos[:t.shape[0], None, :], self.sin[:t.shape[0], None, :]
        a, b = t[..., :half], t[..., half:]
        return self._cat(a * c - b * s, b * c + a * s)

    @staticmethod
    def _cat(a, b):
        import torch
        return torch.cat([a, b], dim=-1)

    def _attention(self, qkv):  # qkv [M][3D] float -> [M][D]
        import torch
        M, D, H, hd = qkv.shape[0], self.D, self.H, self.hd
        q, k, v = (qkv[:, i * D:(i + 1) * D].reshape(M, H, hd) for i in range(3))
        rms = lambda t, w: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + self.eps) * w  # noqa: E731
        q, k = self._rope(rms(q, self.q_norm)), self._rope(rms(k, self.k_norm))
        to = lambda t: t.transpose(0, 1)[None].to(torch.bfloat16)  # noqa: E731  (flash attention runs on bf16)
        o = torch.nn.functional.scaled_dot_product_attention(to(q), to(k), to(v))
        return o[0].transpose(0, 1).reshape(M, D).float()

    # -- the block on the quantised path ---------------------------------------------------------------------------
    def forward(self, x, pending=None):
        """x: Tensor fp32 [m_pad][D], updated in place (the residual stream). pending: post vector of the previous
        block's MLP (a Tensor) with its y in self.y, or None. Returns the post vector left pending (a Tensor)."""
        import torch
        g, M, D, F, blk = self.gpu, self.M, self.D, self.F, self.block
        a8d, a8f = self.a8.view((self.m_pad, D)), self.a8.view((self.m_pad, F))
        fused = {"y": self.y, "post": pending} if pending is not None else {}
        ops.norm_mod_q8(g, x, self._w["pre_attn"], self.rt, a8d, self.sa, M, D, eps=self.eps, block=blk, **fused)
        qkv = self.wide.view((self.m_pad, 3 * D))
        ops.gemm(g, a8d, self.qkv[0], qkv, M, sa=self.sa, tile=(128, 128, 4))
        with torch.cuda.stream(g.stream):
            self.o.torch()[:M] = self._attention(qkv.torch()[:M].float()).to(torch.bfloat16)
        ops.rot_q8(g, self.o, a8d, self.sa, M, D, block=blk)
        ops.gemm(g, a8d, self.out[0], self.y, M, sa=self.sa, tile=(128, 128, 4))
        ops.norm_mod_q8(g, x, self._w["pre_mlp"], self.rt, a8d, self.sa, M, D, eps=self.eps, block=blk, y=self.y,
                        post=self._w["post_attn"])
        h = self.wide.view((self.m_pad, 2 * F))
        ops.gemm(g, a8d, self.fc1[0], h, M, sa=self.sa, tile=(128, 128, 4))
        ops.rot_q8(g, h, a8f, self.sa, M, F, swiglu=True, block=blk)
        ops.gemm(g, a8f, self.fc2[0], self.y, M, sa=self.sa, tile=(128, 128, 4))
        return self._w["post_mlp"]

    def flush(self, x, pending):
        """x += pending * rmsnorm(y): the update a following block would fuse into its first norm (PyTorch)."""
        import torch
        with torch.cuda.stream(self.gpu.stream):
            y = self.y.torch()[:self.M]
            x.torch()[:self.M] += pending.torch() * y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + self.eps)

    # -- the same block in fp32 PyTorch on the dequantised weights -----------------------------------------------------
    def reference_forward(self, x):
        """x: torch fp32 [M][D] -> the residual stream after the block (both updates applied), no quantisation of
        activations, weights dequantised, Hadamard rotation omitted (it cancels between activations and weights)."""
        import torch
        deq = lambda t: t[1].float() * t[2][:, None]  # noqa: E731  (codes, scales) -> fp32 weight in the rotated space
        rms = lambda t: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + self.eps)  # noqa: E731
        H = torch.as_tensor(quant.hadamard(self.block), device=x.device)
        rotate = lambda t: (t.reshape(t.shape[0], -1, self.block) @ H).reshape(t.shape)  # noqa: E731
        lin = lambda t, w: rotate(t) @ deq(w).T  # noqa: E731  the stored weights live in the rotated input space
        a = rms(x) * self.pre_attn[0, 0] + self.pre_attn[0, 1]
        o = self._attention(lin(a, self.qkv))
        x = x + self.post_attn * rms(lin(o, self.out))
        a = rms(x) * self.pre_mlp[0, 0] + self.pre_mlp[0, 1]
        h = lin(a, self.fc1)
        hh = h[:, :self.F] * torch.nn.functional.silu(h[:, self.F:])
        return x + self.post_mlp * rms(lin(hh, self.fc2))

