"""The benchmark configurations of the quantised-linear path and seeded synthetic data of their shapes.

The shapes are those of the transformer blocks the reference runs (Z-Image-Turbo: h3metal/zimage.py:313-346;
FLUX.2 [klein] 4B: h3metal/flux2.py:428-479; a 33B-class DiT: h3metal/dit.py:191-217); the data are synthetic and
seeded and stand in for real checkpoints and activations, as in the reference's own layer benchmarks
(bench/zimage_layer_bench.py:25-38). Activations are bf16 N(0, 1) with a few outlier channels scaled by 20;
weights are fp32 N(0, 0.02), Hadamard-rotated along K and quantised per output channel; biases N(0, 0.01);
LoRA factors N(0, 0.01) rounded to bf16.

Two generators: NumPy (CPU, exact reference pipeline, for parity cases) and torch-on-device (fast, for timing
at full size; it draws the rotated weight directly, which has the same distribution because the rotation is
orthonormal, and quantises with the plain absmax scale).
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import quant


@dataclass(frozen=True)
class Linear:
    name: str
    K: int
    N: int
    swiglu_in: bool = False  # the input is value * silu(gate) of the previous layer's 2K-wide output
    parallel: str = "column"  # how the layer is sharded over GPUs: "column" (N) or "row" (K)


@dataclass(frozen=True)
class Config:
    name: str
    M: int
    layers: tuple
    block: int = 128
    outlier_frac: float = 0.002
    outliers: int | None = None  # fixed count instead of a fraction
    bias: bool = True
    lora_rank: int = 0

    def n_outliers(self, K: int) -> int:
        return self.outliers if self.outliers is not None else int(round(self.outlier_frac * K))

    @property
    def ops(self) -> int:
        return sum(2 * self.M * l.K * l.N for l in self.layers)


def _block(d: int, f: int, qkv: int | None = None):
    return (Linear("qkv", d, qkv or 3 * d), Linear("out", d, d, parallel="row"), Linear("w1w3", d, 2 * f),
            Linear("w2", f, d, swiglu_in=True, parallel="row"))


CONFIGS = {
    0: Config("single-linear-3072", 4096, (Linear("linear", 3072, 3072),), outliers=8),
    1: Config("zimage-turbo-6b-block", 4608, _block(3840, 10240)),
    2: Config("flux2-klein-4b-double-block", 4608,
              (Linear("qkv", 3072, 9216), Linear("out", 3072, 3072, parallel="row"), Linear("mlp_up", 3072, 9216),
               Linear("mlp_down", 9216, 3072, parallel="row")), lora_rank=32),
    # the same block with the MLP as the reference's FLUX.2 runs it: fc1 3072 -> 18432 (value | gate), the SwiGLU
    # quantiser, fc2 9216 -> 3072 (h3metal/flux2.py:142-144), timed beside the literal shape of configuration 2
    5: Config("flux2-klein-4b-double-block-swiglu-mlp", 4608,
              (Linear("qkv", 3072, 9216), Linear("out", 3072, 3072, parallel="row"), Linear("fc1", 3072, 18432),
               Linear("fc2", 9216, 3072, swiglu_in=True, parallel="row")), lora_rank=32),
    3: Config("dit-33b-block-2048px", 17408, _block(6144, 16384)),
    4: Config("dit-33b-block-4096px-lora64", 66560, _block(6144, 16384), lora_rank=64),
}


# ---- NumPy generators (exact pipeline) ------------------------------------------------------------------------------
def activations_np(rng: np.random.Generator, M: int, K: int, n_outliers: int) -> np.ndarray:
    """bf16 bit patterns [M][K]: N(0, 1) with `n_outliers` channels scaled by 20."""
    x = rng.standard_normal((M, K)).astype(np.float32)
    if n_outliers:
        x[:, rng.choice(K, size=n_outliers, replace=False)] *= 20.0
    return quant.bf16_bits(x)


def weight_np(rng: np.random.Generator, N: int, K: int, block: int, search: bool = True):
    """(int8 codes [N][K], fp32 scales [N]) of a N(0, 0.02) weight rotated with `block`-channel Hadamard blocks."""
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    return quant.quant_q8(quant.rotate_in(w, None, block), search=search)


def bias_np(rng: np.random.Generator, N: int) -> np.ndarray:
    return (rng.standard_normal(N) * 0.01).astype(np.float32)


def lora_np(rng: np.random.Generator, r: int, K: int, N: int, block: int):
    """LoRA factors as the path consumes them: A [r][K] already in the rotated input space, B [N][r]; both N(0, 0.01)
    rounded to bf16 and handed on as fp32."""
    A = quant.bf16_to_f32(quant.bf16_bits((rng.standard_normal((r, K)) * 0.01).astype(np.float32)))
    B = quant.bf16_to_f32(quant.bf16_bits((rng.standard_normal((N, r)) * 0.01).astype(np.float32)))
    return quant.rotate_in(A, None, block), B


# ---- device generators (timing at full size) ---------------------------------------------------------------------------
def activations_torch(gen, M: int, K: int, n_outliers: int, device):
    import torch
    x = torch.randn(M, K, generator=gen, device=device, dtype=torch.float32)
    if n_outliers:
        idx = torch.randperm(K, generator=gen, device=device)[:n_outliers]
        x[:, idx] *= 20.0
    return x.to(torch.bfloat16)


def weight_torch(gen, N: int, K: int, device, rows_per_step: int = 4096):
    """(int8 codes [N][K], fp32 scales [N]) of a N(0, 0.02) weight with the plain absmax scale, built in slabs."""
    import torch
    codes = torch.empty(N, K, device=device, dtype=torch.int8)
    scales = torch.empty(N, device=device, dtype=torch.float32)
    for r0 in range(0, N, rows_per_step):
        w = torch.randn(min(rows_per_step, N - r0), K, generator=gen, device=device) * 0.02
        s = (w.abs().amax(dim=1) / 127).clamp_min(1e-12)
        codes[r0:r0 + len(w)] = torch.round(w / s[:, None]).clamp_(-127, 127).to(torch.int8)
        scales[r0:r0 + len(w)] = s
    return codes, scales
