"""BlockLinears: the block's linears strung together, device-resident and with host buffers."""
import numpy as np
import pytest

from h3metal_b200 import workloads
from h3metal_b200.linear import BlockLinears

pytestmark = pytest.mark.gpu

SMALL = workloads.Config("small-block", 384, (workloads.Linear("qkv", 512, 1536), workloads.Linear("out", 512, 512),
                                               workloads.Linear("w1w3", 512, 2048),
                                               workloads.Linear("w2", 1024, 512, swiglu_in=True)), block=128)


@pytest.mark.parametrize("lora", [0, 32])
def test_host_step_equals_device_step(gpu, lora):
    """step_host() (pinned host inputs and outputs, copies overlapped with the kernels on separate streams) gives
    bit for bit what step() gives on device-resident inputs, call after call."""
    import torch
    cfg = workloads.Config(SMALL.name, SMALL.M, SMALL.layers, block=128, lora_rank=lora)
    blk = BlockLinears(gpu, cfg, seed=3)
    blk.step()
    gpu.wait()
    want = [l.out.torch().clone() for l in blk.layers]
    host_in, host_out = blk.host_buffers()
    assert [h is None for h in host_in] == [False, False, False, True]   # w2 reads w1w3's output on the device
    assert [h is None for h in host_out] == [False, False, True, False]  # w1w3's output never leaves the device
    for h, x in zip(host_in, blk.inputs):
        if h is not None:
            h.copy_(x.torch().cpu())
            x.torch().zero_()  # the device copy must really come from the host buffer
    for _ in range(3):
        blk.step_host(host_in, host_out)
    blk.sync_host()
    for h, w in zip(host_out, want):
        if h is not None:
            assert torch.equal(h.view(torch.int16), w.cpu().view(torch.int16))
    assert blk.launches_per_step == (12 if lora else 8)


def test_linear_from_an_h3m_file_with_an_adapter(gpu, tmp_path):
    """A converted layer read from an .h3m file (weights.WeightFile.linear) with a stacked two-adapter LoRA term
    (lora.term / order / stack -> ops.low_rank) gives what the oracle computes from the same arrays."""
    import oracle
    from oracle import gemm_ref
    from h3metal_b200 import lora, ops, quant, weights
    rng = np.random.default_rng(12)
    M, K, N, block = 256, 1024, 768, 128
    signs = quant.random_signs(K, 5)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    codes, scales = quant.quantize("q8", quant.rotate_in(w, signs, block))
    bias = workloads.bias_np(rng, N)
    path = str(tmp_path / "layer.h3m")
    wr = weights.Writer(path, {"block": block})
    wr.linear("blk.0.out", "q8", N, K, codes, scales, bias=bias)
    wr.close()
    wf = weights.WeightFile(gpu, path)
    wt = wf.linear("blk.0.out")
    terms = [lora.term(rng.standard_normal((8, K)).astype(np.float32) * 0.05, rng.standard_normal((N, 8)).astype(np.float32) * 0.05,
                       strength=0.7, scale=2.0, signs=signs, block=block) for _ in range(2)]
    A, B = lora.stack(lora.order(terms))
    wt.low = ops.low_rank(gpu, A, B, ops.Scratch(gpu))
    xh = workloads.activations_np(rng, M, K, 4)
    a8, sa, out = gpu.empty((M, K), "i8"), gpu.empty((M,), "f32"), gpu.empty((M, N), "bf16")
    # activations go through the same signs before the block rotation: fold them into the input here
    x_signed = quant.bf16_bits(quant.bf16_to_f32(xh) * signs[None, :])
    ops.rot_q8(gpu, gpu.upload(x_signed, "bf16"), a8, sa, M, K, block=block)
    ops.gemm(gpu, a8, wt, out, M, sa=sa, tile=(128, 128, 4))
    gpu.wait()
    q, s = oracle.rot_q8_rows(x_signed, K, block=block)
    assert np.array_equal(a8.numpy(), q) and np.array_equal(sa.numpy(), s)
    stored, v, _ = gemm_ref.gemm_q8(q, codes, s, scales, bias, gemm_ref.low_rank_ref(A, B), "bf16")
    got = oracle.bf16_bits_to_f32(out.numpy()).astype(np.float64)
    assert np.linalg.norm(got - oracle.bf16_bits_to_f32(stored)) / np.linalg.norm(v) <= 1e-3
    # and the quantised layer still approximates the float layer with its adapters (int8 error level)
    dense = quant.bf16_to_f32(xh).astype(np.float64) @ w.T.astype(np.float64) + bias
    for t in terms:
        dense += quant.rotate_in(quant.bf16_to_f32(xh) * 1.0, signs, block).astype(np.float64) @ t.A.T.astype(np.float64) @ t.B.T.astype(np.float64)
    assert np.linalg.norm(got - dense) / np.linalg.norm(dense) < 0.03
    wf.close()


def test_zimage_block_matches_fp32_pytorch(gpu):
    """A whole Z-Image-shaped block (both quantising kernels, four int8 products, the fused residual update) against
    the same block in fp32 PyTorch on the dequantised weights: the reference's mini-model bound of 2 % relative
    error for int8 (tests/test_zimage_mini.py:43), with attention supplied by PyTorch on both sides."""
    import torch
    from h3metal_b200.zimage_block import ZImageBlock
    M, D, heads, F = 320, 512, 4, 1024
    blk = ZImageBlock(gpu, M, D, heads, F, block=128, seed=1)
    gen = torch.Generator(device=gpu.torch_device)
    gen.manual_seed(7)
    x0 = torch.randn(blk.m_pad, D, generator=gen, device=gpu.torch_device)
    x0[:, :3] *= 8.0  # outlier channels
    x = gpu.wrap(x0.clone())
    pending = blk.forward(x)
    blk.flush(x, pending)
    gpu.wait()
    want = blk.reference_forward(x0[:M])
    got = x.torch()[:M]
    err = float((got - want).norm() / want.norm())
    assert err < 0.02, err
    delta = float((want - x0[:M]).norm() / x0[:M].norm())
    assert delta > 0.2  # the block changes the stream by far more than the allowed error
