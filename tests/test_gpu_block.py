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
