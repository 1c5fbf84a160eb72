"""The runtime object: the reference's Gpu / Tensor semantics (h3metal/gpu.py:121-265) on CUDA."""
import struct

import numpy as np
import pytest

import oracle
from oracle import gemm_ref
from h3metal_b200 import ops
from h3metal_b200.gpu import GpuError, pack

pytestmark = pytest.mark.gpu


def test_device_and_memory(gpu):
    assert "B200" in gpu.device and gpu.sm_count >= 100 and gpu.working_set > 100 << 30
    t = gpu.empty((3, 5), "f32")
    assert not t.numpy().any()  # zero-filled like the reference's buffers
    arr = np.arange(24, dtype=np.float32).reshape(4, 6)
    up = gpu.upload(arr)
    assert up.dtype == "f32" and np.array_equal(up.numpy(), arr)
    assert np.array_equal(up.row(1, 2).numpy(), arr[1:3])
    assert np.array_equal(up.view((6,), offset_elems=6).numpy(), arr[1])
    bits = np.array([0x3F80, 0xC000], np.uint16)
    assert gpu.upload(bits).dtype == "bf16" and np.array_equal(gpu.upload(bits, "bf16").numpy(), bits)


def test_wait_returns_gpu_seconds_and_profile_lists_launches(gpu):
    rng = np.random.default_rng(0)
    a = gpu.upload(rng.integers(-127, 128, size=(256, 512), dtype=np.int8))
    wt = ops.QWeight("q8", gpu.upload(rng.integers(-127, 128, size=(256, 512), dtype=np.int8)),
                     gpu.upload(np.ones(256, np.float32)), 256, 512)
    sa, out = gpu.upload(np.ones(256, np.float32)), gpu.empty((256, 256), "f16")
    gpu.wait()
    assert gpu.wait() == 0.0
    before = gpu.launch_count
    ops.gemm(gpu, a, wt, out, 256, sa=sa)
    ops.gemm(gpu, a, wt, out, 256, sa=sa)
    dt = gpu.wait()
    assert 0 < dt < 0.1 and gpu.launch_count == before + 2
    gpu.profile(True)
    ops.gemm(gpu, a, wt, out, 256, sa=sa)
    ops.rot_q8(gpu, gpu.empty((4, 512), "bf16"), gpu.empty((4, 512), "i8"), gpu.empty((4,), "f32"), 4, 512)
    took = gpu.profile_take()
    gpu.profile(False)
    assert [n.split("(")[0] for n, _ in took] == ["gemm", "rot_q8"] and all(0 < s < 0.1 for _, s in took)


def test_generic_launch_of_the_reference(gpu, golden):
    """Code written against the reference's kernel()/launch() pair keeps working for the path's two kernels."""
    rng = np.random.default_rng(1)
    M, N, K = 128, 256, 512
    a = rng.integers(-127, 128, size=(M, K), dtype=np.int8)
    w = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    sa = rng.uniform(0.001, 0.01, size=M).astype(np.float32)
    sw = rng.uniform(0.001, 0.01, size=N).astype(np.float32)
    out = gpu.empty((M, N), "f16")
    k = gpu.kernel("gemm.metal", "gemm", WFMT=1, EPI=0, OUT_T="half", TM=64, TN=128, NSG=4, G=128, HAS_BIAS=0,
                   FAST_LAYOUT=0, SWZ=1, LORA=0)
    gpu.launch(k, (N // 128, M // 64, 1), (128, 1, 1),
               [gpu.upload(a), gpu.upload(w), gpu.upload(sw), gpu.upload(sa), out, None, None, None],
               pack("8i", M, N, K, K, N, K, K // 128, N), params_index=8)
    xh = golden["rot_x_bits"]
    q8, s8 = gpu.empty((5, 768), "i8"), gpu.empty((5,), "f32")
    k2 = gpu.kernel("ops.metal", "rot_q8", NSG=3, MAXB=1, IN_T="bfloat", OUT_HR=0)
    gpu.launch(k2, (5, 1, 1), (96, 1, 1), [gpu.upload(xh, "bf16"), q8, s8], pack("4i", 5, 768, 1536, 0))
    gpu.wait()
    stored, _, _ = gemm_ref.gemm_q8(a, w, sa, sw, None, None, "f16")
    assert np.array_equal(out.numpy(), stored)
    q, s = oracle.rot_q8_rows(xh, 768, block=256)
    assert np.array_equal(q8.numpy(), q) and np.array_equal(s8.numpy(), s)
    assert pack("4i", 1, 2, 3, 4) == struct.pack("<4i", 1, 2, 3, 4)


def test_kernels_outside_the_path_are_refused(gpu):
    with pytest.raises(GpuError):
        gpu.kernel("attention.metal", "attention", HD=128)
    k = gpu.kernel("gemm.metal", "gemm", WFMT=2, EPI=0, OUT_T="half")
    with pytest.raises(GpuError):
        gpu.launch(k, (1, 1, 1), (32, 1, 1), [None] * 8, pack("8i", 64, 128, 256, 256, 128, 256, 2, 128), params_index=8)


def test_an_expired_device_wait_surfaces_at_wait_and_the_context_survives(gpu):
    """Every device-side wait is bounded. The self-test kernel waits on a barrier nothing signals; the wait runs out,
    the kernel returns normally, wait() raises with the recorded reason, and the same context then computes a correct
    product (nothing trapped, nothing hung)."""
    from h3metal_b200.gpu import lib
    gpu.wait()
    assert lib().h3b_selftest_expire_wait(gpu.ctx) == 0
    with pytest.raises(GpuError, match="timed out"):
        gpu.wait()
    assert gpu.wait() == 0.0  # the status word was cleared
    rng = np.random.default_rng(2)
    a = rng.integers(-127, 128, size=(128, 256), dtype=np.int8)
    w = rng.integers(-127, 128, size=(64, 256), dtype=np.int8)
    out = gpu.empty((128, 64), "i32")
    ops.gemm(gpu, gpu.upload(a), ops.QWeight("q8", gpu.upload(w), gpu.upload(np.ones(64, np.float32)), 64, 256), out, 128,
             sa=gpu.upload(np.ones(128, np.float32)), tile=(128, 64, 4))
    gpu.wait()
    assert np.array_equal(out.numpy(), gemm_ref.int32_product(a, w))


def test_launch_overlap_changes_no_result(gpu):
    """With programmatic dependent launch every kernel still waits for its predecessor before it touches global
    memory: a chain rotate+quantise -> product -> swiglu rotate+quantise -> product gives the same bits either way."""
    import numpy as np
    import oracle
    from h3metal_b200 import ops
    rng = np.random.default_rng(21)
    M, D, F = 640, 1024, 1536
    x = gpu.upload(oracle.bf16_round_bits((rng.standard_normal((M, D)) * 2).astype(np.float32)), "bf16")
    w1 = ops.QWeight("q8", gpu.upload(rng.integers(-127, 128, size=(2 * F, D), dtype=np.int8)),
                     gpu.upload(rng.uniform(1e-3, 2e-3, size=2 * F).astype(np.float32)), 2 * F, D)
    w2 = ops.QWeight("q8", gpu.upload(rng.integers(-127, 128, size=(D, F), dtype=np.int8)),
                     gpu.upload(rng.uniform(1e-3, 2e-3, size=D).astype(np.float32)), D, F)
    results = []
    for on in (False, True, True):
        gpu.set_launch_overlap(on)
        try:
            a1, s1, h = gpu.empty((M, D), "i8"), gpu.empty((M,), "f32"), gpu.empty((M, 2 * F), "bf16")
            a2, s2, y = gpu.empty((M, F), "i8"), gpu.empty((M,), "f32"), gpu.empty((M, D), "bf16")
            for _ in range(3):  # back to back, so that kernels do follow kernels in the stream
                ops.rot_q8(gpu, x, a1, s1, M, D, block=128)
                ops.gemm(gpu, a1, w1, h, M, sa=s1)
                ops.rot_q8(gpu, h, a2, s2, M, F, swiglu=True, block=128)
                ops.gemm(gpu, a2, w2, y, M, sa=s2)
            gpu.wait()
            results.append((a2.numpy().copy(), y.numpy().copy()))
        finally:
            gpu.set_launch_overlap(True)  # the library's default
    for codes, out in results[1:]:
        assert np.array_equal(codes, results[0][0]) and np.array_equal(out, results[0][1])
