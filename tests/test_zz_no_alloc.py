"""The allocation-free LoRA product, h3b_gemm_w8a8_lora_noalloc, called through the C ABI.

Some hosts of this library cannot allocate device memory while they run it: an inference server whose own allocator
reserved all of HBM at start-up, or a serving loop with a latency bound in which a cudaMalloc would stall the device.
They cannot give the LoRA path the T buffer it normally asks the caller for, so this entry point keeps T in a static
device array inside the library (8 MiB). The test checks that it returns exactly what the ordinary entry point
returns with a caller-provided T, on two different calls in a row (the array keeps the first call's contents, which
must not leak into the second), and that sizes beyond the array are refused.

This file sorts last on purpose: if it fails, a run that stops at the first failure has already run everything else.
"""
import ctypes

import numpy as np
import pytest

from h3metal_b200 import ops
from h3metal_b200.gpu import H3B_BF16, H3B_F32, lib

pytestmark = pytest.mark.gpu


def _case(gpu, seed, M, N, K, rank, out_dtype):
    rng = np.random.default_rng(seed)
    m_pad = ops.pad_rows(M)
    a = gpu.upload(rng.integers(-127, 128, size=(m_pad, K), dtype=np.int8))
    sa = gpu.upload(rng.uniform(0.001, 0.01, size=m_pad).astype(np.float32))
    w = gpu.upload(rng.integers(-127, 128, size=(N, K), dtype=np.int8))
    sw = gpu.upload((rng.uniform(0.001, 0.01, size=N) / 10).astype(np.float32))
    bias = gpu.upload((rng.standard_normal(N) * 0.01).astype(np.float32))
    A_l = (rng.standard_normal((rank, K)) / np.sqrt(K)).astype(np.float32)
    B_l = (rng.standard_normal((N, rank)) * 0.5).astype(np.float32)
    B_l[N // 2:, : rank // 2] = 0  # the second half of the columns touches only the upper ranks
    low = ops.low_rank(gpu, A_l, B_l, ops.Scratch(gpu))

    # the ordinary entry point: T in a buffer the caller (here ops.Scratch) allocated
    want = gpu.empty((m_pad, N), out_dtype)
    ops.gemm(gpu, a, ops.QWeight("q8", w, sw, N, K, bias=bias, low=low), want, M, sa=sa, tile=(128, 32, 4))
    gpu.wait()

    # the allocation-free entry point, straight through the C ABI
    got = gpu.empty((m_pad, N), out_dtype)
    table = low.table(gpu, gpu.gemm_tile_n(N, True))
    rc = lib().h3b_gemm_w8a8_lora_noalloc(
        gpu.ctx, a.ptr, K, w.ptr, K, sw.ptr, sa.ptr, bias.ptr, got.ptr, {"bf16": H3B_BF16, "f32": H3B_F32}[out_dtype],
        N, m_pad, N, K, low.a.w.ptr, K, low.a.sw.ptr, low.b.ptr, low.R, low.R, table.ptr + 8)
    assert rc == 0, lib().h3b_last_error().decode()
    gpu.wait()
    return got.numpy(), want.numpy()


def test_noalloc_product_equals_the_ordinary_one_twice_in_a_row(gpu):
    got, want = _case(gpu, 1, 384, 768, 512, 56, "bf16")
    assert want.any() and np.array_equal(got, want)
    # a second, differently shaped call reuses the same static array; stale T values must not show
    got, want = _case(gpu, 2, 200, 512, 1024, 32, "f32")
    assert want.any() and np.array_equal(got, want)


def test_noalloc_product_refuses_sizes_beyond_its_static_scratch(gpu):
    small = gpu.empty((128, 128), "i8")
    f32 = gpu.empty((128,), "f32")
    out = gpu.empty((128, 128), "bf16")
    half = gpu.empty((128, 128), "f16")
    # 40000 rows x 128 ranks = 5.12 M fp16 values > 4 Mi: refused before anything is launched or read
    rc = lib().h3b_gemm_w8a8_lora_noalloc(gpu.ctx, small.ptr, 128, small.ptr, 128, f32.ptr, f32.ptr, None, out.ptr,
                                          H3B_BF16, 128, 40000, 128, 128, small.ptr, 128, f32.ptr, half.ptr, 128, 128,
                                          None)
    assert rc != 0 and b"static scratch" in lib().h3b_last_error()
    gpu.wait()
