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

import oracle
from oracle import gemm_ref
from h3metal_b200 import ops
from h3metal_b200.gpu import H3B_BF16, H3B_F32, lib
from tests.conftest import rel_fro

pytestmark = pytest.mark.gpu


def _case(gpu, seed, M, N, K, rank, out_dtype, whole_tiles=True):
    """Returns (rows of the allocation-free product, the ordinary product's, the CPU oracle's fp32 values). With
    whole_tiles the call is given the padded row count, as the ordinary path is; without, the ragged M itself, so
    that the last row tile's T stores are masked and its loads zero-filled."""
    rng = np.random.default_rng(seed)
    m_pad = ops.pad_rows(M)
    a_h = rng.integers(-127, 128, size=(m_pad, K), dtype=np.int8)
    sa_h = rng.uniform(0.001, 0.01, size=m_pad).astype(np.float32)
    w_h = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    sw_h = (rng.uniform(0.001, 0.01, size=N) / 10).astype(np.float32)
    bias_h = (rng.standard_normal(N) * 0.01).astype(np.float32)
    a, sa, w, sw, bias = gpu.upload(a_h), gpu.upload(sa_h), gpu.upload(w_h), gpu.upload(sw_h), gpu.upload(bias_h)
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
        N, m_pad if whole_tiles else M, N, K, low.a.w.ptr, K, low.a.sw.ptr, low.b.ptr, low.R, low.R, table.ptr + 8)
    assert rc == 0, lib().h3b_last_error().decode()
    gpu.wait()
    stored, _, _ = gemm_ref.gemm_q8(a_h[:M], w_h, sa_h[:M], sw_h, bias_h, gemm_ref.low_rank_ref(A_l, B_l), out_dtype)
    return got.numpy()[:M], want.numpy()[:M], _as_f32(stored, out_dtype)


def _as_f32(x, dtype):
    return oracle.bf16_bits_to_f32(x) if dtype == "bf16" else x


def test_noalloc_product_equals_the_ordinary_one_twice_in_a_row(gpu):
    got, want, ref = _case(gpu, 1, 384, 768, 512, 56, "bf16")
    assert want.any() and np.array_equal(got, want)
    assert rel_fro(_as_f32(got, "bf16"), ref) <= 1e-3  # against the CPU oracle's values stored in the same type
    # a second, differently shaped call reuses the same static array; stale T values must not show
    got, want, ref = _case(gpu, 2, 200, 512, 1024, 32, "f32")
    assert want.any() and np.array_equal(got, want)
    assert rel_fro(got, ref) <= 1e-3  # the acceptance bound against the CPU oracle, fp32 output


def test_noalloc_product_with_a_ragged_last_row_tile(gpu):
    """M itself (not the padded row count) goes to the call: the last tile's T rows beyond M are neither stored nor
    read as anything but zero, and the rows below M equal the ordinary product's and the oracle's."""
    got, want, ref = _case(gpu, 3, 200, 512, 1024, 32, "f32", whole_tiles=False)
    assert want.any() and np.array_equal(got, want)
    assert rel_fro(got, ref) <= 1e-3


def test_noalloc_product_leaves_device_memory_as_it_found_it(gpu):
    """The property the entry point exists for: once the kernels are loaded (first call), a call changes neither the
    free device memory nor what torch's allocator holds."""
    import torch
    rng = np.random.default_rng(9)
    M, N, K, rank = 256, 512, 512, 32
    a = gpu.upload(rng.integers(-127, 128, size=(M, K), dtype=np.int8))
    sa = gpu.upload(rng.uniform(0.001, 0.01, size=M).astype(np.float32))
    w = gpu.upload(rng.integers(-127, 128, size=(N, K), dtype=np.int8))
    sw = gpu.upload(rng.uniform(1e-4, 1e-3, size=N).astype(np.float32))
    low = ops.low_rank(gpu, (rng.standard_normal((rank, K)) / np.sqrt(K)).astype(np.float32),
                       (rng.standard_normal((N, rank)) * 0.5).astype(np.float32), ops.Scratch(gpu))
    out = gpu.empty((M, N), "bf16")
    table = low.table(gpu, gpu.gemm_tile_n(N, True))

    def call():
        rc = lib().h3b_gemm_w8a8_lora_noalloc(gpu.ctx, a.ptr, K, w.ptr, K, sw.ptr, sa.ptr, None, out.ptr, H3B_BF16, N, M, N,
                                              K, low.a.w.ptr, K, low.a.sw.ptr, low.b.ptr, low.R, low.R, table.ptr + 8)
        assert rc == 0, lib().h3b_last_error().decode()
        gpu.wait()

    call()  # warm-up: loads the two kernels if nothing before did
    torch.cuda.synchronize()
    free0, held0 = torch.cuda.mem_get_info(gpu.torch_device)[0], torch.cuda.memory_allocated(gpu.torch_device)
    call()
    torch.cuda.synchronize()
    free1, held1 = torch.cuda.mem_get_info(gpu.torch_device)[0], torch.cuda.memory_allocated(gpu.torch_device)
    assert (free1, held1) == (free0, held0)


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


def test_noalloc_product_accepts_exactly_its_limit_and_refuses_the_next_step(gpu):
    """M x R = 32768 x 128 = 4 Mi fp16 values is the whole array and runs; one row tile more is refused before launch."""
    rng = np.random.default_rng(11)
    K, N, R = 128, 128, 128
    w = gpu.upload(rng.integers(-127, 128, size=(N, K), dtype=np.int8))
    sw = gpu.upload(rng.uniform(1e-4, 1e-3, size=N).astype(np.float32))
    la = gpu.upload(rng.integers(-127, 128, size=(R, K), dtype=np.int8))
    lsw = gpu.upload(rng.uniform(1e-4, 1e-3, size=R).astype(np.float32))
    lb = gpu.upload((rng.standard_normal((N, R)) * 0.1).astype(np.float16), "f16")
    for M, accepted in ((32768, True), (32896, False)):
        a = gpu.upload(rng.integers(-127, 128, size=(M, K), dtype=np.int8))
        sa = gpu.upload(rng.uniform(0.001, 0.01, size=M).astype(np.float32))
        out = gpu.empty((M, N), "bf16")
        launches = gpu.launch_count
        rc = lib().h3b_gemm_w8a8_lora_noalloc(gpu.ctx, a.ptr, K, w.ptr, K, sw.ptr, sa.ptr, None, out.ptr, H3B_BF16, N, M, N, K,
                                              la.ptr, K, lsw.ptr, lb.ptr, R, R, None)
        if accepted:
            assert rc == 0, lib().h3b_last_error().decode()
            gpu.wait()
            assert gpu.launch_count == launches + 2 and out.numpy().any()
        else:
            assert rc != 0 and b"static scratch" in lib().h3b_last_error()
            assert gpu.launch_count == launches  # nothing was launched


def test_noalloc_product_launches_nothing_when_the_main_product_is_refused(gpu):
    """Both products are checked before the first launch: a bad argument of the MAIN product (here an output stride
    smaller than N) must not leave a T product behind in the shared array."""
    small = gpu.empty((128, 128), "i8")
    f32 = gpu.empty((128,), "f32")
    out = gpu.empty((128, 128), "bf16")
    half = gpu.empty((128, 128), "f16")
    launches = gpu.launch_count
    rc = lib().h3b_gemm_w8a8_lora_noalloc(gpu.ctx, small.ptr, 128, small.ptr, 128, f32.ptr, f32.ptr, None, out.ptr, H3B_BF16,
                                          64, 128, 128, 128, small.ptr, 128, f32.ptr, half.ptr, 128, 128, None)
    assert rc != 0 and b"c_stride" in lib().h3b_last_error()
    assert gpu.launch_count == launches
    gpu.wait()
