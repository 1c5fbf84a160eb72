"""The int8 product on the GPU (ops.gemm -> ctypes -> h3b_gemm_w8a8) against the CPU oracle.

Acceptance: int32 accumulators bit-exact for identical int8 inputs; stored outputs equal to the oracle's fp32
epilogue rounded to the output type (compared like with like), which implies the 1e-3 relative Frobenius bound
on dequantised values; the reference's own bounds (tests/test_gemm.py:85-87) as secondary checks."""
import numpy as np
import pytest

import oracle
from oracle import gemm_ref
from h3metal_b200 import ops
from tests.conftest import rel_fro

pytestmark = pytest.mark.gpu


def _case(rng, M, N, K, full_range=True):
    m_pad = ops.pad_rows(M)
    lo, hi = (-127, 128) if full_range else (-8, 9)
    a = rng.integers(lo, hi, size=(m_pad, K), dtype=np.int8)
    w = rng.integers(lo, hi, size=(N, K), dtype=np.int8)
    sa = rng.uniform(0.001, 0.01, size=m_pad).astype(np.float32)
    sw = rng.uniform(0.001, 0.01, size=N).astype(np.float32)
    return m_pad, a, w, sa, sw


# the product on single CTAs (128-row tiles), on CTA pairs (256 x 256 tiles) with stores from registers, or on pairs
# whose epilogue stages 16-bit outputs in shared memory for TMA stores
PAIR = {"single": -1, "pair": 1, "pair-staged": 1}
STORE = {"single": 0, "pair": -1, "pair-staged": 1}


def _gemm(gpu, a, w, sa, sw, M, out_dtype, bias=None, tile=(64, 32, 2), variant=None, **kw):
    N, K = w.shape
    wt = ops.QWeight("q8", gpu.upload(w), gpu.upload(sw), N, K, bias=gpu.upload(bias) if bias is not None else None)
    out = gpu.empty((a.shape[0], N), out_dtype)
    if variant is not None:
        gpu.set_policy(pair=PAIR[variant])
        gpu.set_store_mode(STORE[variant])
    try:
        ops.gemm(gpu, gpu.upload(a), wt, out, M, sa=gpu.upload(sa), tile=tile, **kw)
        gpu.wait()
    finally:
        if variant is not None:
            gpu.set_policy()
            gpu.set_store_mode(0)
    return out.numpy()


@pytest.mark.parametrize("M,N,K", [(1, 32, 64), (128, 32, 128), (128, 64, 256), (128, 256, 512), (127, 128, 128),
                                   (129, 256, 640), (200, 256, 512), (256, 512, 1024), (384, 768, 3072),
                                   (1000, 1152, 640), (130, 96, 192), (64, 3872, 256), (300, 160, 16384),
                                   (2304, 2560, 1152), (2100, 1056, 384)])
@pytest.mark.parametrize("variant", ["single", "pair"])
def test_accumulators_bit_exact(gpu, variant, M, N, K):
    rng = np.random.default_rng(M + 7 * N + 13 * K)
    m_pad, a, w, sa, sw = _case(rng, M, N, K)
    rows = (M + 63) // 64 * 64  # the rows a (64, ., .) tile writes
    got = _gemm(gpu, a, w, sa, sw, M, "i32", variant=variant)
    assert np.array_equal(got[:rows], gemm_ref.int32_product(a[:rows], w))
    assert not got[rows:].any()  # rows beyond the padded count are not touched


def test_accumulators_at_int32_extremes(gpu):
    """|acc| reaches K * 127^2 = 2.6e8 at K = 16384, beyond 2^24: exact in int32, and rounded once in the epilogue."""
    K = 16384
    a = np.full((128, K), 127, np.int8)
    a[1::2] = -127
    w = np.full((32, K), 127, np.int8)
    w[::3] = -127
    ones_m, ones_n = np.ones(128, np.float32), np.ones(32, np.float32)
    for variant in ("single", "pair"):
        acc = _gemm(gpu, a, w, ones_m, ones_n, 128, "i32", variant=variant)
        assert np.array_equal(acc, gemm_ref.int32_product(a, w)) and abs(int(acc[0, 1])) == K * 127 * 127
        v = _gemm(gpu, a, w, ones_m, ones_n, 128, "f32", variant=variant)
        assert np.array_equal(v, gemm_ref.epilogue_q8(gemm_ref.int32_product(a, w), ones_m, ones_n))


@pytest.mark.parametrize("tile_n", [32, 64, 128, 256])
def test_every_tile_width_is_exact(gpu, tile_n):
    rng = np.random.default_rng(tile_n)
    m_pad, a, w, sa, sw = _case(rng, 384, 512, 1024)
    gpu.set_policy(tile_n, 0)
    try:
        got = _gemm(gpu, a, w, sa, sw, 384, "i32")
    finally:
        gpu.set_policy()
    assert np.array_equal(got, gemm_ref.int32_product(a, w))


@pytest.mark.parametrize("pair", [-1, 1])
@pytest.mark.parametrize("band", [1, 2, 5])
def test_tile_order_does_not_change_results(gpu, band, pair):
    rng = np.random.default_rng(band)
    m_pad, a, w, sa, sw = _case(rng, 1280, 1536, 512)
    gpu.set_policy(0, band, pair=pair)
    try:
        got = _gemm(gpu, a, w, sa, sw, 1280, "i32")
    finally:
        gpu.set_policy()
    assert np.array_equal(got, gemm_ref.int32_product(a, w))


@pytest.mark.parametrize("M,N,K", [(200, 256, 512), (1000, 1152, 640), (2304, 2560, 1152), (130, 96, 192)])
@pytest.mark.parametrize("out_dtype", ["f16", "bf16"])
def test_staged_stores_write_the_same_bits(gpu, out_dtype, M, N, K):
    """CTA pairs with the epilogue staged through shared memory and stored by TMA: ragged M, N not a multiple of the
    256-column tile or of a 64-column panel, several tiles per CTA pair (the staging is reused). Rows beyond the
    written count stay untouched."""
    rng = np.random.default_rng(M + N + K)
    m_pad, a, w, sa, sw = _case(rng, M, N, K)
    bias = (rng.standard_normal(N) * 0.01).astype(np.float32)
    rows = (M + 63) // 64 * 64
    got = _gemm(gpu, a, w, sa, sw, M, out_dtype, bias=bias, variant="pair-staged")
    stored, _, _ = gemm_ref.gemm_q8(a[:rows], w, sa[:rows], sw, bias, None, out_dtype)
    assert np.array_equal(got[:rows], stored)
    assert not got[rows:].any()


@pytest.mark.parametrize("variant", ["single", "pair", "pair-staged"])
@pytest.mark.parametrize("out_dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("with_bias", [False, True])
def test_epilogue_matches_oracle_bit_for_bit(gpu, out_dtype, with_bias, variant):
    rng = np.random.default_rng(17)
    M, N, K = 200, 256, 512
    m_pad, a, w, sa, sw = _case(rng, M, N, K)
    bias = (rng.standard_normal(N) * 0.01).astype(np.float32) if with_bias else None
    got = _gemm(gpu, a, w, sa, sw, M, out_dtype, bias=bias, tile=(64, 128, 4), variant=variant)
    stored, v, _ = gemm_ref.gemm_q8(a, w, sa, sw, bias, None, out_dtype)
    assert np.array_equal(got, stored)
    # acceptance bound on dequantised outputs, like with like
    as_f = oracle.bf16_bits_to_f32(got) if out_dtype == "bf16" else got.astype(np.float32)
    want = oracle.bf16_bits_to_f32(stored) if out_dtype == "bf16" else stored.astype(np.float32)
    assert rel_fro(as_f[:M], want[:M]) <= 1e-3
    # the reference's own check (tests/test_gemm.py:31,85-87)
    ref = (a[:M].astype(np.float64) @ w.T.astype(np.float64)) * sa[:M, None] * sw[None, :] + (0 if bias is None else bias)
    assert np.abs(as_f[:M] - ref).max() / np.abs(ref).max() < (1e-2 if out_dtype == "bf16" else 2e-3)


def test_strided_operands_and_k_slices_add_up(gpu):
    """Views of wider buffers (a_stride, QWeight.ws, c_stride) and linearity over K: the accumulators of two
    K halves, each read in place from the whole operands, sum to the whole product (the arithmetic behind the
    reference's K split, h3metal/ops.py:143-154)."""
    rng = np.random.default_rng(23)
    M, N, K = 256, 384, 1024
    m_pad, a, w, sa, sw = _case(rng, M, N, K)
    A, W = gpu.upload(a), gpu.upload(w)
    SW, SA = gpu.upload(sw), gpu.upload(sa)
    whole = gemm_ref.int32_product(a, w)
    parts = []
    for i in range(2):
        half = ops.QWeight("q8", W.view((N, K // 2), offset_elems=i * K // 2), SW, N, K // 2, ws=K)
        out = gpu.empty((M, 512), "i32")  # wider than N: c_stride
        ops.gemm(gpu, A.view((M, K // 2), offset_elems=i * K // 2), half, out, M, sa=SA, a_stride=K, c_stride=512)
        gpu.wait()
        got = out.numpy()
        assert not got[:, N:].any()
        parts.append(got[:, :N])
        assert np.array_equal(parts[-1], gemm_ref.int32_product(a[:, i * K // 2:(i + 1) * K // 2], w[:, i * K // 2:(i + 1) * K // 2]))
    assert np.array_equal(parts[0] + parts[1], whole)


@pytest.mark.parametrize("name,K,N", [("zimage qkv", 3840, 11520), ("zimage out", 3840, 3840), ("zimage w2", 10240, 3840),
                                      ("flux2 qkv", 3072, 9216), ("flux2 fc1", 3072, 18432), ("flux2 fc2", 9216, 3072)])
def test_model_shapes_on_sampled_rows(gpu, name, K, N):
    """Real shapes and row counts of the models (the reference's check_dit_tiles, tests/test_gemm.py:105-158):
    every output column of a sample of rows against float64, tolerance 2e-3, plus bit-exact accumulators."""
    rng = np.random.default_rng(1)
    M = 4608
    m_pad, a, w, sa, sw = _case(rng, M, N, K)
    rows = np.unique(np.r_[0:40, M - 40:M, rng.integers(0, M, 64)])
    wt = ops.QWeight("q8", gpu.upload(w), gpu.upload(sw), N, K)
    A, SA = gpu.upload(a), gpu.upload(sa)
    out = gpu.empty((m_pad, N), "f16")
    ops.gemm(gpu, A, wt, out, M, sa=SA, tile=(64, 128, 4))
    raw = gpu.empty((m_pad, N), "i32")
    ops.gemm(gpu, A, wt, raw, M, sa=SA, tile=(64, 128, 4))
    gpu.wait()
    acc = gemm_ref.int32_product(a[rows], w)
    assert np.array_equal(raw.numpy()[rows], acc)
    ref = acc.astype(np.float64) * sa[rows, None] * sw[None, :]
    got = out.numpy()[rows].astype(np.float64)
    assert np.abs(got - ref).max() / np.abs(ref).max() < 2e-3
    assert np.array_equal(out.numpy()[rows], gemm_ref.epilogue_q8(acc, sa[rows], sw).astype(np.float16))


def test_refusals_reach_the_caller(gpu):
    from h3metal_b200.gpu import GpuError
    rng = np.random.default_rng(0)
    m_pad, a, w, sa, sw = _case(rng, 64, 256, 256)
    with pytest.raises(ValueError):
        _gemm(gpu, a, w, sa, sw, 64, "f16", tile=(32, 512, 8))
    A = gpu.upload(a)
    wt = ops.QWeight("q8", gpu.upload(w), gpu.upload(sw), 256, 256)
    with pytest.raises(GpuError):  # K-contiguous rows must start on 16-byte boundaries
        ops.gemm(gpu, A.view((64, 240), offset_elems=8), ops.QWeight("q8", wt.w, wt.sw, 256, 240, ws=256),
                 gpu.empty((128, 256), "f16"), 64, sa=gpu.upload(sa), a_stride=256)
    gpu.wait()
