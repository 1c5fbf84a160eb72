"""Guard regions: every output buffer is allocated larger than what a kernel may write and pre-filled with a pattern;
afterwards everything outside the written region must still hold the pattern. Covers the product on single CTAs, on CTA
pairs with stores from registers and with TMA-stored staged tiles (ragged M and N, wide output strides, a low-rank term),
every variant of the rotate+quantise kernel, and the row-parallel push's stores into the owners' staging slots."""
import numpy as np
import pytest

import oracle
from oracle import gemm_ref
from h3metal_b200 import ops

pytestmark = pytest.mark.gpu

CANARY = 0x5A


def _canary(gpu, shape, dtype):
    """A tensor whose every byte is CANARY."""
    t = gpu.empty(shape, dtype)
    t.torch().view(__import__("torch").uint8).fill_(CANARY)
    return t


def _bytes(t):
    return t.torch().view(__import__("torch").uint8).cpu().numpy().reshape(t.shape[0], -1)


@pytest.mark.parametrize("variant,pair,store", [("single", -1, 0), ("pair", 1, -1), ("pair-staged", 1, 1)])
@pytest.mark.parametrize("M,N,K,stride", [(300, 416, 512, 512), (1000, 1152, 640, 1280), (130, 96, 192, 128)])
@pytest.mark.parametrize("out_dtype", ["bf16", "f32"])
def test_product_writes_only_its_rows_and_columns(gpu, variant, pair, store, M, N, K, stride, out_dtype):
    rng = np.random.default_rng(M + N)
    m_pad = ops.pad_rows(M)
    a = rng.integers(-127, 128, size=(m_pad, K), dtype=np.int8)
    w = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    sa = rng.uniform(0.001, 0.01, size=m_pad).astype(np.float32)
    sw = rng.uniform(0.001, 0.01, size=N).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.01).astype(np.float32)
    wt = ops.QWeight("q8", gpu.upload(w), gpu.upload(sw), N, K, bias=gpu.upload(bias))
    out = _canary(gpu, (m_pad + 128, stride), out_dtype)  # 128 guard rows below, stride - N guard columns to the right
    gpu.set_policy(pair=pair)
    gpu.set_store_mode(store)
    try:
        ops.gemm(gpu, gpu.upload(a), wt, out, M, sa=gpu.upload(sa), c_stride=stride, tile=(128, 32, 4))
        gpu.wait()
    finally:
        gpu.set_policy()
        gpu.set_store_mode(0)
    esize = 2 if out_dtype == "bf16" else 4
    raw = _bytes(out)
    assert (raw[m_pad:] == CANARY).all(), "rows below the padded row count were written"
    assert (raw[:, N * esize:] == CANARY).all(), "columns right of N were written"
    stored, _, _ = gemm_ref.gemm_q8(a, w, sa, sw, bias, None, out_dtype)
    assert np.array_equal(out.numpy()[:m_pad, :N], stored)


@pytest.mark.parametrize("pair,store", [(-1, 0), (1, -1), (1, 1)])
def test_product_with_a_low_rank_term_keeps_to_its_region(gpu, pair, store):
    rng = np.random.default_rng(8)
    M, N, K, stride = 700, 768, 512, 1024
    m_pad = ops.pad_rows(M)
    a = rng.integers(-127, 128, size=(m_pad, K), dtype=np.int8)
    w = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    sa = rng.uniform(0.001, 0.01, size=m_pad).astype(np.float32)
    sw = (rng.uniform(0.001, 0.01, size=N) / 10).astype(np.float32)
    A_l = (rng.standard_normal((32, K)) / np.sqrt(K)).astype(np.float32)
    B_l = (rng.standard_normal((N, 32)) * 0.5).astype(np.float32)
    wt = ops.QWeight("q8", gpu.upload(w), gpu.upload(sw), N, K, low=ops.low_rank(gpu, A_l, B_l, ops.Scratch(gpu)))
    out = _canary(gpu, (m_pad + 128, stride), "bf16")
    gpu.set_policy(pair=pair)
    gpu.set_store_mode(store)
    try:
        ops.gemm(gpu, gpu.upload(a), wt, out, M, sa=gpu.upload(sa), c_stride=stride, tile=(128, 32, 4))
        gpu.wait()
    finally:
        gpu.set_policy()
        gpu.set_store_mode(0)
    raw = _bytes(out)
    assert (raw[m_pad:] == CANARY).all() and (raw[:, N * 2:] == CANARY).all()
    stored, _, _ = gemm_ref.gemm_q8(a, w, sa, sw, None, gemm_ref.low_rank_ref(A_l, B_l), "bf16")
    got, want = oracle.bf16_bits_to_f32(out.numpy()[:m_pad, :N]), oracle.bf16_bits_to_f32(stored)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-3


@pytest.mark.parametrize("variant,stages,chunk", [("tma", 0, 0), ("tma_c32", 0, 32), ("tma_c64", 0, 64), ("tma4", 4, 0),
                                                  ("regs", -1, 0)])
@pytest.mark.parametrize("M,D,block,swiglu", [(37, 3072, 128, False), (129, 1280, 256, False), (21, 2048, 64, True),
                                              (300, 6144, 128, False)])
def test_rotate_quantise_writes_only_its_rows(gpu, variant, stages, chunk, M, D, block, swiglu):
    rng = np.random.default_rng(D + M)
    xh = oracle.bf16_round_bits((rng.standard_normal((M, 2 * D if swiglu else D)) * 2).astype(np.float32))
    out = _canary(gpu, (M + 8, D), "i8")   # 8 guard rows
    sa = _canary(gpu, (M + 8,), "f32")
    gpu.set_policy(rot_stages=stages, rot_chunk=chunk)
    try:
        ops.rot_q8(gpu, gpu.upload(xh, "bf16"), out, sa, M, D, swiglu=swiglu, block=block)
        gpu.wait()
    finally:
        gpu.set_policy()
    assert (_bytes(out)[M:] == CANARY).all(), "code rows beyond M were written"
    assert (sa.torch().view(__import__("torch").uint8).cpu().numpy()[4 * M:] == CANARY).all(), "scales beyond M were written"
    q, s = oracle.rot_q8_rows(xh, D, block=block, dtype="bf16", swiglu=swiglu)
    diff = np.abs(out.numpy()[:M].astype(np.int32) - q.astype(np.int32))
    assert diff.max() <= (1 if swiglu else 0)


@pytest.mark.parametrize("stage", ["i32", "bf16"])
def test_push_stores_stay_inside_the_owners_slots(gpu, stage):
    """Two ranks played on one GPU: each owner's staging block holds [guard][slot of rank 0][slot of rank 1][guard];
    the pushed tiles of both ranks fill exactly the two slots (N = 416 columns: a last, partial 256-column tile)."""
    rng = np.random.default_rng(3)
    world, M, N, K = 2, 512, 416, 512
    rows, esize = M // world, 4 if stage == "i32" else 2
    slot = rows * N * esize
    guard = 4096
    blocks = [_canary(gpu, (guard + world * slot + guard,), "u8") for _ in range(world)]
    a = rng.integers(-127, 128, size=(M, K), dtype=np.int8)
    w = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    sa = gpu.upload(rng.uniform(0.01, 0.03, size=M).astype(np.float32))
    sw = gpu.upload(rng.uniform(1e-3, 2e-3, size=N).astype(np.float32))
    kp = K // world
    for r in range(world):
        slots = [blocks[o].ptr + guard + r * slot for o in range(world)]
        gpu.gemm_push_native(gpu.upload(np.ascontiguousarray(a[:, r * kp:(r + 1) * kp])), kp,
                             gpu.upload(np.ascontiguousarray(w[:, r * kp:(r + 1) * kp])), kp, sw, sa, slots, rows, stage, N, M, N, kp)
    gpu.wait()
    for o in range(world):
        raw = blocks[o].numpy()
        assert (raw[:guard] == CANARY).all() and (raw[guard + world * slot:] == CANARY).all(), f"owner {o}: guard bytes written"
        if stage == "i32":
            for r in range(world):
                part = raw[guard + r * slot:guard + (r + 1) * slot].view(np.int32).reshape(rows, N)
                want = gemm_ref.int32_product(a[o * rows:(o + 1) * rows, r * kp:(r + 1) * kp], w[:, r * kp:(r + 1) * kp])
                assert np.array_equal(part, want), f"owner {o}, slot {r}"
