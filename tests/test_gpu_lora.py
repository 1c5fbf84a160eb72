"""The low-rank (LoRA) term of the product on the GPU against the oracle: the reference's check_low_rank
(tests/test_gemm.py:161-251) with its block-structured rank-56 adapter, plus dense adapters of the configs' ranks."""
import numpy as np
import pytest

import oracle
from oracle import gemm_ref
from h3metal_b200 import ops
from tests.conftest import rel_fro

pytestmark = pytest.mark.gpu


def _block_adapter(rng, N, K):
    """rank-16 block per third of the columns, a rank-8 block over all of them, nothing on the last 128 columns"""
    third = (N - 128) // 3
    A_l = rng.standard_normal((56, K)).astype(np.float32) / np.sqrt(K)
    B_l = np.zeros((N, 56), np.float32)
    for i in range(3):
        B_l[i * third:(i + 1) * third, 16 * i:16 * (i + 1)] = rng.standard_normal((third, 16)) * 0.5
    B_l[:N - 128, 48:56] = rng.standard_normal((N - 128, 8)) * 0.5
    return A_l, B_l


def _run(gpu, rng, M, N, K, A_l, B_l, out_dtype, tile_n=0, bias=True, pair=0, store=0):
    m_pad = ops.pad_rows(M)
    a = rng.integers(-127, 128, size=(m_pad, K), dtype=np.int8)
    sa = rng.uniform(0.001, 0.01, size=m_pad).astype(np.float32)
    q = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    sw = (rng.uniform(0.001, 0.01, size=N) / 10).astype(np.float32)
    b = (rng.standard_normal(N) * 0.01).astype(np.float32) if bias else None
    gpu.set_policy(tile_n, 0, pair=pair)
    gpu.set_store_mode(store)
    try:
        scratch = ops.Scratch(gpu)
        lo = ops.low_rank(gpu, A_l, B_l, scratch)
        wt = ops.QWeight("q8", gpu.upload(q), gpu.upload(sw), N, K, bias=gpu.upload(b) if bias else None, low=lo)
        out = gpu.empty((m_pad, N), out_dtype)
        ops.gemm(gpu, gpu.upload(a), wt, out, M, sa=gpu.upload(sa))
        gpu.wait()
    finally:
        gpu.set_policy()
        gpu.set_store_mode(0)
    term = gemm_ref.low_rank_ref(A_l, B_l)
    T = scratch.t.view((m_pad, lo.R)).numpy()
    stored, v, acc = gemm_ref.gemm_q8(a, q, sa, sw, b, term, out_dtype)
    got = out.numpy()
    got_f = oracle.bf16_bits_to_f32(got) if out_dtype == "bf16" else got.astype(np.float32)
    return dict(a=a, sa=sa, q=q, sw=sw, bias=b, term=term, T=T, got=got, got_f=got_f, stored=stored, v=v, acc=acc, M=M)


@pytest.mark.parametrize("out_dtype,tile_n", [("f16", 0), ("bf16", 256), ("f32", 128), ("f32", 256)])
def test_reference_low_rank_check(gpu, out_dtype, tile_n):
    rng = np.random.default_rng(3)
    M, N, K = 200, 768, 512
    A_l, B_l = _block_adapter(rng, N, K)
    r = _run(gpu, rng, M, N, K, A_l, B_l, out_dtype, tile_n, bias=False)
    # T is the same int8 product with an fp16 store: bit-exact against the oracle
    assert np.array_equal(r["T"], gemm_ref.lora_T(r["a"], r["sa"], r["term"]))
    # acceptance: 1e-3 relative Frobenius against the oracle's value, like with like
    want = oracle.bf16_bits_to_f32(r["stored"]) if out_dtype == "bf16" else r["stored"].astype(np.float32)
    assert rel_fro(r["got_f"][:M], want[:M]) <= 1e-3
    # the reference's own expectations and bounds: stored term tight, exact term loose, term/main > 0.3
    x = r["a"].astype(np.float64) * r["sa"][:, None].astype(np.float64)
    main = x @ (r["q"].astype(np.float64) * r["sw"][:, None]).T
    exact = x @ A_l.T.astype(np.float64) @ B_l.T.astype(np.float64)
    Tf = (r["a"].astype(np.float64) @ r["term"].a_codes.astype(np.float64).T) * r["sa"][:, None] * r["term"].a_scales[None, :]
    stored_term = Tf.astype(np.float16).astype(np.float64) @ r["term"].b.astype(np.float64).T
    ref_t, ref_e = (main + stored_term)[:M], (main + exact)[:M]
    got = r["got_f"][:M].astype(np.float64)
    assert np.abs(exact[:M]).max() / np.abs(main[:M]).max() > 0.3
    assert np.abs(got - ref_t).max() / np.abs(ref_t).max() < (2e-3 if out_dtype != "bf16" else 1e-2)
    assert np.abs(got - ref_e).max() / np.abs(ref_e).max() < 1e-2
    # columns no rank touches equal the plain product exactly
    plain = gemm_ref.store_as(gemm_ref.epilogue_q8(r["acc"], r["sa"], r["sw"]), out_dtype)
    assert np.array_equal(r["got"][:M, N - 128:], plain[:M, N - 128:])


@pytest.mark.parametrize("rank,N,K,tile_n", [(32, 1024, 1024, 0), (64, 1024, 1024, 0), (64, 1024, 1024, 128),
                                             (96, 512, 768, 0), (128, 768, 512, 128), (20, 384, 512, 0)])
def test_dense_adapters(gpu, rank, N, K, tile_n):
    rng = np.random.default_rng(rank + N)
    A_l = (rng.standard_normal((rank, K)) / np.sqrt(K)).astype(np.float32)
    B_l = (rng.standard_normal((N, rank)) * 0.5).astype(np.float32)
    r = _run(gpu, rng, 300, N, K, A_l, B_l, "f32", tile_n)
    assert np.array_equal(r["T"], gemm_ref.lora_T(r["a"], r["sa"], r["term"]))
    assert rel_fro(r["got_f"][:300], r["v"][:300]) <= 1e-3
    assert rel_fro(r["got_f"][:300], r["v"][:300]) <= 1e-5  # fp32 accumulation of fp16 products: far inside the bound


@pytest.mark.parametrize("out_dtype,store", [("f32", 0), ("bf16", -1), ("bf16", 1), ("f16", 1)])
@pytest.mark.parametrize("rank", [32, 64, 96, 128])
def test_low_rank_on_cta_pairs(gpu, out_dtype, store, rank):
    """The term inside the CTA-pair product (256 x 256 tiles, one accumulator pair), with stores from registers and
    with the epilogue staged through shared memory; several tiles per pair, ragged M, against the oracle and against
    the single-CTA kernel."""
    M, N, K = 1100, 1280, 768
    A_l = (np.random.default_rng(rank).standard_normal((rank, K)) / np.sqrt(K)).astype(np.float32)
    B_l = (np.random.default_rng(rank + 1).standard_normal((N, rank)) * 0.5).astype(np.float32)
    r = _run(gpu, np.random.default_rng(4), M, N, K, A_l, B_l, out_dtype, pair=1, store=store)
    want = oracle.bf16_bits_to_f32(r["stored"]) if out_dtype == "bf16" else r["stored"].astype(np.float32)
    assert rel_fro(r["got_f"][:M], want[:M]) <= (1e-5 if out_dtype == "f32" else 1e-3)
    single = _run(gpu, np.random.default_rng(4), M, N, K, A_l, B_l, out_dtype, pair=-1)
    assert rel_fro(r["got_f"][:M], single["got_f"][:M]) <= 1e-5
    assert not r["got"][ops.pad_rows(M):].any()


@pytest.mark.parametrize("rank,store", [(32, -1), (96, -1), (96, 1)])
def test_low_rank_over_several_tiles_per_pair(gpu, rank, store):
    """9 x 20 = 180 tiles of 256 x 256 on at most 74 CTA pairs: every pair finishes two or three tiles, so both
    accumulators are handed back and taken again (the int32 one before any arithmetic, the low-rank one on its own
    barrier) with the next tile's main loop already running. Ragged M; rank 96 = one full and one half operand stage."""
    M, N, K = 2300, 5120, 768
    A_l = (np.random.default_rng(rank).standard_normal((rank, K)) / np.sqrt(K)).astype(np.float32)
    B_l = (np.random.default_rng(rank + 1).standard_normal((N, rank)) * 0.5).astype(np.float32)
    r = _run(gpu, np.random.default_rng(5), M, N, K, A_l, B_l, "bf16", pair=1, store=store)
    want = oracle.bf16_bits_to_f32(r["stored"])
    assert rel_fro(r["got_f"][:M], want[:M]) <= 1e-3
    single = _run(gpu, np.random.default_rng(5), M, N, K, A_l, B_l, "bf16", pair=-1)
    assert np.array_equal(r["got"][:M], single["got"][:M]) or rel_fro(r["got_f"][:M], single["got_f"][:M]) <= 1e-5
    assert not r["got"][ops.pad_rows(M):].any()


@pytest.mark.parametrize("store", [-1, 1])
def test_rank_ranges_on_cta_pairs(gpu, store):
    """The reference's block-structured adapter on 256-column pair tiles: tiles use only their own rank range, and the
    columns no rank touches equal the plain product exactly."""
    rng = np.random.default_rng(3)
    M, N, K = 520, 1280, 512
    A_l, B_l = _block_adapter(rng, N, K)
    r = _run(gpu, rng, M, N, K, A_l, B_l, "bf16", bias=False, pair=1, store=store)
    assert np.array_equal(r["T"], gemm_ref.lora_T(r["a"], r["sa"], r["term"]))
    want = oracle.bf16_bits_to_f32(r["stored"])
    assert rel_fro(r["got_f"][:M], want[:M]) <= 1e-3
    plain = gemm_ref.store_as(gemm_ref.epilogue_q8(r["acc"], r["sa"], r["sw"]), "bf16")
    assert np.array_equal(r["got"][:M, N - 128:], plain[:M, N - 128:])


def test_term_is_not_silently_dropped(gpu):
    rng = np.random.default_rng(9)
    A_l = (rng.standard_normal((32, 512)) / np.sqrt(512)).astype(np.float32)
    B_l = (rng.standard_normal((256, 32)) * 0.5).astype(np.float32)
    r = _run(gpu, rng, 128, 256, 512, A_l, B_l, "f32")
    main_only = gemm_ref.epilogue_q8(r["acc"], r["sa"], r["sw"], r["bias"])
    assert rel_fro(r["got_f"], main_only) > 0.1


@pytest.mark.parametrize("K,expect_split", [(8192, 4), (4096, 2), (768, 1)])
def test_k_split_of_the_input_side_product_changes_no_bit(gpu, K, expect_split):
    """T's product split along K (one launch over the activations seen as [M * S][K / S], partial sums added exactly
    by the reduction kernel) against the unsplit product and the oracle."""
    rng = np.random.default_rng(K)
    M, N, rank = 640, 512, 64
    A_l = (rng.standard_normal((rank, K)) / np.sqrt(K)).astype(np.float32)
    B_l = (rng.standard_normal((N, rank)) * 0.5).astype(np.float32)
    lo = ops.low_rank(gpu, A_l, B_l, ops.Scratch(gpu))
    assert ops._t_split(gpu, lo, M, K, None) == expect_split
    results = []
    for split in (4, 0):
        gpu.lora_t_split = split
        try:
            r = _run(gpu, np.random.default_rng(5), M, N, K, A_l, B_l, "bf16")
        finally:
            gpu.lora_t_split = 4
        assert np.array_equal(r["T"], gemm_ref.lora_T(r["a"], r["sa"], r["term"]))
        results.append(r)
    assert np.array_equal(results[0]["T"], results[1]["T"]) and np.array_equal(results[0]["got"], results[1]["got"])
