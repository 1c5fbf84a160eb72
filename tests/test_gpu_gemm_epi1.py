"""The gated-residual epilogue (the reference's EPI 1) on the GPU against the oracle: the reference's checks
check("q8", epi=1, ksplit=...) and check_low_rank("q8", epi=1, ...) of tests/test_gemm.py:74-83,237-246,264-273."""
import numpy as np
import pytest

from oracle import gemm_ref
from h3metal_b200 import ops

pytestmark = pytest.mark.gpu


def _setup(gpu, rng, M, N, K, bias=True):
    m_pad = ops.pad_rows(M)
    a = rng.integers(-127, 128, size=(m_pad, K), dtype=np.int8)
    sa = rng.uniform(0.001, 0.01, size=m_pad).astype(np.float32)
    q = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    sw = rng.uniform(0.001, 0.01, size=N).astype(np.float32)
    b = (rng.standard_normal(N) * 0.01).astype(np.float32) if bias else None
    x0 = rng.standard_normal((m_pad, N)).astype(np.float32)
    types = rng.integers(0, 3, size=m_pad).astype(np.uint8)
    gates = rng.standard_normal((3, N)).astype(np.float32)
    return m_pad, a, sa, q, sw, b, x0, types, gates


@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("M,N,K,ksplit", [(200, 256, 512, 1), (200, 256, 1024, 2), (200, 256, 2048, 4),
                                          (300, 1024, 2048, 4), (129, 384, 768, 1)])
def test_gated_residual_matches_oracle_bit_for_bit(gpu, variant, M, N, K, ksplit):
    rng = np.random.default_rng(K + ksplit)
    m_pad, a, sa, q, sw, b, x0, types, gates = _setup(gpu, rng, M, N, K)
    wt = ops.QWeight("q8", gpu.upload(q), gpu.upload(sw), N, K, bias=gpu.upload(b))
    X = gpu.upload(x0)
    gpu.set_policy(pair=variant)
    try:
        ops.gemm(gpu, gpu.upload(a), wt, X, M, sa=gpu.upload(sa), epi=1, rtype=gpu.upload(types), gate=gpu.upload(gates),
                 tile=(64, 128, 4), ksplit=ksplit)
        gpu.wait()
    finally:
        gpu.set_policy()
    rows = (M + 63) // 64 * 64
    want = x0.copy()
    kp = K // ksplit
    for i in range(ksplit):  # the same sequence of accumulating passes
        acc = gemm_ref.int32_product(a[:rows, i * kp:(i + 1) * kp], q[:, i * kp:(i + 1) * kp])
        v = gemm_ref.epilogue_q8(acc, sa[:rows], sw, b if i == 0 else None)
        want[:rows] = gemm_ref.accumulate_gated(want[:rows], v, gates, types[:rows])
    got = X.numpy()
    assert np.array_equal(got, want)
    # the reference's expectation and bound (tests/test_gemm.py:31,82-87)
    ref = x0[:M].astype(np.float64) + gates[types[:M]] * ((a[:M].astype(np.float64) @ q.T.astype(np.float64)) * sa[:M, None] * sw[None, :] + b)
    assert np.abs(got[:M] - ref).max() / np.abs(ref).max() < 2e-3


@pytest.mark.parametrize("K,ksplit", [(512, 1), (1024, 2)])
def test_gated_residual_with_low_rank_term(gpu, K, ksplit):
    rng = np.random.default_rng(3)
    M, N = 200, 768
    m_pad, a, sa, q, sw, b, x0, types, gates = _setup(gpu, rng, M, N, K, bias=False)
    A_l = (rng.standard_normal((40, K)) / np.sqrt(K)).astype(np.float32)
    B_l = (rng.standard_normal((N, 40)) * 0.5).astype(np.float32)
    lo = ops.low_rank(gpu, A_l, B_l, ops.Scratch(gpu))
    wt = ops.QWeight("q8", gpu.upload(q), gpu.upload(sw / 10), N, K, low=lo)
    X = gpu.upload(x0)
    ops.gemm(gpu, gpu.upload(a), wt, X, M, sa=gpu.upload(sa), epi=1, rtype=gpu.upload(types), gate=gpu.upload(gates),
             ksplit=ksplit)
    gpu.wait()
    term = gemm_ref.low_rank_ref(A_l, B_l)
    low = gemm_ref.lora_low(gemm_ref.lora_T(a, sa, term), term)   # T over the whole K, joins the first slice
    want = x0.copy()
    kp = K // ksplit
    for i in range(ksplit):
        acc = gemm_ref.int32_product(a[:, i * kp:(i + 1) * kp], q[:, i * kp:(i + 1) * kp])
        v = gemm_ref.epilogue_q8(acc, sa, sw / 10, None, low if i == 0 else None)
        want = gemm_ref.accumulate_gated(want, v, gates, types)
    got = X.numpy()
    assert np.linalg.norm(got[:M].astype(np.float64) - want[:M]) / np.linalg.norm(want[:M]) <= 1e-3
    assert np.abs(got[:M] - want[:M]).max() / np.abs(want[:M]).max() < 2e-3
