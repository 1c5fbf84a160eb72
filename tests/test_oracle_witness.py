"""The NumPy restatement of the rotate+quantise kernel against its independent C witness (lane-by-lane butterflies,
oracle/rotq8_witness.c), and against the matmul form of the rotation."""
import numpy as np
import pytest

import oracle
from oracle import build as oracle_build, rotq8_ref


def _inputs(seed, M, D, swiglu):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((M, 2 * D if swiglu else D)) * 2).astype(np.float32)
    x[:, rng.choice(D, size=4, replace=False)] *= 20.0
    bits = oracle.bf16_round_bits(x)
    return bits, oracle.bf16_bits_to_f32(bits)


@pytest.mark.parametrize("block", [64, 128, 256])
@pytest.mark.parametrize("swiglu", [False, True])
def test_numpy_restatement_equals_c_witness(block, swiglu):
    bits, xf = _inputs(block + swiglu, 11, 1536, swiglu)
    q, s = rotq8_ref.rot_q8_rows(bits, 1536, block=block, dtype="bf16", swiglu=swiglu)
    cq, cs, crot = oracle_build.witness_rot_q8(xf, 1536, block, swiglu)
    if not swiglu:
        assert np.array_equal(q, cq) and np.array_equal(s, cs)
    else:
        # numpy's exp and libm's expf may differ in the last place, which can move a code by one step
        assert (q != cq).mean() <= 1e-4 and np.abs(q.astype(int) - cq.astype(int)).max() <= 1
        assert np.allclose(s, cs, rtol=3e-7)


def test_all_zero_row_gets_unit_scale():
    bits = np.zeros((2, 256), np.uint16)
    q, s = rotq8_ref.rot_q8_rows(bits, 256, block=256)
    assert not q.any() and s.tolist() == [1.0, 1.0]
    cq, cs, _ = oracle_build.witness_rot_q8(np.zeros((2, 256), np.float32), 256, 256, False)
    assert not cq.any() and cs.tolist() == [1.0, 1.0]


@pytest.mark.parametrize("block", [64, 128, 256])
def test_kernel_order_rotation_close_to_matmul_rotation(block):
    """Kernel-order butterflies and the fp32 matmul of quant.rotate_in agree to rounding; codes differ on far fewer
    than 1e-4 of the elements and by one step at most (the budget the path's acceptance allows)."""
    bits, xf = _inputs(5, 64, 3072, False)
    q, s = rotq8_ref.rot_q8_rows(bits, 3072, block=block)
    rot = oracle.rotate_in(xf, None, block)
    amax = np.abs(rot).max(1)
    scale = (amax / np.float32(127)).astype(np.float32)
    q2 = np.rint(rot * (np.float32(1) / scale)[:, None]).astype(np.int8)
    assert (q != q2).mean() <= 1e-4
    assert np.abs(q.astype(int) - q2.astype(int)).max() <= 1
    assert np.allclose(s, scale, rtol=2e-6)  # a few fp32 ulps: BLAS sums in another order and folds 1/sqrt(B) into H


def test_rotation_preserves_products():
    """x W^T = rot(x) rot(W)^T (the reference's tests/test_convert.py:19-26), for every block size."""
    rng = np.random.default_rng(0)
    w = rng.standard_normal((64, 512)).astype(np.float32)
    x = rng.standard_normal((8, 512)).astype(np.float32)
    for block in (64, 128, 256):
        s = oracle.random_signs(512, 3)
        assert np.allclose(oracle.rotate_in(x, s, block) @ oracle.rotate_in(w, s, block).T, x @ w.T, atol=1e-3)
