"""norm_mod_q8 on the GPU (ops.norm_mod_q8 -> ctypes -> h3b_norm_mod_q8) against the CPU oracle and the reference
test's expectations (tests/test_ops.py:28-53: shapes D = 5376, 5120, 3072 with LayerNorm).

The row statistics are fp32 sums whose order differs between implementations, so the normalising factor can differ
in its last place: int8 codes are held to "at most 1 LSB on at most 1e-4 of the elements", float outputs to 2e-6,
and the row scales to the largest distance measured over these cases, in units in the last place: 3 for RMSNorm,
8 for LayerNorm, where removing a mean of 50 from values of spread 3 magnifies the order of the mean's summation
(16 over 3000 rows of 3840 channels)."""
import numpy as np
import pytest

import oracle
from h3metal_b200 import ops
from tests.conftest import rel_fro

pytestmark = pytest.mark.gpu


def ulp_distance(a, b):
    """Distance between positive fp32 values in units in the last place (difference of their bit patterns)."""
    return np.abs(a.astype(np.float32).view(np.int32).astype(np.int64) - b.astype(np.float32).view(np.int32).astype(np.int64))


def _case(rng, M, D, ln, types=3):
    x = (rng.standard_normal((M, D)) * 3 + (50 if ln else 0)).astype(np.float32)  # LN: a large mean to remove
    mod = rng.standard_normal((types, 2, D)).astype(np.float32)
    rt = rng.integers(0, types, size=M).astype(np.uint8)
    return x, mod, rt


@pytest.mark.parametrize("M,D,ln,block", [(37, 5376, False, 256), (37, 5120, False, 256), (37, 3072, True, 256),
                                          (129, 3840, False, 128), (64, 6144, False, 128), (5, 16384, False, 64),
                                          (3, 32768, False, 256), (1, 256, True, 128), (700, 1024, True, 64)])
@pytest.mark.parametrize("variant", ["tma", "tma_c64", "regs"])
def test_codes_scales_and_float_outputs(gpu, request, variant, M, D, ln, block):
    """variant "tma": rows staged in shared memory by TMA (D <= 8192); "regs": the register-fed kernel."""
    rng = np.random.default_rng(1)
    x, mod, rt = _case(rng, M, D, ln)
    X, MOD, RT = gpu.upload(x), gpu.upload(mod), gpu.upload(rt)
    gpu.set_policy(rot_stages=-1 if variant == "regs" else 0, rot_chunk=64 if variant == "tma_c64" else 0)
    request.addfinalizer(gpu.set_policy)
    out, sa = gpu.empty((M, D), "i8"), gpu.empty((M,), "f32")
    ops.norm_mod_q8(gpu, X, MOD, RT, out, sa, M, D, eps=1e-5, ln=ln, block=block)
    of = gpu.empty((M, D), "f32")
    ops.norm_mod_q8(gpu, X, MOD, RT, of, None, M, D, eps=1e-5, out_f=True, ln=ln, block=block)
    oh = gpu.empty((M, D), "f16")
    ops.norm_mod_q8(gpu, X, MOD, RT, oh, None, M, D, eps=1e-5, out_h=True, ln=ln, block=block)
    ohr = gpu.empty((M, D), "f16")
    ops.norm_mod_q8(gpu, X, MOD, RT, ohr, None, M, D, eps=1e-5, out_hr=True, ln=ln, block=block)
    gpu.wait()
    q, s = oracle.norm_mod_rows(x, mod, rt, D, eps=1e-5, block=block, ln=ln)
    diff = np.abs(out.numpy().astype(np.int32) - q.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() <= 1e-4
    assert ulp_distance(sa.numpy(), s).max() <= (8 if ln else 3)
    f = oracle.norm_mod_rows(x, mod, rt, D, eps=1e-5, block=block, ln=ln, out="f")
    assert np.allclose(of.numpy(), f, rtol=2e-6, atol=2e-6 * np.abs(f).max())
    assert rel_fro(oh.numpy(), f) < 5e-4
    hr = oracle.norm_mod_rows(x, mod, rt, D, eps=1e-5, block=block, ln=ln, out="hr")
    assert rel_fro(ohr.numpy(), hr) < 5e-4
    # the reference test's own bounds against float64
    xc = x.astype(np.float64) - (x.astype(np.float64).mean(1, keepdims=True) if ln else 0)
    y = xc / np.sqrt((xc ** 2).mean(1, keepdims=True) + 1e-5) * mod[rt, 0] + mod[rt, 1]
    assert np.abs(of.numpy() - y).max() < 1e-3 * np.abs(y).max()
    r = oracle.rotate_rows_matmul(y.astype(np.float32), block)
    got = out.numpy().astype(np.float64) * sa.numpy()[:, None]
    assert np.abs(got - r).max() / np.abs(r).max() < 0.6 / 127
    assert np.abs(ohr.numpy().astype(np.float64) - r).max() / np.abs(r).max() < 2e-3


def test_reference_golden_expectations(gpu, golden):
    for tag, ln in (("rms", False), ("ln", True)):
        x, mod, rt = golden[f"norm_{tag}_x"], golden[f"norm_{tag}_mod"], golden[f"norm_{tag}_rt"]
        out, sa, of = gpu.empty((6, 768), "i8"), gpu.empty((6,), "f32"), gpu.empty((6, 768), "f32")
        X, MOD, RT = gpu.upload(x), gpu.upload(mod), gpu.upload(rt)
        ops.norm_mod_q8(gpu, X, MOD, RT, out, sa, 6, 768, eps=1e-5, ln=ln)
        ops.norm_mod_q8(gpu, X, MOD, RT, of, None, 6, 768, eps=1e-5, ln=ln, out_f=True)
        gpu.wait()
        y, r = golden[f"norm_{tag}_expect_y_f64"], golden[f"norm_{tag}_expect_rot_f64"]
        assert np.abs(of.numpy() - y).max() < 1e-3 * np.abs(y).max()
        assert np.abs(out.numpy().astype(np.float64) * sa.numpy()[:, None] - r).max() / np.abs(r).max() < 0.6 / 127


@pytest.mark.parametrize("M,D", [(33, 3840), (9, 6144)])
def test_fused_residual_update(gpu, M, D):
    """POST: x += post * rmsnorm(y) is written back and the row is then normalised, modulated, rotated, quantised
    (kernels/ops.metal:161-198); wider row stride than D for x."""
    rng = np.random.default_rng(4)
    x, mod, rt = _case(rng, M, D, False)
    xs = np.zeros((M, D + 64), np.float32)
    xs[:, :D] = x
    y = (rng.standard_normal((M, D)) * 2).astype(np.float32)
    post = rng.standard_normal(D).astype(np.float32)
    X, Y, P = gpu.upload(xs), gpu.upload(y), gpu.upload(post)
    out, sa = gpu.empty((M, D), "i8"), gpu.empty((M,), "f32")
    ops.norm_mod_q8(gpu, X, gpu.upload(mod), gpu.upload(rt), out, sa, M, D, eps=1e-6, y=Y, post=P, x_stride=D + 64,
                    block=128)
    gpu.wait()
    q, s, upd = oracle.norm_mod_rows(x, mod, rt, D, eps=1e-6, block=128, y=y, post=post)
    got_x = X.numpy()
    assert np.allclose(got_x[:, :D], upd, rtol=2e-6, atol=2e-6 * np.abs(upd).max()) and not got_x[:, D:].any()
    diff = np.abs(out.numpy().astype(np.int32) - q.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() <= 1e-4
    assert ulp_distance(sa.numpy(), s).max() <= 4


def test_feeds_the_product_like_rot_q8_does(gpu):
    """norm_mod_q8 -> gemm is the other way int8 activations reach the product (h3metal/dit.py:197-200)."""
    from oracle import gemm_ref
    rng = np.random.default_rng(8)
    M, D, N = 256, 1024, 512
    x, mod, rt = _case(rng, M, D, False)
    w = rng.integers(-127, 128, size=(N, D), dtype=np.int8)
    sw = rng.uniform(1e-3, 2e-3, size=N).astype(np.float32)
    a8, sa, out = gpu.empty((M, D), "i8"), gpu.empty((M,), "f32"), gpu.empty((M, N), "bf16")
    ops.norm_mod_q8(gpu, gpu.upload(x), gpu.upload(mod), gpu.upload(rt), a8, sa, M, D, eps=1e-5, block=128)
    ops.gemm(gpu, a8, ops.QWeight("q8", gpu.upload(w), gpu.upload(sw), N, D), out, M, sa=sa, tile=(128, 128, 4))
    gpu.wait()
    stored, _, _ = gemm_ref.gemm_q8(a8.numpy(), w, sa.numpy(), sw, None, None, "bf16")
    assert np.array_equal(out.numpy(), stored)


def test_refusals(gpu):
    from h3metal_b200.gpu import GpuError
    x, mod, rt = gpu.empty((4, 512), "f32"), gpu.empty((1, 2, 512), "f32"), gpu.empty((4,), "u8")
    out, sa = gpu.empty((4, 512), "i8"), gpu.empty((4,), "f32")
    with pytest.raises(ValueError):
        ops.norm_mod_q8(gpu, x, mod, rt, out, sa, 4, 500, eps=1e-5, block=128)
    with pytest.raises(ValueError):
        ops.norm_mod_q8(gpu, x, mod, rt, out, sa, 4, 512, eps=1e-5, y=x)
    with pytest.raises(GpuError):
        ops.norm_mod_q8(gpu, x, mod, rt, out, sa, 4, 512, eps=1e-5, ln=True, y=x, post=mod)
    with pytest.raises(GpuError):
        ops.norm_mod_q8(gpu, x, mod, rt, out, None, 4, 512, eps=1e-5)
    gpu.wait()
