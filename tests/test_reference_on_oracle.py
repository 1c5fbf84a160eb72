"""The reference's own kernel tests, unmodified, driven through the oracle's CPU stand-in for its Gpu object.

Needs the reference source tree (H3METAL_REF; default: a `reference` directory next to this repository); skipped
where it is absent. The
reference's h3metal/ops.py then supplies padding, strides, the LoRA sequence and the parameter blocks, its
tests/test_gemm.py and tests/test_ops.py supply data, expectations and tolerances, and only the arithmetic of the
two kernels comes from the oracle."""
import os
import sys

import pytest

REF = os.environ.get("H3METAL_REF", os.path.abspath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..",
                                                                 "reference")))
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "h3metal")), reason="reference tree not present")


@pytest.fixture(scope="module")
def ref_tests():
    sys.dont_write_bytecode = True
    sys.path.insert(0, REF)
    sys.path.insert(0, os.path.join(REF, "tests"))
    try:
        import test_gemm
        import test_ops
        from oracle.ref_gpu import OracleGpu
        test_gemm.Gpu = OracleGpu
        yield test_gemm, test_ops, OracleGpu
    finally:
        sys.path.remove(REF)
        sys.path.remove(os.path.join(REF, "tests"))


def test_reference_gemm_checks_pass_on_the_oracle(ref_tests):
    test_gemm, _, _ = ref_tests
    test_gemm.check("q8")
    test_gemm.check("q8", out_dtype="bf16")
    test_gemm.check("q8", N=1024, tile=(32, 512, 8))
    test_gemm.check_partial_tiles_refused()


def test_reference_low_rank_checks_pass_on_the_oracle(ref_tests):
    test_gemm, _, _ = ref_tests
    test_gemm.check_low_rank("q8")
    test_gemm.check_low_rank("q8", out_dtype="bf16", tile=(64, 256, 8))
    test_gemm.check_low_rank("q8", out_dtype="f32", tile=(32, 256, 4), swz=4)


def test_reference_rot_checks_pass_on_the_oracle(ref_tests):
    _, test_ops, OracleGpu = ref_tests
    g = OracleGpu()
    test_ops.test_rot(g)
    test_ops.test_rot(g, D=7168, swiglu=False)
