"""CPU oracle for the W8A8 Hadamard-linear path.

TEST INFRASTRUCTURE ONLY. This package restates, on the CPU, the arithmetic of the
reference (audenvenn/h3metal 0.6.4) for one path: offline weight rotation and int8
quantisation, the run-time rotate+quantise row kernel, the int8 product with its
dequantising epilogue, and the low-rank (LoRA) term. It exists so that the CUDA
path can be checked against it; only the test-suite, the smoke entry and the
benchmark's CPU-baseline leg may import it. Nothing in h3metal_b200/ imports it,
and it is never a fallback for the GPU path.

Pinning: the NumPy-level functions (hadamard, random_signs, rotate_in, quant_q8,
dequant, bf16 rounding, low_rank and its rank-range table, the launch geometry and
parameter blocks of ops.gemm / ops.rot_q8) are checked against outputs of the
reference itself, imported from its source tree when the fixtures under
tests/golden/ were generated (tests/golden/make_golden.py). The two Metal kernels
cannot run off Apple hardware, so their restatements (rot_q8_rows, gemm_q8) follow
the kernel source operation by operation and are pinned by the formulas and bounds
of the reference's own kernel tests (tests/test_ops.py:55-78,
tests/test_gemm.py:20-87,161-251), evaluated by the reference's helper functions at
fixture-generation time, and by a second, independent C restatement of the
butterfly (oracle/rotq8_witness.c).
"""

from .quant_ref import (bf16_round_bits, bf16_bits_to_f32, hadamard, random_signs, rotate_in, quant_q8,
                        dequant_q8)
from .rotq8_ref import rot_q8_rows, rotate_rows_matmul
from .normq8_ref import norm_mod_rows
from .gemm_ref import int32_product, epilogue_q8, gemm_q8, low_rank_ref, lora_table, lora_T, LowRankRef
