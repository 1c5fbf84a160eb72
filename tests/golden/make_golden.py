"""Generates tests/golden/ref_golden.npz and ref_dispatch.json from the reference's own Python code.

Run once where the reference source tree is available (path in H3METAL_REF; default: a `reference` directory next
to this repository):

    python tests/golden/make_golden.py

Everything stored here is an OUTPUT OF THE REFERENCE on small seeded inputs: its NumPy quantisation functions
(h3metal/quant.py), its bf16 helpers (h3metal/weights.py), its low-rank preparation and rank-range table
(h3metal/ops.py), the dispatches its ops.gemm / ops.rot_q8 record (geometry, macros, parameter blocks), and the
expected values its kernel tests compute (tests/test_ops.py: rot(); tests/test_gemm.py: the float64 product).
The CPU tests compare the oracle with these files, so they run where the reference tree is absent.
"""

import json
import os
import struct
import sys

import numpy as np

sys.dont_write_bytecode = True
HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("H3METAL_REF", os.path.abspath(os.path.join(HERE, "..", "..", "..", "reference")))
sys.path.insert(0, REF)
sys.path.insert(0, os.path.join(REF, "tests"))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from h3metal import ops as ref_ops, quant as ref_quant  # noqa: E402
from h3metal.weights import bf16_bits, bf16_to_f32  # noqa: E402
import test_ops as ref_test_ops  # noqa: E402  (the reference's tests/test_ops.py: rot(), bf16(), from_bf16())

from oracle.ref_gpu import OracleGpu  # noqa: E402  (array holder + dispatch recorder for the reference's ops.py)


def main():
    out = {}
    rng = np.random.default_rng(11)

    # -- h3metal/quant.py ---------------------------------------------------------------------------------------
    for n in (64, 128, 256):
        out[f"hadamard_{n}"] = ref_quant.hadamard(n)
    out["signs_512_seed3"] = ref_quant.random_signs(512, 3)
    w = (rng.standard_normal((24, 512)) * 0.02).astype(np.float32)
    out["rot_w_in"] = w
    out["rot_w_plain"] = ref_quant.rotate_in(w)
    out["rot_w_signed"] = ref_quant.rotate_in(w, out["signs_512_seed3"])
    codes, scales = ref_quant.quant_q8(out["rot_w_plain"])
    out["q8_codes"], out["q8_scales"] = codes, scales
    codes, scales = ref_quant.quant_q8(out["rot_w_plain"], search=False)
    out["q8_codes_nosearch"], out["q8_scales_nosearch"] = codes, scales
    out["q8_dequant"] = ref_quant.dequant("q8", out["q8_codes"], out["q8_scales"], 24, 512)

    # -- h3metal/weights.py -------------------------------------------------------------------------------------
    vals = np.concatenate([rng.standard_normal(200).astype(np.float32) * 3,
                           np.array([1.0, -2.5, 3.14159265, 1e-3, 65504.0, 0.0, 1.00390625, 1.01171875], np.float32)])
    out["bf16_in"] = vals
    out["bf16_bits"] = bf16_bits(vals)
    out["bf16_back"] = bf16_to_f32(out["bf16_bits"])

    # -- h3metal/ops.py: low_rank() and LowRank.table() ---------------------------------------------------------
    gpu = OracleGpu()
    r, K, N = 24, 512, 512
    A_l = (rng.standard_normal((r, K)) / np.sqrt(K)).astype(np.float32)
    B_l = np.zeros((N, r), np.float32)
    B_l[:128, :8] = rng.standard_normal((128, 8)) * 0.5      # ranks 0..7 touch the first tile only
    B_l[128:384, 8:20] = rng.standard_normal((256, 12)) * 0.5  # ranks 8..19 the middle
    B_l[:384, 20:24] = rng.standard_normal((384, 4)) * 0.5     # ranks 20..23 all but the last 128 columns
    lo = ref_ops.low_rank(gpu, A_l, B_l, ref_ops.Scratch(gpu))
    out["lr_A"], out["lr_B"] = A_l, B_l
    out["lr_codes"], out["lr_scales"] = lo.a.w.numpy().copy(), lo.a.sw.numpy().copy()
    out["lr_b"] = lo.b.numpy().copy()
    out["lr_lo"], out["lr_hi"] = lo.lo, lo.hi
    for tn in (128, 256):
        out[f"lr_table_{tn}"] = lo.table(gpu, tn).numpy().copy()

    # -- the dispatches ops.gemm / ops.rot_q8 record, and what the oracle kernels make of them -------------------
    M = 200
    m_pad = ref_ops.pad_rows(M)
    a = rng.integers(-127, 128, size=(m_pad, K), dtype=np.int8)
    sa = rng.uniform(0.001, 0.01, size=m_pad).astype(np.float32)
    q = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    sw = (rng.uniform(0.001, 0.01, size=N) / 10).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.01).astype(np.float32)
    wt = ref_ops.QWeight("q8", gpu.upload(q), gpu.upload(sw), N, K, bias=gpu.upload(bias), low=lo)
    dst = gpu.empty((m_pad, N), "bf16")
    gpu.launches.clear()
    ref_ops.gemm(gpu, gpu.upload(a), wt, dst, M, sa=gpu.upload(sa), tile=(64, 128, 4))
    x = ref_test_ops.bf16((rng.standard_normal((19, 2 * 512)) * 2).astype(np.float32))
    ref_ops.rot_q8(gpu, gpu.upload(x, "bf16"), gpu.empty((19, 512), "i8"), gpu.empty((19,), "f32"), 19, 512,
                   swiglu=True)
    ref_ops.rot_q8(gpu, gpu.upload(x, "bf16"), gpu.empty((19, 1024), "i8"), gpu.empty((19,), "f32"), 19, 1024)
    dispatch = [{"file": f, "fn": fn, "macros": {k: str(v) for k, v in mac.items()}, "grid": list(grid),
                 "threads": list(thr), "params": list(struct.unpack(f"<{len(p) // 4}i", p))}
                for f, fn, mac, grid, thr, p in gpu.launches]
    with open(os.path.join(HERE, "ref_dispatch.json"), "w") as fh:
        json.dump(dispatch, fh, indent=1)
    out["gemm_a"], out["gemm_sa"], out["gemm_q"], out["gemm_sw"], out["gemm_bias"] = a, sa, q, sw, bias
    # expected values exactly as tests/test_gemm.py:31 and :215-220 write them (float64)
    main_ref = (a.astype(np.float64) @ q.T.astype(np.float64)) * sa[:, None] * sw[None, :]
    T = (a.astype(np.float64) @ out["lr_codes"].astype(np.float64).T) * sa[:, None] * out["lr_scales"][None, :]
    stored = T.astype(np.float16).astype(np.float64) @ out["lr_b"].astype(np.float64).T
    out["gemm_expect_main_f64"] = main_ref[:48]   # a sample of rows keeps the file small
    out["gemm_expect_stored_f64"] = stored[:48]

    # -- tests/test_ops.py: rot() of seeded bf16 rows, plain and value*silu(gate), in float64 --------------------
    xin = (np.random.default_rng(2).standard_normal((5, 2 * 768)) * 2).astype(np.float32)
    xb = ref_test_ops.bf16(xin)
    xf = ref_test_ops.from_bf16(xb).astype(np.float64)
    g = xf[:, 768:]
    out["rot_x_bits"] = xb
    out["rot_expect_plain_f64"] = ref_test_ops.rot(xf[:, :768])
    out["rot_expect_swiglu_f64"] = ref_test_ops.rot(xf[:, :768] * g / (1 + np.exp(-g)))

    # -- tests/test_ops.py:28-53 (test_norm_mod): the float64 expectation the reference's test builds, RMS and LN ---------
    for tag, ln in (("rms", False), ("ln", True)):
        r2 = np.random.default_rng(1)
        xn_in = (r2.standard_normal((6, 768)) * 3 + (50 if ln else 0)).astype(np.float32)
        nmod = r2.standard_normal((3, 2, 768)).astype(np.float32)
        nrt = r2.integers(0, 3, size=6).astype(np.uint8)
        xc = xn_in.astype(np.float64) - (xn_in.astype(np.float64).mean(1, keepdims=True) if ln else 0)
        xn = xc / np.sqrt((xc ** 2).mean(1, keepdims=True) + 1e-5)
        yy = xn * nmod[nrt, 0] + nmod[nrt, 1]
        out[f"norm_{tag}_x"], out[f"norm_{tag}_mod"], out[f"norm_{tag}_rt"] = xn_in, nmod, nrt
        out[f"norm_{tag}_expect_y_f64"] = yy
        out[f"norm_{tag}_expect_rot_f64"] = ref_test_ops.rot(yy)

    # -- h3metal/weights.py: a small .h3m file written by the reference's Writer (stored gzipped: 8 MiB of it are the
    #    reserved, zero-filled header region) ------------------------------------------------------------------------
    import gzip
    import tempfile
    from h3metal.weights import Writer
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "t.h3m")
        wr = Writer(path, {"kind": "test", "hidden": 512})
        wr.tensor("a", np.arange(1000, dtype=np.float32), "f32")
        wr.tensor("cpu_only", np.arange(7, dtype=np.int32), "i32", host_only=True)
        wr.linear("lin", "q8", 24, 512, out["q8_codes"], out["q8_scales"], bias=np.linspace(-1, 1, 24).astype(np.float32))
        wr.close()
        with open(path, "rb") as src, gzip.open(os.path.join(HERE, "ref_file.h3m.gz"), "wb", compresslevel=9) as dst:
            dst.write(src.read())

    # -- h3metal/lora.py:291-310: A scaled and rotated with the layer's signs, ranks stacked side by side -----------------
    from h3metal import lora as ref_lora
    r3 = np.random.default_rng(21)
    A1, B1 = r3.standard_normal((4, 512)).astype(np.float32), r3.standard_normal((96, 4)).astype(np.float32)
    A2, B2 = r3.standard_normal((8, 512)).astype(np.float32), r3.standard_normal((96, 8)).astype(np.float32)
    sgn = out["signs_512_seed3"]
    t1 = ref_lora.Term(ref_quant.rotate_in((A1 * np.float32(0.8 * 2.0)).astype(np.float32), sgn), B1)
    t2 = ref_lora.Term(ref_quant.rotate_in((A2 * np.float32(1.0 * 0.5)).astype(np.float32), sgn), B2)
    sa_, sb_ = ref_lora.stack([t1, t2])
    out["lora_A1"], out["lora_B1"], out["lora_A2"], out["lora_B2"] = A1, B1, A2, B2
    out["lora_stack_A"], out["lora_stack_B"] = sa_, sb_

    np.savez_compressed(os.path.join(HERE, "ref_golden.npz"), **out)
    print("wrote", len(out), "arrays,", os.path.getsize(os.path.join(HERE, "ref_golden.npz")), "bytes;",
          len(dispatch), "dispatches")


if __name__ == "__main__":
    main()
