"""Host side of the launchers (no GPU): the same padding, strides, LoRA sequence and refusals as the reference's
h3metal/ops.py, checked against the dispatches the reference itself records (tests/golden/ref_dispatch.json)."""
import numpy as np
import pytest

from h3metal_b200 import ops, quant
from tests.fakes import RecordingGpu


def test_quant_module_matches_reference(golden):
    for n in (64, 128, 256):
        assert np.array_equal(quant.hadamard(n), golden[f"hadamard_{n}"])
    assert np.array_equal(quant.random_signs(512, 3), golden["signs_512_seed3"])
    assert np.array_equal(quant.rotate_in(golden["rot_w_in"]), golden["rot_w_plain"])
    assert np.array_equal(quant.rotate_in(golden["rot_w_in"], golden["signs_512_seed3"]), golden["rot_w_signed"])
    c, s = quant.quant_q8(golden["rot_w_plain"])
    assert np.array_equal(c, golden["q8_codes"]) and np.array_equal(s, golden["q8_scales"])
    c, s = quant.quant_q8(golden["rot_w_plain"], search=False)
    assert np.array_equal(c, golden["q8_codes_nosearch"]) and np.array_equal(s, golden["q8_scales_nosearch"])
    assert np.array_equal(quant.dequant("q8", golden["q8_codes"], golden["q8_scales"], 24, 512), golden["q8_dequant"])
    assert np.array_equal(quant.bf16_bits(golden["bf16_in"]), golden["bf16_bits"])
    assert np.array_equal(quant.bf16_to_f32(golden["bf16_bits"]), golden["bf16_back"])
    assert quant.RB == 256


def test_rotate_in_refuses_ragged_k():
    with pytest.raises(ValueError):
        quant.rotate_in(np.zeros((2, 200), np.float32))
    with pytest.raises(ValueError):
        quant.rotate_in(np.zeros((2, 192), np.float32), block=128)
    quant.rotate_in(np.zeros((2, 192), np.float32), block=64)


def test_quantiser_round_trip_error():
    """the reference's tests/test_convert.py:35-42: int8 round trip below 1 % relative error"""
    w = np.random.default_rng(2).standard_normal((256, 1024)).astype(np.float32)
    codes, scales = quant.quantize("q8", w)
    back = quant.dequant("q8", codes, scales, 256, 1024)
    assert np.linalg.norm(back - w) / np.linalg.norm(w) < 0.01
    with pytest.raises(ValueError):
        quant.quantize("q4", w)


def test_low_rank_matches_reference(golden):
    g = RecordingGpu()
    lo = ops.low_rank(g, golden["lr_A"], golden["lr_B"], ops.Scratch(g))
    assert lo.R == 32
    assert np.array_equal(lo.a.w.numpy(), golden["lr_codes"]) and np.array_equal(lo.a.sw.numpy(), golden["lr_scales"])
    assert np.array_equal(lo.b.numpy(), golden["lr_b"])
    assert np.array_equal(lo.lo, golden["lr_lo"]) and np.array_equal(lo.hi, golden["lr_hi"])
    for tn in (128, 256):
        assert np.array_equal(lo.table(g, tn).numpy(), golden[f"lr_table_{tn}"])
    # a partial last tile gets the range of the columns it has
    t = lo.table(g, 384).numpy()
    assert t[:2].tolist() == [32, 32] and len(t) == 2 + 2 * 2
    with pytest.raises(ValueError):
        ops.low_rank(g, golden["lr_A"], golden["lr_B"][:, :5], ops.Scratch(g))


def test_gemm_sequence_matches_reference_dispatches(golden, ref_dispatch):
    """Same call as make_golden.py records from the reference: M=200 rows, N=K=512, bias, rank-24 term, tile
    (64, 128, 4). The reference dispatches the narrow T product over whole 128-row tiles, then the main product."""
    g = RecordingGpu(tile_n=128)
    lo = ops.low_rank(g, golden["lr_A"], golden["lr_B"], ops.Scratch(g))
    N = K = 512
    wt = ops.QWeight("q8", g.upload(golden["gemm_q"]), g.upload(golden["gemm_sw"]), N, K,
                     bias=g.upload(golden["gemm_bias"]), low=lo)
    out = g.empty((256, N), "bf16")
    ops.gemm(g, g.upload(golden["gemm_a"]), wt, out, 200, sa=g.upload(golden["gemm_sa"]), tile=(64, 128, 4))
    t_call, main = g.calls
    ref_t, ref_main = ref_dispatch[0], ref_dispatch[1]
    # GemmParams: M_pad, N, K, a_stride, c_stride, w_stride, groups, g_stride
    assert [t_call[k] for k in ("M", "N", "K", "a_stride", "c_stride", "w_stride")] == ref_t["params"][:6]
    assert t_call["out_dtype"] == "f16" and ref_t["macros"]["OUT_T"] == "half" and t_call["bias"] is None
    assert [main[k] for k in ("M", "N", "K", "a_stride", "c_stride", "w_stride")] == ref_main["params"][:6]
    assert main["out_dtype"] == "bf16" and ref_main["macros"]["OUT_T"] == "bfloat"
    assert main["bias"] is not None and ref_main["macros"]["HAS_BIAS"] == "1" and ref_main["macros"]["LORA"] == "1"
    assert main["R"] == 32 and main["t_stride"] == 32 and main["b_stride"] == 32
    assert main["lt"].ptr == t_call["out"].ptr  # the main product reads the T the first product wrote
    assert main["ranges_ptr"] == lo.table(g, 128).ptr + 8


def test_rot_q8_parameters_match_reference_dispatches(ref_dispatch):
    g = RecordingGpu()
    x = g.empty((19, 1024), "bf16")
    ops.rot_q8(g, x, g.empty((19, 512), "i8"), g.empty((19,), "f32"), 19, 512, swiglu=True)
    ops.rot_q8(g, x, g.empty((19, 1024), "i8"), g.empty((19,), "f32"), 19, 1024)
    for call, ref in zip(g.calls, ref_dispatch[2:4]):
        assert [call["M"], call["D"], call["x_stride"], call["mode"]] == ref["params"]
        assert call["block"] == 256
    with pytest.raises(ValueError):
        ops.rot_q8(g, x, g.empty((19, 1000), "i8"), g.empty((19,), "f32"), 19, 1000)


def test_gemm_refusals():
    """h3metal/ops.py:144-145,158-159 and tests/test_gemm.py:90-102: partial tiles and K splits of a storing
    product are refused with ValueError; formats outside the int8 path are refused too."""
    g = RecordingGpu()
    for N, tn in ((5376, 512), (3840, 512), (1152, 256), (1216, 128)):
        wt = ops.QWeight("q8", g.upload(np.zeros((N, 256), np.int8)), g.upload(np.ones(N, np.float32)), N, 256)
        with pytest.raises(ValueError):
            ops.gemm(g, g.upload(np.zeros((64, 256), np.int8)), wt, g.empty((64, N), "f16"), 64,
                     sa=g.upload(np.ones(64, np.float32)), tile=(32, tn, 8))
    wt = ops.QWeight("q8", g.upload(np.zeros((256, 512), np.int8)), g.upload(np.ones(256, np.float32)), 256, 512)
    a, sa, out = g.upload(np.zeros((64, 512), np.int8)), g.upload(np.ones(64, np.float32)), g.empty((64, 256), "f16")
    with pytest.raises(ValueError):
        ops.gemm(g, a, wt, out, 64, sa=sa, ksplit=2)          # K splits exist for the accumulating epilogue only
    with pytest.raises(ValueError):
        ops.gemm(g, a, wt, out, 64, sa=sa, epi=1)             # needs rtype and gate
    with pytest.raises(ValueError):
        ops.gemm(g, a, wt, out, 64, sa=sa, epi=1, rtype=sa, gate=sa)  # fp16 out: the residual stream is fp32
    with pytest.raises(NotImplementedError):
        ops.gemm(g, a, ops.QWeight("q4", wt.w, wt.sw, 256, 512), out, 64, sa=sa)
    with pytest.raises(ValueError):
        ops.gemm(g, a, wt, out, 64)  # int8 activations without their scales
    assert not g.calls
    ops.gemm(g, a, wt, out, 40, sa=sa)
    assert g.calls[0]["M"] == 64 and ops.pad_rows(129) == 256  # rows padded to the tile height, all written


def test_norm_mod_q8_parameters():
    """Defaults of the reference's launcher (h3metal/ops.py:200-211): x_stride = D, mod_stride = 2 D; variants map to
    one output kind; y and post go together."""
    g = RecordingGpu()
    x, mod, rt = g.empty((8, 768), "f32"), g.empty((3, 2, 768), "f32"), g.empty((8,), "u8")
    out, sa = g.empty((8, 768), "i8"), g.empty((8,), "f32")
    ops.norm_mod_q8(g, x, mod, rt, out, sa, 8, 768, eps=1e-5)
    ops.norm_mod_q8(g, x, mod, rt, out, None, 8, 768, eps=1e-5, out_hr=True, ln=True, block=128, x_stride=1024)
    a, b = g.calls
    assert (a["x_stride"], a["mod_stride"], a["block"], a["out_kind"], a["ln"]) == (768, 1536, 256, 0, False)
    assert (b["x_stride"], b["block"], b["out_kind"], b["ln"]) == (1024, 128, 3, True)
    with pytest.raises(ValueError):
        ops.norm_mod_q8(g, x, mod, rt, out, sa, 8, 768, eps=1e-5, post=mod)


def test_k_split_sequence_matches_the_reference():
    """h3metal/ops.py:143-154: ksplit slices of K, each a view of the whole operands (a_stride = w_stride = K), the
    bias and the low-rank term on the first slice only; refused when K is not a multiple of ksplit * 256."""
    g = RecordingGpu()
    N, K = 256, 1024
    wt = ops.QWeight("q8", g.upload(np.zeros((N, K), np.int8)), g.upload(np.ones(N, np.float32)), N, K,
                     bias=g.upload(np.zeros(N, np.float32)))
    a, sa = g.upload(np.zeros((128, K), np.int8)), g.upload(np.ones(128, np.float32))
    x = g.empty((128, N), "f32")
    rt, gate = g.upload(np.zeros(128, np.uint8)), g.upload(np.ones((3, N), np.float32))
    ops.gemm(g, a, wt, x, 100, sa=sa, epi=1, rtype=rt, gate=gate, ksplit=2)
    first, second = g.calls
    assert (first["K"], first["a_stride"], first["w_stride"], first["M"]) == (512, 1024, 1024, 128)
    assert first["a"].ptr == a.ptr and second["a"].ptr == a.ptr + 512 and second["w"].ptr == wt.w.ptr + 512
    assert first["bias"] is not None and second["bias"] is None and first["g_stride"] == N
    with pytest.raises(ValueError):
        ops.gemm(g, a, wt, x, 100, sa=sa, epi=1, rtype=rt, gate=gate, ksplit=3)


def test_low_rank_for_a_slice_of_the_outputs_keeps_the_whole_layers_codes(golden):
    """rows=: the term is prepared from the whole B (same normalisation, same A' codes and scales) and only B' is cut."""
    g = RecordingGpu()
    full = ops.low_rank(g, golden["lr_A"], golden["lr_B"], ops.Scratch(g))
    N = golden["lr_B"].shape[0]
    rows = [(N // 4, N // 2), (3 * N // 4, N)]
    part = ops.low_rank(g, golden["lr_A"], golden["lr_B"], ops.Scratch(g), rows=rows)
    assert np.array_equal(part.a.w.numpy(), full.a.w.numpy()) and np.array_equal(part.a.sw.numpy(), full.a.sw.numpy())
    keep = np.concatenate([np.arange(a, b) for a, b in rows])
    assert np.array_equal(part.b.numpy(), full.b.numpy()[keep])
    assert np.array_equal(part.lo, full.lo[keep]) and np.array_equal(part.hi, full.hi[keep])


def test_split_of_the_input_side_product():
    """When T's product is split along K: only if the GPU asks for it, activations are contiguous and few row tiles
    would leave SMs idle; the split-major copy of A' holds slice s of every rank's K contiguously."""
    rng = np.random.default_rng(0)
    K, N, r = 8192, 256, 32
    g = RecordingGpu()
    lo = ops.low_rank(g, rng.standard_normal((r, K)).astype(np.float32), rng.standard_normal((N, r)).astype(np.float32),
                      ops.Scratch(g))
    assert ops._t_split(g, lo, 4608, K, None) == 1          # the recording stand-in does not ask for a split
    g.lora_t_split, g.sm_count = 4, 148
    assert ops._t_split(g, lo, 4608, K, None) == 4          # 36 row tiles
    assert ops._t_split(g, lo, 4608, K, K) == 4
    assert ops._t_split(g, lo, 4608, K, K + 64) == 1        # strided activations cannot be viewed as [M * S][K / S]
    assert ops._t_split(g, lo, 17408, K, None) == 1         # 136 row tiles already fill the SMs
    assert ops._t_split(g, lo, 4608, 4096, None) == 2       # K / 4 would be too short to pay for a second launch
    assert ops._t_split(g, lo, 4608, 3072, None) == 1
    sm = lo.split_major(g, 4).numpy()
    codes = lo.a.w.numpy()
    assert sm.shape == (4, lo.R, K // 4)
    for s in range(4):
        assert np.array_equal(sm[s], codes[:, s * (K // 4):(s + 1) * (K // 4)])
