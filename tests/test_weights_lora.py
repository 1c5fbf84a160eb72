"""The .h3m container and the LoRA term helpers on the CPU (fake Gpu): byte-level compatibility with a file the
reference's own Writer produced (tests/golden/ref_file.h3m.gz), round trips (the reference's
tests/test_convert.py:51-66), and rotation / stacking of adapter factors against the reference's outputs."""
import gzip
import os

import numpy as np
import pytest

from h3metal_b200 import lora, ops, quant, weights
from tests.conftest import GOLDEN_DIR
from tests.fakes import RecordingGpu


@pytest.fixture()
def ref_file(tmp_path):
    path = tmp_path / "ref.h3m"
    with gzip.open(os.path.join(GOLDEN_DIR, "ref_file.h3m.gz"), "rb") as src:
        path.write_bytes(src.read())
    return str(path)


def test_reads_a_file_written_by_the_reference(ref_file, golden):
    hdr = weights.read_header(ref_file)
    assert hdr["meta"] == {"kind": "test", "hidden": 512} and hdr["chunk"] == weights.CHUNK
    wf = weights.WeightFile(RecordingGpu(), ref_file)
    assert "lin" in wf and "nope" not in wf
    assert np.array_equal(wf.host("a"), np.arange(1000, dtype=np.float32))
    assert np.array_equal(wf.tensor("a").numpy(), np.arange(1000, dtype=np.float32))
    assert np.array_equal(wf.host("cpu_only"), np.arange(7, dtype=np.int32))
    with pytest.raises(ValueError):
        wf.tensor("cpu_only")
    lin = wf.linear("lin")
    assert isinstance(lin, ops.QWeight) and (lin.fmt, lin.N, lin.K, lin.G) == ("q8", 24, 512, 128)
    assert np.array_equal(lin.w.numpy(), golden["q8_codes"]) and np.array_equal(lin.sw.numpy(), golden["q8_scales"])
    assert np.array_equal(lin.bias.numpy(), np.linspace(-1, 1, 24).astype(np.float32))
    assert wf.linear("lin").w is lin.w  # uploaded once, then resident
    assert wf.nbytes(["a", "lin"]) == 4000 + 24 * 512 + 24 * 4 + 24 * 4
    wf.close()


def test_writer_produces_the_reference_layout(tmp_path, ref_file, golden):
    """Writing the same content gives the same bytes as the reference's Writer gave."""
    path = str(tmp_path / "mine.h3m")
    w = weights.Writer(path, {"kind": "test", "hidden": 512})
    w.tensor("a", np.arange(1000, dtype=np.float32), "f32")
    w.tensor("cpu_only", np.arange(7, dtype=np.int32), "i32", host_only=True)
    w.linear("lin", "q8", 24, 512, golden["q8_codes"], golden["q8_scales"], bias=np.linspace(-1, 1, 24).astype(np.float32))
    with pytest.raises(KeyError):
        w.tensor("a", np.zeros(3, np.float32), "f32")
    w.close()
    assert open(path, "rb").read() == open(ref_file, "rb").read()
    for e in weights.read_header(path)["tensors"].values():
        for part in ([e] if "offset" in e else [e[k] for k in ("w", "sw", "bias")]):
            assert part["offset"] % 256 == 0 and part["offset"] >= weights.DATA_START


def test_refuses_other_files_and_formats(tmp_path):
    bad = tmp_path / "bad.h3m"
    bad.write_bytes(b"NOPE" + b"\0" * 64)
    with pytest.raises(ValueError):
        weights.read_header(str(bad))
    path = str(tmp_path / "q4.h3m")
    w = weights.Writer(path, {})
    w.linear("l4", "q4", 8, 64, np.zeros((8, 32), np.uint8), np.ones(8, np.float32))
    w.close()
    with pytest.raises(NotImplementedError):
        weights.WeightFile(RecordingGpu(), path).linear("l4")


def test_lora_terms_match_the_reference(golden):
    sgn = golden["signs_512_seed3"]
    t1 = lora.term(golden["lora_A1"], golden["lora_B1"], strength=0.8, scale=2.0, signs=sgn)
    t2 = lora.term(golden["lora_A2"], golden["lora_B2"], strength=1.0, scale=0.5, signs=sgn)
    A, B = lora.stack([t1, t2])
    assert np.array_equal(A, golden["lora_stack_A"]) and np.array_equal(B, golden["lora_stack_B"])
    # rows placed into a fused layer; ordering by first touched row
    placed = lora.term(golden["lora_A1"], golden["lora_B1"], rotate=False, rows=np.arange(96) + 32, n_out=160)
    assert placed.B.shape == (160, 4) and not placed.B[:32].any() and np.array_equal(placed.B[32:128], golden["lora_B1"])
    assert lora.order([placed, t1])[0] is t1
    # the rotated term equals the dense update in the rotated space: x W'^T with W' = rot(W + s B A)
    x = np.random.default_rng(0).standard_normal((3, 512)).astype(np.float32)
    dense = x @ (np.float32(1.6) * golden["lora_B1"] @ golden["lora_A1"]).T
    assert np.allclose(quant.rotate_in(x, sgn) @ t1.A.T @ t1.B.T, dense, atol=2e-3)
