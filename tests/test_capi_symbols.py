"""The C-ABI library loads and exports every function include/h3b200.h declares (no compute, no GPU needed)."""
import ctypes
import os
import re

from h3metal_b200 import build as lib_build, gpu as gpu_mod

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "h3b200.h")).read()
    return sorted(set(re.findall(r"H3B_API[^;(]*?\b(h3b_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    declared = _declared()
    assert len(declared) >= 18
    assert sorted(gpu_mod._signatures()) == declared


def test_library_exports_every_declared_symbol():
    path = lib_build.build()  # compiles with nvcc if the sources are newer; needs no GPU
    lib = ctypes.CDLL(path)
    for name in _declared():
        assert hasattr(lib, name), name
    lib.h3b_last_error.restype = ctypes.c_char_p
    assert lib.h3b_last_error() == b""


def test_no_torch_types_in_the_abi():
    text = open(os.path.join(ROOT, "include", "h3b200.h")).read()
    assert "torch" not in text.replace("PyTorch", "") and "at::" not in text and "#include <stdint.h>" in text
