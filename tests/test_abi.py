"""CPU-side checks of the C ABI: the library loads, exports every symbol the header declares,
and argument validation answers without touching a GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from flexllm_b200 import build, _lib
    build.build()
    return _lib.load()


def declared_symbols():
    out = []
    for name in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if name.endswith(".h"):
            text = open(os.path.join(ROOT, "include", name)).read()
            out += re.findall(r"FLEXLLM_API\s+[\w\s\*]+?\b(flexllm_\w+)\s*\(", text)
    return out


def test_header_symbols_exported(lib):
    syms = declared_symbols()
    assert len(syms) >= 15
    missing = [s for s in syms if not hasattr(lib, s)]
    assert not missing, missing


def test_python_signatures_cover_header(lib):
    from flexllm_b200 import _lib
    declared = set(declared_symbols())
    bound = set(_lib.SIGNATURES) | {"flexllm_status_string"}
    assert declared <= bound, declared - bound


def test_status_strings(lib):
    assert lib.flexllm_status_string(0) == b"ok"
    assert b"invalid" in lib.flexllm_status_string(-1)
    assert lib.flexllm_version() >= 100


def test_argument_validation_needs_no_gpu(lib):
    # null pointers / bad shapes are rejected on the host before any CUDA call
    assert lib.flexllm_quant_per_token(None, 4, 64, None, None, None) == -1
    assert lib.flexllm_fht(C.c_void_p(16), 1, 100, 1.0, C.c_void_p(16), None) == -1      # not a power of two
    assert lib.flexllm_linear_prefill_i8(C.c_void_p(16), None, C.c_void_p(16), None, 8, 64, 100,
                                         C.c_void_p(16), None, None) == -1              # K % 16 != 0
    assert lib.flexllm_rmsnorm_quant(C.c_void_p(16), C.c_void_p(16), 1, 2048, 1e-5, 3, C.c_void_p(16),
                                     None, None, None) == -1                            # unknown order


def test_no_cpu_fallback_in_product():
    """The product package must not import the oracle."""
    for dirpath, _, files in os.walk(os.path.join(ROOT, "flexllm_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".hpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text and "liboracle" not in text, f
