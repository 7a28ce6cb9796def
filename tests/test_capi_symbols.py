"""The C-ABI library loads without a GPU and exports every symbol include/rg_b200.h declares."""
import os
import re

from refactorgraph_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "rg_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rg_b200_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(capi.SYMBOLS)


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert lib.rg_b200_version() >= 1
    assert lib.rg_b200_status_string(capi.ERR_TIMEOUT) == b"bounded wait expired"


def test_argument_validation_needs_no_gpu(lib):
    # NULL / bad-shape rejections happen before any CUDA call
    p = capi.RmsNormParams(capi.F32, 1, 0, 1e-6, 0)
    assert capi.call("rms_norm", p, [1, 1], [1], check=False) == capi.ERR_SHAPE
    assert capi.call("rms_norm", p, [0, 0], [0], check=False) == capi.ERR_NULL
    t = capi.TopkParams(capi.F32, 1, 10, 65, 0)
    assert capi.call("topk", t, [1], [1, 1], check=False) == capi.ERR_SHAPE
    m = capi.MatMulParams()
    m.dtype = capi.I32
    m.m = m.n = m.k = m.batch = 1
    assert capi.call("mat_mul", m, [1, 1], [1], check=False) == capi.ERR_DTYPE
