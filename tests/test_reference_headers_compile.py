"""The adapters a reference maintainer would add to bind this kernel library compile against the reference's OWN headers (not this repository's mirror of them).

tests/ref_adapters/b200_adapters.cc holds three adapters — RmsNormalization (plain operator), MatMul (attribute struct,
workspace, the weight-is-static hint) and AllReduce (a handle kept in runtime::Resources) — and the collector lines that
register them, written against kernel/kernel.h, kernel/tensor.h, kernel/attributes/*.h and runtime/resource.h of a
reference checkout.  The checkout is taken from RG_REFERENCE_ROOT, else from a directory named `reference` beside this
repository (the rule oracle/Makefile uses); without one the test is skipped: nothing here is needed at run time."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_root():
    ref = os.environ.get("RG_REFERENCE_ROOT") or os.path.abspath(os.path.join(ROOT, "..", "reference"))
    return ref if os.path.isdir(os.path.join(ref, "src", "04kernel", "include")) else None


@pytest.mark.skipif(_reference_root() is None, reason="no reference checkout on this machine")
def test_adapters_compile_against_the_reference_headers():
    import torch
    ref = _reference_root()
    fmt_inc = os.path.join(os.path.dirname(torch.__file__), "include")      # header-only fmt, as the oracle build uses
    cmd = ["g++", "-std=c++20", "-fsyntax-only", "-DFMT_HEADER_ONLY", "-include", "cassert", "-Wall", "-Wno-deprecated-declarations",
           "-I" + os.path.join(ROOT, "oracle", "shim"), "-I" + fmt_inc, "-I" + os.path.join(ROOT, "include")]
    for sub in ("00common", "01graph_topo", "02hardware", "03runtime", "04kernel"):
        cmd.append("-I" + os.path.join(ref, "src", sub, "include"))
    cmd.append(os.path.join(ROOT, "tests", "ref_adapters", "b200_adapters.cc"))
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0, r.stdout[-4000:]
