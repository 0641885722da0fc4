"""The shared library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "realq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rq_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_header_symbols():
    from gptq_plus_mp_quant_b200.csrc import build
    path = build.build()
    lib = ctypes.CDLL(path)
    names = _declared_symbols()
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/realq_b200.h but not exported"


def test_binding_table_matches_header():
    from gptq_plus_mp_quant_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared_symbols()
    assert _lib.lib.rq_version() >= 100
    assert _lib.error_string(0) == "ok"
    assert "wait" in _lib.error_string(_lib.RQ_ERR_TIMEOUT)


def test_no_compute_without_gpu_is_loud():
    import pytest
    import torch
    from gptq_plus_mp_quant_b200.utils import hadamard_utils
    if torch.cuda.is_available():
        pytest.skip("checks the CPU-only behaviour")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        hadamard_utils.matmul_hadU_cuda(torch.randn(4, 64), None, 1)
