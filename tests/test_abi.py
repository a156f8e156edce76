"""The C-ABI library builds, loads without a GPU and exports every symbol the header declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "skv_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(skv_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert "skv_gqa_decode" in names
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/skv_b200.h but not exported"


def test_python_binding_table_matches_header(lib):
    from llm_inference_optimization_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_argument_errors_are_reported_without_a_gpu(lib):
    from llm_inference_optimization_b200 import _lib
    assert lib.skv_abi_version() >= 1
    assert lib.skv_gqa_set_tuning(99, 1) == -1
    assert "tuning" in _lib.last_error()
    rc = lib.skv_gqa_decode(None, None, None, None, None, 0, 1, 1, 1, 1, 128, 0, None, None, 0, 0, 0, None, 1.0, 0, None)
    assert rc == -1 and "null" in _lib.last_error()
    assert lib.skv_gqa_decode_workspace_bytes(1, 65536, 32, 8, 128, 0) > 0
    assert lib.skv_gqa_decode_workspace_bytes(1, 65536, 32, 5, 128, 0) == 0


def test_package_imports_and_has_no_cpu_fallback():
    import llm_inference_optimization_b200 as skv
    import torch
    assert hasattr(skv, "fused_gqa")
    if not torch.cuda.is_available():
        import pytest
        with pytest.raises(RuntimeError):
            skv.fused_gqa(torch.zeros(1, 8, 128).half(), torch.zeros(1, 4, 8, 128).half(),
                          torch.zeros(1, 4, 8, 128).half(), 1.0)
