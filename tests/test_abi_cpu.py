"""CPU: the C-ABI library builds, loads and exports every symbol include/fp4b200.h declares;
host-side argument validation of the shims (no compute calls)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "fp4b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fp4b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    import __graft_entry__ as ge
    ge.build()
    lib = ctypes.CDLL(pkg._lib.LIB_PATH)
    syms = declared_symbols()
    assert len(syms) >= 8
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in include/fp4b200.h but not exported"
    assert lib.fp4b200_abi_version() == 1


def test_ctypes_table_covers_header(pkg):
    assert sorted(pkg._lib.SIGNATURES) == declared_symbols()


def test_shim_rejects_cpu_tensors(pkg):
    import importlib
    import torch
    tkq = importlib.import_module("mfu-fp4-training_b200.tk_quant_v5")
    with pytest.raises(RuntimeError):
        tkq.tk_quantize_for_gemm(torch.zeros(128, 128, dtype=torch.bfloat16), True)
    with pytest.raises(RuntimeError):
        tkq.tk_fused_norm_quantize(torch.zeros(128, 128, dtype=torch.bfloat16), torch.ones(128), 1e-5, False, True)
