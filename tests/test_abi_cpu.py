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


def test_entry_points_validate_before_touching_the_device(pkg):
    """Argument checks come first in every entry point, so bad calls fail with a message on a machine
    without a GPU as well (no kernel is launched here)."""
    lib = pkg._lib.load()
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.cast(buf, ctypes.c_void_p)

    def msg():
        return lib.fp4b200_last_error().decode()

    assert lib.fp4b200_row_rms_reduce(p, 128, 7, 4096, 1e-5, p, None) == -1 and "partition" in msg()
    assert lib.fp4b200_row_rms_reduce(p, 128, 129, 8192, 1e-5, p, None) == -1
    assert lib.fp4b200_row_rms_reduce(p, 128, 16, 4096, -1.0, p, None) == -1 and "eps" in msg()
    assert lib.fp4b200_fp32_to_fp4x2(p, -1, p, None) == -1
    assert lib.fp4b200_tk_nvfp4_quantize(p, 100, 128, p, p, p, 0, None) == -1 and "multiples of 128" in msg()
    assert lib.fp4b200_mxfp4_quantize_weight_2d(p, 128, 100, p, p, p, p, None) == -1
    assert lib.fp4b200_nvfp4_fused_norm_quantize_noalloc(p, p, 1e-5, 65536 + 128, 128, p, p, p, p, p, None) == -1
    assert "65536" in msg()
    # K-split GEMM: segment count, widths and offsets
    offs = (ctypes.c_int64 * 2)(0, 512)
    widths = (ctypes.c_int64 * 2)(512, 500)
    ptrs = (ctypes.c_void_p * 2)(p, p)
    assert lib.fp4b200_mxfp4_gemm_ksplit(p, 1024, 5, offs, widths, ptrs, ptrs, ptrs, p, 0, 128, 256, None) == -1
    assert lib.fp4b200_mxfp4_gemm_ksplit(p, 1024, 2, offs, widths, ptrs, ptrs, ptrs, p, 0, 128, 256, None) == -1
    assert "segment 1" in msg()
    widths = (ctypes.c_int64 * 2)(512, 768)     # runs past the 1024 columns of A
    assert lib.fp4b200_mxfp4_gemm_ksplit(p, 1024, 2, offs, widths, ptrs, ptrs, ptrs, p, 0, 128, 256, None) == -1
    assert lib.fp4b200_nvfp4_gemm(p, p, p, p, p, p, p, 0, None, 128, 200, 256, None) == -1 and "N % 128" in msg()
    # RMSNorm backward: shape limits, then aliasing of outputs with inputs
    assert lib.fp4b200_sum3_rmsnorm_bwd(p, p, p, p, p, p, p, p, p, p, 0, 4, 384, None) == -1 and "multiple of 256" in msg()
    assert lib.fp4b200_sum3_rmsnorm_bwd(p, p, p, p, p, p, p, p, p, p, 0, 4, 16384, None) == -1 and "8192" in msg()
    assert lib.fp4b200_sum3_rmsnorm_bwd(p, p, p, p, p, p, p, p, p, p, 0, 1, 256, None) == -1 and "overlaps" in msg()
    assert lib.fp4b200_rmsnorm_bwd_residual(p, p, p, p, p, p, p, p, 4, 2048, None) == -1 and "4096" in msg()
    # stochastic MXFP4 quantisers: transform block size, axes, outputs
    assert lib.fp4b200_mxfp4_quantize_row_sr(p, 128, 128, 1, 1, 0, 8, 0, 1, 2, p, p, None) == -1 and "16 or 32" in msg()
    assert lib.fp4b200_mxfp4_quantize_row_sr(p, 128, 100, 1, 1, 0, 0, 0, 1, 2, p, p, None) == -1
    assert lib.fp4b200_mxfp4_quantize_row_and_col_sr(p, 128, 128, 1, 1, 0, 16, 1, 0, 0, 1, 2, p, p, p, p, None) == -1
    assert "at least one axis" in msg()
    assert lib.fp4b200_mxfp4_quantize_row_and_col_sr(p, 128, 128, 1, 1, 0, 0, 0, 0, 0, 1, 2, p, p, p, None, None) == -1
    # pitched opt quantiser: the pitch of the wider row-code matrix
    assert lib.fp4b200_nvfp4_quantize_opt_into(p, None, None, 128, 256, p, p, 1, 1, 0, 0, 0, 0, 0, 1, 1, 0, 0, None, 0, p, 100, p, p,
                                               p, None, None) == -1 and "row pitch" in msg()
    # device-side numbering of stochastic launches: argument checks come before any launch
    assert lib.fp4b200_sr_prepare_state(None, 1, 2, 1, None) == -1 and "rng_state" in msg()
    assert lib.fp4b200_sr_prepare_state(p, 1, 2, 0, None) == -1 and "positive" in msg()
    assert lib.fp4b200_sr_get_invocation_offset(None, None) == -1
