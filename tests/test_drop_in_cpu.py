"""CPU: the drop-in tree — four extension modules at the paths and names the reference looks up
under FP4_MATMUL_ROOT — loads the way the reference loads it (by file path) and exposes the symbols
the reference dereferences (tk_gemm.py:3454-3461, tools/check_fp4_runtime_abi.py:16-47)."""
import importlib
import importlib.util
import os

import pytest

REQUIRED = {
    "_tk_quant_v5": ["tk_quantize_for_gemm", "tk_quantize_weight_2d", "tk_fused_norm_quantize",
                     "tk_fused_norm_quantize_from_inv_rms", "tk_silu_quantize_split_for_gemm",
                     "tk_silu_deriv_quantize_split_for_gemm", "tk_silu_deriv_quantize_split_for_gemm_opt",
                     "tk_quantize_for_gemm_opt", "tk_quantize_transpose", "tk_fused_norm_quantize_opt",
                     "tk_quantize_nhsd_wo_for_gemm", "tk_group_quantize_dim1_split3_for_gemm",
                     "tk_group_quantize_dim1_for_gemm",
                     "tk_silu_deriv_quantize_split_for_gemm_opt_alloc", "tk_silu_deriv_quantize_split_for_gemm_opt_launch"],
    # tk_gemm.py:3454-3461 dereferences nvfp4_split_dgrad_sum and nvfp4_batched_accum_gemm unconditionally
    "_C": ["nvfp4_gemm", "nvfp4_gemm_config", "nvfp4_gemm_nopdl", "nvfp4_grouped_gemm", "nvfp4_gemm_residual",
           "nvfp4_batched_gemm", "nvfp4_split_dgrad_sum", "nvfp4_batched_accum_gemm", "nvfp4_forward_rope_packed_qk",
           "nvfp4_inverse_rope_packed_qk", "nvfp4_grouped_gemm_rope_packed_split", "sum3_rmsnorm_bwd_out",
           "rmsnorm_bwd_residual_out", "nvfp4_grouped_gemm_config_nopdl"],
    "mxfp4_quant_v4": ["mxfp4_quantize_for_gemm", "mxfp4_quantize_row_and_col",
                       "mxfp4_fused_rmsnorm_quantize_row_and_col", "mxfp4_fused_silu_mul_quantize_row_and_col",
                       "mxfp4_quantize_for_gemm_opt_rht", "mxfp4_quantize_weight_2d", "mxfp4_quantize_row_and_col_opt",
                       "mxfp4_fused_silu_deriv_quantize_split2_row_and_col_splitcols",
                       "mxfp4_fused_silu_deriv_quantize_split2_row_and_col_splitcols_launch_inplace",
                       "mxfp4_fused_silu_deriv_quantize_split2_row_and_col_strided_combined",
                       "mxfp4_fused_silu_mul_quantize_row_and_col_strided", "mxfp4_quantize_split2_row_and_col",
                       "mxfp4_quantize_split3_row_and_col", "mxfp4_quantize_split3_row_and_col_launch_inplace",
                       "mxfp4_quantize_split3_row_and_col_inverse_rope_live64", "mxfp4_quantize_nhsd_wo_row_and_col",
                       "mxfp4_quantize_col_only"],
    "_C_mx": ["mxfp4_gemm", "mxfp4_gemm_config", "mxfp4_batched_gemm", "mxfp4_batched_gemm_config",
              "mxfp4_gemm_residual", "mxfp4_gemm_residual_config", "mxfp4_split2_dgrad_strided_onepass_gemm",
              "mxfp4_split3_dgrad_strided_onepass_gemm", "mxfp4_gemm_rope_live64", "mxfp4_gemm_rope_live64_config",
              "mxfp4_gemm_rope_live", "mxfp4_gemm_rope", "mxfp4_batched_gemm_rope_live64", "mxfp4_batched_gemm_rope_live"],
}


@pytest.mark.parametrize("name", sorted(REQUIRED))
def test_stub_loads_by_path_and_exports_symbols(name):
    b = importlib.import_module("mfu-fp4-training_b200.build")
    b.build_drop_in()
    path = b.drop_in_path(name)
    assert os.path.isfile(path)
    rel = os.path.relpath(path, b.DROP_IN_ROOT)
    assert rel.startswith(b.DROP_IN[name][0])
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    for sym in REQUIRED[name]:
        assert callable(getattr(mod, sym)), f"{name}.{sym} missing"
