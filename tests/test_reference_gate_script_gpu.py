"""The reference's OWN release-gate code run against this library's drop-in tree.

`tools/check_fp4_runtime_numerics.py` of the reference loads the four extension modules by exact path under a runtime
root (its `_load_extension`), quantises the gate's 512^3 inputs through them and multiplies
(`_nvfp4_gate`: tk_quantize_for_gemm -> nvfp4_gemm; `_mxfp4_gate`: signed-H32 mxfp4_quantize_for_gemm_opt_rht ->
mxfp4_gemm), and asserts its thresholds.  Here those two functions are imported from a checkout of the reference and
pointed at mfu-fp4-training_b200/fp4_runtime: the loader must find the modules at the reference's relative paths and
the gate must print the metrics the reference recorded from its own kernels (release/gpu_gate_receipt.json:47-56).
The script's `main()` is not used: it refuses any CUDA other than 13.0 before doing anything.

Needs the checkout: set FP4_REFERENCE_CHECKOUT to it (the test is skipped where there is none)."""
import importlib.util
import os
import sysconfig
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

RECORDED = {"nvfp4": (0.16246939, 0.98681033, 1.00062418), "mxfp4": (0.16712865, 0.98597604, 0.99495852)}


def _gate_module():
    root = os.environ.get("FP4_REFERENCE_CHECKOUT", "")
    script = Path(root) / "tools" / "check_fp4_runtime_numerics.py"
    if not root or not script.is_file():
        pytest.skip("FP4_REFERENCE_CHECKOUT does not point to a checkout of the reference")
    spec = importlib.util.spec_from_file_location("check_fp4_runtime_numerics", script)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_the_references_gate_functions_pass_on_the_drop_in_tree():
    gate = _gate_module()
    pkg = importlib.import_module("mfu-fp4-training_b200")
    build = importlib.import_module("mfu-fp4-training_b200.build")
    build.build_drop_in()
    root = Path(build.DROP_IN_ROOT).resolve()
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    nv = gate._nvfp4_gate(root, suffix)     # raises AssertionError outside the reference's thresholds
    mx = gate._mxfp4_gate(root, suffix)
    for got, want in ((nv, RECORDED["nvfp4"]), (mx, RECORDED["mxfp4"])):
        assert abs(got["rel_l2"] - want[0]) < 1e-6 and abs(got["cosine"] - want[1]) < 1e-6 and abs(got["norm_ratio"] - want[2]) < 1e-6
    assert pkg is not None
