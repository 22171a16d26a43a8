"""B200-native FP4 training hot path: fused RMSNorm + NVFP4/MXFP4 quantisation, block-scaled
FP4 GEMMs and the quantised SwiGLU producer, as hand-written sm_100a CUDA behind a C ABI
(``include/fp4b200.h``), with Python shims that mirror the reference's extension modules.

The directory name contains a hyphen, so import it with
``importlib.import_module("mfu-fp4-training_b200")``.
"""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
