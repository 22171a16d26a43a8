"""Builds libfp4b200.so (all CUDA kernels + the C ABI) in-tree with nvcc for sm_100a.

    python mfu-fp4-training_b200/build.py [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library lands next to this file so that it travels
with the source tree; nothing is installed into site-packages.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libfp4b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    deps.append(os.path.abspath(__file__))
    return any(os.path.getmtime(d) > t for d in deps)


# extension-module name -> (sub-path under fp4_runtime/, mirror module, levels up to the package's parent)
DROP_IN = {
    "_tk_quant_v5": ("TK_quantisation/nvfp4_v5", "tk_quant_v5", 4),
    "mxfp4_quant_v4": ("TK_quantisation/mxfp4_v4", "mxfp4_quant_v4", 4),
    "_C": ("ThunderKittens/kernels/gemm/nvfp4_b200", "tk_gemm_c", 6),
    "_C_mx": ("ThunderKittens/kernels/gemm/mxfp4_gb200", "tk_gemm_c_mx", 6),
}
DROP_IN_ROOT = os.path.join(HERE, "fp4_runtime")


def drop_in_path(name: str) -> str:
    import sysconfig
    sub = DROP_IN[name][0]
    return os.path.join(DROP_IN_ROOT, sub, name + sysconfig.get_config_var("EXT_SUFFIX"))


def build_drop_in(force: bool = False) -> str:
    """Compiles the four extension-module stubs of the drop-in tree (plain C, CPython API)."""
    import sysconfig
    src = os.path.join(CSRC, "ext_stub.c")
    inc = sysconfig.get_paths()["include"]
    for name, (sub, mirror, up) in DROP_IN.items():
        out = drop_in_path(name)
        if not force and os.path.exists(out) and os.path.getmtime(out) > os.path.getmtime(src):
            continue
        os.makedirs(os.path.dirname(out), exist_ok=True)
        cmd = [os.environ.get("CC", "gcc"), "-O2", "-shared", "-fPIC", f"-I{inc}", f"-DSTUB_NAME={name}",
               f'-DSTUB_MIRROR="{mirror}"', f"-DSTUB_UP={up}", src, "-o", out, "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("stub build failed:\n" + " ".join(cmd) + "\n" + res.stderr)
    return DROP_IN_ROOT


def build(force: bool = False, verbose: bool = False) -> str:
    build_drop_in(force)
    if not force and not _stale():
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc, *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += sources() + ["-o", LIB_PATH]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stdout + res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
