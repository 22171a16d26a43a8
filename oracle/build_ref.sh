#!/bin/bash
# Test infrastructure, not product code.
#
# Compiles the reference's own sm_100a extension modules from the sources where they lie in a checkout of
# MrHuff/mfu-fp4-training (one .cu translation unit each, with the flags of the reference's Makefiles:
# fp4_runtime/TK_quantisation/nvfp4_v5/Makefile:4-27 and fp4_runtime/ThunderKittens/kernels/common.mk) into
# oracle/_ref/.  nvcc cross-compiles without a GPU.  The modules are used only
#   * by tests/golden/make_sr_golden.py, on one GPU, to record the reference kernels' own output bytes, and
#   * by bench.py's --reference-kernels leg, to time the reference's kernels beside this library's.
# Nothing under mfu-fp4-training_b200/ loads them.
#
#   oracle/build_ref.sh <reference checkout> [quant|gemm|mxquant|mxgemm|all]
set -euo pipefail
REF=${1:?usage: build_ref.sh <reference checkout> [quant|gemm|mxquant|mxgemm|all]}
WHAT=${2:-all}
HERE=$(cd "$(dirname "$0")" && pwd)
OUT=$HERE/_ref
mkdir -p "$OUT"
NVCC=${NVCC:-nvcc}
SUFFIX=$(python3 -c "import sysconfig; print(sysconfig.get_config_var('EXT_SUFFIX'))")
PYINC=$(python3 -c "import sysconfig; print('-I' + sysconfig.get_path('include'))")
PBINC=$(python3 -m pybind11 --includes)
THINC=$(python3 -c "from torch.utils.cpp_extension import include_paths; print(' '.join('-I' + p for p in include_paths()))")
THLIBS=$(python3 -c "from torch.utils.cpp_extension import library_paths; print(' '.join(library_paths()))")
THLINK=""
for p in $THLIBS; do THLINK="$THLINK -L$p -Xlinker -rpath -Xlinker $p"; done
COMMON="-std=c++20 -O3 --expt-extended-lambda --expt-relaxed-constexpr -forward-unknown-to-host-compiler
  -Xcompiler=-Wno-psabi -Xcompiler=-fno-strict-aliasing -DNDEBUG -lineinfo -shared -fPIC -diag-suppress 3189,3288
  -DTORCH_API_INCLUDE_EXTENSION_H -DKITTENS_BLACKWELL -gencode arch=compute_100a,code=sm_100a
  $PYINC $PBINC $THINC $THLINK -ltorch_python -ltorch_cuda -ltorch_cpu -ltorch -lc10_cuda -lc10"

if [ "$WHAT" = quant ] || [ "$WHAT" = all ]; then
  # _tk_quant_v5: NVFP4 quantisers (tk_quantize.cu and the headers beside it)
  (cd "$REF/fp4_runtime/TK_quantisation/nvfp4_v5" &&
   $NVCC $COMMON -I../../ThunderKittens/include -Xcudafe --diag_suppress=3288 -DTORCH_EXTENSION_NAME=_tk_quant_v5 \
     tk_quantize.cu -o "$OUT/_tk_quant_v5$SUFFIX")
fi
if [ "$WHAT" = gemm ] || [ "$WHAT" = all ]; then
  # _C: NVFP4 tcgen05 GEMMs (nvfp4_b200_gemm.cu)
  (cd "$REF/fp4_runtime/ThunderKittens/kernels/gemm/nvfp4_b200" &&
   $NVCC $COMMON -I../../../include -I../../../prototype -DTORCH_COMPILE -DTORCH_EXTENSION_NAME=_C \
     -D__CUDA_NO_HALF_OPERATORS__ -D__CUDA_NO_HALF_CONVERSIONS__ -D__CUDA_NO_BFLOAT16_CONVERSIONS__ \
     -D__CUDA_NO_HALF2_OPERATORS__ -L"${CUDA_HOME:-/usr/local/cuda}/lib64/stubs" -lcuda \
     nvfp4_b200_gemm.cu -o "$OUT/_C$SUFFIX")
fi
if [ "$WHAT" = mxquant ] || [ "$WHAT" = all ]; then
  # mxfp4_quant_v4: MXFP4 quantisers (tk_quantize.cu + mxfp4_v3_quantize.cuh; flags of mxfp4_v4/Makefile:32-49)
  (cd "$REF/fp4_runtime/TK_quantisation/mxfp4_v4" &&
   $NVCC $COMMON -diag-suppress 177 -I../nvfp4_v5 -DTORCH_EXTENSION_NAME=mxfp4_quant_v4 \
     -D__CUDA_NO_HALF_OPERATORS__ -D__CUDA_NO_HALF_CONVERSIONS__ -D__CUDA_NO_BFLOAT16_CONVERSIONS__ \
     -D__CUDA_NO_HALF2_OPERATORS__ -L"${CUDA_HOME:-/usr/local/cuda}/lib64/stubs" -lcuda \
     tk_quantize.cu -o "$OUT/mxfp4_quant_v4$SUFFIX")
fi
if [ "$WHAT" = mxgemm ] || [ "$WHAT" = all ]; then
  # _C_mx: MXFP4 tcgen05 GEMMs (mxfp4_gb200_gemm.cu; mxfp4_gb200/Makefile + kernels/common.mk)
  (cd "$REF/fp4_runtime/ThunderKittens/kernels/gemm/mxfp4_gb200" &&
   $NVCC $COMMON -I../../../include -I../../../prototype -DTORCH_COMPILE -DTORCH_EXTENSION_NAME=_C_mx \
     -D__CUDA_NO_HALF_OPERATORS__ -D__CUDA_NO_HALF_CONVERSIONS__ -D__CUDA_NO_BFLOAT16_CONVERSIONS__ \
     -D__CUDA_NO_HALF2_OPERATORS__ -L"${CUDA_HOME:-/usr/local/cuda}/lib64/stubs" -lcuda \
     mxfp4_gb200_gemm.cu -o "$OUT/_C_mx$SUFFIX")
fi
ls -la "$OUT"
