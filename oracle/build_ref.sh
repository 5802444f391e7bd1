#!/usr/bin/env bash
# Test infrastructure, not product code.
#
# Compiles the UNMODIFIED reference extension (csrc/attention_api.cpp +
# csrc/flash_attention.cu + csrc/flash_api.cpp, the source list of the
# reference's setup.py:46-50) from the sources where they lie, into
# oracle/_ref/attention_cutlass_fp8_ref*.so.  Nothing is copied into this repo.
#
# Differences from the reference's own build (setup.py:18-19,55-71), all on the
# command line only:
#   * -gencode arch=compute_89,code=[sm_100,compute_89]: the reference ships
#     sm_89/sm_90 SASS only, which no B200 can load; its sm_89 PTX is assembled
#     for sm_100 here (FP8 mma.sync is legal on every arch >= sm_89).
#   * the CUTLASS submodule (deps/cutlass) is empty in the reference checkout;
#     the CUTLASS headers bundled with the flashinfer wheel are used instead,
#     with a one-line shim for cute/numeric/integer_subbyte.hpp (removed from
#     newer CUTLASS) and three pre-includes to satisfy include-order
#     assumptions of csrc/kernel_traits.h:3.
#   * the python module is named attention_cutlass_fp8_ref so that it can sit
#     beside this repo's own attention_cutlass_fp8.
#
# Usage: oracle/build_ref.sh REFERENCE_DIR     (or FA8_REFERENCE_DIR in the environment)
set -euo pipefail
REF="${1:-${FA8_REFERENCE_DIR:-}}"
if [ -z "$REF" ] || [ ! -d "$REF/csrc" ]; then
  echo "usage: $0 REFERENCE_DIR (a checkout of weishengying/cutlass_flash_atten_fp8)" >&2
  exit 2
fi
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
PY="${PYTHON:-python}"
mkdir -p "$OUT/shim/cute/numeric" "$OUT/obj"
echo '#pragma once
#include <cute/numeric/numeric_types.hpp>' > "$OUT/shim/cute/numeric/integer_subbyte.hpp"

CUTLASS_INC="$($PY - <<'PY'
import importlib.util, os
spec = importlib.util.find_spec("flashinfer")
print(os.path.join(os.path.dirname(spec.origin), "data", "cutlass", "include"))
PY
)"
TORCH_INC="$($PY - <<'PY'
from torch.utils.cpp_extension import include_paths
print(" ".join("-I" + p for p in include_paths()))
PY
)"
PY_INC="$($PY -c 'import sysconfig; print(sysconfig.get_paths()["include"])')"
TORCH_LIB="$($PY -c 'import torch, os; print(os.path.join(os.path.dirname(torch.__file__), "lib"))')"
EXT="$($PY -c 'import sysconfig; print(sysconfig.get_config_var("EXT_SUFFIX"))')"
ABI="$($PY -c 'import torch; print(int(torch._C._GLIBCXX_USE_CXX11_ABI))')"
NAME=attention_cutlass_fp8_ref
COMMON="-DTORCH_EXTENSION_NAME=$NAME -DTORCH_API_INCLUDE_EXTENSION_H -D_GLIBCXX_USE_CXX11_ABI=$ABI \
  -I$OUT/shim -I$REF/csrc -I$REF/include -I$CUTLASS_INC $TORCH_INC -I$PY_INC -I/usr/local/cuda/include"

nvcc -c "$REF/csrc/flash_attention.cu" -o "$OUT/obj/flash_attention.o" \
  -O3 -std=c++17 --use_fast_math -lineinfo --ptxas-options=-O2 \
  -U__CUDA_NO_HALF_OPERATORS__ -U__CUDA_NO_HALF_CONVERSIONS__ -U__CUDA_NO_HALF2_OPERATORS__ \
  -U__CUDA_NO_BFLOAT16_CONVERSIONS__ --expt-relaxed-constexpr --expt-extended-lambda \
  -gencode 'arch=compute_89,code=[sm_100,compute_89]' \
  -include cute/tensor.hpp -include cute/atom/mma_atom.hpp -include cute/atom/copy_atom.hpp \
  -Xcompiler -fPIC $COMMON
g++ -c "$REF/csrc/attention_api.cpp" -o "$OUT/obj/attention_api.o" -O3 -std=c++17 -fPIC $COMMON
g++ -c "$REF/csrc/flash_api.cpp" -o "$OUT/obj/flash_api.o" -O3 -std=c++17 -fPIC $COMMON
g++ -shared -o "$OUT/$NAME$EXT" "$OUT/obj/flash_attention.o" "$OUT/obj/attention_api.o" "$OUT/obj/flash_api.o" \
  -L"$TORCH_LIB" -ltorch -ltorch_cpu -ltorch_cuda -lc10 -lc10_cuda -ltorch_python \
  -L/usr/local/cuda/lib64 -lcudart -Wl,-rpath,"$TORCH_LIB"
echo "built $OUT/$NAME$EXT"
