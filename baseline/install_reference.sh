#!/bin/bash
# Install the unmodified reference under baseline/_ref (git-ignored; travels to the GPU box).
#  1. its CUDA extension (cuda_kernels/, package srrcomp with eden_utils) built for sm_100 with pip from a
#     writable copy, as the reference's own build script does with TORCH_CUDA_ARCH_LIST;
#  2. its kernel benchmark (cuda_kernels/tests/benchmark_scaling_quantization.py), copied byte for byte to
#     _ref/tests/, from where its own import logic finds srrcomp.eden_utils one folder up;
#  3. its hook package and smoke test, copied byte for byte, with eden_utils placed inside
#     new_comm_hooks/ exactly as testbed_evaluation/build_eden_utils_llm.zsh does.
set -euo pipefail
REF=${1:?usage: install_reference.sh <path of the reference checkout>}
HERE="$(cd "$(dirname "$0")" && pwd)"
DST="$HERE/_ref"
mkdir -p "$DST"
if ! ls "$DST"/srrcomp/eden_utils*.so >/dev/null 2>&1; then
  rm -rf /tmp/ref_cuda_kernels && cp -r "$REF/cuda_kernels" /tmp/ref_cuda_kernels && chmod -R u+w /tmp/ref_cuda_kernels
  TORCH_CUDA_ARCH_LIST=10.0 MAX_JOBS=8 python -m pip install --no-index --no-build-isolation --no-deps \
      --find-links /opt/wheelhouse --target "$DST" /tmp/ref_cuda_kernels
fi
mkdir -p "$DST/tests" "$DST/testbed_evaluation"
cp "$REF/cuda_kernels/tests/benchmark_scaling_quantization.py" "$DST/tests/"
cp -r "$REF/testbed_evaluation/new_comm_hooks" "$DST/testbed_evaluation/"
cp "$REF/testbed_evaluation/smoke_test_new_comm_hooks.py" "$DST/testbed_evaluation/"
cp "$DST"/srrcomp/eden_utils*.so "$DST/testbed_evaluation/new_comm_hooks/"
echo "reference installed under $DST"
