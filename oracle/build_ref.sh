#!/usr/bin/env bash
# Builds the reference project's own CUDA kernels for this path, unmodified,
# for sm_100a, from the sources where they lie in the mounted reference tree.
# Output: oracle/_ref/libref_grad.so (git-ignored; test infrastructure only).
#
# The four translation units are the ones that hold the reference's BFP8 block
# codec, the tensor-wide BFP8 gradient reducer, the bucketed BF16 / block-BFP8
# transport and the BF16 gradient norm/scale kernels.  The flags follow the
# reference's own build script (build-cuda.ps1: -O3 --use_fast_math -std=c++17)
# with only the target architecture changed.  No reference source is copied.
set -euo pipefail
REF_ROOT="${NNTRAIN_REFERENCE_ROOT:-}"
if [ -z "$REF_ROOT" ]; then
  echo "set NNTRAIN_REFERENCE_ROOT to the reference project's root" >&2
  exit 0
fi
SRC="$REF_ROOT/NNtrain.Cuda/native"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
OUT="$HERE/_ref"
if [ ! -d "$SRC" ]; then
  echo "reference tree not mounted at $REF_ROOT; keeping any prebuilt $OUT" >&2
  exit 0
fi
mkdir -p "$OUT"
nvcc -O3 --use_fast_math -std=c++17 \
  -gencode arch=compute_100a,code=sm_100a \
  -Xcompiler -fPIC -shared \
  "$SRC/gradient_collectives.cu" "$SRC/cuda_runtime_bridge.cu" \
  "$SRC/tensor_kernels.cu" "$SRC/pure_bfloat16_gradients.cu" \
  -o "$OUT/libref_grad.so"
echo "built $OUT/libref_grad.so"
