#!/usr/bin/env bash
# Compiles the upstream project's own fp32 layers for sm_100a, from its sources under $DF8_REFERENCE_DIR (the checkout of the
# upstream project), into oracle/_ref/libdnn_ref.so.  Only this wrapper (ref_wrap.cu) is ours; no upstream source
# is copied into the repository and upstream's CMake build is not used (it needs network access for GoogleTest,
# and TBB for one app).  Output goes to oracle/_ref/ only, which is git-ignored.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
# the upstream checkout: $DF8_REFERENCE_DIR, else a directory named "reference" beside this repository
REF="${DF8_REFERENCE_DIR:-${REF:-$HERE/../../reference}}"
OUT="$HERE/_ref"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
if [ ! -d "$REF/dnn" ]; then
    echo "ref_build.sh: $REF/dnn not found, nothing to build" >&2
    exit 0
fi
mkdir -p "$OUT"
if [ -f "$OUT/libdnn_ref.so" ] && [ "$OUT/libdnn_ref.so" -nt "$HERE/ref_wrap.cu" ]; then
    exit 0
fi
SRCS=(
    "$REF/dnn/core/tensor.cu" "$REF/dnn/core/tensor_transpose.cu" "$REF/dnn/core/cuda.cu" "$REF/dnn/core/device.cu"
    "$REF/dnn/layers/fully_connected_layer.cu" "$REF/dnn/layers/softmax_layer.cu" "$REF/dnn/layers/layer_norm_layer.cu"
    "$REF/dnn/tokens/token_embedding.cu" "$REF/dnn/tokens/positional_encoding.cu" "$REF/dnn/losses/cross_entropy.cu"
    "$REF/dnn/utils/convert.cu" "$REF/dnn/utils/scalar.cu" "$REF/dnn/utils/infinity.cu"
    "$HERE/ref_wrap.cu"
)
"$NVCC" -std=c++17 -O2 -gencode arch=compute_100a,code=sm_100a -rdc=true -shared -Xcompiler -fPIC -w \
    -I"$REF" -o "$OUT/libdnn_ref.so" "${SRCS[@]}" -lcurand
echo "built $OUT/libdnn_ref.so"
