#!/usr/bin/env bash
# Builds lib/libmllm_b200.so (CUDA kernels + C ABI) for sm_100a, in tree.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
OUT="$HERE/lib"
mkdir -p "$OUT"
SRC=("$HERE"/csrc/host_pack.cpp "$HERE"/csrc/c_api.cu "$HERE"/csrc/repack.cu "$HERE"/csrc/act_quant.cu
     "$HERE"/csrc/gemv.cu "$HERE"/csrc/gemv_stream.cu "$HERE"/csrc/gemm_stream.cu "$HERE"/csrc/gemm_simt.cu "$HERE"/csrc/gemm_tc.cu "$HERE"/csrc/gemm_tcf16.cu
     "$HERE"/csrc/decoder_kernels.cu "$HERE"/csrc/decoder_attn.cu "$HERE"/csrc/decoder.cu "$HERE"/csrc/decoder_batch.cu "$HERE"/csrc/decoder_persistent.cu "$HERE"/csrc/conv3d.cu
     "$HERE"/csrc/host_pack_a16.cpp "$HERE"/csrc/w4a16.cu "$HERE"/csrc/c_api_a16.cu "$HERE"/csrc/tp.cu)
EXTRA=()
[ -f "$HERE/csrc/no_alloc.cu" ] && SRC+=("$HERE/csrc/no_alloc.cu")
"$NVCC" -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -lineinfo -rdc=true \
  -Xcompiler -fPIC,-fvisibility=hidden,-O3 ${PTXAS_V:+-Xptxas -v} \
  -shared -o "$OUT/libmllm_b200.so" "${SRC[@]}" "${EXTRA[@]}" -ldl
echo "built $OUT/libmllm_b200.so"
