#!/bin/sh
# usage: build_ref.sh <reference-checkout>
# Compiles the reference's own CUDA kernels for the stages of the path, from the sources
# where they lie in the reference checkout, into _ref/ beside this script (git-ignored; the
# compiled files travel with the tree to wherever the GPU tests run).  Flags follow the
# reference's build scripts:
#   PTX modules : nvcc -ptx -arch=<sm> -O3 -lineinfo          (kernels/build.sh:72)
#   libfa_sm89  : nvcc -shared -arch=<sm> -O3 --use_fast_math  (kernels/build_fa_sm89_so.sh:13-15)
# Nothing is copied into the repository; only compiler outputs are written.
set -e
if [ -z "$1" ]; then
    echo "usage: $0 <reference-checkout>" >&2
    exit 2
fi
REF="$1"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
if [ ! -d "$REF/kernels" ]; then
    echo "reference checkout not found at $REF; keeping whatever is in $OUT" >&2
    exit 0
fi
mkdir -p "$OUT"
for f in kernels/fused_rmsnorm_fp8_quant.cu kernels/fused_silu_fp8_quant.cu kernels/argmax.cu \
         v3/kernels/fused_gelu_mul_fp8_quant.cu v3/kernels/fp8_channelscale_gemv_ktiled.cu \
         v3/kernels/fp8_channelscale_gemv_splitk.cu v3/kernels/f32_to_f16_sat.cu \
         v3/kernels/fused_rope_partial_fp8kv.cu v3/kernels/fused_rope_cache_fp8kv.cu \
         v3/kernels/fused_qkv_rmsnorm.cu v3/kernels/fused_norm_add_residual_f16.cu \
         v3/kernels/residual_scale_f16.cu v3/kernels/logit_softcap.cu kernels/fp8_gemv.cu \
         kernels/embedding_gather_f16.cu kernels/flash_attention.cu; do
    stem=$(basename "$f" .cu)
    if [ ! -f "$OUT/$stem.ptx" ] || [ "$REF/$f" -nt "$OUT/$stem.ptx" ]; then
        "$NVCC" -ptx -arch=sm_100 -O3 -lineinfo -ccbin /usr/bin/g++ "$REF/$f" -o "$OUT/$stem.ptx"
    fi
done
if [ ! -f "$OUT/libfa_sm89_ref.so" ] || [ "$REF/v3/kernels/fp8_decode_v2.cu" -nt "$OUT/libfa_sm89_ref.so" ]; then
    "$NVCC" -shared -arch=sm_100 -O3 --use_fast_math -ccbin /usr/bin/g++ -Xcompiler -fPIC -cudart static \
        "$REF/v3/kernels/fp8_decode_v2.cu" -o "$OUT/libfa_sm89_ref.so"
fi
ls "$OUT"
