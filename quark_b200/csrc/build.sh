#!/bin/bash
# Builds libquark_b200.so (sm_100a only) next to the Python package.  Usage: build.sh [-v]
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/../libquark_b200.so"
NVCC="${NVCC:-nvcc}"
FLAGS="-gencode arch=compute_100a,code=sm_100a -lineinfo -O3 -std=c++17 -Xcompiler -fPIC"
[ "$1" = "-v" ] && FLAGS="$FLAGS -Xptxas -v"
mkdir -p "$HERE/build"
pids=()
for f in runtime gemm attn attn4 kv glue qkv_post tp; do
  $NVCC $FLAGS -c "$HERE/$f.cu" -o "$HERE/build/$f.o" &
  pids+=($!)
done
for p in "${pids[@]}"; do wait $p; done
$NVCC -shared -o "$OUT" "$HERE"/build/{runtime,gemm,attn,attn4,kv,glue,qkv_post,tp}.o -cudart static
echo "built $OUT"
