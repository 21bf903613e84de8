#!/bin/bash
# Builds the reference's expert-parallel extension (contrib/nccl_ep) from a copy of the reference tree and the small
# client baseline/ref_ep_bench.cu against it. Needs the core reference library already built into
# baseline/_ref/build (see the design record). Output: baseline/_ref/ep/{libnccl_ep.so*, ref_ep_bench}.
#   baseline/build_ref_ep.sh [reference-tree]     (default: the directory "reference" next to this repository)
set -e
ROOT=$(cd "$(dirname "$0")/.." && pwd)
REF=${1:-$(dirname "$ROOT")/reference}
WORK=$(mktemp -d)
mkdir -p "$WORK/contrib" "$ROOT/baseline/_ref/ep"
cp -r "$REF/makefiles" "$WORK/"
cp -r "$REF/contrib/nccl_ep" "$WORK/contrib/"
make -C "$WORK/contrib/nccl_ep" -j8 lib NCCL_HOME="$ROOT/baseline/_ref/build" NCCL_EP_BUILDDIR="$WORK/out" \
     NVCC_GENCODE="-gencode=arch=compute_100,code=sm_100"
cp -a "$WORK"/out/lib/libnccl_ep.so* "$ROOT/baseline/_ref/ep/"
nvcc -std=c++17 -O2 -gencode arch=compute_100,code=sm_100 -I"$WORK/out/include" -I"$ROOT/baseline/_ref/build/include" \
     "$ROOT/baseline/ref_ep_bench.cu" -o "$ROOT/baseline/_ref/ep/ref_ep_bench" \
     -L"$ROOT/baseline/_ref/ep" -lnccl_ep -L"$ROOT/baseline/_ref/build/lib" -lnccl -L/usr/local/cuda/lib64/stubs -lcuda \
     -Xlinker -rpath -Xlinker '$ORIGIN' -Xlinker -rpath -Xlinker '$ORIGIN/../build/lib'
rm -rf "$WORK"
echo built "$ROOT/baseline/_ref/ep/ref_ep_bench"
