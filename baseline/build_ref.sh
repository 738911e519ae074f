#!/usr/bin/env bash
# Builds the reference's C++ control plane (config store, group engine, TCP links) UNMODIFIED, without its Python package and
# without a device back end, and then baseline/ref_store_bench.cpp against it. Output: baseline/_ref/cpp/{lib*.so,ref_store_bench}.
# The reference tree is read-only, so the build runs on a copy.
#
#   baseline/build_ref.sh [reference-dir] [work-dir]
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${1:-/root/reference}"
WORK="${2:-/tmp/mf_refbuild}"
OUT="$HERE/_ref/cpp"
mkdir -p "$WORK" "$OUT"
if [ ! -d "$WORK/src" ]; then
    cp -r "$REF" "$WORK/src"
fi
cmake -S "$WORK/src" -B "$WORK/build" -DCMAKE_BUILD_TYPE=Release -DBUILD_PYTHON=OFF -DXPU_TYPE=NONE -DBUILD_HCOM=OFF \
      -DBUILD_TEST=OFF -DBUILD_UT=OFF > "$WORK/cmake.log" 2>&1
make -C "$WORK/build" -j"$(nproc)" smem_shared hybmm_shared acc_tcp_net_shared > "$WORK/make.log" 2>&1
cp "$WORK/build/src/smem/csrc/libmf_smem.so" "$WORK/build/src/hybm/csrc/libmf_hybm_core.so" \
   "$WORK/build/src/acc_links/csrc/libacc_tcp_net.so" "$OUT/"
S="$WORK/src/src"
INC=$(find "$S/smem/csrc" "$S/smem/include" "$S/util/csrc" "$S/acc_links/include" "$S/hybm/include" -type d | sed 's/^/-I/' | tr '\n' ' ')
# shellcheck disable=SC2086
g++ -std=c++17 -O2 $INC -o "$OUT/ref_store_bench" "$HERE/ref_store_bench.cpp" -L"$OUT" -lmf_smem -Wl,-rpath,'$ORIGIN' -pthread
echo "built $OUT/ref_store_bench"
