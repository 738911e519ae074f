#!/usr/bin/env bash
# Packs a release: builds, then writes output/memfabric_hybrid_b200-<version>-<arch>.tar.gz with
#   lib/            libmf_core.so
#   include/        public C headers and the device header
#   python/         the Python package (with its extension module)
#   examples/ benchmarks/   sources and the built tools
#   install.sh      copies the tree under a prefix (default /usr/local/memfabric_hybrid_b200) and prints the environment to set
# and, when the `wheel` package is importable, a wheel next to it. Counterpart of the reference's
# script/build_and_pack_run.sh + script/run_pkg_maker (a self-installing package of libraries, headers, wheel and tools).
set -euo pipefail
ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
cd "$ROOT"
./build.sh
VERSION="$(python -c 'import memfabric_hybrid_b200 as mf; print(mf.version().split()[1])' 2>/dev/null || echo 0.0.0)"
ARCH="$(uname -m)"
NAME="memfabric_hybrid_b200-${VERSION}-${ARCH}"
OUT="$ROOT/output"
STAGE="$OUT/$NAME"
rm -rf "$STAGE"
mkdir -p "$STAGE/lib" "$STAGE/include" "$STAGE/python" "$STAGE/examples" "$STAGE/benchmarks"
cp memfabric_hybrid_b200/lib/libmf_core.so "$STAGE/lib/"
cp -r include/mf "$STAGE/include/"
rsync -a --exclude '__pycache__' memfabric_hybrid_b200 memfabric_hybrid mf_adapter "$STAGE/python/" 2>/dev/null || cp -r memfabric_hybrid_b200 memfabric_hybrid mf_adapter "$STAGE/python/"
cp -r include/mf "$STAGE/python/memfabric_hybrid_b200/include" 2>/dev/null || { mkdir -p "$STAGE/python/memfabric_hybrid_b200/include"; cp -r include/mf "$STAGE/python/memfabric_hybrid_b200/include/"; }
cp -r examples/. "$STAGE/examples/"
cp benchmarks/*.py benchmarks/*.cpp "$STAGE/benchmarks/"
[ -x benchmarks/store_bench ] && cp benchmarks/store_bench "$STAGE/benchmarks/"
cat > "$STAGE/install.sh" <<'INSTALL'
#!/usr/bin/env bash
set -euo pipefail
PREFIX="${1:-/usr/local/memfabric_hybrid_b200}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
mkdir -p "$PREFIX"
cp -r "$HERE/lib" "$HERE/include" "$HERE/python" "$HERE/examples" "$HERE/benchmarks" "$PREFIX/"
echo "installed under $PREFIX; set:"
echo "  export PYTHONPATH=$PREFIX/python:\$PYTHONPATH"
echo "  export LD_LIBRARY_PATH=$PREFIX/lib:\$LD_LIBRARY_PATH"
echo "  export CPATH=$PREFIX/include:\$CPATH"
INSTALL
chmod +x "$STAGE/install.sh"
tar -C "$OUT" -czf "$OUT/$NAME.tar.gz" "$NAME"
echo "packed $OUT/$NAME.tar.gz"
if python -c 'import wheel' 2>/dev/null; then
    python setup.py -q bdist_wheel -d "$OUT" >/dev/null 2>&1 && echo "wheel in $OUT" || echo "wheel build skipped (setup.py bdist_wheel failed)"
fi
