#!/usr/bin/env bash
# Builds everything in-tree: the core library, the Python extension, the native test binary, the example and benchmark
# programs. Options: --asan also builds the sanitised native tests, --fuzz the sanitised fuzzer, --clean starts from scratch,
# -j N sets the parallelism. Counterpart of the reference's script/build.sh (one entry point for library, bindings and tools).
set -euo pipefail
cd "$(dirname "${BASH_SOURCE[0]}")"
JOBS="$(nproc)"
ASAN=0
FUZZ=0
CLEAN=0
while [ $# -gt 0 ]; do
    case "$1" in
        --asan) ASAN=1 ;;
        --fuzz) FUZZ=1 ;;
        --clean) CLEAN=1 ;;
        -j) shift; JOBS="$1" ;;
        -h|--help) sed -n 2,5p "$0"; exit 0 ;;
        *) echo "unknown option $1" >&2; exit 2 ;;
    esac
    shift
done
if [ "$CLEAN" = 1 ]; then
    make clean
fi
make -j"$JOBS" all examples
if [ "$ASAN" = 1 ]; then
    make -j"$JOBS" asan
fi
if [ "$FUZZ" = 1 ]; then
    make -j"$JOBS" fuzz
fi
python -c "import memfabric_hybrid_b200 as mf; print('built', mf.version())"
