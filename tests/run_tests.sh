#!/usr/bin/env bash
# Runs the test tiers: the native binary, the CPU tier of pytest, and with --gpu the GPU tier (needs at least one B200; cases
# that need more GPUs skip themselves). --asan runs the native tests from the sanitised build as well. Counterpart of the
# reference's script/run_ut.sh (build the tests, run them, fail on the first failing tier).
set -euo pipefail
cd "$(dirname "${BASH_SOURCE[0]}")/.."
GPU=0
ASAN=0
for a in "$@"; do
    case "$a" in
        --gpu) GPU=1 ;;
        --asan) ASAN=1 ;;
        *) echo "unknown option $a" >&2; exit 2 ;;
    esac
done
make -j"$(nproc)" all examples
./csrc/test/mf_native_tests
if [ "$ASAN" = 1 ]; then
    make -j"$(nproc)" asan
    ASAN_OPTIONS=detect_leaks=0:protect_shadow_gap=0 ./build/asan/mf_native_tests_asan
fi
python -m pytest tests -x -q -m "not gpu"
if [ "$GPU" = 1 ]; then
    python -m pytest tests -x -q -m gpu
fi
echo "all requested tiers passed"
