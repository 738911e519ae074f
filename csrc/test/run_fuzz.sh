#!/usr/bin/env bash
# Builds the mutation fuzzer with AddressSanitizer + UBSan and runs it: run_fuzz.sh [seconds-per-seed=20] [seeds=3].
# A failure aborts with the offending input printed as hex. Counterpart of the reference's script/run_fuzz.sh.
set -euo pipefail
cd "$(dirname "${BASH_SOURCE[0]}")/../.."
SECONDS_PER_SEED="${1:-20}"
SEEDS="${2:-3}"
make -j"$(nproc)" fuzz
for seed in $(seq 1 "$SEEDS"); do
    ASAN_OPTIONS=detect_leaks=0:protect_shadow_gap=0 UBSAN_OPTIONS=halt_on_error=1 ./build/asan/mf_fuzz "$SECONDS_PER_SEED" "$seed"
done
