#!/usr/bin/env bash
# Rebuild bin/libs/validation.so from userconfig/deviation_metric_examples/*.c
# Thin entry point with the reference's script name; the work is done by the Python CLI.
cd "$(dirname "$0")/.." || exit 1
exec python3 -m ccbench_b200.cli register-metrics "$@"
