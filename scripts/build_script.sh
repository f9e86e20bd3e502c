#!/usr/bin/env bash
# Build the configured wrappers and generate scripts/run/run_benchmark.*  (--rebuild-bench: also every native artefact)
# Thin entry point with the reference's script name; the work is done by the Python CLI.
cd "$(dirname "$0")/.." || exit 1
exec python3 -m ccbench_b200.cli build "$@"
