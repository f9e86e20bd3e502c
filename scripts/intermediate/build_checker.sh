#!/usr/bin/env bash
# Check the configuration and say what cannot be used (missing files, modes without sources).
# Thin entry point with the reference's script name; the work is done by the Python CLI.
cd "$(dirname "$0")/../.." || exit 1
exec python3 -m ccbench_b200.cli gen-script "$@"
