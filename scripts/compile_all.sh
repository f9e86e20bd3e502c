#!/usr/bin/env bash
# Build every native artefact (core, drivers, libraries, daemons, tools, metric registry)
# Thin entry point with the reference's script name; the work is done by the Python CLI.
cd "$(dirname "$0")/.." || exit 1
exec python3 -m ccbench_b200.cli compile-all "$@"
