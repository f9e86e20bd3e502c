#!/usr/bin/env bash
# Build the benchmark drivers and the core library (the reference's script of this name takes the
# architecture as its argument; every architecture of this repository is built in one go).
# Thin entry point with the reference's script name; the work is done by the Python CLI.
cd "$(dirname "$0")/../.." || exit 1
exec python3 -m ccbench_b200.cli compile-all
