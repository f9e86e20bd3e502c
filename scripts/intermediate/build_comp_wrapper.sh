#!/usr/bin/env bash
# Build the wrappers that the selection files under userconfig/config_in_jsonc describe
# (modes 2 and 3; the three kinds are built together) and regenerate the run script.
# Thin entry point with the reference's script name; the work is done by the Python CLI.
cd "$(dirname "$0")/../.." || exit 1
exec python3 -m ccbench_b200.cli build "$@"
