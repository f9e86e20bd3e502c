#!/usr/bin/env bash
# Configuration snapshots: list | save [name] -m text | load name | compare a [b] | show name | delete name
# Thin entry point with the reference's script name; the work is done by the Python CLI.
cd "$(dirname "$0")/.." || exit 1
exec python3 -m ccbench_b200.cli snapshot "$@"
