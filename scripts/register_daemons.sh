#!/usr/bin/env bash
# Build bin/daemons/daemon_<name> for the selected daemons (--dry-run lists them)
# Thin entry point with the reference's script name; the work is done by the Python CLI.
cd "$(dirname "$0")/.." || exit 1
exec python3 -m ccbench_b200.cli register-daemons "$@"
