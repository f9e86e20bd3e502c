#!/usr/bin/env bash
# Environment-modules planner. SOURCE it:   . scripts/configure_modules.sh [--apply]
# Looks for what the build needs (nvcc, an MPI compiler, nccl.h / libnccl) and, on hosts with
# an environment-modules system, proposes the `module load` lines that would provide what is
# missing (newest match of cuda / nccl / openmpi|mpich / gcc in `module avail`); --apply
# runs them in the current shell. Without a modules system it only reports. Same purpose as
# the reference's interactive scripts/configure_modules.sh, without the prompts.
_ccb_apply=0
[ "$1" = "--apply" ] && _ccb_apply=1

_ccb_have() { command -v "$1" >/dev/null 2>&1; }
_ccb_need=()
_ccb_have nvcc || [ -x /usr/local/cuda/bin/nvcc ] || _ccb_need+=("cuda")
_ccb_have mpicc || _ccb_need+=("openmpi|mpich")
{ [ -f /usr/include/nccl.h ] || [ -n "$NCCL_HOME" ]; } || _ccb_need+=("nccl")
_ccb_have gcc || _ccb_need+=("gcc")

echo "[modules] nvcc:  $(command -v nvcc || echo /usr/local/cuda/bin/nvcc)"
echo "[modules] mpicc: $(command -v mpicc || echo 'none (the single-host MPI subset in csrc/minimpi is used)')"
echo "[modules] nccl:  $([ -f /usr/include/nccl.h ] && echo /usr/include/nccl.h || echo "${NCCL_HOME:-none}")"

if ! type module >/dev/null 2>&1; then
    echo "[modules] no environment-modules system on this host; nothing to load"
elif [ ${#_ccb_need[@]} -eq 0 ]; then
    echo "[modules] everything needed is already on PATH"
else
    _ccb_avail=$(module -t avail 2>&1)
    for _ccb_pat in "${_ccb_need[@]}"; do
        _ccb_pick=$(printf '%s\n' "$_ccb_avail" | grep -Ei "^(${_ccb_pat})(/|$)" | sort -V | tail -1)
        if [ -z "$_ccb_pick" ]; then
            echo "[modules] no module matches '${_ccb_pat}'"
        elif [ $_ccb_apply -eq 1 ]; then
            echo "[modules] module load $_ccb_pick"
            module load "$_ccb_pick"
        else
            echo "[modules] would run: module load $_ccb_pick   (re-source with --apply)"
        fi
    done
fi
unset _ccb_apply _ccb_need _ccb_avail _ccb_pat _ccb_pick
unset -f _ccb_have
