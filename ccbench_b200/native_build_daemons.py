"""Builds bin/daemons/daemon_<name> from userconfig/daemon_code_examples (every
daemon_*.c there is one daemon, as with the reference's scripts/register_daemons.sh),
the shared helper, and the sm_100a burn kernel for the GPU stress daemon."""
from __future__ import annotations

from . import native_build as nb


def daemon_names():
    d = nb.ROOT / "userconfig" / "daemon_code_examples"
    return sorted(p.stem[len("daemon_"):] for p in d.glob("daemon_*.c"))


def build(verbose: bool = False, only=None) -> None:
    root = nb.ROOT
    helper = root / "csrc/daemons/daemon_helper.c"
    src_dir = root / "userconfig/daemon_code_examples"
    out_dir = nb.BIN / "daemons"
    for name in daemon_names():
        if only and name not in only:
            continue
        src = src_dir / f"daemon_{name}.c"
        out = out_dir / f"daemon_{name}"
        if name == "stress_gpu_nvidia":
            cu = root / "csrc/daemons/daemon_gpu_burn_kernel.cu"
            obj = root / "build/obj/daemon_gpu_burn_kernel.o"
            if nb._newer(obj, [cu]):
                obj.parent.mkdir(parents=True, exist_ok=True)
                nb._run(["nvcc", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
                         f"-I{root / 'include/ccb/compat'}", "-c", cu, "-o", obj], verbose)
            nb.cc(out, [src, helper, obj], extra=[f"-I{src_dir}"],
                  libs=[*nb.cuda_libs(), "-lstdc++", "-lpthread", "-lm", "-ldl"], verbose=verbose)
        else:
            nb.cc(out, [src, helper], extra=[f"-I{src_dir}"], libs=["-lpthread", "-lm", "-ldl"], verbose=verbose)
