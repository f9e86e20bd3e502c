"""Command line of the framework (what the reference spreads over scripts/*.sh):

    python -m ccbench_b200.cli build [--rebuild-bench]   wrappers (+ everything native) and the run script
    python -m ccbench_b200.cli gen-script                only regenerate scripts/run/run_benchmark.*
    python -m ccbench_b200.cli compile-all               every native artefact
    python -m ccbench_b200.cli register-metrics          bin/libs/validation.so from userconfig/deviation_metric_examples
    python -m ccbench_b200.cli register-daemons [--dry-run]
    python -m ccbench_b200.cli register-mapper           bin/libs/libjob_device_mapper.so
    python -m ccbench_b200.cli snapshot {list,save,load,compare,show,delete} ...
    python -m ccbench_b200.cli detect-env                JSON description of this host
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="ccbench_b200")
    ap.add_argument("--config-dir", default=str(ROOT / "userconfig/config_in_jsonc"))
    sub = ap.add_subparsers(dest="cmd", required=True)
    b = sub.add_parser("build")
    b.add_argument("--rebuild-bench", action="store_true")
    b.add_argument("-v", "--verbose", action="store_true")
    sub.add_parser("gen-script")
    c = sub.add_parser("compile-all")
    c.add_argument("-v", "--verbose", action="store_true")
    sub.add_parser("register-metrics")
    rd = sub.add_parser("register-daemons")
    rd.add_argument("--dry-run", action="store_true")
    sub.add_parser("register-mapper")
    sub.add_parser("detect-env")
    sn = sub.add_parser("snapshot")
    sn.add_argument("action", choices=["list", "save", "load", "compare", "show", "delete"])
    sn.add_argument("names", nargs="*")
    sn.add_argument("-m", "--message", default="")
    sn.add_argument("--level", default=None)
    a = ap.parse_args(argv)

    from .config import load_config

    if a.cmd in ("build", "gen-script"):
        from . import runscript, wrapper_build

        cfg = load_config(a.config_dir)
        wrong = cfg.problems(ROOT)
        if wrong:
            print("[build_script] the configuration cannot be used:", file=sys.stderr)
            for w in wrong:
                print("  - " + w, file=sys.stderr)
            return 2
        if a.cmd == "build":
            if a.rebuild_bench:
                from .native_build import build_c_targets

                build_c_targets(verbose=a.verbose)
                wrapper_build.register_metrics(verbose=a.verbose)
            wrapper_build.build_wrappers(cfg, verbose=a.verbose)
        path = runscript.write(cfg, ROOT)
        print(f"[build_script] generated {path}")
        if cfg.snapshot_level != "off":
            from . import snapshots

            snapshots.save(None, a.config_dir, cfg.snapshot_dir, level=cfg.snapshot_level, description="auto snapshot at build")
        return 0
    if a.cmd == "compile-all":
        from .native_build import build_c_targets
        from . import wrapper_build

        build_c_targets(verbose=a.verbose)
        wrapper_build.register_metrics(verbose=a.verbose)
        return 0
    if a.cmd == "register-metrics":
        from . import wrapper_build

        print(wrapper_build.register_metrics(verbose=True))
        return 0
    if a.cmd == "register-daemons":
        from . import native_build_daemons as nd

        cfg = load_config(a.config_dir)
        names = [n for n in nd.daemon_names() if not cfg.selected_daemons or n in cfg.selected_daemons]
        if a.dry_run:
            print("would build:", ", ".join(f"bin/daemons/daemon_{n}" for n in names))
            return 0
        nd.build(verbose=True, only=names)
        return 0
    if a.cmd == "register-mapper":
        from . import native_build_mapper as nm

        cfg = load_config(a.config_dir)
        print(nm.build(selected=cfg.selected_daemons, verbose=True))
        return 0
    if a.cmd == "detect-env":
        from .utils import detect_env

        print(json.dumps(detect_env.detect(), indent=2))
        return 0
    if a.cmd == "snapshot":
        from . import snapshots

        return snapshots.main(a.action, a.names, a.config_dir, message=a.message, level=a.level)
    return 1


if __name__ == "__main__":
    sys.exit(main())
