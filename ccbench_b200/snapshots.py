"""Configuration snapshots: env_saves/<name>/{configs/, metadata.json, DESCRIPTION.md}
with metadata {snapshot_level, timestamp, git_commit, description}, the layout of the
reference's scripts/manage_snapshots.sh:82-449 (list / save / load / compare / show /
delete). The levels that script documents but never writes are implemented here:
"summary" adds effective_config.json (the merged configuration), "full" also adds
metadata.runtime.json (host description)."""
from __future__ import annotations

import difflib
import json
import shutil
import subprocess
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _git_commit() -> str:
    try:
        return subprocess.run(["git", "rev-parse", "--short", "HEAD"], cwd=ROOT, capture_output=True, text=True, timeout=5).stdout.strip()
    except Exception:
        return ""


def save(name, config_dir, save_dir="env_saves", level="light", description="") -> Path:
    name = name or time.strftime("snapshot_%Y%m%d_%H%M%S")
    dst = ROOT / save_dir / name
    if dst.exists():
        raise FileExistsError(f"snapshot {name} exists")
    (dst / "configs").mkdir(parents=True)
    for f in sorted(Path(config_dir).glob("*.jsonc")):
        shutil.copy2(f, dst / "configs" / f.name)
    meta = {"snapshot_level": level, "timestamp": time.strftime("%Y-%m-%dT%H:%M:%S"), "git_commit": _git_commit(),
            "description": description}
    (dst / "metadata.json").write_text(json.dumps(meta, indent=2) + "\n")
    (dst / "DESCRIPTION.md").write_text(f"# {name}\n\n{description or '(no description)'}\n")
    if level in ("summary", "full"):
        from .config import load_config

        cfg = load_config(config_dir)
        (dst / "effective_config.json").write_text(json.dumps(cfg.raw, indent=2, sort_keys=True) + "\n")
    if level == "full":
        from .utils import detect_env

        (dst / "metadata.runtime.json").write_text(json.dumps(detect_env.detect(), indent=2) + "\n")
    return dst


def list_snapshots(save_dir="env_saves"):
    base = ROOT / save_dir
    out = []
    for d in sorted(base.glob("*/metadata.json")) if base.exists() else []:
        out.append((d.parent.name, json.loads(d.read_text())))
    return out


def load(name, config_dir, save_dir="env_saves") -> None:
    src = ROOT / save_dir / name / "configs"
    if not src.is_dir():
        raise FileNotFoundError(f"no snapshot {name}")
    for f in src.glob("*.jsonc"):
        shutil.copy2(f, Path(config_dir) / f.name)


def compare(a, b, save_dir="env_saves", config_dir=None) -> str:
    def files(n):
        base = Path(config_dir) if n == "current" and config_dir else ROOT / save_dir / n / "configs"
        return {f.name: f.read_text().splitlines() for f in sorted(base.glob("*.jsonc"))}

    fa, fb = files(a), files(b)
    out = []
    for name in sorted(set(fa) | set(fb)):
        out += list(difflib.unified_diff(fa.get(name, []), fb.get(name, []), f"{a}/{name}", f"{b}/{name}", lineterm=""))
    return "\n".join(out)


def delete(name, save_dir="env_saves") -> None:
    target = ROOT / save_dir / name
    if not (target / "metadata.json").exists():
        raise FileNotFoundError(f"no snapshot {name}")
    shutil.rmtree(target)


def main(action, names, config_dir, message="", level=None, save_dir="env_saves") -> int:
    if action == "list":
        for n, m in list_snapshots(save_dir):
            print(f"{n:32s} {m.get('timestamp', ''):20s} {m.get('snapshot_level', ''):8s} {m.get('description', '')}")
    elif action == "save":
        print(save(names[0] if names else None, config_dir, save_dir, level or "light", message))
    elif action == "load":
        load(names[0], config_dir, save_dir)
    elif action == "compare":
        print(compare(names[0], names[1] if len(names) > 1 else "current", save_dir, config_dir))
    elif action == "show":
        d = ROOT / save_dir / names[0]
        print((d / "metadata.json").read_text())
        print((d / "DESCRIPTION.md").read_text())
    elif action == "delete":
        delete(names[0], save_dir)
    return 0
