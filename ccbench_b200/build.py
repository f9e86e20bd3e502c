"""Builds every native artefact of the repository (in-tree)."""
from __future__ import annotations


def build_all(verbose: bool = False) -> None:
    from ._lib import build_native

    build_native(verbose=verbose)
    try:
        from .native_build import build_c_targets
    except ImportError:
        return
    build_c_targets(verbose=verbose)
    # what the reference's compile_all.sh also leaves behind: the metric override library
    from .wrapper_build import register_metrics

    register_metrics(verbose=verbose)
