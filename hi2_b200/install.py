"""Make an unmodified hi2 checkout call the B200 kernels.

hi2 binds ``hi2.hessian``, ``hi2.encode``, ``hi2.ladder_kernel``, ``hi2.gptq_kernel``,
``hi2.refine_kernel`` (and ``hi2.refine``, ``hi2.stats``) at import time (``from .encode import encode_rows`` in hi2/calibrate.py:17,
``from . import ladder_kernel`` in hi2/encode.py:15, ...), so the replacements have to be in
``sys.modules`` under those names BEFORE ``hi2.calibrate`` / ``hi2.pipeline`` are imported:

    import hi2_b200.install as inst
    inst.install()            # needs hi2 importable
    from hi2 import pipeline  # now runs tabulate / encode on the B200 kernels

The rotation and packing functions of ``hi2.format`` are patched in place (the rest of that
module, the decoder side, stays hi2's own).
"""

from __future__ import annotations

import importlib
import sys

REPLACED = ("hessian", "encode", "ladder_kernel", "gptq_kernel", "refine_kernel", "refine", "stats")
PATCHED_FORMAT = ("fwht_groups", "pack_codes", "assemble")


def install(package: str = "hi2") -> list[str]:
    """Register the replacements; returns the module names that were put in place."""
    late = [f"{package}.{m}" for m in ("calibrate", "pipeline", "layerwise") if f"{package}.{m}" in sys.modules]
    if late:
        raise RuntimeError(f"install() must run before {', '.join(late)} is imported")
    importlib.import_module(package)  # the package itself (its __init__ imports nothing heavy)
    done = []
    for name in REPLACED:
        mod = importlib.import_module(f"hi2_b200.{name}")
        sys.modules[f"{package}.{name}"] = mod
        setattr(sys.modules[package], name, mod)
        done.append(f"{package}.{name}")
    ours = importlib.import_module("hi2_b200.format")
    theirs = importlib.import_module(f"{package}.format")
    for fn in PATCHED_FORMAT:
        setattr(theirs, fn, getattr(ours, fn))
        done.append(f"{package}.format.{fn}")
    return done
