"""etx-megakernel_b200: ETX's decode megakernel, rebuilt for NVIDIA B200 (sm_100a).

The directory name carries a hyphen, so the importable module name is `etx_megakernel_b200` (the loader module of
that name at the repository root registers this directory under it).  Sub-packages mirror the reference's layout for
the decode hot path: ir, frontends, machine, passes, importer, ops, models, runtime (C-ABI session), api, sim.

`install_as_etx()` additionally registers the package as `etx`, so a graph-building module written against the
reference (`from etx.ir import Graph`, `from etx.frontends import hip_link`, `from etx.importer import argblock`) imports
unchanged.
"""
from __future__ import annotations

import importlib
import sys

__version__ = "0.1.0"
_SUBPACKAGES = ("ir", "frontends", "machine", "passes", "importer", "ops", "models", "runtime", "api", "sim", "operators", "external")


def install_as_etx() -> None:
    """Make `import etx.<sub>` resolve to this package's sub-packages (refuses to shadow a real `etx` already imported)."""
    me = sys.modules[__name__]
    cur = sys.modules.get("etx")
    if cur is not None and cur is not me:
        raise ImportError("a different `etx` package is already imported")
    sys.modules["etx"] = me
    for sub in _SUBPACKAGES:
        try:
            sys.modules[f"etx.{sub}"] = importlib.import_module(f"{__name__}.{sub}")
        except ModuleNotFoundError:
            pass
