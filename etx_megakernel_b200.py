"""Import alias: the package directory is `etx-megakernel_b200/` (a hyphen cannot be imported), so this module loads it
and registers it in sys.modules under `etx_megakernel_b200`."""
import importlib.util
import sys
from pathlib import Path

_dir = Path(__file__).resolve().parent / "etx-megakernel_b200"
_spec = importlib.util.spec_from_file_location(__name__, _dir / "__init__.py", submodule_search_locations=[str(_dir)])
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
