"""Import shim: makes ``import blackwell_moe_b200`` load the package that lives
in the ``blackwell-moe_b200/`` directory (a hyphen is not importable)."""

import importlib.util
import sys
from pathlib import Path

_dir = Path(__file__).resolve().parent / "blackwell-moe_b200"
_spec = importlib.util.spec_from_file_location(
    "blackwell_moe_b200", _dir / "__init__.py", submodule_search_locations=[str(_dir)])
_pkg = importlib.util.module_from_spec(_spec)
sys.modules["blackwell_moe_b200"] = _pkg
_spec.loader.exec_module(_pkg)
