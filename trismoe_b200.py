"""Import alias: ``import trismoe_b200`` loads the package directory
``neurips26-tris-moe_b200/`` (whose name is not a valid Python identifier)."""
import importlib
import os
import sys

_root = os.path.dirname(os.path.abspath(__file__))
if _root not in sys.path:
    sys.path.insert(0, _root)
_pkg = importlib.import_module("neurips26-tris-moe_b200")
sys.modules[__name__] = _pkg
for _name in ("_native", "formats", "qlinear_grouped", "moe_block", "synth", "staging", "sidecar", "expert_parallel", "clocks"):
    _mod = sys.modules.get(f"neurips26-tris-moe_b200.{_name}")
    if _mod is not None:
        sys.modules[f"{__name__}.{_name}"] = _mod
