"""Import shim: the package directory is named ``comfy-kitchen_b200`` (not a valid identifier), so this
module loads it under the importable name ``comfy_kitchen_b200`` and replaces itself with it."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "comfy-kitchen_b200")
_spec = importlib.util.spec_from_file_location(
    "comfy_kitchen_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["comfy_kitchen_b200"] = _mod
_spec.loader.exec_module(_mod)
