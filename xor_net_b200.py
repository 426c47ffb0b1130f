"""Import shim: ``import xor_net_b200`` loads the package directory ``xor-net_b200/``.

The package directory carries the project's hyphenated name, which is not a Python identifier;
this module registers it under an importable name.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "xor-net_b200")
_spec = importlib.util.spec_from_file_location(
    "xor_net_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["xor_net_b200"] = _mod
_spec.loader.exec_module(_mod)
