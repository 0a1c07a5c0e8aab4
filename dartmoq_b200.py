"""Import shim: ``import dartmoq_b200`` loads the package kept in ``dartmoq-qwen3.5_b200/``.

The package directory carries the project's name, which is not a valid Python
identifier; this module registers it under an importable alias.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dartmoq-qwen3.5_b200")
_spec = importlib.util.spec_from_file_location(
    "dartmoq_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["dartmoq_b200"] = _mod
_spec.loader.exec_module(_mod)
