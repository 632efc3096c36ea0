"""Import shim: the package directory carries the project's hyphenated name, which Python cannot
import directly; ``import cdssm_b200`` loads it under this name."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cayley-delta-state-space-model_b200")
_spec = importlib.util.spec_from_file_location(
    "cdssm_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["cdssm_b200"] = _mod
_spec.loader.exec_module(_mod)
