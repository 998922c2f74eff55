"""Import shim: the package directory is named ``torch-tpu_b200`` (not a Python identifier), so
``import torch_tpu_b200`` lands here and loads that directory as the package of the same name."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "torch-tpu_b200")
_spec = importlib.util.spec_from_file_location(
    "torch_tpu_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["torch_tpu_b200"] = _mod
_spec.loader.exec_module(_mod)
