"""Import shim: the package directory is named ``flash-llm_b200`` (not a valid Python identifier), so
``import flash_llm_b200`` loads it from there under this importable name."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "flash-llm_b200")
_spec = importlib.util.spec_from_file_location(
    "flash_llm_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_module = importlib.util.module_from_spec(_spec)
sys.modules["flash_llm_b200"] = _module
_spec.loader.exec_module(_module)
