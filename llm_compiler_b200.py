"""Import alias: the package directory is `llm-compiler_b200/` (not a valid Python
identifier), so `import llm_compiler_b200` loads it from there."""

import importlib.util
import sys
from pathlib import Path

_directory = Path(__file__).resolve().parent / "llm-compiler_b200"
_spec = importlib.util.spec_from_file_location(
    "llm_compiler_b200", _directory / "__init__.py", submodule_search_locations=[str(_directory)])
_module = importlib.util.module_from_spec(_spec)
sys.modules["llm_compiler_b200"] = _module
_spec.loader.exec_module(_module)
