"""Import alias: `import lancet_b200` loads the package whose directory name (the repository
name with a `_b200` suffix) is not a valid Python identifier."""
import importlib.util
import os
import sys

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)),
                    "lancet-accelerating-moe-training-via-whole-graph-computation-communication-overlapping_b200")
_spec = importlib.util.spec_from_file_location("lancet_b200", os.path.join(_DIR, "__init__.py"),
                                               submodule_search_locations=[_DIR])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["lancet_b200"] = _mod
_spec.loader.exec_module(_mod)
