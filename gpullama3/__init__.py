"""Import shim: the product lives in the folder ``gpullama3.java_b200`` at the repository root;
this package makes it importable as ``gpullama3.java_b200`` (a dotted folder name cannot be
imported directly)."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "gpullama3.java_b200")
_name = __name__ + ".java_b200"
if _name not in sys.modules:
    _spec = importlib.util.spec_from_file_location(_name, os.path.join(_dir, "__init__.py"),
                                                   submodule_search_locations=[_dir])
    _mod = importlib.util.module_from_spec(_spec)
    sys.modules[_name] = _mod
    _spec.loader.exec_module(_mod)
java_b200 = sys.modules[_name]
