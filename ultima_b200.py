"""Import name for the package that lives in the folder ``ultima.cpp_b200``.

A folder whose name holds a dot cannot be imported by that name, so this module
loads the folder as the package ``ultima_b200`` and puts it in its own place in
``sys.modules``; ``import ultima_b200.engine`` then works as for any package.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ultima.cpp_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
