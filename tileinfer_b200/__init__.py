"""Importable name of the library.

The source tree lives in the sibling folder ``tileinfer.jl_b200/``; a dot cannot be part
of a Python module name, so this package points its search path there and runs that
folder's ``__init__.py`` in its own namespace. ``import tileinfer_b200.config`` therefore
loads ``tileinfer.jl_b200/config/__init__.py``.
"""
import os as _os

_SOURCE = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "tileinfer.jl_b200")
__path__ = [_SOURCE]
with open(_os.path.join(_SOURCE, "__init__.py")) as _f:
    exec(compile(_f.read(), _os.path.join(_SOURCE, "__init__.py"), "exec"))
del _f
