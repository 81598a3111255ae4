"""Importable name of the library.

The source tree is the sibling folder ``tileinfer.jl_b200/`` (the name this library was asked to live
under); a dot cannot be part of a Python module name, so this package's search path points there:
``import tileinfer_b200.config`` loads ``tileinfer.jl_b200/config/__init__.py``. What that folder's
``__init__.py`` exports is imported below.
"""
import os as _os

__path__ = [_os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "tileinfer.jl_b200")]
__version__ = "0.2.0"

from .api import generate, generation_defaults, load_model            # noqa: E402
from .engine import Engine                                            # noqa: E402
from .sampling import SamplingParams                                  # noqa: E402
