from . import ops
from .library import KernelError, lib
