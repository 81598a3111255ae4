"""tileinfer_b200: a small model library with generation of its own for one GPU (B200, sm_100a).

Everything between a request's tokens and its next token, for the Apertus architecture:
typed configuration and registry (``config``), safetensors weights (``weights``), layers
put together from parts (``parts``), a paged cache with a slot per sequence (``cache``), one
step function and a generation loop (``engine``), sampling (``sampling``) and hand-written
CUDA kernels (``csrc``, loaded by ``kernels``).
"""
__version__ = "0.2.0"

from .api import generate, generation_defaults, load_model            # noqa: E402
from .engine import Engine                                            # noqa: E402
from .sampling import SamplingParams                                  # noqa: E402
