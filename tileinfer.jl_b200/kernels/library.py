"""Loads the compiled kernel library and declares its C entry points.

There is no fallback: if the library cannot be built or loaded, importing the kernels
raises with the reason.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_longlong, c_uint, c_void_p

from . import build as _build

_lib = None
# Number of kernels launched through this module so far (a launch inside a CUDA-graph capture counts
# once; its replays are counted by whoever replays the graph).
launch_count = 0
pinned_stream = None          # the stream handle for the launches of a forward pass (see ``stream_scope``)
call_counts = {}              # entry point -> calls that launched (tests read which kernels a step used)


class _Counted:
    """A C entry point that launches ``kernels`` kernels per call; a call that refuses its sizes
    (return code 2) has launched none."""
    __slots__ = ("fn", "kernels", "name")

    def __init__(self, fn, name, kernels=1):
        self.fn, self.name, self.kernels = fn, name, kernels

    def __call__(self, *args):
        global launch_count
        rc = self.fn(*args)
        if rc != 2:
            launch_count += self.kernels
            call_counts[self.name] = call_counts.get(self.name, 0) + 1
        return rc


def current_stream() -> int:
    """The CUDA stream the next launch goes to: the one pinned for the running forward pass, else torch's
    current stream (looking that up costs more than a launch, so a pass looks it up once)."""
    if pinned_stream is not None:
        return pinned_stream
    import torch
    return torch.cuda.current_stream().cuda_stream


class stream_scope:
    """Pins torch's current stream for the launches made inside (a forward pass makes hundreds)."""

    def __enter__(self):
        global pinned_stream
        import torch
        self.before = pinned_stream
        pinned_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global pinned_stream
        pinned_stream = self.before
        return False


def add_launches(n: int) -> None:
    global launch_count
    launch_count += n


class KernelError(RuntimeError):
    pass


_P, _I, _L, _F, _U = c_void_p, c_int, c_longlong, c_float, c_uint
_SIGNATURES = {
    "ti_embed": [_P, _P, _P, _I, _I, _I, _I, _P, _P],
    "ti_gather_rows": [_P, _P, _P, _I, _I, _I, _P],
    "ti_xielu": [_P, _P, _L, _F, _F, _F, _F, _I, _P],
    "ti_rmsnorm": [_P, _P, _P, _I, _I, _F, _I, _P],
    "ti_add_rmsnorm": [_P, _P, _P, _I, _L, _P, _P, _I, _I, _F, _I, _P],
    "ti_add": [_P, _P, _L, _I, _P],
    "ti_attention_inputs": [_P, _L, _P, _I, _L, _P, _P, _P, _P, _P, _F, _P, _I, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "ti_attention_plain": [_P, _P, _P, _P, _P, _I, _P, _P, _F, _I, _I, _I, _I, _I, _I, _I, _P],
    "ti_gemm_plain": [_P, _L, _P, _L, _P, _I, _I, _I, _I, _F, _F, _F, _F, _I, _P],
    "ti_argmax": [_P, _L, _I, _I, _P, _P, _P, _P, _P, _P],
    "ti_sample": [_P, _L, _I, _I, _F, _I, _F, _P, _P, _P, _P, _P],
    "ti_sample_shared": [_P, _L, _I, _I, _F, _I, _F, _P, _P, _P, _P, _I, _P],
    "ti_random_normal": [_P, _I, _L, _L, _U, _U, _F, _F, _P],
    "ti_wait_probe": [_P, _I, _I, _P, _P],
}


def lib():
    """The loaded library (built at the first call if the sources changed)."""
    global _lib
    if _lib is not None:
        return _lib
    try:
        path = _build.build()
        handle = ctypes.CDLL(path)
    except Exception as e:                      # BuildError, OSError
        raise KernelError(f"tileinfer_b200 cannot run without its CUDA kernel library: {e}") from e
    handle.ti_last_error.restype = c_char_p
    handle.ti_last_error.argtypes = []
    handle.ti_sampling_uniform.restype = c_float
    handle.ti_sampling_uniform.argtypes = [_U, _U]
    handle.ti_argmax_chunks.restype = c_int
    handle.ti_argmax_chunks.argtypes = [c_int]
    handle.ti_gemm_tcgen05_decode_plan.restype = c_int
    handle.ti_gemm_tcgen05_decode_plan.argtypes = [c_int] * 5 + [ctypes.POINTER(c_int)] * 2
    class _Lib:
        pass
    wrapped = _Lib()
    wrapped.ti_last_error = handle.ti_last_error
    wrapped.ti_sampling_uniform = handle.ti_sampling_uniform
    wrapped.ti_argmax_chunks = handle.ti_argmax_chunks
    wrapped.ti_gemm_tcgen05_decode_plan = handle.ti_gemm_tcgen05_decode_plan
    wrapped.handle = handle
    for name, args in _SIGNATURES.items():
        fn = getattr(handle, name)
        fn.restype = c_int
        fn.argtypes = args
        setattr(wrapped, name, _Counted(fn, name))
    _lib = wrapped
    return wrapped


def set_pdl(enabled: bool) -> None:
    """Launch kernels as programmatic dependents of their predecessors (default) or strictly one
    after the other."""
    h = lib().handle
    h.ti_set_pdl.restype = None
    h.ti_set_pdl.argtypes = [c_int]
    h.ti_set_pdl(1 if enabled else 0)


def declare(name: str, argtypes, restype=c_int):
    """Declare one more entry point (used by kernel files added later)."""
    fn = getattr(lib().handle, name)
    fn.restype = restype
    fn.argtypes = argtypes
    return fn


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what}: {lib().ti_last_error().decode()}")

_SIGNATURES_FAST = {
    "ti_gemv_bf16": [_P, _L, _P, _L, _P, _I, _I, _I, _I, _I, _F, _F, _F, _F, _P],
    "ti_gemm_tcgen05": [_P, _L, _P, _L, _P, _I, _I, _I, _I, _I, _F, _F, _F, _F, _P, _P],
    "ti_gemm_tcgen05_decode": [_P, _L, _P, _L, _P, _I, _I, _I, _I, _I, _I, _F, _F, _F, _F, _P, _P],
    "ti_attention_prefill": [_P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _F, _I, _I, _I, _I, _I, _P],
    "ti_attention_decode": [_P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _F, _I, _I, _I, _I, _I, _I, _I, _P],
    "ti_attention_decode_shared": [_P, _P, _P, _P, _P, _I, _P, _P, _P, _P, _P, _P, _F, _I, _I, _I, _I, _I, _I, _I, _P],
    "ti_attention_prefill_tc": [_P, _P, _P, _P, _I, _P, _I, _P, _P, _P, _I, _I, _I, _F, _I, _I, _I, _I, _I, _P, _P],
}
_SIGNATURES.update(_SIGNATURES_FAST)
