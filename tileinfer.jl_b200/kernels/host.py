"""The host runtime's C entry points (``csrc/host/``, ``csrc/decode_loop.cu``), declared for ctypes.

The cache's books (slots, lengths, block tables, page pools), the step planner (one pinned
upload per step) and the decode loop's per-step enqueue are C++; this module only gives their
functions argument types. They are compiled into the same library as the kernels and need no
device to run, so the host-side tests drive them on a machine without a GPU.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_longlong, c_void_p

from .library import lib

_INTS, _LONGS = POINTER(c_int), POINTER(c_longlong)
_DECLS = {
    "ti_pool_create": (c_void_p, [c_int]), "ti_pool_destroy": (None, [c_void_p]), "ti_pool_take": (c_int, [c_void_p]),
    "ti_pool_give": (c_int, [c_void_p, c_int]), "ti_pool_free": (c_int, [c_void_p]), "ti_pool_held": (c_int, [c_void_p]),
    "ti_pool_is_held": (c_int, [c_void_p, c_int]),
    "ti_cache_create": (c_void_p, [c_int, c_longlong, c_int]), "ti_cache_destroy": (None, [c_void_p]),
    "ti_cache_add_group": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int]),
    "ti_cache_group_storage": (None, [c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_int, c_longlong, c_longlong, c_int]),
    "ti_cache_alloc_slot": (c_int, [c_void_p]), "ti_cache_free_slot": (c_int, [c_void_p, c_int]),
    "ti_cache_length": (c_longlong, [c_void_p, c_int]), "ti_cache_lengths": (None, [c_void_p, c_int, _INTS, _LONGS]),
    "ti_cache_slots_held": (c_int, [c_void_p]), "ti_cache_slot_is_held": (c_int, [c_void_p, c_int]),
    "ti_cache_reserve": (c_int, [c_void_p, c_int, _INTS, _LONGS, c_longlong, c_void_p, _LONGS, _LONGS]),
    "ti_cache_prepare": (c_int, [c_void_p, c_int, _INTS, _LONGS, c_void_p]),
    "ti_cache_advance": (c_int, [c_void_p, c_int, c_longlong]), "ti_cache_advance_many": (c_int, [c_void_p, c_int, _INTS, _LONGS]),
    "ti_cache_truncate": (c_int, [c_void_p, c_int, c_longlong]),
    "ti_group_pages_free": (c_int, [c_void_p, c_int]), "ti_group_pages_held": (c_int, [c_void_p, c_int]),
    "ti_group_page_is_held": (c_int, [c_void_p, c_int, c_int]), "ti_group_table": (c_int, [c_void_p, c_int, c_int, _INTS, c_int]),
    "ti_group_first": (c_int, [c_void_p, c_int, c_int]), "ti_group_host_table": (c_void_p, [c_void_p, c_int]),
    "ti_group_peak_pages": (c_longlong, [c_void_p, c_int, c_int, _INTS, _LONGS, c_longlong]),
    "ti_planner_create": (c_void_p, [c_void_p, c_int, c_int]), "ti_planner_destroy": (None, [c_void_p]),
    "ti_planner_attach_plan": (None, [c_void_p, c_int, c_void_p]), "ti_group_plan_destroy": (None, [c_void_p]),
    "ti_planner_capacity": (c_int, [c_void_p]), "ti_planner_set_meta": (None, [c_void_p, c_void_p]),
    "ti_planner_layout": (None, [c_void_p, c_int, c_int, c_int, _INTS]),
    "ti_planner_plan": (c_int, [c_void_p, c_int, _INTS, _INTS, _INTS, _INTS, _INTS, c_void_p]),
    "ti_planner_plan_decode": (c_int, [c_void_p, c_int, _INTS, _INTS, c_void_p, _LONGS]),
    "ti_planner_last_upload_bytes": (c_longlong, [c_void_p]),
    "ti_split_kv_plan_create": (c_void_p, [c_int, c_int, c_longlong, c_int, c_int]), "ti_split_kv_plan_splits": (c_int, [c_void_p, c_int]),
    "ti_split_kv_tables": (c_int, [c_int, c_int, c_int, c_int, _LONGS, _INTS, _INTS]),
    "ti_loop_create": (c_void_p, [c_void_p, c_void_p, c_int, c_int] + [c_void_p] * 6), "ti_loop_destroy": (None, [c_void_p]),
    "ti_loop_enqueue": (c_int, [c_void_p, c_void_p, c_longlong, c_int, c_float, c_int, c_float, c_int, _INTS, _INTS, c_void_p, c_void_p,
                                c_void_p, _LONGS, _LONGS]),
    "ti_loop_wait": (c_int, [c_void_p, _INTS, c_int]),
    "ti_range_push": (None, [c_char_p]), "ti_range_pop": (None, []),
}
_api = None


class _Api:
    pass


def api():
    """The declared functions, as attributes without the ``ti_`` prefix."""
    global _api
    if _api is None:
        handle = lib().handle
        a = _Api()
        for name, (restype, argtypes) in _DECLS.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = restype, argtypes
            setattr(a, name[3:], fn)
        _api = a
    return _api


def ints(values):
    """A C array of ints from a sequence."""
    values = list(values)
    return (c_int * len(values))(*values)


def longs(values):
    values = list(values)
    return (c_longlong * len(values))(*values)


def last_error() -> str:
    return lib().ti_last_error().decode()


class nvtx_range:
    """An NVTX range around a phase of a step (a no-op unless a profiler is attached), as the reference marks
    its prefill, upload, replay and sampling (src/engine/runner.jl:77-97, 171-175)."""

    def __init__(self, name: str):
        self.name = name.encode()

    def __enter__(self):
        api().range_push(self.name)
        return self

    def __exit__(self, *exc):
        api().range_pop()
        return False
