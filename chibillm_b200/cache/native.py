"""Loads the host-side runtime (``csrc/runtime.cc``: cache manager, batch packing,
scheduler) and declares its C entry points."""
from __future__ import annotations

import ctypes
import threading
from ctypes import POINTER, c_char_p, c_int, c_longlong, c_void_p

from ..csrc import build

_lock = threading.Lock()
_lib = None

IP = POINTER(c_int)
LP = POINTER(c_longlong)

_SIGNATURES = {
    "chibi_rt_error": ([], c_char_p),
    "chibi_pool_new": ([c_int], c_void_p),
    "chibi_pool_delete": ([c_void_p], None),
    "chibi_pool_free_count": ([c_void_p], c_int),
    "chibi_pool_take": ([c_void_p, c_int, IP], c_int),
    "chibi_pool_give": ([c_void_p, c_int], c_int),
    "chibi_cache_new": ([c_int, IP, IP, IP, IP, c_int], c_void_p),
    "chibi_cache_delete": ([c_void_p], None),
    "chibi_cache_admit": ([c_void_p, c_longlong], c_int),
    "chibi_cache_has": ([c_void_p, c_longlong], c_int),
    "chibi_cache_count": ([c_void_p], c_int),
    "chibi_cache_info": ([c_void_p, c_longlong, IP], c_int),
    "chibi_cache_table": ([c_void_p, c_longlong, c_int, IP, c_int], c_int),
    "chibi_cache_reserve": ([c_void_p, c_longlong, c_int], c_int),
    "chibi_cache_commit": ([c_void_p, c_longlong, c_int], c_int),
    "chibi_cache_advance": ([c_void_p, c_int, c_int, LP, IP], c_int),
    "chibi_cache_release": ([c_void_p, c_longlong], c_int),
    "chibi_cache_free_pages": ([c_void_p, c_int], c_int),
    "chibi_cache_free_slots": ([c_void_p], c_int),
    "chibi_cache_pending_updates": ([c_void_p, c_int], c_int),
    "chibi_cache_drain": ([c_void_p, c_int, IP, c_int], c_int),
    "chibi_cache_check": ([c_void_p], c_int),
    "chibi_sched_new": ([c_void_p, c_int, c_int, c_int, c_int], c_void_p),
    "chibi_sched_delete": ([c_void_p], None),
    "chibi_sched_fits_cache": ([c_void_p, c_int, c_int], c_int),
    "chibi_sched_admission": ([c_void_p, c_int, c_int], c_int),
    "chibi_sched_add": ([c_void_p, c_longlong, IP, c_int, c_int, c_int], c_int),
    "chibi_sched_has_work": ([c_void_p], c_int),
    "chibi_sched_active": ([c_void_p], c_int),
    "chibi_sched_schedule": ([c_void_p, LP, c_int, IP], c_int),
    "chibi_sched_complete": ([c_void_p, c_int, IP, c_int, LP, c_int], c_int),
    "chibi_sched_abort": ([c_void_p, c_int], c_int),
    "chibi_sched_cancel": ([c_void_p, c_longlong], c_int),
    "chibi_sched_remove": ([c_void_p, c_longlong], c_int),
    "chibi_sched_info": ([c_void_p, c_longlong, IP], c_int),
    "chibi_sched_tokens": ([c_void_p, c_longlong, c_int, c_int, IP], c_int),
    "chibi_sched_queue": ([c_void_p, c_int, LP, c_int], c_int),
    "chibi_sched_check": ([c_void_p], c_int),
    "chibi_pack_step": ([c_void_p, c_int, LP, IP, IP, IP, IP, c_int, c_int, c_int, c_void_p, c_int, IP, c_int],
                        c_int),
}

# negative status -> the code a CacheError carries
ERROR_CODES = {-1: "capacity_exhausted", -2: "invalid_release", -3: "unknown_request", -4: "duplicate_request",
               -5: "invalid_reservation", -6: "invalid_commit", -7: "invalid_configuration", -8: "invariant",
               -9: "batch", -10: "buffer_too_small"}


def runtime():
    """The library, compiled at the first call if its current version is absent."""
    global _lib
    with _lock:
        if _lib is None:
            lib = ctypes.CDLL(build.runtime_library())
            for name, (argtypes, restype) in _SIGNATURES.items():
                fn = getattr(lib, name)
                fn.argtypes = argtypes
                fn.restype = restype
            _lib = lib
        return _lib


def error_message() -> str:
    return runtime().chibi_rt_error().decode("utf-8", "replace")
