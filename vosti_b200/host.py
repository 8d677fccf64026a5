"""Python face of the C++ host core (vosti_b200/csrc/host/engine_core.cpp): page pools,
cache accounting and the scheduler live there; this module loads the library and turns its
error codes into exceptions."""
from __future__ import annotations

import ctypes
from typing import Optional

from .csrc import build as _build

_LIB: Optional[ctypes.CDLL] = None

i32p = ctypes.POINTER(ctypes.c_int32)
i64p = ctypes.POINTER(ctypes.c_int64)


class OutOfPages(RuntimeError):
    """An allocation asked for more pages than are free or evictable."""


class PageAccountingError(AssertionError):
    """A page was released twice, acquired while vacant, or lost."""


class OutOfSlots(RuntimeError):
    pass


OK, OUT_OF_PAGES, ACCOUNTING, BAD_ARGUMENT, OUT_OF_SLOTS, UNKNOWN_REQUEST = 0, -1, -2, -3, -4, -5
_ERRORS = {OUT_OF_PAGES: OutOfPages, ACCOUNTING: PageAccountingError, BAD_ARGUMENT: ValueError,
           OUT_OF_SLOTS: OutOfSlots, UNKNOWN_REQUEST: KeyError}


def library() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        lib = ctypes.CDLL(str(_build.host_library_path()))
        lib.vh_last_error.restype = ctypes.c_char_p
        lib.vh_chain_hash.restype = ctypes.c_uint64
        lib.vh_chain_hash.argtypes = [ctypes.c_uint64, i32p, ctypes.c_int]
        lib.vh_pool_create.restype = ctypes.c_void_p
        lib.vh_pool_publish.restype = ctypes.c_uint64
        lib.vh_pool_publish.argtypes = [ctypes.c_void_p, ctypes.c_int, i32p, ctypes.c_int, ctypes.c_uint64,
                                        ctypes.c_int, ctypes.c_int, i32p]
        lib.vh_pool_evictions.restype = ctypes.c_int64
        lib.vh_create.restype = ctypes.c_void_p
        lib.vh_group_pool.restype = ctypes.c_void_p
        lib.vh_counter.restype = ctypes.c_int64
        for name in ("vh_pool_destroy", "vh_pool_available", "vh_pool_num_pages", "vh_pool_evictions",
                     "vh_pool_refcount", "vh_pool_allocate", "vh_pool_acquire", "vh_pool_release", "vh_pool_match",
                     "vh_pool_list", "vh_pool_set_published_tokens", "vh_pool_check", "vh_destroy",
                     "vh_configure_scheduler", "vh_group_pool", "vh_prefix_reuse", "vh_available_pages",
                     "vh_counter", "vh_begin", "vh_is_live", "vh_pages_needed", "vh_can_extend", "vh_extend",
                     "vh_trim", "vh_publish", "vh_finish", "vh_length", "vh_slot", "vh_residency_field",
                     "vh_block_row", "vh_free_slots", "vh_live_ids", "vh_check", "vh_add_request", "vh_abort",
                     "vh_unfinished", "vh_queue", "vh_plan", "vh_commit", "vh_commit_ahead", "vh_resolve", "vh_request_field", "vh_request_tokens",
                     "vh_forget", "vh_step_extend", "vh_step_fill", "vh_take_fresh_slots"):
            getattr(lib, name).argtypes = None      # variadic-style calls; handles are wrapped below
        _LIB = lib
    return _LIB


def check(code: int) -> int:
    """Return `code` if it is not an error, else raise what the code stands for."""
    if code >= 0:
        return code
    message = library().vh_last_error().decode()
    raise _ERRORS.get(code, RuntimeError)(message)


def ints(values) -> ctypes.Array:
    values = list(values)
    return (ctypes.c_int32 * max(len(values), 1))(*values)


def handle(pointer) -> ctypes.c_void_p:
    return ctypes.c_void_p(pointer)
