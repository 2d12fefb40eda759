"""Python face of the host library (C++ under ``csrc/host/``): page pools, the cache
manager, the scheduler and the packing of a step's index arrays. The bookkeeping runs in the library;
the classes in ``cache`` and ``engine.runner`` hold its handles.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, byref, c_int, c_int32, c_int64, c_void_p

from .csrc import build as _build

OK, CACHE_ERROR, OUT_OF_PAGES, NO_FREE_SLOT, BAD_ARGUMENT = range(5)

# Order of the arrays in a packed step (StepArray in csrc/host/cache_manager.hpp).
(TOKEN_IDS, POSITIONS, TOKEN_REQ, Q_START, N_NEW, CACHED_LEN, SLOT_IDS, WANT_ROWS, PEND_DST, PEND_SRC,
 FIRST_TABLE) = range(11)

_configured = False


def lib() -> ctypes.CDLL:
    global _configured
    library = _build.host_library()
    if not _configured:
        i32p, i64p, intp = POINTER(c_int32), POINTER(c_int64), POINTER(c_int)
        sigs = {
            "llmrs_pool_create": [c_int, POINTER(c_void_p)],
            "llmrs_pool_destroy": [c_void_p],
            "llmrs_pool_allocate": [c_void_p, i32p],
            "llmrs_pool_free": [c_void_p, c_int32, intp],
            "llmrs_pool_increment_ref": [c_void_p, c_int32],
            "llmrs_pool_ref_count": [c_void_p, c_int32, intp],
            "llmrs_pool_counts": [c_void_p, intp, intp],
            "llmrs_cm_create": [intp, intp, c_int, c_int, c_int, POINTER(c_void_p)],
            "llmrs_cm_destroy": [c_void_p],
            "llmrs_cm_admit": [c_void_p, c_int64, intp],
            "llmrs_cm_release": [c_void_p, c_int64],
            "llmrs_cm_pages_needed": [c_void_p, c_int, c_int64, c_int, c_int, intp],
            "llmrs_cm_reserve": [c_void_p, c_int64, c_int],
            "llmrs_cm_cancel": [c_void_p, c_int64],
            "llmrs_cm_commit": [c_void_p, c_int64, c_int],
            "llmrs_cm_info": [c_void_p, c_int64, intp, i64p],
            "llmrs_cm_table": [c_void_p, c_int64, c_int, i32p, c_int, intp],
            "llmrs_cm_pool_counts": [c_void_p, c_int, intp, intp],
            "llmrs_cm_check_invariants": [c_void_p],
            "llmrs_sched_create": [c_void_p, c_int, i32p, c_int, c_int, c_int, c_int, POINTER(c_void_p)],
            "llmrs_sched_destroy": [c_void_p],
            "llmrs_sched_add": [c_void_p, c_int64, c_int, c_int, c_int],
            "llmrs_sched_has_work": [c_void_p, intp],
            "llmrs_sched_schedule": [c_void_p, i64p, i32p, c_int, intp, i64p],
            "llmrs_sched_on_launched": [c_void_p, c_int64],
            "llmrs_sched_cancel": [c_void_p, c_int64],
            "llmrs_sched_on_result": [c_void_p, c_int64, i32p, c_int, i64p, i32p, c_int, intp],
            "llmrs_sched_abort_all": [c_void_p, c_int, i64p, i32p, c_int, intp],
            "llmrs_sched_take": [c_void_p, c_int, i64p, c_int, intp],
            "llmrs_sched_get": [c_void_p, c_int64, i32p],
            "llmrs_sched_forget": [c_void_p, c_int64],
            "llmrs_sched_stats": [c_void_p, i64p],
            "llmrs_pack_step": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, i64p, intp],
            "llmrs_plan_paged_attention": [c_int, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_void_p, c_int64,
                                           c_void_p, intp],
        }
        for name, argtypes in sigs.items():
            fn = getattr(library, name)
            fn.argtypes = argtypes
            fn.restype = None if name.endswith("_destroy") else c_int
        _configured = True
    return library


def plan_paged_attention(n_new, cached_len, tile: int):
    """The host library's plan of paged attention for a step (int32 numpy arrays of the step's requests in,
    ``(tiles [n, 2], decode list, max_decode_kv_len, long_portions)`` out)."""
    import numpy as np
    R = int(n_new.shape[0])
    # Requests that bring one token take no tile: n // tile + 1 bounds a longer portion's tiles.
    tiles_cap = int(n_new.sum()) // tile + R
    tiles = np.empty((max(tiles_cap, 1), 2), np.int32)
    decode = np.empty(max(R, 1), np.int32)
    plan = np.zeros(4, np.int32)
    written = c_int()
    n_new = np.ascontiguousarray(n_new, np.int32)
    cached_len = np.ascontiguousarray(cached_len, np.int32)
    rc = lib().llmrs_plan_paged_attention(R, n_new.ctypes.data, cached_len.ctypes.data, tile, tiles.ctypes.data,
                                          tiles_cap, decode.ctypes.data, R, plan.ctypes.data, byref(written))
    if rc != 0 or not written.value:
        raise RuntimeError(f"attention plan failed: {last_error() if rc else 'capacity'}")
    return tiles[:plan[0]], decode[:plan[1]], int(plan[2]), bool(plan[3])


def last_error() -> str:
    return lib().llmrs_host_last_error().decode("utf-8", "replace")


__all__ = ["lib", "last_error", "byref", "c_int", "c_int32", "c_int64", "c_void_p"]
