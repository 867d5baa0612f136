"""ctypes face of csrc/host_runtime.cpp: the cache manager's bookkeeping in C++."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_longlong, c_void_p

from ..csrc.build import load_library

_lib = None


def lib():
    global _lib
    if _lib is None:
        L = load_library("host_runtime")
        sig = {
            "qvh_pool_create": (c_void_p, [c_int]), "qvh_pool_destroy": (None, [c_void_p]),
            "qvh_pool_num_free": (c_int, [c_void_p]), "qvh_pool_alloc": (c_int, [c_void_p, c_int, POINTER(c_int)]),
            "qvh_pool_free": (c_int, [c_void_p, POINTER(c_int), c_int]), "qvh_pool_is_held": (c_int, [c_void_p, c_int]),
            "qvh_create": (c_void_p, [c_int, POINTER(c_int), c_int, c_int, c_int]), "qvh_destroy": (None, [c_void_p]),
            "qvh_has": (c_int, [c_void_p, c_longlong]), "qvh_length": (c_int, [c_void_p, c_longlong]),
            "qvh_slot": (c_int, [c_void_p, c_longlong]), "qvh_epoch": (c_longlong, [c_void_p, c_longlong]),
            "qvh_free_slots": (c_int, [c_void_p]), "qvh_num_live": (c_int, [c_void_p]),
            "qvh_free_pages": (c_int, [c_void_p, c_int]), "qvh_held_pages": (c_int, [c_void_p, c_int]),
            "qvh_admit": (c_int, [c_void_p, c_longlong]),
            "qvh_pages_needed": (c_int, [c_void_p, c_longlong, c_int, c_int, c_int]),
            "qvh_can_reserve": (c_int, [c_void_p, c_int, POINTER(c_longlong), POINTER(c_int), POINTER(c_int)]),
            "qvh_reserve": (c_int, [c_void_p, c_longlong, c_int]), "qvh_commit": (c_int, [c_void_p, c_longlong, c_int]),
            "qvh_release": (c_int, [c_void_p, c_longlong]),
            "qvh_one_more_token_fits": (c_int, [c_void_p, c_int, POINTER(c_longlong)]),
            "qvh_table_len": (c_int, [c_void_p, c_longlong, c_int]),
            "qvh_table_copy": (c_int, [c_void_p, c_longlong, c_int, POINTER(c_int), c_int]),
            "qvh_youngest": (c_int, [c_void_p, c_int, POINTER(c_longlong)]),
            "qvh_check": (c_int, [c_void_p, c_char_p, c_int]),
            "qvh_decode_variant": (c_int, [c_int, c_int]), "qvh_decode_splits": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int]),
            "qvh_folded_norm_enabled": (c_int, [c_int]), "qvh_fused_rope_enabled": (c_int, [c_int]),
            "qvh_fill_decode": (c_int, [c_void_p, c_int, POINTER(c_longlong), POINTER(c_int), c_int, c_int, c_int, c_int,
                                        c_void_p, c_void_p, c_void_p]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def ints(values):
    return (c_int * len(values))(*values)


def longs(values):
    return (c_longlong * len(values))(*values)
