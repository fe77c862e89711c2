"""ctypes binding of the native host core (``csrc/host_core.cpp``): page pools, the cache
manager's state, the scheduler's planner and the routine that fills a step's metadata buffer.  The shared object
is host-only code, compiled at first use like the kernels."""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_int32, c_uint32, c_void_p

from ..ops import build

_lib = None


class RlLayout(ctypes.Structure):
    _fields_ = [(n, c_int32) for n in (
        "token_ids", "token_src", "positions", "seq_of_token", "state_slot", "decode_info", "tile_seq",
        "tile_tok", "tile_rows", "logit_rows", "temperature", "top_k", "top_p", "seed_lo", "seed_hi",
        "sample_pos", "words")]


class RlSegment(ctypes.Structure):
    _fields_ = [("rid", c_int32), ("start_pos", c_int32), ("num_tokens", c_int32), ("src_row", c_int32),
                ("token_off", c_int32), ("want_off", c_int32), ("num_want", c_int32), ("has_sampling", c_int32),
                ("temperature", c_float), ("top_p", c_float), ("top_k", c_int32), ("seed_lo", c_uint32),
                ("seed_hi", c_uint32)]


class RlSchedCfg(ctypes.Structure):
    _fields_ = [("max_num_seqs", c_int32), ("budget", c_int32), ("max_seq_len", c_int32), ("mix", c_int32),
                ("watermark", c_double)]


SCHED_SEQ_FIELDS = ("rid", "known", "pending", "computed", "prompt_len", "max_new", "pending_ok", "pending_row",
                    "where", "preempted", "cache_changed")       # RlSchedSeq: int32 each
SCHED_ENTRY_FIELDS = ("seq", "start_pos", "num_tokens", "sample", "from_device", "src_row")   # RlSchedEntry


# the same record as a numpy dtype (a step's segments are marshalled in one call)
SEGMENT_DTYPE = None


def _segment_dtype():
    import numpy as np
    return np.dtype([("rid", "<i4"), ("start_pos", "<i4"), ("num_tokens", "<i4"), ("src_row", "<i4"),
                     ("token_off", "<i4"), ("want_off", "<i4"), ("num_want", "<i4"), ("has_sampling", "<i4"),
                     ("temperature", "<f4"), ("top_p", "<f4"), ("top_k", "<i4"), ("seed_lo", "<u4"),
                     ("seed_hi", "<u4")])


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = build.compile_module("host_core", "host_core.cpp")
        L = ctypes.CDLL(path)
        i32p = POINTER(c_int32)
        sig = {
            "rl_pool_create": (c_void_p, [c_int, c_int]),
            "rl_pool_destroy": (None, [c_void_p]),
            "rl_pool_allocate": (c_int, [c_void_p]),
            "rl_pool_free": (c_int, [c_void_p, i32p, c_int, POINTER(c_int)]),
            "rl_pool_num_free": (c_int, [c_void_p]),
            "rl_pool_num_usable": (c_int, [c_void_p]),
            "rl_pool_is_held": (c_int, [c_void_p, c_int]),
            "rl_hc_create": (c_void_p, [c_int, i32p, i32p, c_int, c_int]),
            "rl_hc_destroy": (None, [c_void_p]),
            "rl_hc_open": (c_int, [c_void_p]),
            "rl_hc_close": (c_int, [c_void_p, c_int, POINTER(c_int)]),
            "rl_hc_reserve": (c_int, [c_void_p, c_int, c_int]),
            "rl_hc_release_passed": (c_int, [c_void_p, c_int, c_int]),
            "rl_hc_state_slot": (c_int, [c_void_p, c_int]),
            "rl_hc_num_tokens": (c_int, [c_void_p, c_int]),
            "rl_hc_released_upto": (c_int, [c_void_p, c_int, c_int]),
            "rl_hc_table": (c_int, [c_void_p, c_int, c_int, POINTER(i32p)]),
            "rl_hc_num_free": (c_int, [c_void_p, c_int]),
            "rl_hc_num_usable": (c_int, [c_void_p, c_int]),
            "rl_hc_num_open": (c_int, [c_void_p]),
            "rl_hc_check": (c_int, [c_void_p, c_char_p, c_int]),
            "rl_hc_build": (c_int, [c_void_p, c_void_p, POINTER(RlLayout), i32p, i32p, c_int, c_int, c_int,
                                    c_void_p, c_void_p, c_void_p, c_int, c_int, i32p]),
            "rl_hc_pad": (None, [c_void_p, POINTER(RlLayout), c_int, c_int]),
            "rl_sched_plan": (c_int, [c_void_p, POINTER(RlSchedCfg), c_void_p, c_int, c_int, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p]),
        }
        for name, (res, args) in sig.items():
            f = getattr(L, name)
            f.restype = res
            f.argtypes = args
        _lib = L
    return _lib


SEGMENT_DTYPE = _segment_dtype()
assert SEGMENT_DTYPE.itemsize == ctypes.sizeof(RlSegment)
