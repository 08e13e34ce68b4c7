"""ctypes binding of the C ABI declared in include/diffcache_b200.h.

There is no CPU fallback: if the shared library is missing this module raises.
"""
from __future__ import annotations

import ctypes
import os

from . import _build

_i32, _i64, _u64, _f32, _vp = ctypes.c_int, ctypes.c_int64, ctypes.c_uint64, ctypes.c_float, ctypes.c_void_p

# name -> (restype, argtypes); mirrors include/diffcache_b200.h one to one
SIGNATURES = {
    "dc_last_error": (ctypes.c_char_p, []),
    "dc_version": (_i32, []),
    "dc_create": (_i32, [_i32, _i32, _i32, _i32, _i64, _i32, _i32, ctypes.POINTER(_vp)]),
    "dc_destroy": (_i32, [_vp]),
    "dc_set_row_offset": (_i32, [_vp, _i64]),
    "dc_prefill": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _u64]),
    "dc_insert": (_i32, [_vp, _vp, _vp, _u64]),
    "dc_ctx_len": (_i32, [_vp, ctypes.POINTER(_i64)]),
    "dc_query": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _u64]),
    "dc_check_status": (_i32, [_vp, _u64]),
    "dc_get_keys": (_i32, [_vp, _vp]),
    "dc_export_rows": (_i32, [_vp, _vp, _vp]),
    "dc_update_r_sq": (_i32, [_vp, _vp, _i32]),
    "dc_decode_attend": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _f32, _vp, _vp, _vp, _u64]),
    "dc_decode_attend_strided": (_i32, [_vp, _vp, _i64, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _i32, _i32, _f32, _vp, _vp,
                                        _vp, _u64]),
    "dc_window_push": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _vp, _u64]),
    "dc_window_advance": (_i32, [_vp, _u64]),
    "dc_decode_attend_dyn": (_i32, [_vp, _vp, _i64, _vp, _vp, _i64, _i64, _vp, _i32, _i32, _f32, _vp, _vp, _vp, _u64]),
    "dc_set_adaptive_budget": (_i32, [_vp, _vp, _i32, _f32]),
    "dc_get_budget": (_i32, [_vp, _vp, _u64]),
    "dc_adaptive_budget": (_i32, [_vp, _i64, _i32, _i32, _i32, _vp, _i32, _f32, _vp, _u64]),
    "dc_set_phase_timing": (_i32, [_vp, _i32]),
    "dc_get_phase_times": (_i32, [_vp, ctypes.POINTER(_f32), ctypes.POINTER(_f32), ctypes.POINTER(_f32),
                                  ctypes.POINTER(_i32)]),
    "dc_trace_begin": (_i32, [_vp, _i32]),
    "dc_trace_read": (_i32, [_vp, _vp, ctypes.POINTER(_i32)]),
    "dc_local_topk": (_i32, [_vp, _vp, _i32, _vp, _vp, _u64]),
    "dc_attend_owned": (_i32, [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _f32, _vp, _vp, _vp, _u64]),
    "dc_xchg_create": (_i32, [_i32, _i32, _i32, _vp, _i32, ctypes.POINTER(_vp)]),
    "dc_xchg_destroy": (_i32, [_vp]),
    "dc_xchg_handle_bytes": (_i32, []),
    "dc_xchg_get_handle": (_i32, [_vp, _vp]),
    "dc_xchg_open_peer": (_i32, [_vp, _i32, _vp]),
    "dc_xchg_set_peer": (_i32, [_vp, _i32, _vp]),
    "dc_xchg_local": (_vp, [_vp]),
    "dc_xchg_set_timeout_ms": (_i32, [_vp, _i32]),
    "dc_xchg_push": (_i32, [_vp, _i32, _vp, _i64, _u64]),
    "dc_xchg_push_rows": (_i32, [_vp, _i32, _vp, _i64, _i64, _u64]),
    "dc_xchg_collect": (_i32, [_vp, _i32, _vp, _i64, _u64]),
    "dc_xchg_check": (_i32, [_vp, _u64]),
    "dc_set_output_exchange": (_i32, [_vp, _vp, _i32]),
    "dc_set_output_gather": (_i32, [_vp, _vp]),
    "dc_sharded_slot_bytes": (_i32, [_vp, _i32, _vp]),
    "dc_sharded_local": (_i32, [_vp, _vp, _vp, _i32, _u64]),
    "dc_sharded_attend": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _f32, _u64]),
    "dc_sharded_combine": (_i32, [_vp, _vp, _vp, _vp, _u64]),
    "dc_sharded_decode_attend": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _f32, _vp, _vp, _u64]),
    "dc_merge_sorted_count": (_i32, [_vp, _i32, _i32, _i32, _i32, _vp, _u64]),
    "dc_score_scan": (_i32, [_vp, _i64, _i32, _i64, _i32, _i32, _vp, _i32, _i32, _vp, _i64, _vp, _u64]),
    "dc_select_scratch_bytes": (_i64, [_i32]),
    "dc_topk_select": (_i32, [_vp, _vp, _i64, _i32, _i64, _i32, _vp, _vp, _vp, _i64, _vp, _u64]),
    "dc_attend_scratch_bytes": (_i64, [_i32, _i32, _i32]),
    "dc_sparse_attend": (_i32, [_vp, _vp, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _i64, _i32, _i64, _vp,
                                _vp, _vp, _vp, _i64, _i64, _i32, _f32, _vp, _vp, _vp, _vp, _vp, _u64]),
    "dc_sparse_attend_noalloc": (_i32, [_vp, _vp, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _i64, _i32, _i64,
                                        _vp, _vp, _vp, _vp, _i64, _i64, _i32, _f32, _vp, _vp, _vp, _vp, _u64]),
    "dc_lse_combine": (_i32, [_vp, _i64, _vp, _i64, _i32, _i64, _i32, _i32, _vp, _vp, _u64]),
    "dc_gather_rows": (_i32, [_vp, _i64, _i32, _i32, _vp, _i64, _i32, _vp, _u64]),
    "dc_pq_build_lut": (_i32, [_vp, _i32, _i32, _i32, _vp, _i32, _i32, _i32, _vp, _u64]),
    "dc_pq_adc_scan": (_i32, [_vp, _i64, _i32, _i64, _i32, _vp, _vp, _i64, _vp, _u64]),
    "dc_rerank_scores": (_i32, [_vp, _i64, _i32, _i32, _i32, _vp, _i32, _i32, _vp, _i64, _i32, _vp, _u64]),
}

_lib = None


class DiffCacheError(RuntimeError):
    """A C-ABI call returned a non-zero status (the reference panics in the same situations)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"diffcache_b200 error {code}: {message}")
        self.code = code


def load() -> ctypes.CDLL:
    """Load (building first if the sources are newer) the CUDA shared library."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    if _build.is_stale():
        if os.environ.get("DIFFCACHE_B200_NO_BUILD") == "1" and os.path.exists(path):
            pass
        else:
            path = _build.build()
    if not os.path.exists(path):
        raise ImportError(f"diffcache_b200: CUDA extension {path} is missing and could not be built")
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != 0:
        msg = load().dc_last_error()
        raise DiffCacheError(code, msg.decode() if msg else "")
