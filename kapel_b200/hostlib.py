"""The host library (`csrc/host/*.cpp`: the cache manager's bookkeeping and the host sampler), built
with the C++ compiler alone at first use and loaded through ctypes."""
from __future__ import annotations

import ctypes
from typing import Optional

_LIB: Optional[ctypes.CDLL] = None


def host_library() -> ctypes.CDLL:
    """The host library, built if need be; raises if it cannot be built or loaded."""
    global _LIB
    if _LIB is None:
        from .csrc.build import ensure_host_built

        lib = ctypes.CDLL(str(ensure_host_built(verbose=True)))
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        ip = ctypes.POINTER(ctypes.c_int)
        sigs = {
            "kp_create": (vp, [i32]), "kp_destroy": (None, [vp]), "kp_take": (i32, [vp]), "kp_give": (i32, [vp, i32]),
            "kp_free": (i32, [vp]), "kp_is_held": (i32, [vp, i32]), "kp_check": (i32, [vp, ctypes.c_char_p, i32]),
            "kc_create": (vp, [i32, i32, ip, ip, i32]), "kc_destroy": (None, [vp]), "kc_add": (i32, [vp]),
            "kc_remove": (i32, [vp, i32]), "kc_length": (i32, [vp, i32]), "kc_free_slots": (i32, [vp]),
            "kc_released_pages": (i64, [vp]), "kc_free_pages": (None, [vp, ip]), "kc_held_pages": (i32, [vp, i32, ip]),
            "kc_pages_of": (i32, [vp, i32, i32, ip, i32]), "kc_pages_needed": (i32, [vp, i32, i32, ip]),
            "kc_plan_prepare": (i32, [vp, i32, vp, vp, vp]),
            "kc_plan_fill": (i32, [vp, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, vp, i32]),
            "kc_commit": (i64, [vp, i32, vp, vp]), "kc_abort": (i32, [vp, i32, vp]),
            "kc_check": (i32, [vp, ctypes.c_char_p, i32]),
            "ks_seed": (None, [ctypes.c_ulonglong, vp]), "ks_uniform": (ctypes.c_double, [vp]),
            "ks_choose": (i32, [vp, i32, i32, vp, i32, vp, i32, i32, vp, vp, i32]),
            "ks_choose_many": (None, [i32, vp, i64, i32, i32, vp, vp, vp, vp, vp, vp, vp, i32]),
        }
        for name, (res, args) in sigs.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _LIB = lib
    return _LIB
