"""ctypes binding of ``libmoe_b200.so`` (the C ABI in ``include/moe_b200.h``).

There is no fallback: if the shared library is missing or a call fails, an
exception is raised.  Build the library with ``python -m tilelang_moe_b200.build``.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

# MOE_B200_LIBRARY selects another build of the same ABI (the tile-timeline build, libmoe_b200_trace.so)
LIB_PATH = Path(os.environ.get("MOE_B200_LIBRARY") or Path(__file__).resolve().parent / "libmoe_b200.so")

# every symbol declared in include/moe_b200.h: name -> (restype, argtypes)
_i64, _i32, _vp, _sz = C.c_int64, C.c_int, C.c_void_p, C.c_size_t
SIGNATURES = {
    "moe_last_error": (C.c_char_p, []),
    "moe_abi_version": (_i32, []),
    "moe_device_info": (_i32, [_i32, C.POINTER(_i32), C.POINTER(_i32), C.POINTER(_i32)]),
    "moe_topk_softmax": (_i32, [_vp, _i64, _i64, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp]),
    "moe_route_histogram_workspace": (_sz, [_i64, _i32]),
    "moe_route_histogram": (_i32, [_vp, _i32, _i64, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _vp]),
    "moe_route_histogram_static": (_i32, [_vp, _i32, _i64, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "moe_gather_rows": (_i32, [_vp, _vp, _i32, _i64, _i64, _vp, _vp, _vp, _vp]),
    "moe_grouped_gemm": (_i32, [_i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _vp, _vp]),
    "moe_grouped_gemm_gathered": (_i32, [_i32, _vp, _i64, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64,
                                         _i32, _i32, _i32, _i32, _vp, _vp]),
    "moe_combine": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i64, _i32, _vp, _vp]),
    "moe_ep_regroup": (_i32, [_vp, _i32, _i32, _vp, _vp, _vp]),
    "moe_ep_plan": (_i32, [_vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp]),
    "moe_ep_dispatch": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i64, _i64, C.POINTER(C.c_void_p), _i32, _vp]),
    "moe_ep_unique": (_i32, [_vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp]),
    "moe_ep_plan_dedup": (_i32, [_vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "moe_ep_dispatch_dedup": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i64, _i64, _i64,
                                     C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), _i32, _vp]),
    "moe_ep_barrier": (_i32, [C.POINTER(C.c_void_p), _i32, _i32, _i32, _i32, _i64, _vp, _vp]),
    "moe_ep_share_counts": (_i32, [_vp, _i32, _vp, _i32, C.POINTER(C.c_void_p), _i32, C.POINTER(C.c_void_p), _i32, _i32,
                                   _i32, _i32, _i64, _vp, _vp]),
    "moe_debug_wait_probe": (_i32, [_i64, _vp, _vp, _vp]),
    "moe_debug_bounds_status": (_i32, [C.POINTER(C.c_int32), _vp]),
    "moe_grouped_gemm_peer_scatter": (_i32, [_vp, _vp, _vp, _vp, _vp, C.POINTER(C.c_void_p), _i32, _i64, _i64, _i64,
                                             _i32, _i32, _i32, _i32, _vp, _vp]),
    "moe_layer_workspace": (_sz, [_i64, _i32, _i32, _i32, _i32, _i32]),
    "moe_layer_forward": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _i32,
                                 _vp, _sz, _vp, _vp, _vp, _vp]),
    "moe_mhc_pre_workspace": (_sz, [_i64, _i32, _i64]),
    "moe_mhc_split_weights": (_i32, [_vp, _i32, _i64, _vp, _vp]),
    "moe_mhc_pre": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i64, C.c_float, C.c_float, C.c_float, C.c_float, _i32,
                           _vp, _sz, _vp, _vp, _vp, _vp, _vp]),
    "moe_mhc_post": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i64, _vp, _vp]),
    "moe_router_topk": (_i32, [_vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "moe_router_topk_splitk_workspace": (_sz, [_i64, _i32, _i32]),
    "moe_router_topk_splitk": (_i32, [_vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _vp]),
    "moe_router_logits": (_i32, [_vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp]),
}


class MoeLibraryError(RuntimeError):
    pass


_lib = None


def load() -> C.CDLL:
    """Load the shared library once and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise MoeLibraryError(
            f"{LIB_PATH} is missing: build it with `python -m tilelang_moe_b200.build` "
            "(there is no CPU or PyTorch fallback)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise MoeLibraryError(f"{LIB_PATH} does not export {name}; rebuild it") from e
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().moe_last_error()
        raise MoeLibraryError(f"{what} failed with status {rc}: {msg.decode(errors='replace') if msg else ''}")
