"""Loads libtq_b200.so. There is no fallback: if the CUDA library is missing or
does not export a symbol the header declares, importing callers fail loudly."""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
_LIB = None

u32, i32p, f32, vp = C.c_uint32, C.c_void_p, C.c_float, C.c_void_p

# name -> (restype, argtypes); one entry per symbol include/tq_b200.h declares.
SIGNATURES = {
    "tq_version": (C.c_char_p, []),
    "tq_status_string": (C.c_char_p, [C.c_int]),
    "tq_reshape_and_cache": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32,
                                       u32, u32, f32, vp]),
    "tq_reshape_and_cache_warp_mma": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32,
                                       u32, u32, f32, vp]),
    "tq_reshape_and_cache_tcgen05": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32,
                                       u32, u32, f32, vp]),
    "tq_ingest_set_wait_budget": (None, [C.c_longlong]),
    "tq_reshape_and_cache_varlen": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32,
                                              u32, u32, f32, vp]),
    "tq_reshape_scatter": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32,
                                     u32, u32, f32, vp]),
    "tq_decode_splitk": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32,
                                   u32, u32, u32, u32, u32, u32, u32, f32, f32, vp]),
    "tq_decode_splitk_levels": (C.c_int, [vp] * 12 + [u32] * 12 + [f32, vp]),
    "tq_decode_step": (C.c_int, [vp] * 14 + [u32] * 11 + [f32, f32, vp]),
    "tq_decode_splitk_persistent": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32,
                                              u32, u32, u32, u32, u32, u32, f32, f32, vp]),
    "tq_decode_splitk_precise": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32,
                                           u32, u32, u32, u32, u32, u32, u32, f32, f32, vp]),
    "tq_decode_splitk_nz": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32,
                                      u32, u32, u32, u32, u32, u32, u32, f32, f32, f32, u32, vp]),
    "tq_decode_splitk_elem": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32,
                                        u32, u32, u32, u32, u32, u32, u32, f32, f32, vp]),
    "tq_decode_splitk_mtp": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32,
                                       u32, u32, u32, u32, u32, u32, u32, u32, f32, f32, vp]),
    "tq_decode_splitk_prerotated": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32,
                                              u32, u32, u32, u32, u32, u32, u32, u32, u32, f32, vp]),
    "tq_rotate_query_pi": (C.c_int, [vp, vp, u32, vp, vp, u32, u32]),
    "tq_nz_kv4_import": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, f32]),
    "tq_decode_splitk_static": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32,
                                          u32, u32, u32, u32, u32, u32, u32, u32, f32, f32, vp]),
    "tq_decode_splitk_export": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32,
                                          u32, u32, u32, u32, u32, f32, f32, vp]),
    "tq_decode_choose_splits": (u32, [u32, u32, u32, u32, u32]),
    "tq_decode_worker_census": (C.c_int, [vp, u32]),
    "tq_decode_workspace_floats": (C.c_size_t, [u32, u32, u32, u32, u32]),
    "tq_decode_splitk_partials": (C.c_int, [vp, vp, vp, u32, vp, vp, vp, vp, vp, vp, u32, u32,
                                            u32, u32, u32, u32, u32, u32, u32, u32, u32, f32, f32,
                                            vp]),
    "tq_splitk_combine": (C.c_int, [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, u32, f32,
                                    vp]),
    "tq_rotate_query": (C.c_int, [vp, vp, vp, vp, u32, u32, f32]),
    "tq_hadamard16": (C.c_int, [vp, vp, vp, u32, u32]),
    "tq_lloydmax4_quantize": (C.c_int, [vp, vp, vp, vp, C.c_size_t]),
    "tq_icdf_quantize": (C.c_int, [vp, vp, u32, vp, C.c_size_t]),
    "tq_reshape_and_cache_lloydmax": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32,
                                                u32, f32, vp]),
    "tq_decode_lloydmax_export": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32,
                                            u32, u32, u32, f32, vp]),
    # reference-named launchers (C++ callers; listed so their export is checked)
    "launch_turboquant_reshape_and_cache_a8": (None, None),
    "launch_turboquant_reshape_and_cache_bf16": (None, None),
    "launch_turboquant_reshape_scatter_aiv": (None, None),
    "launch_turboquant_paged_decode_splitk_aic": (None, None),
    "launch_fused_decode_opt": (None, None),
    "launch_fused_decode_opt_raw_query": (None, None),
}


class TqError(RuntimeError):
    def __init__(self, status: int, what: str):
        super().__init__(f"{what}: status {status} ({status_string(status)})")
        self.status = status


def library_path() -> str:
    return os.path.join(PKG, "libtq_b200.so")


def load_library(build_if_missing: bool = True) -> C.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.exists(path):
        if not build_if_missing:
            raise FileNotFoundError(f"{path} is missing; run ascend_micro_harness_b200/build.py")
        from . import build as _build
        _build.build()
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = the library lacks a declared symbol
        if args is not None:
            fn.restype, fn.argtypes = res, args
    _LIB = lib
    return lib


def status_string(status: int) -> str:
    return load_library().tq_status_string(status).decode()
