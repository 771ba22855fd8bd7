"""ctypes binding of libmortar_b200.so (the C ABI declared in include/mortar_b200.h).

There is no fallback: if the shared library is missing the import of any op raises with
the build command, and any non-zero status from the library becomes a Python exception.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libmortar_b200.so")

OK = 0
F32, BF16 = 0, 1
OUT_F32, OUT_BF16, OUT_PLANES = 0, 1, 2
FLAG_SWIGLU, FLAG_ROUND_BF16, FLAG_GATES_ON_INPUT, FLAG_ACCUMULATE = 1, 2, 4, 8
PATH_FLAGS = {"auto": 0, "plain": 16, "staged": 32, "persistent": 48}

_SHAPE_ERRORS = {-2, -3, -4, -5, -6, -7, -8}


class MortarError(RuntimeError):
    def __init__(self, status: int, where: str, detail: str):
        super().__init__(f"{where}: {detail} (status {status})")
        self.status = status


class Stream(C.Structure):
    """mirror of `mortar_stream`"""
    _fields_ = [("grp_codes", C.c_void_p), ("grp_cols", C.c_void_p), ("grp_ptr", C.c_void_p),
                ("n_groups", C.c_int32), ("tile_rows", C.c_int32), ("tile_cols", C.c_int32),
                ("scale", C.c_float), ("row_scale", C.c_void_p)]


class HcPost(C.Structure):
    """mirror of `mortar_hc_post`"""
    _fields_ = [("hres", C.c_void_p), ("hpost_row", C.c_void_p), ("carrier_in", C.c_void_p),
                ("carrier_out", C.c_void_p), ("term", C.c_void_p), ("n_streams", C.c_int32)]


class Sched(C.Structure):
    """mirror of `mortar_sched`"""
    _fields_ = [("step_data", C.c_void_p), ("step_off", C.c_void_p), ("step_meta", C.c_void_p),
                ("panel_step_ptr", C.c_void_p), ("panel_mask", C.c_void_p),
                ("n_tiles", C.c_int64), ("n_runs", C.c_int64), ("n_steps", C.c_int64),
                ("data_units", C.c_int64), ("n_panels", C.c_int32), ("tile_rows", C.c_int32),
                ("tile_cols", C.c_int32), ("swiglu", C.c_int32), ("scale", C.c_float),
                ("arith", C.c_int32)]


class GemvPack(C.Structure):
    """mirror of `mortar_gemv_pack`"""
    _fields_ = [("row_words", C.c_void_p), ("blk_ptr", C.c_void_p), ("blk_col", C.c_void_p), ("items", C.c_void_p),
                ("n_blocks", C.c_int64), ("n_items", C.c_int32), ("out_features", C.c_int32),
                ("in_features", C.c_int32), ("swiglu", C.c_int32), ("scale", C.c_float)]


class Blocks(C.Structure):
    """mirror of `mortar_blocks`"""
    _fields_ = [("data", C.c_void_p), ("pair_ptr", C.c_void_p), ("steps", C.c_void_p), ("n_blocks", C.c_int64),
                ("n_pairs", C.c_int32), ("n_steps", C.c_int32), ("out_features", C.c_int32),
                ("in_features", C.c_int32), ("swiglu", C.c_int32), ("scale", C.c_float)]


_lib = None

_i32, _i64, _f32, _vp = C.c_int32, C.c_int64, C.c_float, C.c_void_p

_SIGNATURES = {
    "mortar_version": (C.c_char_p, []),
    "mortar_status_string": (C.c_char_p, [C.c_int]),
    "mortar_last_cuda_error": (C.c_char_p, []),
    "mortar_validate_bcsr": (C.c_int, [_vp, _vp, _vp, _i32, _i32, _i64]),
    "mortar_stream_groups": (_i64, [_vp, _i32]),
    "mortar_build_stream": (C.c_int, [_vp, _vp, _vp, _i32, _i32, _i64, _vp, _vp, _vp]),
    "mortar_unpack_stream": (C.c_int, [_vp, _vp, _vp, _vp, _i32, _vp, _vp]),
    "mortar_split_blocks": (C.c_int, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "mortar_act_prep": (C.c_int, [_vp, C.c_int, _i64, _i32, _i64, _vp, _f32, _vp, _i32, _i64, _i64, _vp]),
    "mortar_linear": (C.c_int, [C.POINTER(Stream), _vp, _i32, _i64, _i64, _i64, _vp, _i32, _i32, _i64,
                                _i64, _i32, _vp, _i64, _i32, _vp, _i64, _vp, _i64, _vp]),
    "mortar_linear_hc": (C.c_int, [C.POINTER(Stream), _vp, _i32, _i64, _i64, _i64, C.POINTER(HcPost), _i64, _i32,
                                   _vp, _i64, _vp]),
    "mortar_mlp_decode_hc": (C.c_int, [C.POINTER(Stream), C.POINTER(Stream), _vp, C.c_int, _i64, _i64, _vp, _f32,
                                       _vp, _i64, _i32, C.POINTER(HcPost), _i64, _i32, _i32, _vp, _i64, _vp]),
    "mortar_route_flags": (C.c_int, [_vp, _i64, _i64, _vp, _vp, _i32, _vp, _vp, _i32, _vp, _i64, _vp,
                                     _i64, _vp]),
    "mortar_route_gather": (C.c_int, [_vp, _i64, _i64, _i32, _i32, _vp, _vp, _i64, _vp]),
    "mortar_linear_gathered": (C.c_int, [C.POINTER(Stream), _vp, _i32, _i64, _i64, _i64, _vp, _i32, _i32, _i64,
                                         _i64, _i32, _vp, _i64, _i32, _vp, _vp, _i64, _vp]),
    "mortar_mlp_workspace_bytes": (_i64, [_i64, _i32, _i32, _i32]),
    "mortar_mlp_decode": (C.c_int, [C.POINTER(Stream), C.POINTER(Stream), _vp, C.c_int, _i64, _i64, _vp,
                                    _f32, _vp, _i64, _i32, _vp, C.c_int, _i64, _i32, _i32, _vp, _i64,
                                    _vp]),
    "mortar_mlp_static_scratch_bytes": (_i64, []),
    "mortar_mlp_decode_static": (C.c_int, [C.POINTER(Stream), C.POINTER(Stream), _vp, C.c_int, _i64, _i64,
                                           _vp, _f32, _vp, _i64, _i32, _vp, C.c_int, _i64, _i32, _i32,
                                           _vp]),
    "mortar_stack_decode": (C.c_int, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _i64, _i64,
                                      _f32, _i32, _vp, _vp]),
    "mortar_sched_sizes": (C.c_int, [_vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp]),
    "mortar_build_sched": (C.c_int, [_vp, _vp, _vp, _i32, _i32, _i64, _i32, _vp, _vp, _vp, _vp, _vp]),
    "mortar_linear_tc": (C.c_int, [C.POINTER(Sched), _vp, _i64, _i64, _vp, _i64, _vp, _i64, _i32, _vp]),
    "mortar_gemv_xprep": (C.c_int, [_vp, _i32, _i64, _i64, _i64, _i32, _vp, _vp]),
    "mortar_gemv_xprep_swiglu": (C.c_int, [_vp, _i64, _i64, _i32, _i32, _vp, _vp]),
    "mortar_gemv_blocks": (C.c_int, [C.POINTER(GemvPack), _vp, _i64, _i32, _vp, _i32, _i32, _i64, _i64, _vp]),
    "mortar_gemv_blocks_error": (C.c_int, [_vp, _i32]),
    "mortar_linear_blocks": (C.c_int, [C.POINTER(Blocks), _vp, _i64, _i64, _vp, _i64, _vp, _i64, _i32, _vp]),
    "mortar_linear_blocks_mode": (C.c_int, [_i32]),
    "mortar_mlp_prefill_blocks": (C.c_int, [C.POINTER(Blocks), C.POINTER(Blocks), _vp, _i64, _i64, _vp, _i64, _i32,
                                            _vp, _i64, _vp, _i64, _vp]),
    "mortar_sched_sizes_i8": (C.c_int, [_vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp]),
    "mortar_build_sched_i8": (C.c_int, [_vp, _vp, _vp, _i32, _i32, _i64, _i32, _vp, _vp, _vp, _vp, _vp]),
    "mortar_quantize_rows": (C.c_int, [_vp, _i64, _i64, _i32, _vp, _i64, _vp, _vp]),
    "mortar_linear_tc_i8": (C.c_int, [C.POINTER(Sched), _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _i32, _vp]),
    "mortar_mlp_prefill": (C.c_int, [C.POINTER(Sched), C.POINTER(Sched), _vp, _i64, _i64, _vp, _i64,
                                     _i32, _vp, _i64, _vp, _i64, _vp]),
    "mortar_sdd_tiles": (C.c_int, [_vp, _i64, _vp, _i64, _i64, _vp, _vp, _i32, _i32, _vp, _vp, _i32, _vp, _i32, _vp]),
    "mortar_sdd_blocks": (C.c_int, [_vp, _i64, _vp, _i64, _i64, _i32, _i32, _vp, _vp, _i32, _i32, _i64, _vp, _i64,
                                    _vp, _i32, _vp]),
    "mortar_sdd_error": (C.c_int, [_vp, _i32]),
    "mortar_prefill_error": (C.c_int, [_vp, _i32]),
    "mortar_linear_error": (C.c_int, [_vp, _i32]),
    "mortar_router_gates": (C.c_int, [_vp, _i64, _i64, _i32, _vp, _vp, _vp, _vp, _f32, _vp, _vp, _i32, _vp,
                                      _i32, _i32, _vp, _vp, _i64, _vp]),
}

# entry points added by later translation units; bound when present in the header list
_OPTIONAL = {}


def exported_symbols() -> list[str]:
    return list(_SIGNATURES) + list(_OPTIONAL)


def lib():
    """Load the shared library once.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: the CUDA extension must be built first "
                f"(python {os.path.join(PKG, 'build.py')}); there is no CPU fallback")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in {**_SIGNATURES, **_OPTIONAL}.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int, where: str) -> None:
    if status == OK:
        return
    L = lib()
    detail = L.mortar_status_string(int(status)).decode()
    if status == -9:
        detail += ": " + L.mortar_last_cuda_error().decode()
    err = MortarError(int(status), where, detail)
    if status in _SHAPE_ERRORS or status == -1:
        raise ValueError(str(err)) from err
    raise err
