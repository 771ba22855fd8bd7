"""Argument validation of the device entry points, which happens on the host before any CUDA call:
NULL pointers, shapes, alignment and modes come back as status codes.  Runs without a GPU (the
pointers are host addresses that are never dereferenced)."""
import ctypes as C

import numpy as np

import mortar_b200 as mb

L = mb._lib.lib()
NULL, SHAPE, ALIGN, DTYPE, CAP = -1, -2, -6, -7, -8


def _buf(nbytes=4096):
    a = np.zeros(nbytes + 256, dtype=np.uint8)
    base = a.ctypes.data
    return a, C.c_void_p((base + 255) & ~255)


def test_block_path_entry_points_validate():
    keep, p = _buf()
    blk = mb._lib.Blocks(p, p, p, 1, 1, 1, 256, 256, 0, 1.0)
    f = L.mortar_linear_blocks
    assert f(None, p, 256, 8, p, 256, None, 0, 0, None) == NULL
    assert f(C.byref(blk), None, 256, 8, p, 256, None, 0, 0, None) == NULL
    assert f(C.byref(blk), p, 128, 8, p, 256, None, 0, 0, None) == SHAPE          # ldx < in_features
    assert f(C.byref(blk), p, 256, -1, p, 256, None, 0, 0, None) == SHAPE
    assert f(C.byref(blk), C.c_void_p(p.value + 2), 256, 8, p, 256, None, 0, 0, None) == ALIGN
    assert f(C.byref(blk), p, 256, 8, p, 256, p, 4, 16, None) == SHAPE             # gates without a swiglu layout
    assert f(C.byref(blk), p, 256, 0, p, 256, None, 0, 0, None) == 0               # no rows: nothing to do
    sw = mb._lib.Blocks(p, p, p, 1, 1, 1, 2 * 192, 256, 1, 1.0)                    # one pair of block rows cannot hold 192 hidden columns
    assert f(C.byref(sw), p, 256, 8, p, 192, None, 0, 0, None) == SHAPE
    g = L.mortar_mlp_prefill_blocks
    assert g(C.byref(blk), C.byref(blk), p, 256, 8, None, 0, 0, p, 256, p, 1 << 20, None) == SHAPE   # first must be swiglu


def test_backward_and_gemv_entry_points_validate():
    keep, p = _buf()
    f = L.mortar_sdd_blocks
    assert f(None, 256, p, 256, 8, 256, 256, p, p, 1, 1, 4, None, 0, p, 0, None) == NULL
    assert f(p, 128, p, 256, 8, 256, 256, p, p, 1, 1, 4, None, 0, p, 0, None) == SHAPE   # ld_dy < out_features
    assert f(p, 256, p, 256, 8, 256, 256, p, p, 1, 1, 4, None, 0, p, 5, None) == DTYPE
    assert f(p, 256, p, 256, 8, 256, 256, p, p, 0, 1, 4, None, 0, p, 0, None) == 0        # no blocks
    assert f(p, 256, p, 256, 1000, 256, 256, p, p, 1, 4, 4, None, 0, p, 0, None) == CAP   # splits need scratch
    pack = mb._lib.GemvPack(p, p, p, p, 1, 1, 256, 256, 0, 1.0)
    g = L.mortar_gemv_blocks
    assert g(None, p, 1, 3, p, 0, 0, 0, 256, None) == NULL
    assert g(C.byref(pack), p, 6, 3, p, 0, 0, 0, 256, None) == SHAPE                       # 18 columns > 16
    assert g(C.byref(pack), p, 1, 3, p, 7, 0, 0, 256, None) == DTYPE
    assert g(C.byref(pack), p, 1, 3, p, 0, 0, 0, 128, None) == SHAPE                       # ld_out < out_features
    bad = mb._lib.GemvPack(p, p, p, p, 1, 1, 200, 256, 0, 1.0)
    assert g(C.byref(bad), p, 1, 3, p, 0, 0, 0, 256, None) == SHAPE                        # not a multiple of 128
    assert L.mortar_gemv_xprep(p, 3, 256, 256, 6, 256, p, None) == SHAPE
    assert L.mortar_gemv_xprep(p, 3, 256, 256, 1, 250, p, None) == SHAPE
    assert L.mortar_gemv_xprep_swiglu(None, 512, 1, 256, 3, p, None) == NULL


def test_int8_arm_entry_points_validate():
    keep, p = _buf()
    assert L.mortar_quantize_rows(None, 256, 8, 256, p, 256, p, None) == NULL
    assert L.mortar_quantize_rows(p, 256, 8, 250, p, 256, p, None) == SHAPE                # cols not a multiple of 8
    assert L.mortar_quantize_rows(p, 256, 8, 256, p, 250, p, None) == SHAPE
    assert L.mortar_quantize_rows(p, 256, 0, 256, p, 256, p, None) == 0
    sched = mb._lib.Sched(p, p, p, p, p, 1, 1, 1, 1, 2, 16, 16, 0, 1.0, 0)                 # a bf16 schedule
    assert L.mortar_linear_tc_i8(C.byref(sched), p, 256, p, 8, p, 256, None, 0, 0, None) == DTYPE
    assert L.mortar_linear_tc_i8(C.byref(sched), p, 256, None, 8, p, 256, None, 0, 0, None) == NULL
