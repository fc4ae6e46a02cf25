"""The C-ABI library loads on a machine without a GPU and exports every symbol include/b200k.h declares;
host-only helpers behave; device entry points fail with a status code (not a crash) when no device exists."""
import ctypes
import os
import re

import numpy as np

from armnn_b200 import _abi, lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_loads_and_exports_every_declared_symbol():
    l = lib.load_library()
    header = open(os.path.join(ROOT, "include", "b200k.h")).read()
    declared = set(re.findall(r"\b(b200k_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in the header"
    for sym in sorted(declared):
        assert hasattr(l, sym), "libb200k.so does not export %s" % sym
    assert declared == set(_abi.EXPORTED_SYMBOLS), declared ^ set(_abi.EXPORTED_SYMBOLS)
    assert b"sm_100a" in l.b200k_version()


def test_struct_layouts_match_the_header():
    l = lib.load_library()
    l.b200k_sizeof_params.restype = ctypes.c_size_t
    for i, name in enumerate(["conv2d_q8", "fully_connected_q8", "batch_matmul_q8", "pool2d_q8", "mean_hw_q8",
                              "eltwise_q8", "activation_q8", "softmax_q8", "convert_q", "qlstm_step", "pad_q",
                              "view_copy_q", "resize_q", "reduce_q", "unary_q", "arg_min_max_q", "gather_q",
                              "batch_norm_q", "instance_norm_q", "normalization_q", "conv3d_q", "pool3d_q", "gather_nd_q", "lstm_step_f32", "reverse_q"]):
        assert l.b200k_sizeof_params(i) == ctypes.sizeof(_abi.KERNEL_ENTRY_POINTS[name]), name


def test_activation_clamp_matches_quantize_formula():
    l = lib.load_library()
    lo, hi = ctypes.c_int32(), ctypes.c_int32()
    assert l.b200k_activation_clamp(1, 0, 0, 0.05, -128, _abi.S8, ctypes.byref(lo), ctypes.byref(hi)) == 0
    assert (lo.value, hi.value) == (-128, 127)
    assert l.b200k_activation_clamp(1, 0, 0, 0.05, 3, _abi.S8, ctypes.byref(lo), ctypes.byref(hi)) == 0
    assert (lo.value, hi.value) == (3, 127)
    assert l.b200k_activation_clamp(2, 6.0, 0.0, 0.05, 0, _abi.U8, ctypes.byref(lo), ctypes.byref(hi)) == 0
    assert (lo.value, hi.value) == (0, 120)
    assert l.b200k_activation_clamp(0, 0, 0, 1.0, 0, _abi.U8, ctypes.byref(lo), ctypes.byref(hi)) == 0
    assert (lo.value, hi.value) == (0, 255)
    assert l.b200k_activation_clamp(7, 0, 0, 1.0, 0, _abi.U8, ctypes.byref(lo), ctypes.byref(hi)) == _abi.E_INVALID


def test_no_device_is_an_error_code_not_a_crash():
    l = lib.load_library()
    if l.b200k_device_count() == 0:
        assert l.b200k_device_open(0) == _abi.E_NODEVICE
        assert b"no CUDA device" in l.b200k_last_error()
