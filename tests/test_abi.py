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
                              "batch_norm_q", "instance_norm_q", "normalization_q", "conv3d_q", "pool3d_q", "gather_nd_q", "lstm_step_f32", "reverse_q", "convert_fp16", "scatter_nd_q"]):
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


def _refused(l, name, params, code, text):
    rc = getattr(l, "b200k_" + name)(ctypes.byref(params), None)
    assert rc == code, (name, rc, l.b200k_last_error())
    assert text in l.b200k_last_error(), (name, l.b200k_last_error())


def test_malformed_parameters_are_refused_before_any_launch():
    """Argument checks of the layer entry points run on the host: they return an error code and a message, with or
    without a device."""
    l = lib.load_library()
    buf = (ctypes.c_uint8 * 4096)()
    ptr = ctypes.addressof(buf)

    def tensor(dtype=_abi.S8, scale=0.05):
        t = _abi.QTensor()
        t.data, t.dtype, t.scale, t.zero_point = ptr, dtype, scale, 0
        return t
    p = _abi.ViewCopyParams(); p.x, p.y, p.rank = tensor(), tensor(), 7
    _refused(l, "view_copy_q", p, _abi.E_UNSUPPORTED, b"rank 7")
    p = _abi.ViewCopyParams(); p.x, p.y, p.rank = tensor(_abi.S8), tensor(_abi.U8), 1
    _refused(l, "view_copy_q", p, _abi.E_UNSUPPORTED, b"types differ")
    p = _abi.EltwiseParams(); p.a, p.b, p.out, p.rank, p.op = tensor(), tensor(), tensor(), 1, 9
    _refused(l, "eltwise_q8", p, _abi.E_UNSUPPORTED, b"unsupported binary operation")
    p = _abi.UnaryParams(); p.x, p.y, p.count, p.operation = tensor(), tensor(), 4, 10
    _refused(l, "unary_q", p, _abi.E_UNSUPPORTED, b"unsupported unary operation")
    p = _abi.ActivationParams(); p.x, p.y, p.count, p.function, p.a, p.b = tensor(), tensor(), 4, 50, 0.0, 1.0
    _refused(l, "activation_q8", p, _abi.E_INVALID, b"FakeQuantization takes Float32")
    p = _abi.PadParams(); p.x, p.y, p.rank, p.mode = tensor(), tensor(), 1, 1
    p.shape[0], p.pad_before[0], p.pad_after[0] = 4, 4, 0
    _refused(l, "pad_q", p, _abi.E_INVALID, b"mirrored padding wider")
    p = _abi.ArgMinMaxParams(); p.x, p.y, p.outer, p.axis_size, p.inner, p.function = tensor(), ptr, 1, 4, 1, 2
    _refused(l, "arg_min_max_q", p, _abi.E_INVALID, b"neither Min")
    p = _abi.GatherNdParams(); p.x, p.y, p.indices, p.n_indices, p.nd, p.inner = tensor(), tensor(), ptr, 1, 9, 1
    _refused(l, "gather_nd_q", p, _abi.E_INVALID, b"bad shape")
    p = _abi.InstanceNormParams(); p.x, p.y, p.n, p.c, p.hw = tensor(), tensor(), 1, 1, 4
    _refused(l, "instance_norm_q", p, _abi.E_UNSUPPORTED, b"Float32 tensors only")
    p = _abi.NormalizationParams(); p.x, p.y, p.n, p.c, p.h, p.w, p.channel_type, p.norm_size = tensor(), tensor(), 1, 2, 2, 2, 1, 3
    _refused(l, "normalization_q", p, _abi.E_UNSUPPORTED, b"Within indexes the tensor as NCHW")
    p = _abi.Conv3dParams(); p.x, p.w, p.y = tensor(_abi.F32), tensor(_abi.S8), tensor(_abi.F32)
    for k in ("n", "d", "h", "wd", "c", "od", "oh", "ow", "oc", "kd", "kh", "kw", "stride_d", "stride_h", "stride_w", "dil_d", "dil_h", "dil_w"):
        setattr(p, k, 1)
    _refused(l, "conv3d_q", p, _abi.E_UNSUPPORTED, b"Float32 input needs Float32 weights")
    p = _abi.LstmParams(); p.batch, p.input_size, p.num_units, p.output_size = 1, 2, 4, 3
    for k in ("input", "output_state_in", "cell_state_in", "output_state_out", "cell_state_out", "output",
              "w_i2f", "w_i2c", "w_i2o", "w_r2f", "w_r2c", "w_r2o", "b_f", "b_c", "b_o"):
        setattr(p, k, ptr)
    p.activation = 4
    _refused(l, "lstm_step_f32", p, _abi.E_INVALID, b"without projection the output size")
    p.output_size, p.activation = 4, 2
    _refused(l, "lstm_step_f32", p, _abi.E_UNSUPPORTED, b"unsupported activation function")
    p = _abi.ReverseParams(); p.x, p.y, p.axes, p.rank = tensor(), tensor(_abi.U8), ptr, 2
    _refused(l, "reverse_q", p, _abi.E_UNSUPPORTED, b"one supported element type")
