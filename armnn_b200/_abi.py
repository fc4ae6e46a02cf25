"""ctypes mirror of include/b200k.h: the parameter structs and function prototypes of the C ABI.

The structs are declared once here and used for two different shared objects: the product library
(libb200k.so, device pointers) and — in tests only — the CPU oracle, which takes the same structs
with host pointers.  Field order and types must match the header exactly.
"""
import ctypes as C

U8, S8, S16, S32, F32 = 0, 1, 2, 3, 4

OK, E_INVALID, E_CUDA, E_UNSUPPORTED, E_NODEVICE, E_TIMEOUT, E_TOOBIG = 0, -1, -2, -3, -4, -5, -6


class QTensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int32), ("scale", C.c_float),
                ("zero_point", C.c_int32), ("scales", C.c_void_p)]


class Conv2dParams(C.Structure):
    _fields_ = [("x", QTensor), ("w", QTensor), ("bias", QTensor), ("y", QTensor),
                ("n", C.c_int32), ("h", C.c_int32), ("wd", C.c_int32), ("c", C.c_int32),
                ("oh", C.c_int32), ("ow", C.c_int32), ("oc", C.c_int32),
                ("kh", C.c_int32), ("kw", C.c_int32),
                ("stride_h", C.c_int32), ("stride_w", C.c_int32),
                ("pad_top", C.c_int32), ("pad_left", C.c_int32),
                ("dil_h", C.c_int32), ("dil_w", C.c_int32),
                ("clamp_lo", C.c_int32), ("clamp_hi", C.c_int32),
                ("acc_out", C.c_void_p), ("algo", C.c_int32), ("packed", C.c_void_p),
                ("add_operand", QTensor), ("add_out", QTensor),
                ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t), ("selftest_us", C.c_int32)]


class FcParams(C.Structure):
    _fields_ = [("x", QTensor), ("w", QTensor), ("bias", QTensor), ("y", QTensor),
                ("m", C.c_int32), ("k", C.c_int32), ("n", C.c_int32), ("transpose_w", C.c_int32),
                ("clamp_lo", C.c_int32), ("clamp_hi", C.c_int32),
                ("acc_out", C.c_void_p), ("algo", C.c_int32), ("packed", C.c_void_p)]


class BmmParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor), ("out", QTensor),
                ("batch", C.c_int32), ("m", C.c_int32), ("k", C.c_int32), ("n", C.c_int32),
                ("transpose_x", C.c_int32), ("transpose_y", C.c_int32),
                ("batch_stride_x", C.c_int64), ("batch_stride_y", C.c_int64),
                ("acc_out", C.c_void_p), ("algo", C.c_int32)]


class Pool2dParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor),
                ("n", C.c_int32), ("h", C.c_int32), ("wd", C.c_int32), ("c", C.c_int32),
                ("oh", C.c_int32), ("ow", C.c_int32),
                ("pool_h", C.c_int32), ("pool_w", C.c_int32), ("stride_h", C.c_int32), ("stride_w", C.c_int32),
                ("pad_top", C.c_int32), ("pad_bottom", C.c_int32), ("pad_left", C.c_int32), ("pad_right", C.c_int32),
                ("pool_type", C.c_int32), ("padding_method", C.c_int32)]


class MeanParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor),
                ("n", C.c_int32), ("h", C.c_int32), ("wd", C.c_int32), ("c", C.c_int32)]


class EltwiseParams(C.Structure):
    _fields_ = [("a", QTensor), ("b", QTensor), ("out", QTensor), ("rank", C.c_int32),
                ("shape_a", C.c_int32 * 4), ("shape_b", C.c_int32 * 4), ("shape_out", C.c_int32 * 4),
                ("op", C.c_int32), ("clamp_lo", C.c_int32), ("clamp_hi", C.c_int32)]


class ActivationParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor), ("count", C.c_int64), ("function", C.c_int32),
                ("a", C.c_float), ("b", C.c_float)]


class SoftmaxParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor), ("outer", C.c_int32), ("axis_size", C.c_int32),
                ("inner", C.c_int32), ("beta", C.c_float)]


class ArgMinMaxParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", C.c_void_p), ("outer", C.c_int32), ("axis_size", C.c_int32), ("inner", C.c_int32),
                ("function", C.c_int32), ("out_int64", C.c_int32)]


class GatherParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor), ("indices", C.c_void_p), ("outer", C.c_int32), ("axis_size", C.c_int32),
                ("inner", C.c_int32), ("n_indices", C.c_int32)]


class ConvertFp16Params(C.Structure):
    _fields_ = [("x", C.c_void_p), ("y", C.c_void_p), ("count", C.c_int64), ("to_half", C.c_int32)]


class ScatterNdParams(C.Structure):
    _fields_ = [("x", QTensor), ("updates", QTensor), ("y", QTensor), ("indices", C.c_void_p), ("n_indices", C.c_int32),
                ("nd", C.c_int32), ("inner", C.c_int32), ("dims", C.c_int32 * 8), ("function", C.c_int32)]


class ReverseParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor), ("axes", C.c_void_p), ("n_axes", C.c_int32), ("rank", C.c_int32),
                ("shape", C.c_int32 * 6)]


class GatherNdParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor), ("indices", C.c_void_p), ("n_indices", C.c_int32), ("nd", C.c_int32),
                ("inner", C.c_int32), ("dims", C.c_int32 * 8)]


class BatchNormParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor), ("mean", QTensor), ("variance", QTensor), ("beta", QTensor), ("gamma", QTensor),
                ("n", C.c_int32), ("c", C.c_int32), ("hw", C.c_int64), ("nchw", C.c_int32), ("eps", C.c_float),
                ("scratch", C.c_void_p)]


class InstanceNormParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor), ("n", C.c_int32), ("c", C.c_int32), ("hw", C.c_int64), ("nchw", C.c_int32),
                ("gamma", C.c_float), ("beta", C.c_float), ("eps", C.c_float)]


class NormalizationParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor), ("n", C.c_int32), ("c", C.c_int32), ("h", C.c_int32), ("w", C.c_int32),
                ("nchw", C.c_int32), ("channel_type", C.c_int32), ("norm_size", C.c_uint32),
                ("alpha", C.c_float), ("beta", C.c_float), ("kappa", C.c_float)]


class Conv3dParams(C.Structure):
    _fields_ = [("x", QTensor), ("w", QTensor), ("bias", QTensor), ("y", QTensor)] + [(k, C.c_int32) for k in (
        "n", "d", "h", "wd", "c", "od", "oh", "ow", "oc", "kd", "kh", "kw", "stride_d", "stride_h", "stride_w",
        "pad_front", "pad_top", "pad_left", "dil_d", "dil_h", "dil_w", "clamp_lo", "clamp_hi")]


class Pool3dParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor)] + [(k, C.c_int32) for k in (
        "n", "d", "h", "wd", "c", "od", "oh", "ow", "pool_d", "pool_h", "pool_w", "stride_d", "stride_h", "stride_w",
        "pad_front", "pad_back", "pad_top", "pad_bottom", "pad_left", "pad_right", "pool_type", "padding_method")]


class ConvertParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor), ("count", C.c_int64)]


class PadParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor), ("rank", C.c_int32), ("shape", C.c_int32 * 4),
                ("pad_before", C.c_int32 * 4), ("pad_after", C.c_int32 * 4), ("pad_value", C.c_float), ("mode", C.c_int32)]


class ViewCopyParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor), ("rank", C.c_int32), ("shape", C.c_int32 * 6),
                ("src_strides", C.c_int64 * 6), ("dst_strides", C.c_int64 * 6),
                ("src_offset", C.c_int64), ("dst_offset", C.c_int64)]


class UnaryParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor), ("count", C.c_int64), ("operation", C.c_int32)]


class ReduceParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor), ("rank", C.c_int32), ("shape", C.c_int32 * 6), ("axis_mask", C.c_int32),
                ("op", C.c_int32)]


class ResizeParams(C.Structure):
    _fields_ = [("x", QTensor), ("y", QTensor), ("n", C.c_int32), ("c", C.c_int32), ("in_h", C.c_int32), ("in_w", C.c_int32),
                ("out_h", C.c_int32), ("out_w", C.c_int32), ("method", C.c_int32), ("align_corners", C.c_int32),
                ("half_pixel_centers", C.c_int32), ("nchw", C.c_int32)]


_P, _F, _I = C.c_void_p, C.c_float, C.c_int32


class QLstmParams(C.Structure):
    _fields_ = [
        ("batch", _I), ("input_size", _I), ("num_units", _I), ("output_size", _I),
        ("input", _P), ("input_scale", _F), ("input_zp", _I),
        ("output_state_in", _P), ("output_state_scale", _F), ("output_state_zp", _I),
        ("cell_state_in", _P), ("cell_state_scale", _F),
        ("output_state_out", _P), ("cell_state_out", _P),
        ("output", _P), ("output_scale", _F), ("output_zp", _I),
        ("w_i2i", _P), ("w_i2f", _P), ("w_i2c", _P), ("w_i2o", _P),
        ("s_i2i", _F), ("s_i2f", _F), ("s_i2c", _F), ("s_i2o", _F),
        ("w_r2i", _P), ("w_r2f", _P), ("w_r2c", _P), ("w_r2o", _P),
        ("s_r2i", _F), ("s_r2f", _F), ("s_r2c", _F), ("s_r2o", _F),
        ("w_c2i", _P), ("w_c2f", _P), ("w_c2o", _P),
        ("s_c2i", _F), ("s_c2f", _F), ("s_c2o", _F),
        ("b_i", _P), ("b_f", _P), ("b_c", _P), ("b_o", _P),
        ("s_bi", _F), ("s_bf", _F), ("s_bc", _F), ("s_bo", _F),
        ("ln_i", _P), ("ln_f", _P), ("ln_c", _P), ("ln_o", _P),
        ("s_lni", _F), ("s_lnf", _F), ("s_lnc", _F), ("s_lno", _F),
        ("w_proj", _P), ("s_proj", _F),
        ("b_proj", _P), ("s_bproj", _F),
        ("cell_clip", _F), ("projection_clip", _F),
        ("input_intermediate_scale", _F), ("forget_intermediate_scale", _F),
        ("cell_intermediate_scale", _F), ("output_intermediate_scale", _F),
        ("hidden_state_scale", _F), ("hidden_state_zp", _I),
    ]


class LstmParams(C.Structure):
    _fields_ = ([("batch", _I), ("input_size", _I), ("num_units", _I), ("output_size", _I),
                 ("input", _P), ("input_stride", C.c_int64), ("output_state_in", _P), ("cell_state_in", _P),
                 ("output_state_out", _P), ("cell_state_out", _P), ("output", _P), ("output_stride", C.c_int64)] +
                [(k, _P) for k in ("w_i2i", "w_i2f", "w_i2c", "w_i2o", "w_r2i", "w_r2f", "w_r2c", "w_r2o", "w_c2i", "w_c2f", "w_c2o",
                                   "b_i", "b_f", "b_c", "b_o", "ln_i", "ln_f", "ln_c", "ln_o", "w_proj", "b_proj")] +
                [("activation", _I), ("cell_clip", _F), ("projection_clip", _F), ("layer_norm_eps", _F)])


# name -> (parameter struct, takes a stream argument in the product library)
KERNEL_ENTRY_POINTS = {
    "conv2d_q8": Conv2dParams,
    "dwconv2d_q8": Conv2dParams,
    "transpose_conv2d_q8": Conv2dParams,
    "conv2d_f32": Conv2dParams,
    "dwconv2d_f32": Conv2dParams,
    "fully_connected_f32": FcParams,
    "fully_connected_q8": FcParams,
    "batch_matmul_q8": BmmParams,
    "batch_matmul_f32": BmmParams,
    "pool2d_q8": Pool2dParams,
    "mean_hw_q8": MeanParams,
    "eltwise_q8": EltwiseParams,
    "activation_q8": ActivationParams,
    "softmax_q8": SoftmaxParams,
    "log_softmax_q": SoftmaxParams,
    "l2_normalization_q": SoftmaxParams,
    "arg_min_max_q": ArgMinMaxParams,
    "gather_q": GatherParams,
    "reverse_q": ReverseParams,
    "scatter_nd_q": ScatterNdParams,
    "gather_nd_q": GatherNdParams,
    "batch_norm_q": BatchNormParams,
    "instance_norm_q": InstanceNormParams,
    "normalization_q": NormalizationParams,
    "conv3d_q": Conv3dParams,
    "pool3d_q": Pool3dParams,
    "convert_q": ConvertParams,
    "cast_q": ConvertParams,
    "convert_fp16": ConvertFp16Params,
    "qlstm_step": QLstmParams,
    "lstm_step_f32": LstmParams,
    "pad_q": PadParams,
    "view_copy_q": ViewCopyParams,
    "resize_q": ResizeParams,
    "reduce_q": ReduceParams,
    "unary_q": UnaryParams,
}

# every symbol include/b200k.h declares
EXPORTED_SYMBOLS = ["b200k_" + k for k in KERNEL_ENTRY_POINTS] + [
    "b200k_device_open", "b200k_device_count", "b200k_last_error", "b200k_version",
    "b200k_activation_clamp", "b200k_conv2d_pack_bytes", "b200k_conv2d_pack", "b200k_conv2d_scratch_bytes", "b200k_conv2d_q8_static", "b200k_sizeof_params", "b200k_poll_status",
    "b200k_kernel_launches", "b200k_int8_mma_peak",
]


def declare_product(lib):
    """Attach prototypes to a loaded libb200k.so."""
    for name, struct in KERNEL_ENTRY_POINTS.items():
        fn = getattr(lib, "b200k_" + name)
        fn.argtypes = [C.POINTER(struct), C.c_void_p]
        fn.restype = C.c_int
    lib.b200k_kernel_launches.argtypes = []
    lib.b200k_kernel_launches.restype = C.c_ulonglong
    lib.b200k_device_open.argtypes = [C.c_int]
    lib.b200k_device_open.restype = C.c_int
    lib.b200k_device_count.restype = C.c_int
    lib.b200k_last_error.restype = C.c_char_p
    lib.b200k_version.restype = C.c_char_p
    lib.b200k_activation_clamp.argtypes = [C.c_int, C.c_float, C.c_float, C.c_float, C.c_int32, C.c_int32,
                                           C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.b200k_activation_clamp.restype = C.c_int
    lib.b200k_conv2d_pack_bytes.argtypes = [C.c_int32] * 4
    lib.b200k_conv2d_pack_bytes.restype = C.c_size_t
    lib.b200k_conv2d_pack.argtypes = [C.POINTER(Conv2dParams), C.c_void_p, C.c_void_p]
    lib.b200k_conv2d_pack.restype = C.c_int
    lib.b200k_poll_status.restype = C.c_int
    lib.b200k_int8_mma_peak.argtypes = [C.POINTER(C.c_double), C.c_void_p]
    lib.b200k_int8_mma_peak.restype = C.c_int
    lib.b200k_conv2d_q8_static.argtypes = [C.POINTER(Conv2dParams), C.c_void_p]
    lib.b200k_conv2d_q8_static.restype = C.c_int
    lib.b200k_conv2d_scratch_bytes.argtypes = [C.POINTER(Conv2dParams)]
    lib.b200k_conv2d_scratch_bytes.restype = C.c_size_t
    return lib
