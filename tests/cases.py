"""The seeded parity cases, shared by the CPU tests (oracle vs golden / real CpuRef), the fixture generator and
the GPU tests (CUDA vs oracle).  Every case is small enough for the oracle to finish in well under a second,
and covers the edge cases the reference's own layer tests exercise: odd channel counts, strides, dilation,
padding wider than the kernel, per-axis and per-tensor quantisation, both 8-bit signednesses and their mix,
broadcast, ragged tails that do not fill a vector or a tile."""
import numpy as np

from q8util import (RANGE, NP_OF, FcCase, MoveCase, SimpleCase, _abi, activation_clamp, qt, qt_out, random_conv_case,
                    random_fc_case, random_qlstm_case)

U8, S8, S16, S32, F32 = _abi.U8, _abi.S8, _abi.S16, _abi.S32, _abi.F32


def conv_cases():
    c = {}
    # the single-layer benchmark config, as specified (output scale 0.05 saturates ~2/3 of outputs) ...
    c["config1_as_specified"] = lambda: random_conv_case(1234, 1, 56, 56, 64, 64, 3, 3, pad=(1, 1, 1, 1), act=(1, 0, 0),
                                                         y_scale=0.05, y_zp=-128)
    # ... and with an output scale that leaves most values unsaturated
    c["config1_unsaturated"] = lambda: random_conv_case(1234, 1, 56, 56, 64, 64, 3, 3, pad=(1, 1, 1, 1), act=(1, 0, 0))
    c["1x1_s1"] = lambda: random_conv_case(1, 2, 14, 14, 64, 128, 1, 1)
    c["1x1_s2_shortcut"] = lambda: random_conv_case(2, 2, 14, 14, 64, 96, 1, 1, stride=(2, 2))
    c["3x3_s2"] = lambda: random_conv_case(3, 1, 15, 15, 32, 48, 3, 3, stride=(2, 2), pad=(1, 1, 1, 1), act=(1, 0, 0))
    c["7x7_s2_stem_c3"] = lambda: random_conv_case(4, 1, 32, 32, 3, 64, 7, 7, stride=(2, 2), pad=(2, 3, 2, 3), act=(1, 0, 0))
    c["3x3_dilation2"] = lambda: random_conv_case(5, 1, 12, 12, 16, 16, 3, 3, pad=(2, 2, 2, 2), dil=(2, 2))
    c["odd_channels_c5_oc7"] = lambda: random_conv_case(6, 2, 9, 7, 5, 7, 3, 3, pad=(1, 1, 1, 1))
    c["c4_words"] = lambda: random_conv_case(7, 1, 10, 10, 12, 20, 3, 3, pad=(1, 1, 1, 1))
    c["pad_wider_than_kernel"] = lambda: random_conv_case(8, 1, 6, 6, 16, 16, 3, 3, pad=(4, 4, 4, 4))
    c["u8_u8_per_tensor_relu6"] = lambda: random_conv_case(9, 1, 12, 12, 32, 32, 3, 3, pad=(1, 1, 1, 1), x_dtype=U8, w_dtype=U8,
                                                           y_dtype=U8, per_axis=False, x_q=(0.02, 121), y_zp=0, act=(2, 6.0, 0.0),
                                                           y_scale=0.04)
    c["u8_act_s8_per_axis"] = lambda: random_conv_case(10, 1, 8, 8, 16, 24, 1, 1, x_dtype=U8, y_dtype=U8, x_q=(0.5, 128))
    c["s8_per_tensor_no_bias"] = lambda: random_conv_case(11, 1, 8, 8, 16, 16, 3, 3, pad=(1, 1, 1, 1), per_axis=False, bias=False)
    c["rect_kernel_3x1_stride_1x2"] = lambda: random_conv_case(12, 1, 9, 11, 8, 8, 3, 1, stride=(1, 2), pad=(1, 1, 0, 0))
    c["k_not_multiple_of_64"] = lambda: random_conv_case(13, 1, 5, 5, 48, 80, 3, 3, pad=(1, 1, 1, 1))
    c["fused_add_relu_1x1"] = lambda: random_conv_case(14, 2, 14, 14, 64, 256, 1, 1, act=(1, 0, 0), fused_add=True)
    c["fused_add_3x3_odd"] = lambda: random_conv_case(15, 1, 7, 9, 12, 20, 3, 3, pad=(1, 1, 1, 1), fused_add=True)
    c["fused_add_u8"] = lambda: random_conv_case(16, 1, 8, 8, 16, 24, 1, 1, x_dtype=U8, y_dtype=U8, x_q=(0.5, 128), fused_add=True)
    # 1x1 convolutions that run as a GEMM over groups of 2, 4 or 8 consecutive pixels (block-diagonal weights): the
    # MobileNet-v2 bottleneck shapes, every weight type, a pixel count the group does not divide (another path)
    c["grouped_c16_oc96_u8_everything"] = lambda: random_conv_case(17, 2, 28, 28, 16, 96, 1, 1, x_dtype=U8, w_dtype=U8, y_dtype=U8,
                                                                   per_axis=False, x_q=(0.02, 117), y_zp=0, act=(2, 6.0, 0.0),
                                                                   y_scale=0.02)
    c["c24_oc144_u8_everything_padded_input"] = lambda: random_conv_case(18, 2, 28, 28, 24, 144, 1, 1, x_dtype=U8, w_dtype=U8, y_dtype=U8,
                                                                    per_axis=False, x_q=(0.02, 131), y_zp=0, act=(2, 6.0, 0.0),
                                                                    y_scale=0.02)
    c["grouped_c96_oc24_u8_everything"] = lambda: random_conv_case(19, 2, 28, 28, 96, 24, 1, 1, x_dtype=U8, w_dtype=U8, y_dtype=U8,
                                                                   per_axis=False, x_q=(0.02, 3))
    c["grouped_c8_oc40_per_axis"] = lambda: random_conv_case(20, 1, 12, 12, 8, 40, 1, 1, act=(1, 0, 0))
    c["grouped_c12_oc20_s8_weight_zero_point"] = lambda: random_conv_case(21, 1, 8, 8, 12, 20, 1, 1, per_axis=False, w_zp=11)
    c["grouped_c2_oc6_group8"] = lambda: random_conv_case(22, 1, 8, 8, 2, 6, 1, 1, bias=False)
    c["grouped_c32_oc16_narrow_output"] = lambda: random_conv_case(24, 2, 12, 12, 32, 16, 1, 1, x_dtype=U8, w_dtype=U8, y_dtype=U8,
                                                                   per_axis=False, x_q=(0.02, 120))
    c["grouped_c192_oc32_per_axis"] = lambda: random_conv_case(25, 1, 14, 14, 192, 32, 1, 1)
    c["c24_oc144_odd_pixel_count"] = lambda: random_conv_case(23, 1, 7, 9, 24, 144, 1, 1)
    return c


def dwconv_cases():
    c = {}
    c["3x3_s1_c32"] = lambda: random_conv_case(21, 2, 14, 14, 32, None, 3, 3, pad=(1, 1, 1, 1), depthwise=True, act=(2, 6.0, 0.0),
                                               x_dtype=U8, w_dtype=U8, y_dtype=U8, per_axis=False, x_q=(0.02, 0), y_zp=0, y_scale=0.03)
    c["3x3_s2_c96"] = lambda: random_conv_case(22, 1, 15, 15, 96, None, 3, 3, stride=(2, 2), pad=(0, 1, 0, 1), depthwise=True,
                                               x_dtype=U8, w_dtype=U8, y_dtype=U8, per_axis=False, x_q=(0.02, 3), y_zp=0, y_scale=0.03)
    c["s8_per_axis_c20"] = lambda: random_conv_case(23, 1, 9, 9, 20, None, 3, 3, pad=(1, 1, 1, 1), depthwise=True)
    c["odd_c7"] = lambda: random_conv_case(24, 1, 7, 7, 7, None, 3, 3, pad=(1, 1, 1, 1), depthwise=True)
    c["multiplier2"] = lambda: random_conv_case(25, 1, 6, 6, 8, None, 3, 3, pad=(1, 1, 1, 1), depthwise=True, depth_multiplier=2)
    c["5x5_dilation2"] = lambda: random_conv_case(26, 1, 12, 12, 16, None, 5, 5, pad=(4, 4, 4, 4), dil=(2, 2), depthwise=True)
    # the row-sliding 3x3 kernel (signed symmetric weights): eight, four, two and one output rows per thread, ragged
    # right and bottom edges, both strides, the three ways its requantisation ends, both input signednesses
    c["rows8_s1_c32_relu6"] = lambda: random_conv_case(27, 32, 111, 113, 32, None, 3, 3, pad=(1, 1, 1, 1), depthwise=True,
                                                       act=(2, 6.0, 0.0), x_q=(0.05, -7))
    c["rows4_s2_c64"] = lambda: random_conv_case(28, 32, 113, 111, 64, None, 3, 3, stride=(2, 2), pad=(0, 1, 0, 1), depthwise=True,
                                                 x_q=(0.02, 5))
    c["rows2_s1_u8_activations"] = lambda: random_conv_case(29, 16, 56, 56, 64, None, 3, 3, pad=(1, 1, 1, 1), depthwise=True,
                                                            x_dtype=U8, y_dtype=U8, x_q=(0.02, 131))
    c["rows1_s2_c96_relu"] = lambda: random_conv_case(30, 1, 15, 15, 96, None, 3, 3, stride=(2, 2), pad=(1, 1, 1, 1), depthwise=True,
                                                      act=(1, 0., 0.), per_axis=False)
    c["rows1_s1_c8_no_bias"] = lambda: random_conv_case(31, 3, 5, 6, 8, None, 3, 3, pad=(1, 1, 1, 1), depthwise=True, bias=False)
    c["rows_s2_u8_activations_pad0"] = lambda: random_conv_case(32, 2, 17, 19, 24, None, 3, 3, stride=(2, 2), depthwise=True,
                                                                x_dtype=U8, y_dtype=U8, x_q=(0.03, 128), act=(2, 6.0, 0.0))
    c["rows4_s1_u8_everything"] = lambda: random_conv_case(33, 32, 56, 56, 64, None, 3, 3, pad=(1, 1, 1, 1), depthwise=True,
                                                           act=(2, 6.0, 0.0), x_dtype=U8, w_dtype=U8, y_dtype=U8, per_axis=False,
                                                           x_q=(0.02, 117), y_zp=0, y_scale=0.03)
    c["rows2_s2_u8_everything"] = lambda: random_conv_case(34, 16, 57, 55, 96, None, 3, 3, stride=(2, 2), pad=(0, 1, 0, 1), depthwise=True,
                                                           x_dtype=U8, w_dtype=U8, y_dtype=U8, per_axis=False, x_q=(0.02, 3))
    c["rows1_s1_s8_weight_zero_point"] = lambda: random_conv_case(35, 2, 9, 10, 12, None, 3, 3, pad=(1, 1, 1, 1), depthwise=True,
                                                                  per_axis=False, w_zp=-9)
    return c


def fc_cases():
    c = {}
    c["m1_k1024"] = lambda: random_fc_case(31, 1, 1024, 1024)
    c["m16_k1024"] = lambda: random_fc_case(32, 16, 1024, 1024)
    c["m256_k1024"] = lambda: random_fc_case(33, 256, 1024, 1024)
    c["m16_k4096_n512"] = lambda: random_fc_case(34, 16, 4096, 512)
    c["odd_m3_k37_n11"] = lambda: random_fc_case(35, 3, 37, 11)
    c["not_transposed"] = lambda: random_fc_case(36, 5, 64, 24, transpose_w=False)
    c["u8_per_tensor_relu"] = lambda: random_fc_case(37, 8, 128, 64, x_dtype=U8, w_dtype=U8, y_dtype=U8, per_axis=False,
                                                     x_q=(0.03, 120), act=(1, 0., 0.))
    c["classifier_2048_1001"] = lambda: random_fc_case(38, 4, 2048, 1001, per_axis=False)
    # the row kernel: N not a multiple of 16, several row chunks and K chunks, every operand signedness, zero points
    c["rows_m70_k2048_n1001"] = lambda: random_fc_case(39, 70, 2048, 1001, per_axis=False)
    c["rows_m33_k4112_n40_per_axis"] = lambda: random_fc_case(40, 33, 4112, 40)
    c["rows_u8_zero_points"] = lambda: random_fc_case(41, 37, 1280, 1001, x_dtype=U8, w_dtype=U8, y_dtype=U8, per_axis=False,
                                                      x_q=(0.03, 119), act=(1, 0, 0))
    c["rows_s8x_u8w"] = lambda: random_fc_case(42, 9, 256, 21, w_dtype=U8, per_axis=False)
    c["rows_u8x_s8w"] = lambda: random_fc_case(43, 9, 256, 21, x_dtype=U8, y_dtype=U8, per_axis=True, x_q=(0.03, 100))
    # the weight-streaming kernel (at most 16 rows, K a multiple of 64): the sweep's largest point, row-count and column
    # tails, one and two row halves, both zero points, every operand signedness
    c["stream_m16_k4096_n4096"] = lambda: random_fc_case(44, 16, 4096, 4096)
    c["stream_m1_k4096_n4096"] = lambda: random_fc_case(45, 1, 4096, 4096)
    c["stream_m7_k8192_n1000_u8_zp"] = lambda: random_fc_case(46, 7, 8192, 1000, x_dtype=U8, w_dtype=U8, y_dtype=U8, per_axis=False,
                                                             x_q=(0.03, 119), act=(1, 0, 0))
    c["stream_m1_k64_n7"] = lambda: random_fc_case(47, 1, 64, 7)
    c["stream_m13_k192_n130"] = lambda: random_fc_case(48, 13, 192, 130, x_dtype=U8, y_dtype=U8, x_q=(0.03, 100))
    c["stream_m9_k1024_n2500_s8x_u8w"] = lambda: random_fc_case(49, 9, 1024, 2500, w_dtype=U8, per_axis=False)
    return c


def _rand(rng, dtype, shape):
    lo, hi = RANGE[dtype]
    return rng.integers(lo, hi + 1, size=shape).astype(NP_OF[dtype])


def bmm_cases():
    def make(seed, batch, m, k, n, tx, ty, bcast_y=False, xd=S8, yd=S8):
        def build(mem):
            rng = np.random.default_rng(seed)
            xs = (batch, k, m) if tx else (batch, m, k)
            ys = ((1,) if bcast_y else (batch,)) + ((n, k) if ty else (k, n))
            p = _abi.BmmParams()
            p.x = qt(mem, _rand(rng, xd, xs), xd, 0.02, 3 if xd == S8 else 130)
            p.y = qt(mem, _rand(rng, yd, ys), yd, 0.01, -2 if yd == S8 else 120)
            p.out, out = qt_out(mem, (batch, m, n), S8, 0.02 * 0.01 * 74 * 74 * np.sqrt(k) * 3 / 127, 1)
            p.batch, p.m, p.k, p.n = batch, m, k, n
            p.transpose_x, p.transpose_y = int(tx), int(ty)
            p.batch_stride_x = m * k
            p.batch_stride_y = 0 if bcast_y else k * n
            acc, p.acc_out = mem.out((batch, m, n), np.int32)
            return p, [out, acc]
        return lambda: SimpleCase("batch_matmul_q8", build)
    c = {"plain": make(41, 3, 17, 33, 9, False, False), "transpose_x": make(42, 2, 8, 16, 8, True, False),
         "transpose_y": make(43, 2, 8, 16, 12, False, True), "broadcast_y": make(44, 4, 5, 20, 6, False, False, True),
         "u8": make(45, 1, 16, 16, 16, False, False, xd=U8, yd=U8)}
    # the tensor-core kernel: several 128 x 128 tiles with ragged edges, every layout of either operand (16-byte
    # aligned rows and not), K beyond one 64-byte step and not a multiple of it, every signedness, broadcast
    for i, (tx, ty) in enumerate(((False, False), (False, True), (True, False), (True, True))):
        c["tiles_tx%d_ty%d" % (tx, ty)] = make(50 + i, 2, 200, 150, 170, tx, ty)
        c["aligned_tx%d_ty%d" % (tx, ty)] = make(54 + i, 3, 256, 128, 144, tx, ty)
    c["attention_qk"] = make(58, 12, 128, 64, 128, False, True)
    c["attention_pv_u8x"] = make(59, 12, 128, 128, 64, False, False, xd=U8)
    c["u8y_transposed_both"] = make(60, 2, 70, 96, 130, True, True, yd=U8)
    c["broadcast_y_tiles"] = make(61, 5, 130, 80, 64, False, False, True)
    c["k1"] = make(62, 1, 3, 1, 5, False, False)
    # the CUDA-core kernel stays reachable
    def generic(case):
        def build():
            sc = case()
            inner = sc.build
            def build2(mem):
                p, outs = inner(mem)
                p.algo = 1
                return p, outs
            sc.build = build2
            return sc
        return build
    c["generic_plain"] = generic(make(63, 3, 17, 33, 9, False, False))
    c["generic_transposed"] = generic(make(64, 2, 40, 50, 30, True, True, xd=U8))
    return c


def pool_cases():
    def make(seed, n, h, w, c, ptype, k, s, pad, method, dtype=S8, out_scale_mul=1.0):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.Pool2dParams()
            zp = -5 if dtype == S8 else 7
            p.x = qt(mem, _rand(rng, dtype, (n, h, w, c)), dtype, 0.1, zp)
            oh = (h + pad[0] + pad[1] - k[0]) // s[0] + 1
            ow = (w + pad[2] + pad[3] - k[1]) // s[1] + 1
            p.y, y = qt_out(mem, (n, oh, ow, c), dtype, 0.1 * out_scale_mul, zp)
            p.n, p.h, p.wd, p.c, p.oh, p.ow = n, h, w, c, oh, ow
            p.pool_h, p.pool_w = k
            p.stride_h, p.stride_w = s
            p.pad_top, p.pad_bottom, p.pad_left, p.pad_right = pad
            p.pool_type, p.padding_method = ptype, method
            return p, [y]
        return lambda: SimpleCase("pool2d_q8", build)
    return {
        "max_3x3_s2_pad1_c64": make(51, 2, 16, 16, 64, 0, (3, 3), (2, 2), (1, 1, 1, 1), 1),
        "avg_global_7x7_c2048": make(52, 2, 7, 7, 2048, 1, (7, 7), (1, 1), (0, 0, 0, 0), 1, out_scale_mul=0.5),
        "avg_3x3_exclude_pad": make(53, 1, 9, 9, 20, 1, (3, 3), (2, 2), (1, 1, 1, 1), 1),
        "avg_3x3_ignore_value": make(54, 1, 9, 9, 20, 1, (3, 3), (2, 2), (1, 1, 1, 1), 0),
        "l2_2x2_u8_c5": make(55, 1, 8, 8, 5, 2, (2, 2), (2, 2), (0, 0, 0, 0), 1, dtype=U8),
        "max_u8_odd_c3": make(56, 1, 7, 7, 3, 0, (2, 2), (1, 1), (0, 0, 0, 0), 1, dtype=U8),
        "avg_pad2_window3_ignore": make(57, 1, 5, 5, 8, 1, (3, 3), (2, 2), (2, 2, 2, 2), 0),
        "max_pad2_window3": make(58, 1, 5, 5, 8, 0, (3, 3), (2, 2), (2, 2, 2, 2), 1),
    }


def mean_cases():
    def make(seed, n, h, w, c, dtype=S8):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.MeanParams()
            p.x = qt(mem, _rand(rng, dtype, (n, h, w, c)), dtype, 0.05, 3)
            p.y, y = qt_out(mem, (n, c), dtype, 0.02, 1)
            p.n, p.h, p.wd, p.c = n, h, w, c
            return p, [y]
        return lambda: SimpleCase("mean_hw_q8", build)
    return {"7x7x1280_u8": make(61, 2, 7, 7, 1280, U8), "5x3x10": make(62, 3, 5, 3, 10)}


def eltwise_cases():
    def make(seed, sa, sb, op, dtype=S8, act=(0, 0., 0.), extra=(), nonzero=False):
        def build(mem):
            rng = np.random.default_rng(seed)
            so = tuple(max(a, b) for a, b in zip(sa, sb))
            p = _abi.EltwiseParams()
            za, zb, zo = (3, -7, -128 if act[0] else 5) if dtype == S8 else (120, 131, 0 if act[0] else 128)
            a, b = _rand(rng, dtype, sa), _rand(rng, dtype, sb)
            if nonzero:
                # strictly positive operands: no division by zero, no negative base under a fractional exponent
                za = zb = -128 if dtype == S8 else 0
                a, b = np.maximum(a, za + 1).astype(a.dtype), np.maximum(b, zb + 1).astype(b.dtype)
            p.a = qt(mem, a, dtype, 0.031, za)
            p.b = qt(mem, b, dtype, 0.017, zb)
            oscale = {0: 0.05, 4: 0.06, 5: 0.05, 2: 0.035, 3: 0.035, 1: 0.5, 6: 0.3, 7: 0.9, 8: 0.4, 100: 0.025}[op]
            p.out, out = qt_out(mem, so, dtype, oscale, zo)
            p.rank = len(so)
            for i in range(len(so)):
                p.shape_a[i], p.shape_b[i], p.shape_out[i] = sa[i], sb[i], so[i]
            p.op = op
            p.clamp_lo, p.clamp_hi = activation_clamp(act[0], act[1], act[2], oscale, zo, dtype)
            return p, [out]
        return lambda: SimpleCase("eltwise_q8", build, extra)
    def boolean(seed, sa, sb, op, dtype=S8, coarse=False):
        """Comparison (op 200 + ComparisonOperation) of quantised tensors, or LogicalBinary (210 / 211) of Boolean ones;
        the output is a Boolean tensor: B200K_U8, scale 1, zero point 0."""
        def build(mem):
            rng = np.random.default_rng(seed)
            so = tuple(max(a, b) for a, b in zip(sa, sb))
            p = _abi.EltwiseParams()
            if op >= 210:
                p.a = qt(mem, rng.integers(0, 3, size=sa).astype(np.uint8), U8, 1.0, 0)
                p.b = qt(mem, rng.integers(0, 3, size=sb).astype(np.uint8), U8, 1.0, 0)
            else:
                a, b = _rand(rng, dtype, sa), _rand(rng, dtype, sb)
                if coarse:                              # few distinct values with one quantisation: many equal pairs
                    a, b = (a // 64 * 64).astype(a.dtype), (b // 64 * 64).astype(b.dtype)
                q = (0.05, 3) if dtype == S8 else (0.05, 120)
                p.a = qt(mem, a, dtype, *q)
                p.b = qt(mem, b, dtype, *(q if coarse else (0.04, q[1] - 2)))
            p.out, out = qt_out(mem, so, U8, 1.0, 0)
            p.rank = len(so)
            for i in range(len(so)):
                p.shape_a[i], p.shape_b[i], p.shape_out[i] = sa[i], sb[i], so[i]
            p.op, p.clamp_lo, p.clamp_hi = op, 0, 255
            return p, [out]
        return lambda: SimpleCase("eltwise_q8", build, none)
    import ctypes as C
    relu = (C.c_int(1), C.c_float(0), C.c_float(0))
    none = (C.c_int(0), C.c_float(0), C.c_float(0))
    return {
        "add_residual_relu": make(71, (2, 14, 14, 64), (2, 14, 14, 64), 0, act=(1, 0., 0.), extra=relu),
        "add_u8": make(72, (1, 7, 7, 24), (1, 7, 7, 24), 0, dtype=U8, extra=none),
        "mul": make(73, (2, 5, 5, 16), (2, 5, 5, 16), 4, extra=none),
        "sub_ragged": make(74, (1, 3, 5, 7), (1, 3, 5, 7), 5, extra=none),
        "add_broadcast_channel": make(75, (2, 6, 6, 10), (1, 1, 1, 10), 0, extra=none),
        "mul_broadcast_scalar": make(76, (1, 1, 1, 1), (2, 4, 4, 8), 4, extra=none),
        "maximum": make(77, (3, 17), (3, 17), 2, extra=none),
        "minimum_broadcast_row": make(78, (4, 1), (4, 9), 3, extra=none),
        "div": make(79, (2, 5, 5, 16), (2, 5, 5, 16), 1, extra=none, nonzero=True),
        "sqdiff_u8": make(80, (1, 6, 6, 12), (1, 1, 1, 12), 6, dtype=U8, extra=none),
        "power_u8": make(61, (1, 9, 9, 16), (1, 9, 9, 16), 7, dtype=U8, extra=none, nonzero=True),
        "floor_div": make(62, (3, 7, 11), (3, 7, 11), 8, extra=none, nonzero=True),
        "floor_div_broadcast_u8": make(63, (2, 4, 4, 8), (1, 1, 1, 8), 8, dtype=U8, extra=none, nonzero=True),
        "prelu_channel_alpha": make(64, (2, 9, 9, 24), (1, 1, 1, 24), 100, extra=none),
        "prelu_u8_same_shape": make(65, (1, 5, 5, 32), (1, 5, 5, 32), 100, dtype=U8, extra=none),
        "equal_coarse": boolean(66, (2, 5, 5, 16), (2, 5, 5, 16), 200, coarse=True),
        "greater_broadcast": boolean(67, (2, 6, 6, 10), (1, 1, 1, 10), 201),
        "greater_or_equal_u8_coarse": boolean(68, (3, 17), (3, 17), 202, dtype=U8, coarse=True),
        "less": boolean(69, (1, 7, 7, 24), (1, 7, 7, 24), 203),
        "less_or_equal_coarse": boolean(70, (4, 1), (4, 9), 204, coarse=True),
        "not_equal_coarse_u8": boolean(56, (1, 3, 5, 7), (1, 3, 5, 7), 205, dtype=U8, coarse=True),
        "logical_and": boolean(57, (2, 5, 5, 16), (2, 5, 5, 16), 210),
        "logical_or_broadcast": boolean(58, (2, 4, 4, 8), (1, 1, 1, 8), 211),
    }


# std::pow: the CUDA and glibc implementations may differ in the last ulp
TRANSCENDENTAL_ELTWISE = ("power_u8",)


def activation_cases():
    def make(seed, fn, a, b, dtype=S8, count=1000, in_q=(0.05, 2), out_q=(0.05, 2)):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.ActivationParams()
            p.x = qt(mem, _rand(rng, dtype, (count,)), dtype, *in_q)
            p.y, y = qt_out(mem, (count,), dtype, *out_q)
            p.count, p.function, p.a, p.b = count, fn, a, b
            return p, [y]
        return lambda: SimpleCase("activation_q8", build)

    def make_fake(seed, lo, hi, count=777):
        def build(mem):
            p = _abi.ActivationParams()
            p.x = qt(mem, (np.random.default_rng(seed).standard_normal(count) * 3).astype(np.float32), F32)
            p.y, y = qt_out(mem, (count,), F32)
            p.count, p.function, p.a, p.b = count, 50, lo, hi
            return p, [y]
        return lambda: SimpleCase("activation_q8", build)
    return {
        "relu": make(81, 3, 0, 0), "bounded_relu6": make(82, 4, 6.0, 0.0, out_q=(0.03, -128)),
        "sigmoid_u8": make(83, 0, 0, 0, dtype=U8, in_q=(0.05, 128), out_q=(1 / 256., 0)),
        "tanh": make(84, 1, 1.0, 1.0, out_q=(1 / 128., 0)), "linear": make(85, 2, 0.7, -0.3),
        "leaky_relu": make(86, 6, 0.1, 0), "abs": make(87, 7, 0, 0), "square": make(88, 9, 0, 0, out_q=(0.3, -128)),
        "hard_swish": make(89, 11, 0, 0, count=1003), "sqrt_u8": make(90, 8, 0, 0, dtype=U8, in_q=(0.05, 0), out_q=(0.02, 0)),
        "elu": make(91, 10, 1.0, 0), "soft_relu": make(92, 5, 0, 0),
        "fake_quantization_float": make_fake(95, -3.0, 5.0), "fake_quantization_float_narrow": make_fake(96, -0.5, 0.25),
        "gelu": make(93, 12, 0, 0, in_q=(0.04, 0), out_q=(0.04, 0)), "gelu_u8": make(94, 12, 0, 0, dtype=U8, in_q=(0.03, 128), out_q=(0.016, 11)),
    }


# activations that go through libm exp / tanh / log: the CUDA and glibc implementations may differ in the last
# ulp, which can move a value across a rounding boundary
TRANSCENDENTAL_ACTIVATIONS = ("sigmoid_u8", "tanh", "elu", "soft_relu", "gelu", "gelu_u8")


def softmax_cases():
    def make(seed, outer, axis, inner, dtype=S8, beta=1.0):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.SoftmaxParams()
            p.x = qt(mem, _rand(rng, dtype, (outer, axis, inner)), dtype, 0.06, 0 if dtype == S8 else 128)
            p.y, y = qt_out(mem, (outer, axis, inner), dtype, 1 / 256., -128 if dtype == S8 else 0)
            p.outer, p.axis_size, p.inner, p.beta = outer, axis, inner, beta
            return p, [y]
        return lambda: SimpleCase("softmax_q8", build)
    return {"classifier_1001": make(101, 8, 1001, 1), "u8_rows_10": make(102, 5, 10, 1, dtype=U8),
            "inner_axis": make(103, 3, 7, 4, beta=0.5), "single_element": make(104, 4, 1, 1)}


def rows_cases():
    """LogSoftmax, L2Normalization and ArgMinMax: independent rows along one axis (outer x inner of them)."""
    def log_softmax(seed, outer, axis, inner, dtype=S8, beta=1.0):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.SoftmaxParams()
            if dtype == F32:
                p.x = qt(mem, (rng.standard_normal((outer, axis, inner)) * 3).astype(np.float32), F32)
                p.y, y = qt_out(mem, (outer, axis, inner), F32)
            else:
                p.x = qt(mem, _rand(rng, dtype, (outer, axis, inner)), dtype, 0.06, 0 if dtype == S8 else 128)
                p.y, y = qt_out(mem, (outer, axis, inner), dtype, 1 / 16., 127 if dtype == S8 else 255)
            p.outer, p.axis_size, p.inner, p.beta = outer, axis, inner, beta
            return p, [y]
        return lambda: SimpleCase("log_softmax_q", build)

    def l2norm(seed, outer, axis, inner, dtype=S8, eps=1e-12, zero_rows=False):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.SoftmaxParams()
            if dtype == F32:
                p.x = qt(mem, rng.standard_normal((outer, axis, inner)).astype(np.float32), F32)
                p.y, y = qt_out(mem, (outer, axis, inner), F32)
            else:
                zp = 3 if dtype == S8 else (128 if dtype == U8 else 0)
                x = _rand(rng, dtype, (outer, axis, inner))
                if zero_rows:
                    x[0] = zp                       # a row of zeros: the sum of squares is below eps
                p.x = qt(mem, x, dtype, 0.04, zp)
                p.y, y = qt_out(mem, (outer, axis, inner), dtype, 1 / 128. if dtype != S16 else 1 / 32768., 0 if dtype != U8 else 128)
            p.outer, p.axis_size, p.inner, p.beta = outer, axis, inner, eps
            return p, [y]
        return lambda: SimpleCase("l2_normalization_q", build)

    def argminmax(seed, outer, axis, inner, function, dtype=S8, out64=False, few_values=False):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.ArgMinMaxParams()
            if dtype == F32:
                p.x = qt(mem, rng.standard_normal((outer, axis, inner)).astype(np.float32), F32)
            else:
                x = _rand(rng, dtype, (outer, axis, inner))
                if few_values:
                    x = (x % 3).astype(x.dtype)    # many equal elements: the first one must win
                p.x = qt(mem, x, dtype, 0.05, 1)
            y, p.y = mem.out((outer, inner), np.int64 if out64 else np.int32)
            p.outer, p.axis_size, p.inner, p.function, p.out_int64 = outer, axis, inner, function, int(out64)
            return p, [y]
        return lambda: SimpleCase("arg_min_max_q", build)
    return {
        "log_softmax_classifier_1001": log_softmax(301, 4, 1001, 1),
        "log_softmax_u8_inner_axis": log_softmax(302, 3, 9, 5, dtype=U8, beta=0.5),
        "log_softmax_float": log_softmax(303, 6, 40, 1, dtype=F32, beta=2.0),
        "l2norm_nhwc_channels": l2norm(304, 50, 64, 1),
        "l2norm_nchw_u8": l2norm(305, 2, 24, 35, dtype=U8),
        "l2norm_eps_and_zero_row": l2norm(306, 3, 16, 1, eps=0.5, zero_rows=True),
        "l2norm_s16": l2norm(307, 4, 33, 1, dtype=S16),
        "l2norm_float": l2norm(308, 7, 19, 3, dtype=F32),
        "argmax_classifier_1001": argminmax(309, 16, 1001, 1, 1),
        "argmax_segmentation_inner": argminmax(310, 2, 21, 33 * 17, 1, dtype=U8),
        "argmin_ties_first_wins": argminmax(311, 9, 200, 1, 0, few_values=True),
        "argmax_ties_inner_int64": argminmax(312, 3, 50, 7, 1, out64=True, few_values=True),
        "argmin_float_short_axis": argminmax(313, 10, 5, 1, 0, dtype=F32),
        "argmax_s16_single_element": argminmax(314, 4, 1, 3, 1, dtype=S16),
    }


# expf / logf of the device against glibc: the last ulp may move a value across a rounding boundary
TRANSCENDENTAL_ROWS = ("log_softmax_classifier_1001", "log_softmax_u8_inner_axis", "log_softmax_float")


def norm_cases():
    """Gather, BatchNormalization and InstanceNormalization."""
    def gather(seed, outer, axis, inner, n_idx, dtype=S8, requant=False, negative=False):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.GatherParams()
            xq = (0.05, 0) if dtype != F32 else (1.0, 0)
            yq = (0.07, 5) if requant else xq
            if dtype == F32:
                p.x = qt(mem, rng.standard_normal((outer, axis, inner)).astype(np.float32), F32)
            else:
                p.x = qt(mem, _rand(rng, dtype, (outer, axis, inner)), dtype, *xq)
            idx = rng.integers(-axis if negative else 0, axis, size=(n_idx,)).astype(np.int32)
            p.indices = mem.inp(idx)
            p.y, y = qt_out(mem, (outer, n_idx, inner), dtype, *yq)
            p.outer, p.axis_size, p.inner, p.n_indices = outer, axis, inner, n_idx
            return p, [y]
        return lambda: SimpleCase("gather_q", build)

    def batch_norm(seed, n, c, hw, nchw=False, dtype=S8, param_dtype=None):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.BatchNormParams()
            pd = dtype if param_dtype is None else param_dtype
            shape = (n, c, hw) if nchw else (n, hw, c)
            if dtype == F32:
                p.x = qt(mem, rng.standard_normal(shape).astype(np.float32), F32)
                p.y, y = qt_out(mem, shape, F32)
            else:
                p.x = qt(mem, _rand(rng, dtype, shape), dtype, 0.05, 3 if dtype == S8 else 120)
                p.y, y = qt_out(mem, shape, dtype, 0.04, -5 if dtype == S8 else 110)
            if pd == F32:
                p.mean = qt(mem, rng.standard_normal(c).astype(np.float32), F32)
                p.variance = qt(mem, (rng.random(c) * 2 + 0.1).astype(np.float32), F32)
                p.beta = qt(mem, rng.standard_normal(c).astype(np.float32), F32)
                p.gamma = qt(mem, (rng.standard_normal(c) + 1).astype(np.float32), F32)
            else:
                lo = RANGE_LO[pd]
                p.mean = qt(mem, _rand(rng, pd, (c,)), pd, 0.02, lo + 128)
                p.variance = qt(mem, _rand(rng, pd, (c,)), pd, 0.01, lo)            # never negative
                p.beta = qt(mem, _rand(rng, pd, (c,)), pd, 0.02, lo + 100)
                p.gamma = qt(mem, _rand(rng, pd, (c,)), pd, 0.01, lo + 20)
            p.n, p.c, p.hw, p.nchw, p.eps = n, c, hw, int(nchw), 1e-3
            _, p.scratch = mem.out((2 * c,), np.float32)
            return p, [y]
        return lambda: SimpleCase("batch_norm_q", build)

    def instance_norm(seed, n, c, hw, nchw=False, dtype=S8, gamma=1.3, beta=-0.2):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.InstanceNormParams()
            shape = (n, c, hw) if nchw else (n, hw, c)
            if dtype == F32:
                p.x = qt(mem, rng.standard_normal(shape).astype(np.float32), F32)
                p.y, y = qt_out(mem, shape, F32)
            else:
                p.x = qt(mem, _rand(rng, dtype, shape), dtype, 0.05, 3 if dtype == S8 else 120)
                p.y, y = qt_out(mem, shape, dtype, 0.03, 0 if dtype == S8 else 128)
            p.n, p.c, p.hw, p.nchw = n, c, hw, int(nchw)
            p.gamma, p.beta, p.eps = gamma, beta, 1e-5
            return p, [y]
        return lambda: SimpleCase("instance_norm_q", build)
    def lrn(seed, n, c, h, w, channel_type, size, nchw=False, dtype=S8, alpha=1e-2, beta=0.75, kappa=1.0):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.NormalizationParams()
            shape = (n, c, h, w) if nchw else (n, h, w, c)
            if dtype == F32:
                p.x = qt(mem, (rng.standard_normal(shape) * 3).astype(np.float32), F32)
                p.y, y = qt_out(mem, shape, F32)
            else:
                # the reference encodes the output with the input's quantisation
                q = (0.05, 3) if dtype == S8 else (0.05, 120)
                p.x = qt(mem, _rand(rng, dtype, shape), dtype, *q)
                p.y, y = qt_out(mem, shape, dtype, *q)
            p.n, p.c, p.h, p.w, p.nchw, p.channel_type, p.norm_size = n, c, h, w, int(nchw), channel_type, size
            p.alpha, p.beta, p.kappa = alpha, beta, kappa
            return p, [y]
        return lambda: SimpleCase("normalization_q", build)
    def gather_nd(seed, dims, inner, n_idx, dtype=S8, requant=False):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.GatherNdParams()
            shape = tuple(dims) + (inner,)
            xq = (0.05, 0) if dtype != F32 else (1.0, 0)
            yq = (0.07, 5) if requant else xq
            if dtype == F32:
                p.x = qt(mem, rng.standard_normal(shape).astype(np.float32), F32)
            else:
                p.x = qt(mem, _rand(rng, dtype, shape), dtype, *xq)
            idx = np.stack([rng.integers(0, n, size=(n_idx,)) for n in dims], axis=1).astype(np.int32)
            p.indices = mem.inp(idx)
            p.y, y = qt_out(mem, (n_idx, inner), dtype, *yq)
            p.n_indices, p.nd, p.inner = n_idx, len(dims), inner
            for i, n in enumerate(dims):
                p.dims[i] = n
            return p, [y]
        return lambda: SimpleCase("gather_nd_q", build)
    def reverse(seed, shape, axes, dtype=S8, requant=False):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.ReverseParams()
            xq = (0.05, -3) if dtype != F32 else (1.0, 0)
            if dtype == F32:
                p.x = qt(mem, rng.standard_normal(shape).astype(np.float32), F32)
            else:
                p.x = qt(mem, _rand(rng, dtype, shape), dtype, *xq)
            p.y, y = qt_out(mem, shape, dtype, *((0.07, 5) if requant else xq))
            p.axes = mem.inp(np.array(axes, np.int32))
            p.n_axes, p.rank = len(axes), len(shape)
            for i, n in enumerate(shape):
                p.shape[i] = n
            return p, [y]
        return lambda: SimpleCase("reverse_q", build)
    def scatter(seed, dims, inner, n_idx, fn, dtype=S8, with_input=True, duplicates=False):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.ScatterNdParams()
            shape = tuple(dims) + (inner,)
            q = (0.05, 2) if dtype == S8 else ((0.05, 120) if dtype == U8 else (1.0, 0))
            rand = lambda sh: rng.standard_normal(sh).astype(np.float32) if dtype == F32 else _rand(rng, dtype, sh)
            if with_input:
                p.x = qt(mem, rand(shape), dtype, *q)
            p.updates = qt(mem, rand((n_idx, inner)), dtype, *((0.04, -1) if dtype == S8 else q))
            p.y, y = qt_out(mem, shape, dtype, *((0.09, 0) if dtype == S8 else q))
            rows = int(np.prod(dims))
            flat = rng.integers(0, rows, n_idx) if duplicates else rng.permutation(rows)[:n_idx]
            if duplicates:
                flat[-1] = flat[0]                         # the last tuple repeats the first: it must win
            p.indices = mem.inp(np.stack(np.unravel_index(flat, dims), axis=1).astype(np.int32))
            p.n_indices, p.nd, p.inner, p.function = n_idx, len(dims), inner, fn
            for i, n in enumerate(dims):
                p.dims[i] = n
            return p, [y]
        return lambda: SimpleCase("scatter_nd_q", build)
    return {
        "scatter_update_rows": scatter(344, (12,), 16, 5, 0),
        "scatter_add_duplicates_last_wins": scatter(345, (4, 5), 3, 9, 1, duplicates=True),
        "scatter_sub_u8_pixels": scatter(346, (3, 4, 5), 2, 7, 2, dtype=U8),
        "scatter_max_float_elements": scatter(347, (6, 7), 1, 10, 3, dtype=F32, duplicates=True),
        "scatter_min_shape_variant": scatter(348, (5, 3), 4, 6, 4, with_input=False),
        "scatter_mul_float_shape_variant": scatter(349, (9,), 8, 4, 5, dtype=F32, with_input=False),
        "scatter_update_shape_variant_u8": scatter(350, (4, 4), 2, 8, 0, dtype=U8, with_input=False),
        "reverse_width_and_batch": reverse(341, (2, 5, 7, 8), (2, 0)),
        "reverse_negative_axis_u8_requantise": reverse(342, (4, 6, 5), (-1,), dtype=U8, requant=True),
        "reverse_all_axes_float": reverse(343, (3, 4, 5), (0, 1, 2), dtype=F32),
        "gather_nd_pixels": gather_nd(338, (2, 7, 9), 16, 40),
        "gather_nd_u8_requantise": gather_nd(339, (5, 4), 3, 11, dtype=U8, requant=True),
        "gather_nd_float_rank1_tuples": gather_nd(340, (30,), 5, 12, dtype=F32),
        "lrn_across_nhwc": lrn(333, 2, 24, 6, 7, 0, 5),
        "lrn_across_nchw_u8": lrn(334, 1, 9, 5, 8, 0, 3, nchw=True, dtype=U8, alpha=1e-1, beta=0.5, kappa=2.0),
        "lrn_across_float": lrn(335, 2, 16, 4, 4, 0, 5, dtype=F32, alpha=1e-4),
        "lrn_within_nchw": lrn(336, 2, 3, 9, 10, 1, 3, nchw=True),
        "lrn_within_float": lrn(337, 1, 4, 7, 5, 1, 5, nchw=True, dtype=F32, alpha=2e-2, beta=1.0),
        "gather_embedding_rows": gather(321, 1, 500, 64, 37),
        "gather_axis1_requantise": gather(322, 3, 11, 5, 7, dtype=U8, requant=True),
        "gather_negative_indices_s16": gather(323, 2, 9, 3, 12, dtype=S16, negative=True),
        "gather_float_scalars": gather(324, 1, 40, 1, 25, dtype=F32),
        "gather_float_rows_aligned": gather(325, 2, 30, 8, 9, dtype=F32, negative=True),
        "batch_norm_nhwc": batch_norm(326, 2, 24, 35),
        "batch_norm_nchw_u8": batch_norm(327, 2, 10, 49, nchw=True, dtype=U8),
        "batch_norm_float": batch_norm(328, 3, 17, 20, dtype=F32),
        "batch_norm_s8_float_parameters": batch_norm(329, 1, 32, 64, param_dtype=F32),
        "instance_norm_nhwc": instance_norm(330, 2, 16, 13 * 11, dtype=F32),
        "instance_norm_nchw": instance_norm(331, 2, 5, 100, nchw=True, dtype=F32),
        "instance_norm_one_channel": instance_norm(332, 1, 1, 333, dtype=F32, gamma=0.7, beta=0.1),
    }


RANGE_LO = {U8: 0, S8: -128, S16: -32768}

# powf of the device against glibc: the last ulp may move a value across a rounding boundary
TRANSCENDENTAL_NORM = ("lrn_across_nhwc", "lrn_across_nchw_u8", "lrn_across_float", "lrn_within_nchw", "lrn_within_float")

# RefGatherWorkload.cpp:40-47 throws on a negative index before armnn::Gather (Gather.cpp:55-57), which would wrap it,
# runs: these cases have no CpuRef output and pin the wrapping against the restatement of Gather.cpp only
CPUREF_REFUSES = {("norm", "gather_negative_indices_s16"), ("norm", "gather_float_rows_aligned")}


def volume_cases():
    """Convolution3d and Pooling3d on NDHWC tensors."""
    def conv3d(seed, n, dims, c, oc, k, stride=(1, 1, 1), pad=(0, 0, 0, 0, 0, 0), dil=(1, 1, 1), dtype=S8, per_axis=False, bias=True):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.Conv3dParams()
            d, h, w = dims
            pf, pb, pt, pbm, pl, pr = pad
            od = (d + pf + pb - dil[0] * (k[0] - 1) - 1) // stride[0] + 1
            oh = (h + pt + pbm - dil[1] * (k[1] - 1) - 1) // stride[1] + 1
            ow = (w + pl + pr - dil[2] * (k[2] - 1) - 1) // stride[2] + 1
            if dtype == F32:
                p.x = qt(mem, rng.standard_normal((n, d, h, w, c)).astype(np.float32), F32)
                p.w = qt(mem, (rng.standard_normal(k + (c, oc)) * 0.3).astype(np.float32), F32)
                if bias:
                    p.bias = qt(mem, rng.standard_normal(oc).astype(np.float32), F32)
                p.y, y = qt_out(mem, (n, od, oh, ow, oc), F32)
            else:
                sx = 0.05
                p.x = qt(mem, _rand(rng, dtype, (n, d, h, w, c)), dtype, sx, 3 if dtype == S8 else 120)
                wd = S8 if (per_axis or dtype == S8) else U8
                wdata = _rand(rng, wd, k + (c, oc))
                if per_axis:
                    scales = (rng.random(oc) * 0.02 + 0.005).astype(np.float32)
                    p.w = qt(mem, wdata, S8, 1.0, 0, scales=scales)
                    bsc = (scales * np.float32(sx)).astype(np.float32)
                    if bias:
                        p.bias = qt(mem, rng.integers(-2000, 2000, size=(oc,)).astype(np.int32), S32, 1.0, 0, scales=bsc)
                else:
                    sw = 0.01
                    p.w = qt(mem, wdata, wd, sw, 0 if wd == S8 else 131)
                    if bias:
                        p.bias = qt(mem, rng.integers(-2000, 2000, size=(oc,)).astype(np.int32), S32, sx * sw, 0)
                fan = k[0] * k[1] * k[2] * c
                p.y, y = qt_out(mem, (n, od, oh, ow, oc), dtype, 0.05 * 0.01 * 64 * np.sqrt(fan), -5 if dtype == S8 else 110)
                lo, hi = RANGE[dtype]
                p.clamp_lo, p.clamp_hi = lo, hi
            p.n, p.d, p.h, p.wd, p.c, p.od, p.oh, p.ow, p.oc = n, d, h, w, c, od, oh, ow, oc
            p.kd, p.kh, p.kw = k
            p.stride_d, p.stride_h, p.stride_w = stride
            p.pad_front, p.pad_top, p.pad_left = pf, pt, pl
            p.dil_d, p.dil_h, p.dil_w = dil
            return p, [y]
        return lambda: SimpleCase("conv3d_q", build)

    def pool3d(seed, n, dims, c, pool, stride, pad=(0, 0, 0, 0, 0, 0), pool_type=0, method=1, dtype=S8):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.Pool3dParams()
            d, h, w = dims
            pf, pb, pt, pbm, pl, pr = pad
            od, oh, ow = (d + pf + pb - pool[0]) // stride[0] + 1, (h + pt + pbm - pool[1]) // stride[1] + 1, (w + pl + pr - pool[2]) // stride[2] + 1
            if dtype == F32:
                p.x = qt(mem, rng.standard_normal((n, d, h, w, c)).astype(np.float32), F32)
                p.y, y = qt_out(mem, (n, od, oh, ow, c), F32)
            else:
                q = (0.05, 3) if dtype == S8 else (0.05, 120)
                p.x = qt(mem, _rand(rng, dtype, (n, d, h, w, c)), dtype, *q)
                p.y, y = qt_out(mem, (n, od, oh, ow, c), dtype, *q)
            p.n, p.d, p.h, p.wd, p.c, p.od, p.oh, p.ow = n, d, h, w, c, od, oh, ow
            p.pool_d, p.pool_h, p.pool_w = pool
            p.stride_d, p.stride_h, p.stride_w = stride
            p.pad_front, p.pad_back, p.pad_top, p.pad_bottom, p.pad_left, p.pad_right = pad
            p.pool_type, p.padding_method = pool_type, method
            return p, [y]
        return lambda: SimpleCase("pool3d_q", build)
    return {
        "conv3d_3x3x3_same": conv3d(401, 1, (5, 6, 7), 4, 8, (3, 3, 3), pad=(1, 1, 1, 1, 1, 1)),
        "conv3d_u8_stride2_ragged": conv3d(402, 2, (6, 5, 7), 3, 5, (2, 3, 2), stride=(2, 1, 2), pad=(0, 0, 1, 0, 0, 1), dtype=U8),
        "conv3d_per_axis_dilated": conv3d(403, 1, (7, 7, 6), 6, 10, (2, 2, 2), dil=(2, 1, 3), per_axis=True),
        "conv3d_no_bias_1x1x1": conv3d(404, 2, (3, 4, 5), 16, 7, (1, 1, 1), bias=False),
        "conv3d_float": conv3d(405, 1, (4, 5, 6), 3, 6, (3, 2, 3), stride=(1, 2, 1), pad=(1, 1, 0, 1, 1, 1), dtype=F32),
        "pool3d_max_2x2x2": pool3d(406, 2, (6, 8, 6), 5, (2, 2, 2), (2, 2, 2)),
        "pool3d_average_exclude_padded_u8": pool3d(407, 1, (5, 6, 7), 3, (3, 3, 3), (2, 2, 2), pad=(1, 1, 1, 1, 1, 1), pool_type=1, dtype=U8),
        "pool3d_average_ignore_value_padded": pool3d(408, 1, (4, 5, 5), 4, (2, 3, 2), (1, 2, 2), pad=(1, 0, 1, 1, 0, 1), pool_type=1, method=0),
        "pool3d_l2_float": pool3d(409, 2, (4, 4, 6), 3, (2, 2, 3), (2, 2, 3), pool_type=2, dtype=F32),
        "pool3d_max_padded_float": pool3d(410, 1, (5, 5, 5), 2, (3, 3, 3), (2, 2, 2), pad=(1, 1, 1, 1, 1, 1), dtype=F32),
    }


def lstm_cases():
    """One Float32 LSTM step with every combination of options the reference implements."""
    def make(seed, batch, n_in, units, n_out, cifg=False, peephole=False, layer_norm=False, projection=False, activation=4,
             cell_clip=0.0, proj_clip=0.0):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.LstmParams()
            f = lambda *shape, s=0.4: mem.inp((rng.standard_normal(shape) * s).astype(np.float32))
            p.batch, p.input_size, p.num_units, p.output_size = batch, n_in, units, n_out
            p.input, p.input_stride = f(batch, n_in, s=1.0), n_in
            p.output_state_in, p.cell_state_in = f(batch, n_out, s=0.7), f(batch, units, s=0.7)
            hs, p.output_state_out = mem.out((batch, n_out), np.float32)
            cs, p.cell_state_out = mem.out((batch, units), np.float32)
            out, p.output = mem.out((batch, n_out), np.float32)
            p.output_stride = n_out
            for g in "ifco":
                if g == "i" and cifg:
                    continue
                setattr(p, "w_i2" + g, f(units, n_in)); setattr(p, "w_r2" + g, f(units, n_out)); setattr(p, "b_" + g, f(units))
                if peephole and g != "c":
                    setattr(p, "w_c2" + g, f(units))
                if layer_norm:
                    setattr(p, "ln_" + g, f(units, s=1.0))
            if projection:
                p.w_proj, p.b_proj = f(n_out, units), f(n_out)
            p.activation, p.cell_clip, p.projection_clip, p.layer_norm_eps = activation, cell_clip, proj_clip, 1e-8
            return p, [hs, cs, out]
        return lambda: SimpleCase("lstm_step_f32", build)
    return {
        "plain_tanh": make(421, 3, 20, 32, 32),
        "cifg_peephole": make(422, 2, 12, 24, 24, cifg=True, peephole=True),
        "layer_norm_projection": make(423, 4, 40, 64, 24, layer_norm=True, projection=True, cell_clip=1.5, proj_clip=0.8),
        "everything_relu6": make(424, 2, 16, 48, 20, peephole=True, layer_norm=True, projection=True, activation=3, cell_clip=3.0),
        "no_activation_cifg_layer_norm": make(425, 2, 10, 16, 16, cifg=True, layer_norm=True, activation=0),
        "sigmoid_wide": make(426, 1, 300, 520, 520, activation=6),
    }


def convert_cases():
    def fp16(seed, to_half):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.ConvertFp16Params()
            if to_half:
                # normal halves, ties at bit 13, the subnormal range, underflow to zero, overflow to infinity, infinities
                x = np.concatenate([rng.standard_normal(3000) * 10 ** rng.uniform(-9, 6, 3000),
                                    np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, -65536.0, 1e9, np.inf, -np.inf, 6.1e-5, 6.0e-8, 2.9e-8, 3.0e-8, 1e-10]),
                                    (np.arange(2048, 4096, dtype=np.float64) + 0.5) * 2.0 ** -11,        # exact ties
                                    (np.arange(0, 1100, dtype=np.float64) * 0.5) * 2.0 ** -24]).astype(np.float32)
                p.x = mem.inp(x)
                y, p.y = mem.out(x.shape, np.uint16)
            else:
                codes = np.arange(65536, dtype=np.uint16)
                codes = codes[~(((codes & 0x7c00) == 0x7c00) & ((codes & 0x3ff) != 0))]                    # every code but the NaNs
                p.x = mem.inp(codes)
                y, p.y = mem.out(codes.shape, np.float32)
            p.count, p.to_half = (x if to_half else codes).size, int(to_half)
            return p, [y]
        return lambda: SimpleCase("convert_fp16", build)

    def make(seed, xd, yd, count=1001, xq=(0.05, 3), yq=(0.07, -4), entry="convert_q", fscale=4):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.ConvertParams()
            if xd == F32:
                x = (rng.standard_normal(count) * fscale).astype(np.float32)
                p.x = qt(mem, x, F32)
            elif xd == S32:
                p.x = qt(mem, rng.integers(-70000, 70000, size=(count,)).astype(np.int32), S32, 1.0, 0)
            else:
                p.x = qt(mem, _rand(rng, xd, (count,)), xd, *xq)
            p.y, y = qt_out(mem, (count,), yd, *yq)
            p.count = count
            return p, [y]
        return lambda: SimpleCase(entry, build)
    return {"quantize_f32_s8": make(111, F32, S8), "quantize_f32_u8": make(112, F32, U8, yq=(0.05, 128)),
            "quantize_f32_s16": make(113, F32, S16, yq=(0.001, 0)), "dequantize_s8": make(114, S8, F32),
            "dequantize_u8": make(115, U8, F32, xq=(0.1, 120)), "requantize_u8_s8": make(116, U8, S8, xq=(0.05, 128)),
            "requantize_s16_s8": make(117, S16, S8, xq=(0.0005, 0)),
            # Cast ignores both quantisations: the stored numbers are converted
            "cast_f32_s8": make(118, F32, S8, entry="cast_q", fscale=40), "cast_f32_s32": make(119, F32, S32, entry="cast_q", fscale=1e5),
            "cast_u8_f32": make(120, U8, F32, entry="cast_q", xq=(0.1, 120)), "cast_s16_u8": make(110, S16, U8, entry="cast_q", xq=(0.0005, 0)),
            "cast_s32_s16": make(109, S32, S16, entry="cast_q"), "cast_s8_s32": make(108, S8, S32, entry="cast_q"),
            "fp32_to_fp16_every_range": fp16(107, True), "fp16_to_fp32_every_code": fp16(106, False)}


def pad_cases():
    def make(seed, shape, pads, value, dtype=S8, xq=(0.05, -7), yq=None, mode=0):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.PadParams()
            p.mode = mode
            p.x = qt(mem, _rand(rng, dtype, shape) if dtype != F32 else rng.standard_normal(shape).astype(np.float32), dtype, *xq)
            out_shape = tuple(s + a + b for s, (a, b) in zip(shape, pads))
            p.y, y = qt_out(mem, out_shape, dtype, *(yq or xq))
            p.rank = len(shape)
            for i, (a, b) in enumerate(pads):
                p.shape[i], p.pad_before[i], p.pad_after[i] = shape[i], a, b
            p.pad_value = value
            return p, [y]
        return lambda: SimpleCase("pad_q", build)
    return {
        "nhwc_hw_zero_point": make(131, (2, 9, 7, 24), ((0, 0), (1, 1), (2, 1), (0, 0)), -7),
        "nhwc_channels_u8": make(132, (1, 5, 5, 3), ((0, 0), (0, 0), (0, 0), (2, 3)), 200, dtype=U8, xq=(0.1, 128)),
        "rank2_requantise": make(133, (7, 11), ((3, 0), (0, 5)), 9, xq=(0.05, 2), yq=(0.08, -4)),
        "rank1": make(134, (33,), ((4, 4),), -128),
        "rank3_float": make(135, (3, 4, 5), ((1, 0), (0, 2), (1, 1)), 1.5, dtype=F32, xq=(1.0, 0)),
        "reflect_nhwc_hw": make(136, (2, 6, 5, 8), ((0, 0), (2, 3), (4, 1), (0, 0)), 0, mode=1),
        "reflect_widest_u8_requantise": make(137, (3, 4), ((2, 2), (3, 3)), 0, dtype=U8, xq=(0.1, 128), yq=(0.13, 100), mode=1),
        "symmetric_nhwc_hw": make(138, (1, 5, 7, 6), ((0, 0), (1, 2), (3, 3), (0, 0)), 0, mode=2),
        "symmetric_widest_float": make(139, (2, 3, 4), ((2, 2), (3, 3), (0, 4)), 0, dtype=F32, xq=(1.0, 0), mode=2),
    }


def qlstm_cases():
    return {
        "proj_ln": lambda: random_qlstm_case(121, 3, 40, 64, 32),
        "proj_ln_zero_state": lambda: random_qlstm_case(122, 2, 40, 64, 32, state="zero"),
        "peephole": lambda: random_qlstm_case(123, 2, 24, 32, 16, peephole=True),
        "cifg": lambda: random_qlstm_case(124, 2, 24, 32, 16, cifg=True),
        "no_layer_norm": lambda: random_qlstm_case(125, 2, 24, 32, 16, layer_norm=False),
        "no_projection": lambda: random_qlstm_case(126, 2, 20, 32, 32, projection=False),
        "cifg_peephole_unaligned": lambda: random_qlstm_case(127, 2, 13, 19, 11, cifg=True, peephole=True),
        "config5_layer2_shape": lambda: random_qlstm_case(128, 2, 256, 512, 256),
    }


def f32_cases():
    """The Float32 variants of Convolution2d, DepthwiseConvolution2d and FullyConnected: bit-exact against CpuRef."""
    def conv(seed, n, h, w, c, oc, k, stride=(1, 1), pad=(0, 0), dil=(1, 1), depthwise=False, bias=True):
        def build(mem):
            rng = np.random.default_rng(seed)
            oh = (h + 2 * pad[0] - dil[0] * (k[0] - 1) - 1) // stride[0] + 1
            ow = (w + 2 * pad[1] - dil[1] * (k[1] - 1) - 1) // stride[1] + 1
            p = _abi.Conv2dParams()
            p.x = qt(mem, rng.standard_normal((n, h, w, c)).astype(np.float32), F32)
            wshape = (1, k[0], k[1], oc) if depthwise else (oc, k[0], k[1], c)
            p.w = qt(mem, (rng.standard_normal(wshape) * 0.2).astype(np.float32), F32)
            if bias:
                p.bias = qt(mem, rng.standard_normal(oc).astype(np.float32), F32)
            p.y, y = qt_out(mem, (n, oh, ow, oc), F32)
            p.n, p.h, p.wd, p.c, p.oh, p.ow, p.oc, p.kh, p.kw = n, h, w, c, oh, ow, oc, k[0], k[1]
            p.stride_h, p.stride_w, p.pad_top, p.pad_left, p.dil_h, p.dil_w = stride[0], stride[1], pad[0], pad[1], dil[0], dil[1]
            return p, [y]
        return lambda: SimpleCase("dwconv2d_f32" if depthwise else "conv2d_f32", build)

    def fc(seed, m, k, n, transpose=True, bias=True):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.FcParams()
            p.x = qt(mem, rng.standard_normal((m, k)).astype(np.float32), F32)
            p.w = qt(mem, (rng.standard_normal((n, k) if transpose else (k, n)) * 0.1).astype(np.float32), F32)
            if bias:
                p.bias = qt(mem, rng.standard_normal(n).astype(np.float32), F32)
            p.y, y = qt_out(mem, (m, n), F32)
            p.m, p.k, p.n, p.transpose_w = m, k, n, int(transpose)
            return p, [y]
        return lambda: SimpleCase("fully_connected_f32", build)

    def bmm(seed, batch, m, k, n, tx=False, ty=False, bcast_y=False):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.BmmParams()
            p.x = qt(mem, rng.standard_normal((batch, k, m) if tx else (batch, m, k)).astype(np.float32), F32)
            p.y = qt(mem, rng.standard_normal(((1,) if bcast_y else (batch,)) + ((n, k) if ty else (k, n))).astype(np.float32), F32)
            p.out, out = qt_out(mem, (batch, m, n), F32)
            p.batch, p.m, p.k, p.n, p.transpose_x, p.transpose_y = batch, m, k, n, int(tx), int(ty)
            p.batch_stride_x, p.batch_stride_y = m * k, 0 if bcast_y else k * n
            return p, [out]
        return lambda: SimpleCase("batch_matmul_f32", build)
    return {
        "bmm_plain": bmm(358, 3, 17, 33, 9), "bmm_transpose_both": bmm(359, 2, 8, 40, 12, tx=True, ty=True),
        "bmm_attention_qk_broadcast_y": bmm(360, 4, 16, 64, 16, ty=True, bcast_y=True),
        "conv3x3_pad1": conv(351, 2, 9, 8, 12, 20, (3, 3), pad=(1, 1)),
        "conv1x1": conv(352, 1, 7, 7, 32, 16, (1, 1), bias=False),
        "conv5x5_s2_dilation2": conv(353, 1, 17, 15, 5, 7, (5, 5), stride=(2, 2), pad=(4, 4), dil=(2, 2)),
        "dwconv3x3_s1": conv(354, 2, 10, 9, 16, 16, (3, 3), pad=(1, 1), depthwise=True),
        "dwconv3x3_s2_multiplier2": conv(355, 1, 11, 11, 6, 12, (3, 3), stride=(2, 2), pad=(1, 1), depthwise=True),
        "fc_m5_k64_n24": fc(356, 5, 64, 24),
        "fc_not_transposed_no_bias": fc(357, 3, 37, 11, transpose=False, bias=False),
    }


def tconv_cases():
    """TransposeConvolution2d (NHWC, weights OHWI): the up-sampling shapes of decoder networks, every operand type,
    channel counts with and without the 4-byte vector path, padding that crops the output."""
    def make(seed, n, h, w, c, oc, k, stride, pad=(0, 0), x_dtype=S8, w_dtype=S8, y_dtype=S8, per_axis=True, x_q=(0.02, -3),
             bias=True, out_pad=(0, 0)):
        def build(mem):
            rng = np.random.default_rng(seed)
            oh = (h - 1) * stride[0] + k[0] - 2 * pad[0] + out_pad[0]
            ow = (w - 1) * stride[1] + k[1] - 2 * pad[1] + out_pad[1]
            p = _abi.Conv2dParams()
            p.x = qt(mem, _rand(rng, x_dtype, (n, h, w, c)), x_dtype, *x_q)
            wq = _rand(rng, w_dtype, (oc, k[0], k[1], c))
            if per_axis and w_dtype == S8:
                ws = rng.uniform(0.001, 0.01, size=oc).astype(np.float32)
                p.w = qt(mem, wq, w_dtype, 1.0, 0, scales=ws)
                bs = (np.float32(x_q[0]) * ws).astype(np.float32)
                mean_sw = float(ws.mean())
            else:
                sw = float(np.float32(rng.uniform(0.001, 0.01)))
                zw = 0 if w_dtype == S8 else int(rng.integers(100, 156))
                p.w = qt(mem, wq, w_dtype, sw, zw)
                bs, mean_sw = None, sw
            if bias:
                bq = rng.integers(-1000, 1001, size=oc).astype(np.int32)
                p.bias = qt(mem, bq, S32, float(np.float32(x_q[0]) * np.float32(mean_sw)), 0, scales=bs)
            taps = max(1, (k[0] // stride[0]) * (k[1] // stride[1])) * c
            y_scale = float(np.float32(x_q[0] * mean_sw * 74.0 * 74.0 * np.sqrt(taps) * 3.0 / 127.0))
            p.y, y = qt_out(mem, (n, oh, ow, oc), y_dtype, y_scale, 0 if y_dtype == S8 else 128)
            p.n, p.h, p.wd, p.c, p.oh, p.ow, p.oc, p.kh, p.kw = n, h, w, c, oh, ow, oc, k[0], k[1]
            p.stride_h, p.stride_w, p.pad_top, p.pad_left, p.dil_h, p.dil_w = stride[0], stride[1], pad[0], pad[1], 1, 1
            lo, hi = RANGE[y_dtype]
            p.clamp_lo, p.clamp_hi = lo, hi
            return p, [y]
        return lambda: SimpleCase("transpose_conv2d_q8", build)
    return {
        "up2_k2_s2": make(341, 2, 7, 6, 16, 24, (2, 2), (2, 2)),
        "up2_k4_s2_pad1": make(342, 1, 6, 5, 32, 16, (4, 4), (2, 2), pad=(1, 1)),
        "k3_s1_pad1_same_size": make(343, 1, 9, 8, 12, 20, (3, 3), (1, 1), pad=(1, 1)),
        "u8_everything_k3_s2": make(344, 1, 5, 7, 8, 12, (3, 3), (2, 2), x_dtype=U8, w_dtype=U8, y_dtype=U8, per_axis=False, x_q=(0.02, 121)),
        "odd_channels_c5_oc7_no_bias": make(345, 2, 4, 4, 5, 7, (3, 2), (2, 3), bias=False),
        "u8_activations_s8_weights_s3": make(346, 1, 4, 5, 16, 8, (5, 5), (3, 3), pad=(2, 2), x_dtype=U8, y_dtype=U8, x_q=(0.03, 100)),
    }


# unary operations whose result depends on libm's exp / log / sin (the device functions differ in the last bit)
TRANSCENDENTAL_UNARY = ("exp_s8", "log_u8", "sin_s8", "exp_float")


def unary_cases():
    """ElementwiseUnary: every supported operation on quantised and float tensors."""
    def make(seed, count, op, dtype=S8, xq=(0.05, -3), yq=None, positive=False):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.UnaryParams()
            if dtype == F32:
                x = rng.standard_normal(count).astype(np.float32) * 2
                x = np.abs(x) + np.float32(0.1) if positive else x
            else:
                x = _rand(rng, dtype, (count,))
                if positive:                              # dequantised values > 0
                    lo, hi = RANGE[dtype]
                    x = np.clip(x, xq[1] + 1, hi).astype(NP_OF[dtype])
            p.x = qt(mem, x, dtype, *xq)
            p.y, y = qt_out(mem, (count,), dtype, *(yq or xq))
            p.count, p.operation = count, op
            return p, [y]
        return lambda: SimpleCase("unary_q", build)
    ABS, EXP, SQRT, RSQRT, NEG, LOG, SIN, CEIL, FLOOR = 0, 1, 2, 3, 4, 6, 7, 8, 9

    def logical_not():
        def build(mem):
            p = _abi.UnaryParams()
            p.x = qt(mem, np.random.default_rng(372).integers(0, 3, size=(500,)).astype(np.uint8), U8, 1.0, 0)
            p.y, y = qt_out(mem, (500,), U8, 1.0, 0)
            p.count, p.operation = 500, 5
            return p, [y]
        return SimpleCase("unary_q", build)
    return {
        "logical_not_boolean": logical_not,
        "floor_layer_float": make(371, 333, FLOOR, dtype=F32, xq=(1.0, 0)),
        "abs_s8": make(361, 1000, ABS),
        "neg_u8_requantise": make(362, 777, NEG, dtype=U8, xq=(0.1, 128), yq=(0.12, 120)),
        "sqrt_u8": make(363, 513, SQRT, dtype=U8, xq=(0.07, 10), yq=(0.02, 0), positive=True),
        "rsqrt_s8": make(364, 300, RSQRT, xq=(0.05, -100), yq=(0.05, -128), positive=True),
        "ceil_s16": make(365, 999, CEIL, dtype=S16, xq=(0.013, 0), yq=(0.5, 0)),
        "ceil_float": make(366, 257, CEIL, dtype=F32, xq=(1.0, 0)),
        "exp_s8": make(367, 1000, EXP, xq=(0.02, 5), yq=(0.1, -128)),
        "log_u8": make(368, 900, LOG, dtype=U8, xq=(0.05, 0), yq=(0.05, 128), positive=True),
        "sin_s8": make(369, 1111, SIN, xq=(0.05, 0), yq=(0.008, 0)),
        "exp_float": make(370, 400, EXP, dtype=F32, xq=(1.0, 0)),
    }


def reduce_cases():
    """Reduce: every operation, inner / outer / several / all axes, re-quantisation, float."""
    def make(seed, shape, axes, op, dtype=S8, xq=(0.05, -3), yq=None):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.ReduceParams()
            p.x = qt(mem, _rand(rng, dtype, shape) if dtype != F32 else rng.standard_normal(shape).astype(np.float32), dtype, *xq)
            out_shape = tuple(s for d, s in enumerate(shape) if d not in axes) or (1,)
            p.y, y = qt_out(mem, out_shape, dtype, *(yq or xq))
            p.rank = len(shape)
            for i, s in enumerate(shape):
                p.shape[i] = s
            p.axis_mask = sum(1 << d for d in axes)
            p.op = op
            return p, [y]
        return lambda: SimpleCase("reduce_q", build)
    SUM, MAX, MEAN, MIN, PROD = 0, 1, 2, 3, 4
    return {
        "sum_channels_nhwc": make(321, (2, 5, 6, 24), (3,), SUM, yq=(0.4, 10)),
        "sum_hw_u8": make(322, (2, 7, 9, 16), (1, 2), SUM, dtype=U8, xq=(0.02, 128), yq=(0.3, 120)),
        "mean_hw_requantise": make(323, (3, 6, 5, 20), (1, 2), MEAN, yq=(0.03, 4)),
        "mean_outer_axis": make(324, (9, 4, 11), (0,), MEAN),
        "max_width": make(325, (2, 4, 13, 8), (2,), MAX),
        "min_batch_and_channels": make(326, (3, 5, 4, 7), (0, 3), MIN, dtype=U8, xq=(0.1, 77)),
        "prod_small_float": make(327, (4, 3, 5), (1,), PROD, dtype=F32, xq=(1.0, 0)),
        "prod_quantised": make(328, (2, 3, 6), (1,), PROD, xq=(0.02, 1), yq=(0.05, 0)),
        "sum_all_axes_float": make(329, (3, 7, 5), (0, 1, 2), SUM, dtype=F32, xq=(1.0, 0)),
        "max_rank1_s16": make(330, (37,), (0,), MAX, dtype=S16, xq=(0.01, 0)),
    }


def resize_cases():
    """Resize: both methods, both coordinate conventions, both layouts, up- and down-sampling, re-quantisation."""
    def make(seed, n, c, ih, iw, oh, ow, method, align=0, half=0, nchw=0, dtype=S8, xq=(0.05, -3), yq=None):
        def build(mem):
            rng = np.random.default_rng(seed)
            p = _abi.ResizeParams()
            in_shape = (n, c, ih, iw) if nchw else (n, ih, iw, c)
            out_shape = (n, c, oh, ow) if nchw else (n, oh, ow, c)
            p.x = qt(mem, _rand(rng, dtype, in_shape) if dtype != F32 else rng.standard_normal(in_shape).astype(np.float32), dtype, *xq)
            p.y, y = qt_out(mem, out_shape, dtype, *(yq or xq))
            p.n, p.c, p.in_h, p.in_w, p.out_h, p.out_w = n, c, ih, iw, oh, ow
            p.method, p.align_corners, p.half_pixel_centers, p.nchw = method, align, half, nchw
            return p, [y]
        return lambda: SimpleCase("resize_q", build)
    return {
        "bilinear_up2_nhwc": make(301, 2, 16, 7, 9, 14, 18, 0),
        "bilinear_up_odd_align_corners": make(302, 1, 5, 6, 5, 11, 13, 0, align=1),
        "bilinear_up_half_pixel": make(303, 1, 8, 5, 7, 15, 14, 0, half=1),
        "bilinear_down_u8_requantise": make(304, 2, 3, 17, 19, 5, 8, 0, dtype=U8, xq=(0.1, 128), yq=(0.07, 100)),
        "bilinear_nchw_float": make(305, 1, 4, 6, 6, 9, 13, 0, nchw=1, dtype=F32, xq=(1.0, 0)),
        "bilinear_down_half_pixel_nchw": make(306, 1, 3, 16, 12, 5, 7, 0, half=1, nchw=1),
        "nearest_up2_nhwc": make(307, 2, 24, 6, 5, 12, 10, 1),
        "nearest_align_corners": make(308, 1, 7, 5, 9, 12, 4, 1, align=1),
        "nearest_half_pixel_down": make(309, 1, 4, 13, 11, 6, 5, 1, half=1, dtype=U8, xq=(0.2, 9)),
        "nearest_nchw_s16": make(310, 1, 3, 4, 6, 10, 9, 1, nchw=1, dtype=S16, xq=(0.01, 0)),
    }


def move_cases():
    """Concat, Splitter, Permute, Transpose, StridedSlice and Slice as the reference's descriptors state them."""
    q = (S8, 0.05, -3)
    c = {}
    # channel-wise Concat of NHWC tensors (the 128-bit row path), equal quantisation
    c["concat_channels_nhwc"] = lambda: MoveCase("concat", 201, ((2, 7, 5, 80),) + q,
                                                  [((2, 7, 5, 32),) + q, ((2, 7, 5, 48),) + q], origins=[(0, 0, 0, 0), (0, 0, 0, 32)])
    # inputs with their own quantisation: every element goes through Q_out(deq_in(.))
    c["concat_requantise_u8"] = lambda: MoveCase("concat", 202, ((1, 4, 6, 11), U8, 0.07, 120),
                                                 [((1, 4, 6, 3), U8, 0.05, 128), ((1, 4, 6, 8), U8, 0.11, 100)],
                                                 origins=[(0, 0, 0, 0), (0, 0, 0, 3)])
    c["concat_height_three_inputs"] = lambda: MoveCase("concat", 203, ((1, 9, 4, 6),) + q,
                                                       [((1, 2, 4, 6),) + q, ((1, 3, 4, 6),) + q, ((1, 4, 4, 6),) + q],
                                                       origins=[(0, 0, 0, 0), (0, 2, 0, 0), (0, 5, 0, 0)])
    c["concat_batch_rank2_float"] = lambda: MoveCase("concat", 204, ((5, 7), F32, 1.0, 0), [((2, 7), F32, 1.0, 0), ((3, 7), F32, 1.0, 0)],
                                                     origins=[(0, 0), (2, 0)])
    c["split_channels_nhwc"] = lambda: MoveCase("split", 205, ((2, 5, 5, 96),) + q,
                                                [((2, 5, 5, 32),) + q, ((2, 5, 5, 64),) + q], origins=[(0, 0, 0, 0), (0, 0, 0, 32)])
    c["split_width_requantise"] = lambda: MoveCase("split", 206, ((1, 3, 10, 4), S8, 0.05, 2),
                                                   [((1, 3, 4, 4), S8, 0.05, 2), ((1, 3, 6, 4), S8, 0.08, -5)],
                                                   origins=[(0, 0, 0, 0), (0, 0, 4, 0)])
    c["split_s16_rank3"] = lambda: MoveCase("split", 207, ((4, 6, 5), S16, 0.01, 0), [((4, 2, 5), S16, 0.01, 0), ((4, 4, 5), S16, 0.01, 0)],
                                            origins=[(0, 0, 0), (0, 2, 0)])
    c["permute_nhwc_to_nchw"] = lambda: MoveCase("permute", 208, ((2, 5, 7, 3),) + q, [((2, 3, 5, 7),) + q], perm=(0, 2, 3, 1))
    c["permute_rank3_u8"] = lambda: MoveCase("permute", 209, ((4, 6, 5), U8, 0.1, 7), [((5, 4, 6), U8, 0.1, 7)], perm=(1, 2, 0))
    c["transpose_nchw_to_nhwc"] = lambda: MoveCase("transpose", 210, ((2, 3, 5, 7),) + q, [((2, 5, 7, 3),) + q], perm=(0, 2, 3, 1))
    c["transpose_rank2_float"] = lambda: MoveCase("transpose", 211, ((9, 13), F32, 1.0, 0), [((13, 9), F32, 1.0, 0)], perm=(1, 0))
    c["transpose_rank5"] = lambda: MoveCase("transpose", 212, ((2, 3, 4, 5, 6),) + q, [((6, 2, 5, 3, 4),) + q], perm=(4, 0, 3, 1, 2))
    c["strided_slice_plain"] = lambda: MoveCase("strided_slice", 213, ((3, 8, 9, 4),) + q, [((2, 3, 4, 4),) + q],
                                                begin=(1, 1, 0, 0), end=(3, 7, 8, 4), stride=(1, 2, 2, 1))
    c["strided_slice_negative_stride_and_masks"] = lambda: MoveCase("strided_slice", 214, ((2, 6, 7, 5), U8, 0.2, 9), [((2, 6, 4, 2), U8, 0.2, 9)],
                                                                    begin=(0, 0, -1, 1), end=(0, 0, 0, 5), stride=(1, -1, -2, 2),
                                                                    begin_mask=0b0011, end_mask=0b0111)
    c["strided_slice_shrink_axis"] = lambda: MoveCase("strided_slice", 215, ((4, 5, 6),) + q, [((5, 3),) + q],
                                                      begin=(2, 0, 1), end=(3, 5, 6), stride=(1, 1, 2), shrink_axis_mask=0b001)
    c["slice_block"] = lambda: MoveCase("slice", 216, ((2, 9, 8, 16),) + q, [((1, 4, 5, 16),) + q], begin=(1, 2, 3, 0), end=(1, 4, 5, 16))
    c["depth_to_space_nhwc_block2"] = lambda: MoveCase("depth_to_space", 218, ((2, 3, 5, 32),) + q, [((2, 6, 10, 8),) + q], perm=(2, 0))
    c["depth_to_space_nchw_block3"] = lambda: MoveCase("depth_to_space", 219, ((1, 18, 4, 3), U8, 0.1, 7), [((1, 2, 12, 9), U8, 0.1, 7)], perm=(3, 1))
    c["space_to_depth_nhwc_block2"] = lambda: MoveCase("space_to_depth", 220, ((2, 6, 10, 8),) + q, [((2, 3, 5, 32),) + q], perm=(2, 0))
    c["space_to_depth_nchw_requantise"] = lambda: MoveCase("space_to_depth", 221, ((1, 3, 6, 9), S8, 0.05, 1), [((1, 27, 2, 3), S8, 0.08, -4)],
                                                           perm=(3, 1))
    c["channel_shuffle_nhwc_groups4"] = lambda: MoveCase("channel_shuffle", 222, ((2, 5, 4, 24),) + q, [((2, 5, 4, 24),) + q], perm=(3, 4))
    c["channel_shuffle_nchw_axis1_requantise"] = lambda: MoveCase("channel_shuffle", 223, ((2, 12, 3, 5), U8, 0.1, 100), [((2, 12, 3, 5), U8, 0.07, 90)],
                                                                  perm=(1, 3))
    c["stack_axis0"] = lambda: MoveCase("stack", 224, ((3, 4, 5),) + q, [((4, 5),) + q] * 3, perm=(0,))
    c["stack_axis2_rank4_out"] = lambda: MoveCase("stack", 225, ((2, 3, 2, 7), U8, 0.1, 9), [((2, 3, 7), U8, 0.1, 9)] * 2, perm=(2,))
    c["stack_last_axis_requantise"] = lambda: MoveCase("stack", 226, ((4, 6, 3), S8, 0.06, 2), [((4, 6), S8, 0.05, -1), ((4, 6), S8, 0.07, 3), ((4, 6), S8, 0.06, 2)],
                                                       perm=(2,))
    c["slice_rank2_s32"] = lambda: MoveCase("slice", 217, ((7, 9), S32, 1.0, 0), [((3, 4), S32, 1.0, 0)], begin=(2, 5), end=(3, 4))
    c["tile_rank3"] = lambda: MoveCase("tile", 235, ((2, 3, 5),) + q, [((4, 9, 5),) + q], perm=(2, 3, 1))
    c["tile_rank4_requantise_u8"] = lambda: MoveCase("tile", 236, ((1, 2, 3, 4), U8, 0.1, 9), [((2, 2, 6, 12), U8, 0.13, 20)], perm=(2, 1, 2, 3))
    c["tile_all_ones_float"] = lambda: MoveCase("tile", 237, ((3, 7), F32, 1.0, 0), [((3, 7), F32, 1.0, 0)], perm=(1, 1))
    c["broadcast_to_channels"] = lambda: MoveCase("broadcast_to", 238, ((1, 1, 1, 16),) + q, [((2, 5, 6, 16),) + q])
    c["broadcast_to_higher_rank_requantise"] = lambda: MoveCase("broadcast_to", 239, ((3, 1), S8, 0.05, 2), [((4, 2, 3, 7), S8, 0.08, -4)])
    c["broadcast_to_scalar_float"] = lambda: MoveCase("broadcast_to", 240, ((1,), F32, 1.0, 0), [((5, 9), F32, 1.0, 0)])
    # BatchToSpaceNd / SpaceToBatchNd: begin = block shape, end / stride = crops or padding before / after
    c["batch_to_space_2x2"] = lambda: MoveCase("batch_to_space", 227, ((8, 5, 6, 16),) + q, [((2, 10, 12, 16),) + q],
                                               perm=(0,), begin=(2, 2), end=(0, 0), stride=(0, 0))
    c["batch_to_space_crops"] = lambda: MoveCase("batch_to_space", 228, ((12, 4, 5, 7), U8, 0.1, 9), [((2, 5, 11, 7), U8, 0.1, 9)],
                                                 perm=(0,), begin=(2, 3), end=(1, 3), stride=(2, 1))
    c["batch_to_space_nchw_requantise"] = lambda: MoveCase("batch_to_space", 229, ((6, 3, 4, 5), S8, 0.05, 2), [((1, 3, 11, 9), S8, 0.08, -4)],
                                                           perm=(1,), begin=(3, 2), end=(0, 1), stride=(1, 0))
    c["batch_to_space_rank3"] = lambda: MoveCase("batch_to_space", 230, ((6, 5, 9),) + q, [((2, 12, 9),) + q],
                                                 perm=(0,), begin=(3,), end=(2,), stride=(1,))
    c["space_to_batch_2x2"] = lambda: MoveCase("space_to_batch", 231, ((2, 8, 6, 16),) + q, [((8, 4, 3, 16),) + q],
                                               perm=(0,), begin=(2, 2), end=(0, 0), stride=(0, 0))
    c["space_to_batch_padded_u8"] = lambda: MoveCase("space_to_batch", 232, ((2, 5, 7, 6), U8, 0.1, 131), [((12, 4, 4, 6), U8, 0.1, 131)],
                                                     perm=(0,), begin=(2, 3), end=(1, 3), stride=(2, 2))
    c["space_to_batch_nchw_requantise"] = lambda: MoveCase("space_to_batch", 233, ((1, 3, 7, 5), S8, 0.05, 2), [((6, 3, 3, 3), S8, 0.08, -4)],
                                                           perm=(1,), begin=(3, 2), end=(2, 0), stride=(0, 1))
    c["space_to_batch_rank3_dilation"] = lambda: MoveCase("space_to_batch", 234, ((2, 13, 8),) + q, [((8, 4, 8),) + q],
                                                          perm=(0,), begin=(4,), end=(2,), stride=(1,))
    return c


ALL_GROUPS = {"conv": conv_cases, "dwconv": dwconv_cases, "fc": fc_cases, "bmm": bmm_cases, "pool": pool_cases,
              "mean": mean_cases, "eltwise": eltwise_cases, "activation": activation_cases, "softmax": softmax_cases,
              "convert": convert_cases, "pad": pad_cases, "qlstm": qlstm_cases, "move": move_cases, "resize": resize_cases, "reduce": reduce_cases, "tconv": tconv_cases, "f32": f32_cases, "unary": unary_cases,
              "rows": rows_cases, "norm": norm_cases, "volume": volume_cases, "lstm": lstm_cases}


def run_case(case, where):
    """Outputs of a case as a list of arrays: [y, acc] for contractions, the case's output list otherwise."""
    if where == "oracle":
        r = case.run_oracle()
    elif where == "cpuref":
        r = case.run_cpuref()
    else:
        r = case.run_gpu()
    if isinstance(r, tuple):
        return [a for a in r if a is not None]
    if isinstance(r, list):
        return r
    return [r]
