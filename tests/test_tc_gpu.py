"""The tcgen05 implicit-GEMM kernel (algo = 2, forced) against the CPU oracle: int32 accumulators and quantised
outputs bit-exact.  Covers both activation fetch modes (2-D tile for 1x1/FullyConnected, TMA im2col for the rest),
both swizzle widths (C = 64 -> 64-byte, C % 128 == 0 -> 128-byte), every N-tile width (64 / 128 / 256), ragged M
tails, input zero points with and without padding (prefix-table correction), strides, dilation, uint8 inputs."""
import numpy as np
import pytest

from q8util import _abi, diff_stats, random_conv_case, random_fc_case

pytestmark = pytest.mark.gpu

U8, S8 = _abi.U8, _abi.S8

CONV = {
    "gemm_c64_oc64": lambda: random_conv_case(201, 2, 14, 14, 64, 64, 1, 1),
    "gemm_c128_oc128_tail": lambda: random_conv_case(202, 1, 13, 11, 128, 128, 1, 1, act=(1, 0, 0)),
    "gemm_c256_oc256": lambda: random_conv_case(203, 2, 14, 14, 256, 256, 1, 1),
    "gemm_c64_oc256_zx0": lambda: random_conv_case(204, 1, 28, 28, 64, 256, 1, 1, x_q=(0.02, 0)),
    "gemm_u8_input": lambda: random_conv_case(205, 1, 14, 14, 128, 64, 1, 1, x_dtype=U8, y_dtype=U8, x_q=(0.02, 131)),
    "gemm_k2048": lambda: random_conv_case(206, 1, 7, 7, 2048, 512, 1, 1),
    "im2col_3x3_c64_config1": lambda: random_conv_case(1234, 1, 56, 56, 64, 64, 3, 3, pad=(1, 1, 1, 1), act=(1, 0, 0)),
    "im2col_3x3_c128_batch3": lambda: random_conv_case(207, 3, 14, 14, 128, 128, 3, 3, pad=(1, 1, 1, 1)),
    "im2col_3x3_zx0": lambda: random_conv_case(208, 2, 14, 14, 64, 64, 3, 3, pad=(1, 1, 1, 1), x_q=(0.02, 0)),
    "im2col_3x3_stride2": lambda: random_conv_case(209, 2, 28, 28, 128, 128, 3, 3, stride=(2, 2), pad=(1, 1, 1, 1), act=(1, 0, 0)),
    "im2col_3x3_stride2_tf_same": lambda: random_conv_case(210, 2, 28, 28, 64, 64, 3, 3, stride=(2, 2), pad=(0, 1, 0, 1)),
    "im2col_1x1_stride2": lambda: random_conv_case(211, 2, 28, 28, 256, 512, 1, 1, stride=(2, 2)),
    "im2col_3x3_dilation2": lambda: random_conv_case(212, 1, 14, 14, 64, 64, 3, 3, pad=(2, 2, 2, 2), dil=(2, 2)),
    "im2col_7x7_pad3": lambda: random_conv_case(213, 1, 14, 14, 64, 64, 7, 7, pad=(3, 3, 3, 3)),
    "im2col_no_pad_valid": lambda: random_conv_case(214, 1, 12, 12, 64, 128, 3, 3),
    "im2col_rect_3x1": lambda: random_conv_case(215, 1, 9, 11, 64, 64, 3, 1, stride=(1, 2), pad=(1, 1, 0, 0)),
    "gemm_fused_add_relu": lambda: random_conv_case(217, 2, 28, 28, 128, 512, 1, 1, act=(1, 0, 0), fused_add=True),
    # wide tiles + fused-add table leave a ring of two stages: several tiles per CTA, several K-slices per tile, so the
    # ring wraps many times with more producer warps than stages
    "gemm_fused_add_short_ring": lambda: random_conv_case(219, 24, 56, 56, 256, 256, 1, 1, act=(1, 0, 0), fused_add=True),
    "im2col_fused_add": lambda: random_conv_case(218, 2, 14, 14, 64, 64, 3, 3, pad=(1, 1, 1, 1), fused_add=True),
    "gemm_many_tiles_persistent": lambda: random_conv_case(219, 4, 56, 56, 64, 256, 1, 1, act=(1, 0, 0)),
    "im2col_many_tiles_persistent": lambda: random_conv_case(220, 6, 28, 28, 128, 128, 3, 3, pad=(1, 1, 1, 1)),
    "rowwin_stem_7x7_s2_c3": lambda: random_conv_case(240, 2, 64, 64, 3, 64, 7, 7, stride=(2, 2), pad=(2, 3, 2, 3), act=(1, 0, 0)),
    "rowwin_stem_224": lambda: random_conv_case(241, 1, 224, 224, 3, 64, 7, 7, stride=(2, 2), pad=(2, 3, 2, 3), act=(1, 0, 0)),
    "rowwin_3x3_s2_c3_u8": lambda: random_conv_case(242, 2, 32, 32, 3, 64, 3, 3, stride=(2, 2), pad=(0, 1, 0, 1), x_dtype=U8,
                                                     y_dtype=U8, x_q=(0.02, 128)),
    "rowwin_3x3_s1_c4": lambda: random_conv_case(243, 1, 20, 20, 4, 128, 3, 3, pad=(1, 1, 1, 1)),
    "rowwin_5x5_s1_c16_dil_h2": lambda: random_conv_case(244, 1, 24, 24, 16, 64, 5, 5, pad=(4, 4, 2, 2), dil=(2, 1)),
    "rowwin_1x1_c8_zx0": lambda: random_conv_case(245, 2, 9, 9, 8, 64, 1, 1, x_q=(0.02, 0)),
    "im2col_odd_image_7x7": lambda: random_conv_case(216, 5, 7, 7, 512, 512, 3, 3, pad=(1, 1, 1, 1), act=(1, 0, 0)),
    # channel counts that are multiples of 16 only: the last K-slice and the last N-tile are padding
    "gemm_c96_oc144": lambda: random_conv_case(250, 2, 14, 14, 96, 144, 1, 1, act=(1, 0, 0)),
    "gemm_c16_oc96": lambda: random_conv_case(251, 1, 28, 28, 32, 96, 1, 1),
    "gemm_c192_oc32": lambda: random_conv_case(252, 2, 14, 14, 192, 32, 1, 1),
    "gemm_c960_oc320": lambda: random_conv_case(253, 1, 7, 7, 960, 320, 1, 1),
    "im2col_3x3_c32_oc48": lambda: random_conv_case(254, 2, 14, 14, 32, 48, 3, 3, pad=(1, 1, 1, 1)),
    # per-tensor uint8 weights with a zero point: row sums of the activations from a second, 16-column MMA
    "gemm_u8w_c64_oc64": lambda: random_conv_case(260, 2, 14, 14, 64, 64, 1, 1, x_dtype=U8, w_dtype=U8, y_dtype=U8, x_q=(0.02, 128)),
    "gemm_u8w_c144_oc32_relu6": lambda: random_conv_case(261, 2, 28, 28, 144, 32, 1, 1, x_dtype=U8, w_dtype=U8, y_dtype=U8,
                                                          x_q=(0.03, 0), act=(2, 6.0, 0.0), y_zp=0),
    "gemm_u8w_c32_oc192_zx": lambda: random_conv_case(262, 1, 28, 28, 32, 192, 1, 1, x_dtype=U8, w_dtype=U8, y_dtype=U8, x_q=(0.02, 117)),
    "gemm_u8w_c320_oc1280": lambda: random_conv_case(263, 2, 7, 7, 320, 1280, 1, 1, x_dtype=U8, w_dtype=U8, y_dtype=U8, x_q=(0.02, 128)),
    "gemm_u8w_s8x": lambda: random_conv_case(264, 1, 14, 14, 128, 128, 1, 1, w_dtype=U8),
    "im2col_u8w_3x3_pad": lambda: random_conv_case(265, 2, 14, 14, 64, 64, 3, 3, pad=(1, 1, 1, 1), x_dtype=U8, w_dtype=U8, y_dtype=U8,
                                                    x_q=(0.02, 121)),
    "gemm_u8w_fused_add": lambda: random_conv_case(266, 2, 14, 14, 192, 32, 1, 1, x_dtype=U8, w_dtype=U8, y_dtype=U8, x_q=(0.02, 128),
                                                    fused_add=True),
    "rowwin_u8w_stem_3x3_s2_oc32": lambda: random_conv_case(267, 2, 64, 64, 3, 32, 3, 3, stride=(2, 2), pad=(0, 1, 0, 1), x_dtype=U8,
                                                            w_dtype=U8, y_dtype=U8, x_q=(0.02, 128), act=(2, 6.0, 0.0), y_zp=0),
    # channel counts that are multiples of 8 only: zero-padded copies in scratch (input) and / or a padded output
    "padded_c24_oc144_u8w": lambda: random_conv_case(270, 2, 28, 28, 24, 144, 1, 1, x_dtype=U8, w_dtype=U8, y_dtype=U8,
                                                     x_q=(0.02, 128), act=(2, 6.0, 0.0), y_zp=0),
    "padded_c144_oc24_u8w": lambda: random_conv_case(271, 2, 28, 28, 144, 24, 1, 1, x_dtype=U8, w_dtype=U8, y_dtype=U8, x_q=(0.02, 111)),
    "padded_c24_oc24_s8_3x3": lambda: random_conv_case(272, 1, 14, 14, 24, 24, 3, 3, pad=(1, 1, 1, 1)),
    "padded_c40_oc72_stride2": lambda: random_conv_case(273, 2, 14, 14, 40, 72, 3, 3, stride=(2, 2), pad=(0, 1, 0, 1), act=(1, 0, 0)),
    "rowwin_u8w_5x5_c4": lambda: random_conv_case(268, 1, 20, 20, 4, 48, 5, 5, pad=(2, 2, 2, 2), x_dtype=U8, w_dtype=U8, y_dtype=U8,
                                                  x_q=(0.02, 100)),
    # per-tensor weight zero points at the ends of their type's range: -zw = +128 does not fit one int8 tile value
    "gemm_s8w_zp_minus128": lambda: random_conv_case(280, 2, 14, 14, 64, 64, 1, 1, per_axis=False, w_zp=-128),
    "gemm_s8w_zp_plus127": lambda: random_conv_case(281, 2, 14, 14, 128, 96, 1, 1, per_axis=False, w_zp=127),
    "im2col_s8w_zp_minus128_pad": lambda: random_conv_case(282, 1, 14, 14, 64, 64, 3, 3, pad=(1, 1, 1, 1), per_axis=False, w_zp=-128),
    "gemm_u8w_zp_255": lambda: random_conv_case(283, 1, 14, 14, 64, 128, 1, 1, x_dtype=U8, w_dtype=U8, y_dtype=U8, x_q=(0.02, 7), w_zp=255),
    "gemm_u8w_zp_128": lambda: random_conv_case(284, 1, 14, 14, 64, 64, 1, 1, x_dtype=U8, w_dtype=U8, y_dtype=U8, x_q=(0.02, 255), w_zp=128),
    # fused Add whose last n-tile is partly padding (some epilogue warps have no columns in its second unit), in
    # row-window mode and as a plain GEMM: the operand buffers' release must not run ahead of slower warps
    "rowwin_fused_add_partial_tile": lambda: random_conv_case(5713, 18, 42, 24, 16, 160, 1, 1, fused_add=True),
    "gemm_fused_add_partial_tile": lambda: random_conv_case(287, 8, 28, 28, 64, 160, 1, 1, act=(1, 0, 0), fused_add=True),
    # explicit clamp narrower than the type on both sides (BoundedReLu with a non-zero lower bound), int8 and uint8
    "gemm_clamp_both_s8": lambda: random_conv_case(285, 2, 14, 14, 64, 128, 1, 1, act=(2, 3.0, -1.0)),
    "gemm_clamp_both_u8": lambda: random_conv_case(286, 2, 14, 14, 64, 64, 1, 1, x_dtype=U8, y_dtype=U8, x_q=(0.02, 128), act=(2, 2.0, -2.0)),
}

FC = {
    "fc_m1": lambda: random_fc_case(221, 1, 1024, 1024),
    "fc_m16": lambda: random_fc_case(222, 16, 1024, 1024),
    "fc_m256": lambda: random_fc_case(223, 256, 1024, 1024),
    "fc_m300_k4096_n256": lambda: random_fc_case(224, 300, 4096, 256),
}


def _poll():
    from armnn_b200 import lib
    lib.check(lib.load_library().b200k_poll_status())


@pytest.mark.parametrize("name", list(CONV))
def test_tcgen05_conv_bit_exact(built, name):
    case = CONV[name]()
    y, acc = case.run_oracle()
    gy, gacc = case.run_gpu(algo=2)
    _poll()
    assert np.array_equal(acc, gacc), (name, diff_stats(acc, gacc))
    assert np.array_equal(y, gy), (name, diff_stats(y, gy))
    # the accumulator dump goes through the kernel's cold pass: the plain launch must agree as well
    gy2, _ = case.run_gpu(want_acc=False, algo=2)
    _poll()
    assert np.array_equal(y, gy2), (name, diff_stats(y, gy2))


@pytest.mark.parametrize("name", list(FC))
def test_tcgen05_fully_connected_bit_exact(built, name):
    case = FC[name]()
    y, acc = case.run_oracle()
    gy, gacc = case.run_gpu(algo=2)
    _poll()
    assert np.array_equal(acc, gacc), (name, diff_stats(acc, gacc))
    assert np.array_equal(y, gy), (name, diff_stats(y, gy))


def test_tcgen05_equals_cuda_core_kernel_at_full_size(built):
    """At a size the oracle cannot finish quickly, the two independent CUDA implementations must agree exactly."""
    case = random_conv_case(230, 32, 56, 56, 64, 64, 3, 3, pad=(1, 1, 1, 1), act=(1, 0, 0))
    y1, a1 = case.run_gpu(algo=1)
    y2, a2 = case.run_gpu(algo=2)
    _poll()
    assert np.array_equal(a1, a2) and np.array_equal(y1, y2)
    case = random_conv_case(231, 32, 14, 14, 1024, 256, 1, 1, act=(1, 0, 0))
    y1, a1 = case.run_gpu(algo=1)
    y2, a2 = case.run_gpu(algo=2)
    _poll()
    assert np.array_equal(a1, a2) and np.array_equal(y1, y2)


def test_bounded_waits_give_up_and_report_a_timeout(built):
    """The failure path of the tcgen05 kernel, injected from the host: with selftest_us set the TMA producers issue no
    loads, so the MMA issuer, the epilogue warps and (once the ring is full) the producers all run into their wait
    limit of a few milliseconds, the kernel returns by itself and the status word says so.  The device stays usable:
    the next ordinary launch is bit-exact."""
    import ctypes as C
    import time
    from q8util import Cuda, gpu_pack
    from armnn_b200 import lib
    l = lib.load_library()
    case = random_conv_case(290, 2, 14, 14, 64, 64, 1, 1)
    mem = Cuda()
    p, y, _ = case.params(mem, False, 2)
    p.packed = gpu_pack(mem, p)
    p.selftest_us = 3000
    t0 = time.perf_counter()
    lib.call("conv2d_q8", p)
    rc = l.b200k_poll_status()                      # synchronises
    elapsed = time.perf_counter() - t0
    assert rc == _abi.E_TIMEOUT, rc
    assert b"wait gave up" in l.b200k_last_error()
    assert elapsed < 1.0, elapsed                   # a handful of 3 ms limits, not the two-second default
    assert l.b200k_poll_status() == 0               # the status word was cleared by the poll
    want, _ = case.run_oracle(want_acc=False)
    got, _ = case.run_gpu(want_acc=False, algo=2)
    _poll()
    assert np.array_equal(want, got)


def test_zero_points_outside_the_type_range_are_refused(built):
    from armnn_b200 import lib
    case = random_conv_case(291, 1, 8, 8, 64, 64, 1, 1, per_axis=False, w_zp=-128)
    case.w_q = (case.w_q[0], -200)                  # not an int8 value: the tcgen05 path must not take it
    with pytest.raises(lib.B200KError) as e:
        case.run_gpu(algo=2)
    assert e.value.code == _abi.E_UNSUPPORTED


def test_ineligible_shapes_are_refused_when_forced(built):
    from armnn_b200 import lib
    # channel counts that are not multiples of 8 cannot even use the zero-padded copies (a 1x1 convolution could run on
    # groups of pixels instead: 3x3 here)
    case = random_conv_case(232, 1, 8, 8, 20, 28, 3, 3, pad=(1, 1, 1, 1))
    with pytest.raises(lib.B200KError) as e:
        case.run_gpu(algo=2)
    assert e.value.code == _abi.E_UNSUPPORTED
    # multiples of 8 can, but only with the packed tables and the scratch: without them the forced launch is refused
    case = random_conv_case(233, 1, 8, 8, 24, 24, 1, 1)
    with pytest.raises(lib.B200KError) as e:
        case.run_gpu(algo=2, pack=False)
    assert e.value.code == _abi.E_UNSUPPORTED


@pytest.mark.parametrize("seed,big", [(1, False), (2, False), (7, True)])
def test_tcgen05_random_shapes_agree_with_cuda_core_kernel(built, seed, big):
    """Randomised geometry, channel counts, types, strides, padding and fused Adds: the tcgen05 kernel (stages of
    several K-slices, two producers, epilogue groups, all tile widths) against the CUDA-core kernel, which the other
    tests pin to the oracle.  `big`: many tiles per CTA, so that rings and accumulator buffers wrap many times."""
    rng = np.random.default_rng(seed)
    ran = 0
    for it in range(40):
        k = int(rng.choice([1, 1, 3, 3, 5, 7]))
        c = int(rng.choice([16, 32, 48, 64, 96, 128, 192, 256, 512]))
        oc = int(rng.choice([16, 32, 64, 80, 128, 160, 256, 320, 512]))
        if big:
            n, h, w = int(rng.integers(4, 24)), int(rng.integers(max(k, 20), 72)), int(rng.integers(max(k, 20), 72))
        else:
            n, h, w = int(rng.integers(1, 5)), int(rng.integers(max(k, 6), 40)), int(rng.integers(max(k, 6), 40))
        stride = int(rng.choice([1, 1, 2]))
        pad = k // 2 if rng.random() < 0.7 else 0
        kw = dict(stride=(stride, stride), pad=(pad, pad, pad, pad), fused_add=bool(rng.random() < 0.35))
        if rng.random() < 0.3:
            kw.update(x_dtype=U8, w_dtype=U8, y_dtype=U8, x_q=(0.02, int(rng.integers(0, 255))))
        if rng.random() < 0.5:
            kw["act"] = (1, 0, 0)
        case = random_conv_case(5000 + 100 * seed + it, n, h, w, c, oc, k, k, **kw)
        try:
            y2, a2 = case.run_gpu(algo=2)
        except Exception:
            continue                                       # a shape the tcgen05 path refuses (forced algo): not this test's subject
        y1, a1 = case.run_gpu(algo=1)
        _poll()
        ran += 1
        assert np.array_equal(a1, a2) and np.array_equal(y1, y2), (seed, it, n, h, w, c, oc, k, stride, pad, kw)
    assert ran >= 30
