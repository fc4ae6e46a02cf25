"""Host-side logic of the INetwork -> Optimize -> LoadNetwork mirror, and whole graphs on the CPU oracle against
the real Arm NN runtime on CpuRef (free-running, graph level).  No GPU needed."""
import numpy as np
import pytest

from armnn_b200 import configs, network
from armnn_b200.network import (ActivationFunction, DataType, INetwork, InvalidArgumentException, Optimize, TensorInfo)
from q8util import diff_stats, have_cpuref

needs_cpuref = pytest.mark.skipif(not have_cpuref(), reason="oracle/_ref not built (reference sources absent)")


def _conv_relu(out_q_conv, out_q_act):
    net = INetwork.Create()
    il = net.AddInputLayer(0)
    il.GetOutputSlot(0).SetTensorInfo(TensorInfo((1, 4, 4, 16), DataType.QAsymmS8, 0.1, 0))
    w = net.AddConstantLayer(np.ones((16, 1, 1, 16), np.int8), TensorInfo((16, 1, 1, 16), DataType.QSymmS8, 0.1, 0))
    cl = net.AddConvolution2dLayer(bias_enabled=False)
    il.GetOutputSlot(0).Connect(cl.GetInputSlot(0))
    w.GetOutputSlot(0).Connect(cl.GetInputSlot(1))
    cl.GetOutputSlot(0).SetTensorInfo(TensorInfo((1, 4, 4, 16), DataType.QAsymmS8, *out_q_conv))
    al = net.AddActivationLayer(ActivationFunction.ReLu)
    cl.GetOutputSlot(0).Connect(al.GetInputSlot(0))
    al.GetOutputSlot(0).SetTensorInfo(TensorInfo((1, 4, 4, 16), DataType.QAsymmS8, *out_q_act))
    ol = net.AddOutputLayer(0)
    al.GetOutputSlot(0).Connect(ol.GetInputSlot(0))
    return net


def test_optimize_fuses_relu_only_when_quantisation_matches():
    opt = Optimize(_conv_relu((0.2, -128), (0.2, -128)))
    types = [l.type for l in opt.layers]
    assert "Activation" not in types
    conv = [l for l in opt.layers if l.type == "Convolution2d"][0]
    assert conv.fused_activation[0] == ActivationFunction.ReLu
    opt = Optimize(_conv_relu((0.2, -128), (0.1, -128)))
    assert "Activation" in [l.type for l in opt.layers]


def test_optimize_refuses_unsupported_layers_there_is_no_cpu_fallback():
    net = INetwork.Create()
    il = net.AddInputLayer(0)
    il.GetOutputSlot(0).SetTensorInfo(TensorInfo((2, 3, 4), DataType.QAsymmS8, 0.1, 0))
    il2 = net.AddInputLayer(1)
    il2.GetOutputSlot(0).SetTensorInfo(TensorInfo((2, 4, 4), DataType.QAsymmS8, 0.1, 0))
    b = net.AddBatchMatMulLayer(adjoint_y=True)
    il.GetOutputSlot(0).Connect(b.GetInputSlot(0))
    il2.GetOutputSlot(0).Connect(b.GetInputSlot(1))
    b.GetOutputSlot(0).SetTensorInfo(TensorInfo((2, 3, 4), DataType.QAsymmS8, 0.1, 0))
    with pytest.raises(InvalidArgumentException, match="adjoint"):
        Optimize(net)
    with pytest.raises(InvalidArgumentException):
        Optimize(_conv_relu((0.2, 0), (0.2, 0)), ["CpuRef"])


def test_resnet50_layer_list_and_mac_count():
    net, info = configs.resnet50(1, 224)
    convs = [l for l in info["layers"] if l[1].startswith("conv")]
    assert len(convs) == 53                                   # stem + 16 blocks x 3 + 4 projection shortcuts
    assert info["macs"] == 4089186304                         # 4.09 GMAC per 224x224 image
    opt = Optimize(net)
    assert sum(1 for l in opt.layers if l.type == "Activation") == 0      # every ReLU fused
    # every residual Add (+ ReLU) is folded into the epilogue of the block's last convolution
    assert sum(1 for l in opt.layers if l.type == "ElementwiseBinary") == 0
    assert sum(1 for l in opt.layers if getattr(l, "fused_add", None) is not None) == 16


def _run_pair(net, info, dtype):
    import hostnet
    rng = np.random.default_rng(3)
    lo, hi = (0, 256) if dtype == np.uint8 else (-128, 128)
    x = rng.integers(lo, hi, size=info["input_shape"]).astype(dtype)
    want = hostnet.ArmnnNetwork(net, "CpuRef").run({0: x})[0]
    got = hostnet.OracleNetwork(Optimize(net)).run({0: x})[0]
    return want, got


@needs_cpuref
def test_single_conv_graph_oracle_vs_armnn_cpuref(built):
    want, got = _run_pair(*configs.single_conv(), np.int8)
    st = diff_stats(want, got)
    assert st["max_abs"] <= 1 and st["mismatch_frac"] < 1e-3, st


@needs_cpuref
def test_resnet50_reduced_oracle_vs_armnn_cpuref_free_running(built):
    """Whole ResNet-50 graph (2 x 64 x 64 input) through the real Arm NN Optimizer/Runtime on CpuRef versus the
    fused graph on the integer oracle: class scores within +-1 LSB."""
    want, got = _run_pair(*configs.resnet50(2, 64), np.int8)
    st = diff_stats(want, got)
    assert st["max_abs"] <= 1 and st["mismatch_frac"] < 0.02, st
    assert np.array_equal(want.argmax(1), got.argmax(1))


@needs_cpuref
def test_mobilenet_v2_reduced_oracle_vs_armnn_cpuref_free_running(built):
    want, got = _run_pair(*configs.mobilenet_v2(1, 64), np.uint8)
    st = diff_stats(want, got)
    assert st["max_abs"] <= 2 and st["mismatch_frac"] < 0.05, st


@needs_cpuref
def test_qlstm_stack_three_steps_oracle_vs_armnn_cpuref(built):
    """The 3-layer QLstm graph through the real Arm NN runtime on CpuRef versus the oracle, states fed back for three
    timesteps: identical int8 outputs and int16 cell states (the oracle restates CpuRef operation by operation)."""
    import hostnet
    net, info = configs.qlstm_stack(batch=2, num_units=64, output_size=32)
    ref_net = hostnet.ArmnnNetwork(net, "CpuRef")
    on = hostnet.OracleNetwork(Optimize(net))
    rng = np.random.default_rng(4)
    state = {}
    for l in range(info["layers"]):
        state[1 + 2 * l] = np.zeros((2, 32), np.int8)
        state[2 + 2 * l] = np.zeros((2, 64), np.int16)
    for step in range(3):
        x = rng.integers(-128, 128, size=info["input_shape"]).astype(np.int8)
        ins = {0: x}
        ins.update(state)
        want = ref_net.run(ins)
        got = on.run(ins)
        for k in want:
            assert np.array_equal(want[k], got[k]), (step, k)
        state = {k: want[k] for k in state}


@needs_cpuref
def test_data_movement_graph_mirror_views_vs_armnn_cpuref(built):
    """Splitter, Transpose, Permute, StridedSlice, Slice and a re-quantising Concat in one graph: the views the Python
    mirror derives from the descriptors (armnn_b200/views.py), executed by the oracle, against the real runtime on
    CpuRef.  Copies and fp32-faithful re-quantisation: identical bytes."""
    import hostnet
    from test_plugin import _data_movement_net
    net, info = _data_movement_net()
    x = np.random.default_rng(12).integers(-128, 128, size=info["input_shape"]).astype(np.int8)
    want = hostnet.ArmnnNetwork(net, "CpuRef").run({0: x})
    got = hostnet.OracleNetwork(Optimize(net)).run({0: x})
    assert sorted(want) == sorted(got) == [0, 1]
    for k in want:
        assert want[k].shape == got[k].shape and np.array_equal(want[k], got[k]), k
    assert np.array_equal(got[1], x[..., :16])


@needs_cpuref
def test_transpose_convolution_graph_oracle_vs_armnn_cpuref(built):
    """Two TransposeConvolution2d layers (per-axis weights + bias + fused ReLU; per-tensor weights without bias) through
    the real runtime on CpuRef versus the mirror's graph on the integer oracle: +-1 LSB."""
    from test_plugin import _tconv_net
    want, got = _run_pair(*_tconv_net(), np.int8)
    assert want.shape == got.shape
    st = diff_stats(want, got)
    assert st["max_abs"] <= 1 and st["mismatch_frac"] < 5e-3, st


@needs_cpuref
def test_space_depth_shuffle_stack_graph_mirror_views_vs_armnn_cpuref(built):
    import hostnet
    from test_plugin import _shuffle_net
    net, info = _shuffle_net()
    x = np.random.default_rng(16).integers(-128, 128, size=info["input_shape"]).astype(np.int8)
    want = hostnet.ArmnnNetwork(net, "CpuRef").run({0: x})
    got = hostnet.OracleNetwork(Optimize(net)).run({0: x})
    for k in (0, 1):
        assert want[k].shape == got[k].shape and np.array_equal(want[k], got[k]), k


@needs_cpuref
def test_float32_graph_oracle_equals_armnn_cpuref(built):
    """The fp32 Convolution2d / DepthwiseConvolution2d / FullyConnected restatements inside a graph (with a separate
    ReLU): identical bits to the real runtime on CpuRef."""
    import hostnet
    from test_plugin import _float_net
    net, info = _float_net()
    x = np.random.default_rng(18).standard_normal(info["input_shape"]).astype(np.float32)
    want = hostnet.ArmnnNetwork(net, "CpuRef").run({0: x})[0]
    got = hostnet.OracleNetwork(Optimize(net)).run({0: x})[0]
    assert want.shape == got.shape and np.array_equal(want, got)


@needs_cpuref
def test_space_to_batch_graph_mirror_views_vs_armnn_cpuref(built):
    """SpaceToBatchNd (zero fill + strided blocks) -> depthwise convolution -> BatchToSpaceNd with crops, and a rank-3
    SpaceToBatchNd that re-quantises: the mirror's views against the real runtime on CpuRef."""
    import hostnet
    from test_plugin import _dilated_by_batching_net
    net = _dilated_by_batching_net()
    rng = np.random.default_rng(32)
    xs = {0: rng.integers(-128, 128, size=(2, 9, 11, 16)).astype(np.int8), 1: rng.integers(0, 256, size=(3, 10, 12)).astype(np.uint8)}
    want = hostnet.ArmnnNetwork(net, "CpuRef").run(xs)
    got = hostnet.OracleNetwork(Optimize(net)).run(xs)
    assert want[1].shape == got[1].shape and np.array_equal(want[1], got[1])
    # the convolution in the middle: CpuRef accumulates in fp32, the oracle exactly (a rounding tie may differ by one)
    st = diff_stats(want[0], got[0])
    assert want[0].shape == got[0].shape and st["max_abs"] <= 1 and st["mismatch_frac"] < 5e-3, st


@needs_cpuref
def test_prelu_and_binary_graph_oracle_equals_armnn_cpuref(built):
    import hostnet
    from armnn_b200.network import BinaryOperation, DataType, INetwork, TensorInfo
    rng = np.random.default_rng(24)
    shape = (2, 6, 5, 16)
    net = INetwork.Create()
    il = net.AddInputLayer(0, "input")
    il.GetOutputSlot(0).SetTensorInfo(TensorInfo(shape, DataType.QAsymmS8, 0.04, 3))
    alpha = rng.integers(-128, 128, size=(16,)).astype(np.int8)
    al = net.AddConstantLayer(alpha, TensorInfo((16,), DataType.QAsymmS8, 0.01, 0), "alpha")
    pl = net.AddPreluLayer("prelu")
    il.GetOutputSlot(0).Connect(pl.GetInputSlot(0))
    al.GetOutputSlot(0).Connect(pl.GetInputSlot(1))
    pl.GetOutputSlot(0).SetTensorInfo(TensorInfo(shape, DataType.QAsymmS8, 0.03, -20))
    c = np.maximum(rng.integers(-128, 128, size=(1, 1, 1, 16)), -100).astype(np.int8)
    cl = net.AddConstantLayer(c, TensorInfo(c.shape, DataType.QAsymmS8, 0.02, -128), "divisor")
    fd = net.AddElementwiseBinaryLayer(BinaryOperation.FloorDiv, "floor_div")
    pl.GetOutputSlot(0).Connect(fd.GetInputSlot(0))
    cl.GetOutputSlot(0).Connect(fd.GetInputSlot(1))
    fd.GetOutputSlot(0).SetTensorInfo(TensorInfo(shape, DataType.QAsymmS8, 0.25, 0))
    ol = net.AddOutputLayer(0, "output")
    fd.GetOutputSlot(0).Connect(ol.GetInputSlot(0))
    x = rng.integers(-128, 128, size=shape).astype(np.int8)
    want = hostnet.ArmnnNetwork(net, "CpuRef").run({0: x})[0]
    got = hostnet.OracleNetwork(Optimize(net)).run({0: x})[0]
    assert np.array_equal(want, got)


@needs_cpuref
def test_l2_normalization_arg_max_log_softmax_graph_oracle_equals_armnn_cpuref(built):
    import hostnet
    from test_plugin import _rows_net
    net, shape = _rows_net()
    x = np.random.default_rng(38).integers(-128, 128, size=shape).astype(np.int8)
    want = hostnet.ArmnnNetwork(net, "CpuRef").run({0: x})
    got = hostnet.OracleNetwork(Optimize(net)).run({0: x})
    assert want[1].dtype == np.int32
    for k in (0, 1, 2):
        assert want[k].shape == got[k].shape and np.array_equal(want[k], got[k]), k


@needs_cpuref
def test_gather_batch_norm_instance_norm_graph_oracle_equals_armnn_cpuref(built):
    import hostnet
    from test_plugin import _norm_inputs, _norm_net
    net, xs = _norm_net(), _norm_inputs(44)
    want = hostnet.ArmnnNetwork(net, "CpuRef").run(xs)
    got = hostnet.OracleNetwork(Optimize(net)).run(xs)
    for k in (0, 1):
        assert want[k].shape == got[k].shape and np.array_equal(want[k], got[k]), k


@needs_cpuref
def test_tile_and_broadcast_to_graph_mirror_views_vs_armnn_cpuref(built):
    import hostnet
    from test_plugin import _repeat_inputs, _repeat_net
    net, xs = _repeat_net(), _repeat_inputs(48)
    want = hostnet.ArmnnNetwork(net, "CpuRef").run(xs)[0]
    got = hostnet.OracleNetwork(Optimize(net)).run(xs)[0]
    assert want.shape == got.shape and np.array_equal(want, got)


@needs_cpuref
def test_normalization_graph_oracle_equals_armnn_cpuref(built):
    import hostnet
    from test_plugin import _lrn_net
    net = _lrn_net()
    x = np.random.default_rng(54).integers(0, 256, size=(2, 6, 7, 16)).astype(np.uint8)
    want = hostnet.ArmnnNetwork(net, "CpuRef").run({0: x})[0]
    got = hostnet.OracleNetwork(Optimize(net)).run({0: x})[0]
    assert want.shape == got.shape and np.array_equal(want, got)


@needs_cpuref
def test_mirror_pad_gelu_floor_graph_oracle_equals_armnn_cpuref(built):
    import hostnet
    from test_plugin import _gelu_floor_mirror_inputs, _gelu_floor_mirror_net
    net, xs = _gelu_floor_mirror_net(), _gelu_floor_mirror_inputs(60)
    want = hostnet.ArmnnNetwork(net, "CpuRef").run(xs)
    got = hostnet.OracleNetwork(Optimize(net)).run(xs)
    for k in range(4):
        assert want[k].shape == got[k].shape and np.array_equal(want[k], got[k]), k


@needs_cpuref
def test_comparison_and_logical_graph_oracle_equals_armnn_cpuref(built):
    import hostnet
    from test_plugin import _boolean_inputs, _boolean_net
    net, shape = _boolean_net()
    xs = _boolean_inputs(62, shape)
    want = hostnet.ArmnnNetwork(net, "CpuRef").run(xs)[0]
    got = hostnet.OracleNetwork(Optimize(net)).run(xs)[0]
    assert set(np.unique(want)) <= {0, 1} and np.array_equal(want, got)


@needs_cpuref
def test_cast_and_fill_graph_oracle_equals_armnn_cpuref(built):
    import hostnet
    from test_plugin import _cast_fill_net
    net, shape = _cast_fill_net()
    xs = {0: np.random.default_rng(68).integers(-128, 128, size=shape).astype(np.int8), 1: np.array(shape, np.int32)}
    want = hostnet.ArmnnNetwork(net, "CpuRef").run(xs)[0]
    got = hostnet.OracleNetwork(Optimize(net)).run(xs)[0]
    assert want.dtype == np.int32 and np.array_equal(want, got)


@needs_cpuref
def test_volume_graph_oracle_vs_armnn_cpuref(built):
    import hostnet
    from test_plugin import _volume_net
    net = _volume_net()
    x = np.random.default_rng(74).integers(-128, 128, size=(1, 6, 8, 8, 4)).astype(np.int8)
    want = hostnet.ArmnnNetwork(net, "CpuRef").run({0: x})[0]
    got = hostnet.OracleNetwork(Optimize(net)).run({0: x})[0]
    st = diff_stats(want, got)
    assert want.shape == got.shape and st["max_abs"] <= 1 and st["mismatch_frac"] < 5e-3, st


@needs_cpuref
def test_shape_and_rank_graph_mirror_equals_armnn_cpuref(built):
    import hostnet
    from test_plugin import _shape_rank_net
    x = np.zeros((2, 3, 5, 7), np.uint8)
    want = hostnet.ArmnnNetwork(_shape_rank_net(with_rank=False), "CpuRef").run({0: x})
    got = hostnet.OracleNetwork(Optimize(_shape_rank_net())).run({0: x})
    assert list(want[0]) == [2, 3, 5, 7] and list(got[2]) == [4]
    for k in range(2):
        assert np.array_equal(want[k], got[k]), k


@needs_cpuref
def test_gather_nd_graph_oracle_equals_armnn_cpuref(built):
    import hostnet
    from test_plugin import _gather_nd_inputs, _gather_nd_net
    net, xs = _gather_nd_net(), _gather_nd_inputs(84)
    want = hostnet.ArmnnNetwork(net, "CpuRef").run(xs)
    got = hostnet.OracleNetwork(Optimize(net)).run(xs)
    for k in (0, 1):
        assert want[k].shape == got[k].shape and np.array_equal(want[k], got[k]), k


@needs_cpuref
@pytest.mark.parametrize("sequence,time_major", [(False, False), (True, False), (True, True)])
def test_float_lstm_graph_oracle_equals_armnn_cpuref(built, sequence, time_major):
    """The Lstm layer and UnidirectionalSequenceLstm in both layouts: the restatement run step by step through the mirror
    returns the real runtime's bits."""
    import hostnet
    from test_plugin import _lstm_net
    net, xs = _lstm_net(sequence, time_major)
    want = hostnet.ArmnnNetwork(net, "CpuRef").run(xs)
    got = hostnet.OracleNetwork(Optimize(net)).run(xs)
    # the reference's sequence workload keeps the states in buffers of its own and leaves its two state outputs unwritten
    # (RefUnidirectionalSequenceLstmWorkload.cpp:95-123); here they receive the final states
    for k in ((2,) if sequence else range(3)):
        assert want[k].shape == got[k].shape and np.array_equal(want[k], got[k]), k


@needs_cpuref
def test_reverse_v2_graph_oracle_equals_armnn_cpuref(built):
    import hostnet
    from test_plugin import _reverse_net
    net = _reverse_net()
    xs = {0: np.random.default_rng(98).integers(-128, 128, size=(2, 5, 6, 8)).astype(np.int8), 1: np.array([2, -3], np.int32)}
    want = hostnet.ArmnnNetwork(net, "CpuRef").run(xs)[0]
    got = hostnet.OracleNetwork(Optimize(net)).run(xs)[0]
    assert np.array_equal(want, xs[0][:, ::-1, ::-1, :]) and np.array_equal(want, got)


def test_fake_quantization_in_the_mirror_matches_the_formula(built):
    """armnn::INetwork cannot state a FakeQuantization layer, so the runtime bridge cannot either: the mirror's layer runs
    on the restatement (itself checked against the real RefFakeQuantizationFloat32Workload) and against the formula."""
    import hostnet
    from armnn_b200.network import DataType, INetwork, TensorInfo
    net = INetwork.Create()
    il = net.AddInputLayer(0, "input")
    il.GetOutputSlot(0).SetTensorInfo(TensorInfo((3, 50), DataType.Float32))
    fq = net.AddFakeQuantizationLayer(-2.0, 6.0, "fake_quantization")
    il.GetOutputSlot(0).Connect(fq.GetInputSlot(0))
    fq.GetOutputSlot(0).SetTensorInfo(TensorInfo((3, 50), DataType.Float32))
    ol = net.AddOutputLayer(0, "out")
    fq.GetOutputSlot(0).Connect(ol.GetInputSlot(0))
    x = (np.random.default_rng(101).standard_normal((3, 50)) * 4).astype(np.float32)
    got = hostnet.OracleNetwork(Optimize(net)).run({0: x})[0]
    scale, offset = np.float32(8.0) / np.float32(255.0), int(np.float32(2.0 * 255.0) / np.float32(8.0))
    q = x / scale
    want = np.clip(np.where(q >= 0, np.floor(q + np.float32(0.5)), np.ceil(q - np.float32(0.5))) + offset, 0, 255).astype(np.float32)
    assert np.array_equal(got, want)


@needs_cpuref
def test_fp16_conversion_graph_oracle_equals_armnn_cpuref(built):
    """The mirror's explicit conversion layers around a Float32 Activation against CpuRef's Float16 Activation (its
    decoder widens and its encoder narrows with the same FloatingPointConverter, saturation included)."""
    import hostnet
    from test_plugin import _fp16_net
    x = (np.random.default_rng(110).standard_normal((2, 40)) * 60).astype(np.float16)
    x[0, 0], x[1, 3] = 300.0, -280.0
    want = hostnet.ArmnnNetwork(_fp16_net(False), "CpuRef").run({0: x})[0]
    got = hostnet.OracleNetwork(Optimize(_fp16_net(True))).run({0: x})[0]
    assert want.dtype == np.float16 and want.max() == np.float16(65504)          # an overflowing square saturates
    assert np.array_equal(want.view(np.uint16), got.view(np.uint16))


@needs_cpuref
def test_scatter_nd_graph_oracle_equals_armnn_cpuref(built):
    import hostnet
    from test_plugin import _scatter_inputs, _scatter_net
    net, xs = _scatter_net(), _scatter_inputs(114)
    want = hostnet.ArmnnNetwork(net, "CpuRef").run(xs)
    got = hostnet.OracleNetwork(Optimize(net)).run(xs)
    for k in (0, 1):
        assert want[k].shape == got[k].shape and np.array_equal(want[k], got[k]), k
