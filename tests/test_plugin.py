"""The C++ backend plugin (armnn_b200/backend -> Nv_B200Acc_backend.so) inside the unmodified Arm NN runtime:
dynamic loading and registration (no GPU needed), and — on a GPU — whole graphs through INetwork -> Optimize({B200Acc})
-> LoadNetwork -> EnqueueWorkload against the same graph on CpuRef in the same process."""
import os

import numpy as np
import pytest

from q8util import diff_stats, have_cpuref

import hostnet

needs_plugin = pytest.mark.skipif(not (have_cpuref() and os.path.exists(hostnet.PLUGIN_PATH)),
                                  reason="Arm NN runtime (oracle/_ref) or the plugin is not built")


@needs_plugin
def test_plugin_is_found_loaded_and_registered_by_the_runtime():
    assert hostnet.ArmnnNetwork.backend_available("CpuRef")
    assert hostnet.ArmnnNetwork.backend_available("B200Acc")


@needs_plugin
def test_optimize_folds_activations_and_residual_adds_into_the_convolutions():
    """Optimize({B200Acc}) inside the unmodified runtime: B200Backend::OptimizeSubgraphView leaves no Activation layer
    and replaces Convolution2d -> Add -> ReLu by one PreCompiled layer wherever the channel count allows it."""
    from collections import Counter
    from armnn_b200 import configs
    net, _ = configs.resnet50(1, 64)
    kinds = Counter(t for t, _ in hostnet.ArmnnNetwork(net, "B200Acc", optimize_only=True).optimized_layers)
    assert kinds["PreCompiled"] == 16 and kinds["ElementwiseBinary"] == 0 and kinds["Activation"] == 0
    assert kinds["Convolution2d"] == 53 - 16
    net, _ = configs.mobilenet_v2(1, 64)
    kinds = Counter(t for t, _ in hostnet.ArmnnNetwork(net, "B200Acc", optimize_only=True).optimized_layers)
    # ten residual Adds; the one with 24 channels (not a multiple of 16) stays a layer of its own
    assert kinds["PreCompiled"] == 9 and kinds["ElementwiseBinary"] == 1 and kinds["Activation"] == 0
    # the same graphs on CpuRef keep every layer
    kinds = Counter(t for t, _ in hostnet.ArmnnNetwork(net, "CpuRef", optimize_only=True).optimized_layers)
    assert kinds["PreCompiled"] == 0 and kinds["ElementwiseBinary"] == 10


def _pair(net, info, dtype, seed=3):
    rng = np.random.default_rng(seed)
    lo, hi = (0, 256) if dtype == np.uint8 else (-128, 128)
    x = rng.integers(lo, hi, size=info["input_shape"]).astype(dtype)
    ref = hostnet.ArmnnNetwork(net, "CpuRef").run({0: x})[0]
    got = hostnet.ArmnnNetwork(net, "B200Acc").run({0: x})[0]
    return x, ref, got


@needs_plugin
@pytest.mark.gpu
def test_single_conv_through_the_runtime_matches_cpuref():
    from armnn_b200 import configs
    for args in ({}, {"output_scale": 0.33}):
        _, ref, got = _pair(*configs.single_conv(**args), np.int8)
        st = diff_stats(ref, got)
        assert st["max_abs"] <= 1 and st["mismatch_frac"] < 1e-3, st


@needs_plugin
@pytest.mark.gpu
def test_resnet50_reduced_through_the_runtime_matches_cpuref_and_the_python_mirror():
    from armnn_b200 import configs, network
    net, info = configs.resnet50(2, 64)
    x, ref, got = _pair(net, info, np.int8)
    st = diff_stats(ref, got)
    assert st["max_abs"] <= 1 and st["mismatch_frac"] < 0.02, st
    assert np.array_equal(ref.argmax(1), got.argmax(1))
    # the plugin and the Python host mirror drive the same kernels: identical class scores
    rt = network.IRuntime.Create(0)
    ln = rt.GetLoadedNetwork(rt.LoadNetwork(network.Optimize(net)))
    y = np.zeros(info["output_shape"], np.int8)
    ln.EnqueueWorkload({0: x}, {0: y})
    assert diff_stats(y, got)["max_abs"] <= 1


@needs_plugin
@pytest.mark.gpu
def test_mobilenet_v2_reduced_through_the_runtime_matches_cpuref():
    from armnn_b200 import configs
    _, ref, got = _pair(*configs.mobilenet_v2(1, 64), np.uint8)
    st = diff_stats(ref, got)
    assert st["max_abs"] <= 2 and st["mismatch_frac"] < 0.05, st


@needs_plugin
@pytest.mark.gpu
def test_unsupported_layer_makes_optimize_fail_instead_of_falling_back():
    from armnn_b200.network import DataType, INetwork, TensorInfo
    net = INetwork.Create()
    il = net.AddInputLayer(0)
    il.GetOutputSlot(0).SetTensorInfo(TensorInfo((1, 8), DataType.Float32))
    sl = net.AddSoftmaxLayer()
    il.GetOutputSlot(0).Connect(sl.GetInputSlot(0))
    sl.GetOutputSlot(0).SetTensorInfo(TensorInfo((1, 8), DataType.Float32))
    ml = net.AddMeanLayer((1,))
    sl.GetOutputSlot(0).Connect(ml.GetInputSlot(0))
    ml.GetOutputSlot(0).SetTensorInfo(TensorInfo((1,), DataType.Float32))
    ol = net.AddOutputLayer(0)
    ml.GetOutputSlot(0).Connect(ol.GetInputSlot(0))
    with pytest.raises(RuntimeError):
        hostnet.ArmnnNetwork(net, "B200Acc")


@needs_plugin
@pytest.mark.gpu
def test_qlstm_stack_through_the_runtime_matches_cpuref():
    from armnn_b200 import configs
    net, info = configs.qlstm_stack(batch=4, num_units=64, output_size=32)
    ref_net = hostnet.ArmnnNetwork(net, "CpuRef")
    gpu_net = hostnet.ArmnnNetwork(net, "B200Acc")
    rng = np.random.default_rng(6)
    state = {}
    for l in range(info["layers"]):
        state[1 + 2 * l] = np.zeros((4, 32), np.int8)
        state[2 + 2 * l] = np.zeros((4, 64), np.int16)
    for step in range(3):
        x = rng.integers(-128, 128, size=info["input_shape"]).astype(np.int8)
        ins = {0: x}
        ins.update(state)
        want = ref_net.run(ins)
        got = gpu_net.run(ins)
        for k in want:
            st = diff_stats(want[k], got[k])
            tol = 2 if want[k].dtype == np.int16 else 1
            assert st["max_abs"] <= tol and st["mismatch_frac"] <= 0.01, (step, k, st)
        state = {k: want[k] for k in state}


@needs_plugin
@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["import", "preimport"])
def test_imported_io_buffers_match_copied_ones(mode):
    """INetworkProperties{Malloc, Malloc} (the core calls ITensorHandle::Import on every EnqueueWorkload) and
    IRuntime::ImportInputs / ImportOutputs (imported once, buffers rewritten in place between inferences) give the
    results of the copying path, inference after inference."""
    from armnn_b200 import configs
    net, info = configs.resnet50(2, 64)
    copied = hostnet.ArmnnNetwork(net, "B200Acc")
    imported = hostnet.ArmnnNetwork(net, "B200Acc", import_io=(mode == "import"))
    rng = np.random.default_rng(11)
    x = np.zeros(info["input_shape"], np.int8)
    y = np.zeros(info["output_shape"], np.int8)
    seen = set()
    for _ in range(4):
        x[...] = rng.integers(-128, 128, size=x.shape)
        want = copied.run({0: x})[0]
        y[...] = 0
        imported.run_into({0: x}, {0: y}, preimported=(mode == "preimport"))
        assert np.array_equal(want, y)
        seen.add(y.tobytes())
    assert len(seen) > 1


@needs_plugin
@pytest.mark.gpu
@pytest.mark.parametrize("tx,ty", [(False, False), (False, True), (True, False)])
def test_batch_matmul_through_the_runtime_matches_cpuref(tx, ty):
    """BatchMatMul (attention-shaped: a batch of 8 heads, 64 x 32 by 32 x 48) with transposed operands through the real
    runtime on both backends; QAsymmS8 per-tensor operands as RefLayerSupport.cpp:697-740 allows."""
    from armnn_b200.network import DataType, INetwork, TensorInfo
    b, m, k, n = 8, 64, 32, 48
    net = INetwork.Create()
    x_shape = (b, k, m) if tx else (b, m, k)
    y_shape = (b, n, k) if ty else (b, k, n)
    ix = net.AddInputLayer(0)
    ix.GetOutputSlot(0).SetTensorInfo(TensorInfo(x_shape, DataType.QAsymmS8, 0.05, 3))
    iy = net.AddInputLayer(1)
    iy.GetOutputSlot(0).SetTensorInfo(TensorInfo(y_shape, DataType.QAsymmS8, 0.04, -5))
    l = net.AddBatchMatMulLayer(transpose_x=tx, transpose_y=ty)
    ix.GetOutputSlot(0).Connect(l.GetInputSlot(0))
    iy.GetOutputSlot(0).Connect(l.GetInputSlot(1))
    l.GetOutputSlot(0).SetTensorInfo(TensorInfo((b, m, n), DataType.QAsymmS8, 0.9, 7))
    ol = net.AddOutputLayer(0)
    l.GetOutputSlot(0).Connect(ol.GetInputSlot(0))
    rng = np.random.default_rng(21)
    x = rng.integers(-128, 128, size=x_shape).astype(np.int8)
    y = rng.integers(-128, 128, size=y_shape).astype(np.int8)
    ref = hostnet.ArmnnNetwork(net, "CpuRef").run({0: x, 1: y})[0]
    got = hostnet.ArmnnNetwork(net, "B200Acc").run({0: x, 1: y})[0]
    st = diff_stats(ref, got)
    assert st["max_abs"] <= 1 and st["mismatch_frac"] < 0.01, st
    assert np.unique(ref).size > 50                          # not saturated
