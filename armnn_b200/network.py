"""Host-side mirror of the Arm NN flow for the B200Acc backend:

    INetwork (Add*Layer, slots, TensorInfo)  ->  Optimize(network, ["B200Acc"])  ->
    IRuntime.LoadNetwork  ->  LoadedNetwork.EnqueueWorkload(inputs, outputs)

Names, argument meaning and error behaviour follow the reference (include/armnn/INetwork.hpp,
include/armnn/IRuntime.hpp, src/armnn/Network.cpp:2026-2271, src/armnn/LoadedNetwork.cpp:783-981 of the
Arm NN tree): weights and biases are Constant layers feeding input slots 1 and 2, activations are separate
layers that Optimize fuses into the producer when the quantisation allows it (what Neon/CL do in
OptimizeSubgraphView, src/backends/cl/ClBackend.cpp:326-390), every layer must be supported by the backend or
Optimize raises, and one workload per layer is enqueued on a CUDA stream.  Each workload is one call of the
C ABI in include/b200k.h; torch is used for device memory, streams and events only.

The C++ plugin under armnn_b200/backend/ implements the same decisions against the real IBackendInternal
interface; this module is what the tests and the benchmark drive when no Arm NN runtime is around.
"""
import ctypes
from enum import IntEnum

import numpy as np

from . import _abi, lib, views


class DataType(IntEnum):            # include/armnn/Types.hpp:48-60
    Float16 = 0                     # only as the other side of ConvertFp16ToFp32 / ConvertFp32ToFp16
    Float32 = 1
    QAsymmU8 = 2
    Signed32 = 3
    Boolean = 4
    QSymmS16 = 5
    QSymmS8 = 6
    QAsymmS8 = 7


class ActivationFunction(IntEnum):  # include/armnn/Types.hpp:86-101
    Sigmoid = 0
    TanH = 1
    Linear = 2
    ReLu = 3
    BoundedReLu = 4
    SoftReLu = 5
    LeakyReLu = 6
    Abs = 7
    Sqrt = 8
    Square = 9
    Elu = 10
    HardSwish = 11
    Gelu = 12


class BinaryOperation(IntEnum):     # include/armnn/Types.hpp:138-149
    Add = 0
    Div = 1
    Maximum = 2
    Minimum = 3
    Mul = 4
    Sub = 5
    SqDiff = 6
    Power = 7
    FloorDiv = 8


class PoolingAlgorithm(IntEnum):
    Max = 0
    Average = 1
    L2 = 2


class PaddingMethod(IntEnum):
    IgnoreValue = 0
    Exclude = 1


# a Boolean tensor travels through the C ABI as bytes with scale 1 and zero point 0 (non-zero = true, results 0 or 1)
_ABI_DTYPE = {DataType.Float32: _abi.F32, DataType.QAsymmU8: _abi.U8, DataType.Signed32: _abi.S32,
              DataType.QSymmS16: _abi.S16, DataType.QSymmS8: _abi.S8, DataType.QAsymmS8: _abi.S8, DataType.Boolean: _abi.U8}
_NP_DTYPE = {DataType.Float32: np.float32, DataType.QAsymmU8: np.uint8, DataType.Signed32: np.int32,
             DataType.QSymmS16: np.int16, DataType.QSymmS8: np.int8, DataType.QAsymmS8: np.int8, DataType.Boolean: np.uint8,
             DataType.Float16: np.float16}
_TYPE_RANGE = {DataType.QAsymmU8: (0, 255), DataType.QAsymmS8: (-128, 127), DataType.QSymmS8: (-128, 127),
               DataType.QSymmS16: (-32768, 32767), DataType.Signed32: (-(1 << 31), (1 << 31) - 1)}


class InvalidArgumentException(ValueError):
    """armnn::InvalidArgumentException"""


class BackendUnavailableException(RuntimeError):
    """armnn::BackendUnavailableException"""


class TensorInfo:
    """armnn::TensorInfo: shape, data type and per-tensor or per-axis quantisation."""

    def __init__(self, shape, dtype, scale=1.0, offset=0, scales=None, quant_dim=None, constant=False):
        self.shape = tuple(int(s) for s in shape)
        self.dtype = DataType(dtype)
        self.scale = float(np.float32(scale))
        self.offset = int(offset)
        self.scales = None if scales is None else np.asarray(scales, dtype=np.float32)
        self.quant_dim = quant_dim
        self.constant = constant

    def GetNumElements(self):
        return int(np.prod(self.shape)) if self.shape else 1

    def GetNumBytes(self):
        return self.GetNumElements() * np.dtype(_NP_DTYPE[self.dtype]).itemsize

    def HasPerAxisQuantization(self):
        return self.scales is not None

    def same_quantization(self, other):
        return (self.dtype == other.dtype and self.scales is None and other.scales is None and
                self.scale == other.scale and self.offset == other.offset)

    def __repr__(self):
        return "TensorInfo(%s, %s, scale=%g, offset=%d%s)" % (self.shape, self.dtype.name, self.scale, self.offset,
                                                               ", per-axis" if self.scales is not None else "")


class OutputSlot:
    def __init__(self, layer, index):
        self.layer, self.index, self.info, self.connections = layer, index, None, []

    def SetTensorInfo(self, info):
        self.info = info

    def GetTensorInfo(self):
        return self.info

    def Connect(self, input_slot):
        if input_slot.source is not None:
            raise InvalidArgumentException("input slot %d of %s is already connected" % (input_slot.index, input_slot.layer.name))
        input_slot.source = self
        self.connections.append(input_slot)


class InputSlot:
    def __init__(self, layer, index):
        self.layer, self.index, self.source = layer, index, None


class Layer:
    def __init__(self, ltype, name, n_in, n_out, desc=None):
        self.type, self.name, self.desc = ltype, name or ltype, dict(desc or {})
        self.inputs = [InputSlot(self, i) for i in range(n_in)]
        self.outputs = [OutputSlot(self, i) for i in range(n_out)]
        self.fused_activation = None       # (function, a, b) set by Optimize
        self.const_data = None             # Constant layers: numpy array

    def GetInputSlot(self, i):
        return self.inputs[i]

    def GetOutputSlot(self, i=0):
        return self.outputs[i]

    def GetName(self):
        return self.name


class INetwork:
    """Graph builder; one Add*Layer per reference method used on the hot path (include/armnn/INetwork.hpp)."""

    def __init__(self):
        self.layers = []

    @staticmethod
    def Create():
        return INetwork()

    def _add(self, layer):
        self.layers.append(layer)
        return layer

    def AddInputLayer(self, binding_id, name=None):
        return self._add(Layer("Input", name, 0, 1, {"id": binding_id}))

    def AddOutputLayer(self, binding_id, name=None):
        return self._add(Layer("Output", name, 1, 0, {"id": binding_id}))

    def AddConstantLayer(self, data, info, name=None):
        info.constant = True
        layer = self._add(Layer("Constant", name, 0, 1))
        layer.const_data = np.ascontiguousarray(np.asarray(data).astype(_NP_DTYPE[info.dtype], copy=False)).reshape(info.shape)
        layer.outputs[0].SetTensorInfo(info)
        return layer

    def AddConvolution2dLayer(self, stride=(1, 1), pad=(0, 0, 0, 0), dilation=(1, 1), bias_enabled=True, name=None, nchw=False):
        """pad = (top, bottom, left, right); NHWC; inputs: 0 data, 1 weights [O,H,W,I], 2 bias.  nchw=True states the layer
        in DataLayout::NCHW (weights [O,I,H,W]): the B200Acc plugin runs it through a re-layout around the NHWC kernels;
        this Python runtime executes NHWC graphs only."""
        return self._add(Layer("Convolution2d", name, 3 if bias_enabled else 2, 1,
                               {"stride": stride, "pad": pad, "dilation": dilation, "bias": bias_enabled, "nchw": bool(nchw)}))

    def AddConvolution3dLayer(self, stride=(1, 1, 1), pad=(0, 0, 0, 0, 0, 0), dilation=(1, 1, 1), bias_enabled=True, name=None):
        """armnn::Convolution3dDescriptor, NDHWC: stride / dilation = (depth, height, width), pad = (front, back, top,
        bottom, left, right); inputs: 0 data [N,D,H,W,C], 1 weights [D,H,W,I,O], 2 bias."""
        return self._add(Layer("Convolution3d", name, 3 if bias_enabled else 2, 1,
                               {"stride": tuple(stride), "pad": tuple(pad), "dilation": tuple(dilation), "bias": bias_enabled}))

    def AddPooling3dLayer(self, pool_type, pool=(2, 2, 2), stride=(2, 2, 2), pad=(0, 0, 0, 0, 0, 0),
                          padding_method=PaddingMethod.Exclude, name=None):
        """armnn::Pooling3dDescriptor, NDHWC: pool / stride = (depth, height, width), pad = (front, back, top, bottom,
        left, right)."""
        return self._add(Layer("Pooling3d", name, 1, 1, {"type": PoolingAlgorithm(pool_type), "pool": tuple(pool), "stride": tuple(stride),
                                                          "pad": tuple(pad), "method": PaddingMethod(padding_method)}))

    def AddDepthwiseConvolution2dLayer(self, stride=(1, 1), pad=(0, 0, 0, 0), dilation=(1, 1), bias_enabled=True, name=None, nchw=False):
        """weights [1,H,W,I*M] (in both data layouts)"""
        return self._add(Layer("DepthwiseConvolution2d", name, 3 if bias_enabled else 2, 1,
                               {"stride": stride, "pad": pad, "dilation": dilation, "bias": bias_enabled, "nchw": bool(nchw)}))

    def AddFullyConnectedLayer(self, transpose_weights=False, bias_enabled=True, name=None):
        return self._add(Layer("FullyConnected", name, 3 if bias_enabled else 2, 1,
                               {"transpose": transpose_weights, "bias": bias_enabled}))

    def AddBatchMatMulLayer(self, transpose_x=False, transpose_y=False, adjoint_x=False, adjoint_y=False, name=None):
        return self._add(Layer("BatchMatMul", name, 2, 1, {"tx": transpose_x, "ty": transpose_y,
                                                            "ax": adjoint_x, "ay": adjoint_y}))

    def AddActivationLayer(self, function, a=0.0, b=0.0, name=None):
        return self._add(Layer("Activation", name, 1, 1, {"function": ActivationFunction(function), "a": float(a), "b": float(b)}))

    def AddPooling2dLayer(self, pool_type, pool=(2, 2), stride=(2, 2), pad=(0, 0, 0, 0),
                          padding_method=PaddingMethod.Exclude, name=None, nchw=False):
        return self._add(Layer("Pooling2d", name, 1, 1, {"type": PoolingAlgorithm(pool_type), "pool": pool, "stride": stride,
                                                          "pad": pad, "method": PaddingMethod(padding_method), "nchw": bool(nchw)}))

    def AddElementwiseBinaryLayer(self, operation, name=None):
        return self._add(Layer("ElementwiseBinary", name, 2, 1, {"op": BinaryOperation(operation)}))

    def AddAdditionLayer(self, name=None):
        return self.AddElementwiseBinaryLayer(BinaryOperation.Add, name)

    def AddMultiplicationLayer(self, name=None):
        return self.AddElementwiseBinaryLayer(BinaryOperation.Mul, name)

    def AddComparisonLayer(self, operation, name=None):
        """armnn::ComparisonDescriptor: 0 Equal, 1 Greater, 2 GreaterOrEqual, 3 Less, 4 LessOrEqual, 5 NotEqual; the
        output is a Boolean tensor."""
        if int(operation) not in range(6):
            raise InvalidArgumentException("Comparison: unknown operation %d" % operation)
        return self._add(Layer("Comparison", name, 2, 1, {"op": int(operation)}))

    def AddLogicalBinaryLayer(self, operation, name=None):
        """armnn::LogicalBinaryDescriptor: 0 LogicalAnd, 1 LogicalOr, on Boolean tensors."""
        if int(operation) not in (0, 1):
            raise InvalidArgumentException("LogicalBinary: unknown operation %d" % operation)
        return self._add(Layer("LogicalBinary", name, 2, 1, {"op": int(operation)}))

    def AddSubtractionLayer(self, name=None):
        return self.AddElementwiseBinaryLayer(BinaryOperation.Sub, name)

    def AddDivisionLayer(self, name=None):
        return self.AddElementwiseBinaryLayer(BinaryOperation.Div, name)

    def AddMaximumLayer(self, name=None):
        return self.AddElementwiseBinaryLayer(BinaryOperation.Maximum, name)

    def AddMinimumLayer(self, name=None):
        return self.AddElementwiseBinaryLayer(BinaryOperation.Minimum, name)

    def AddPreluLayer(self, name=None):
        """armnn::INetwork::AddPreluLayer: input 0 is the tensor, input 1 alpha (broadcast, aligned to the innermost
        dimensions when its rank is lower)."""
        return self._add(Layer("Prelu", name, 2, 1, {}))

    def AddSoftmaxLayer(self, beta=1.0, axis=-1, name=None):
        return self._add(Layer("Softmax", name, 1, 1, {"beta": float(beta), "axis": int(axis)}))

    def AddLogSoftmaxLayer(self, beta=1.0, axis=-1, name=None):
        return self._add(Layer("LogSoftmax", name, 1, 1, {"beta": float(beta), "axis": int(axis)}))

    def AddL2NormalizationLayer(self, eps=1e-12, nchw=False, name=None):
        """armnn::L2NormalizationDescriptor: normalises over the channel dimension of a tensor of up to 4 dimensions."""
        return self._add(Layer("L2Normalization", name, 1, 1, {"eps": float(eps), "nchw": bool(nchw)}))

    def AddArgMinMaxLayer(self, function, axis=-1, name=None):
        """armnn::ArgMinMaxDescriptor: function 0 Min, 1 Max; the output (Signed32) drops the axis."""
        if int(function) not in (0, 1):
            raise InvalidArgumentException("ArgMinMax: function must be 0 (Min) or 1 (Max)")
        return self._add(Layer("ArgMinMax", name, 1, 1, {"function": int(function), "axis": int(axis)}))

    def AddMeanLayer(self, axis=(1, 2), keep_dims=False, name=None):
        return self._add(Layer("Mean", name, 1, 1, {"axis": tuple(axis), "keep_dims": keep_dims}))

    def AddReshapeLayer(self, target_shape, name=None):
        return self._add(Layer("Reshape", name, 1, 1, {"shape": tuple(target_shape)}))

    def AddPadLayer(self, pad_list, pad_value=0.0, name=None, padding_mode=0):
        """pad_list: one (before, after) pair per dimension, outermost first (armnn::PadDescriptor::m_PadList);
        constant padding with pad_value — for quantised tensors a quantised number (normally the zero point), as
        armnn::Pad takes it (src/backends/reference/workloads/Pad.cpp:76-83).  padding_mode follows armnn::PaddingMode:
        0 Constant, 1 Reflect, 2 Symmetric (workloads/MirrorPad.cpp)."""
        return self._add(Layer("Pad", name, 1, 1, {"pads": tuple((int(a), int(b)) for a, b in pad_list), "value": float(pad_value),
                                                   "mode": int(padding_mode)}))

    def AddShapeLayer(self, name=None):
        """armnn::ShapeLayer: the input's shape as a Signed32 vector."""
        return self._add(Layer("Shape", name, 1, 1, {}))

    def AddRankLayer(self, name=None):
        """armnn::RankLayer: the input's number of dimensions as one Signed32 element."""
        return self._add(Layer("Rank", name, 1, 1, {}))

    def AddFakeQuantizationLayer(self, minimum, maximum, name=None):
        """armnn::FakeQuantizationDescriptor (Float32 tensors): every value becomes its 8-bit code over [min, max]."""
        return self._add(Layer("FakeQuantization", name, 1, 1, {"min": float(minimum), "max": float(maximum)}))

    def AddConvertFp16ToFp32Layer(self, name=None):
        return self._add(Layer("ConvertFp16ToFp32", name, 1, 1, {}))

    def AddConvertFp32ToFp16Layer(self, name=None):
        return self._add(Layer("ConvertFp32ToFp16", name, 1, 1, {}))

    def AddCastLayer(self, name=None):
        return self._add(Layer("Cast", name, 1, 1, {}))

    def AddFillLayer(self, value, name=None):
        """armnn::FillDescriptor: the input is the (ignored) shape tensor, every output element is `value`."""
        return self._add(Layer("Fill", name, 1, 1, {"value": float(value)}))

    def AddFloorLayer(self, name=None):
        return self._add(Layer("Floor", name, 1, 1, {}))

    def AddConcatLayer(self, view_origins, name=None):
        """view_origins: per input, the coordinates of its block in the output (armnn::OriginsDescriptor)."""
        origins = tuple(tuple(int(x) for x in o) for o in view_origins)
        return self._add(Layer("Concat", name, len(origins), 1, {"origins": origins}))

    def AddSplitterLayer(self, view_origins, name=None):
        """view_origins: per output, the coordinates of its block in the input (armnn::ViewsDescriptor); the view sizes
        are the outputs' shapes."""
        origins = tuple(tuple(int(x) for x in o) for o in view_origins)
        return self._add(Layer("Splitter", name, 1, len(origins), {"origins": origins}))

    def AddPermuteLayer(self, dim_mappings, name=None):
        """dim_mappings[i]: the destination dimension of source dimension i (armnn::PermuteDescriptor)."""
        return self._add(Layer("Permute", name, 1, 1, {"mappings": tuple(int(x) for x in dim_mappings)}))

    def AddTransposeLayer(self, dim_mappings, name=None):
        """dim_mappings[i]: the source dimension of destination dimension i (armnn::TransposeDescriptor)."""
        return self._add(Layer("Transpose", name, 1, 1, {"mappings": tuple(int(x) for x in dim_mappings)}))

    def AddStridedSliceLayer(self, begin, end, stride, begin_mask=0, end_mask=0, shrink_axis_mask=0, name=None):
        """armnn::StridedSliceDescriptor without ellipsis and new-axis masks."""
        return self._add(Layer("StridedSlice", name, 1, 1, {"begin": tuple(int(x) for x in begin), "end": tuple(int(x) for x in end),
                                                            "stride": tuple(int(x) for x in stride), "begin_mask": int(begin_mask),
                                                            "end_mask": int(end_mask), "shrink_axis_mask": int(shrink_axis_mask)}))

    def AddSliceLayer(self, begin, size, name=None):
        return self._add(Layer("Slice", name, 1, 1, {"begin": tuple(int(x) for x in begin), "size": tuple(int(x) for x in size)}))

    def AddDepthToSpaceLayer(self, block_size, nchw=False, name=None):
        return self._add(Layer("DepthToSpace", name, 1, 1, {"block": int(block_size), "nchw": bool(nchw)}))

    def AddSpaceToDepthLayer(self, block_size, nchw=False, name=None):
        return self._add(Layer("SpaceToDepth", name, 1, 1, {"block": int(block_size), "nchw": bool(nchw)}))

    def AddBatchToSpaceNdLayer(self, block_shape, crops, nchw=False, name=None):
        """armnn::BatchToSpaceNdDescriptor: one block extent and one (before, after) crop pair per spatial dimension."""
        return self._add(Layer("BatchToSpaceNd", name, 1, 1, {"block": tuple(int(b) for b in block_shape),
                                                              "edges": tuple((int(a), int(b)) for a, b in crops), "nchw": bool(nchw)}))

    def AddSpaceToBatchNdLayer(self, block_shape, pad_list, nchw=False, name=None):
        """armnn::SpaceToBatchNdDescriptor: one block extent and one (before, after) padding pair per spatial dimension."""
        return self._add(Layer("SpaceToBatchNd", name, 1, 1, {"block": tuple(int(b) for b in block_shape),
                                                              "edges": tuple((int(a), int(b)) for a, b in pad_list), "nchw": bool(nchw)}))

    def AddTileLayer(self, multiples, name=None):
        return self._add(Layer("Tile", name, 1, 1, {"multiples": tuple(int(m) for m in multiples)}))

    def AddBroadcastToLayer(self, shape, name=None):
        return self._add(Layer("BroadcastTo", name, 1, 1, {"shape": tuple(int(n) for n in shape)}))

    def AddChannelShuffleLayer(self, axis, num_groups, name=None):
        return self._add(Layer("ChannelShuffle", name, 1, 1, {"axis": int(axis), "groups": int(num_groups)}))

    def AddStackLayer(self, axis, num_inputs, name=None):
        """armnn::StackDescriptor (the input shape is taken from the connected inputs)."""
        return self._add(Layer("Stack", name, int(num_inputs), 1, {"axis": int(axis)}))

    def AddTransposeConvolution2dLayer(self, stride=(1, 1), pad=(0, 0, 0, 0), bias_enabled=True, name=None, nchw=False):
        """pad = (top, bottom, left, right); NHWC; inputs: 0 data, 1 weights [O,H,W,I], 2 bias (Constant layers: the Arm NN
        API takes them as ConstTensor arguments of the layer, armnn::INetwork::AddTransposeConvolution2dLayer)."""
        return self._add(Layer("TransposeConvolution2d", name, 3 if bias_enabled else 2, 1,
                               {"stride": tuple(stride), "pad": tuple(pad), "bias": bool(bias_enabled), "nchw": bool(nchw)}))

    def AddElementwiseUnaryLayer(self, operation, name=None):
        """armnn::UnaryOperation: 0 Abs, 1 Exp, 2 Sqrt, 3 Rsqrt, 4 Neg, 6 Log, 7 Sin, 8 Ceil (5 LogicalNot is not supported)."""
        return self._add(Layer("ElementwiseUnary", name, 1, 1, {"op": int(operation)}))

    def AddReduceLayer(self, axis, operation, keep_dims=False, name=None):
        """armnn::ReduceDescriptor; operation follows armnn::ReduceOperation (0 Sum, 1 Max, 2 Mean, 3 Min, 4 Prod)."""
        return self._add(Layer("Reduce", name, 1, 1, {"axis": tuple(int(a) for a in axis), "op": int(operation), "keep_dims": bool(keep_dims)}))

    def AddResizeLayer(self, target_height, target_width, method=0, align_corners=False, half_pixel_centers=False,
                       nchw=False, name=None):
        """armnn::ResizeDescriptor; method 0 = Bilinear, 1 = NearestNeighbor (armnn::ResizeMethod)."""
        return self._add(Layer("Resize", name, 1, 1, {"height": int(target_height), "width": int(target_width), "method": int(method),
                                                      "align_corners": bool(align_corners),
                                                      "half_pixel_centers": bool(half_pixel_centers), "nchw": bool(nchw)}))

    def AddQuantizeLayer(self, name=None):
        return self._add(Layer("Quantize", name, 1, 1))

    def AddDequantizeLayer(self, name=None):
        return self._add(Layer("Dequantize", name, 1, 1))

    def AddNormalizationLayer(self, channel_type, norm_size, alpha, beta, k, nchw=False, name=None):
        """armnn::NormalizationDescriptor with NormalizationAlgorithmMethod::LocalBrightness; channel_type 0 Across,
        1 Within."""
        if int(channel_type) not in (0, 1):
            raise InvalidArgumentException("Normalization: channel type must be 0 (Across) or 1 (Within)")
        return self._add(Layer("Normalization", name, 1, 1, {"channel_type": int(channel_type), "norm_size": int(norm_size),
                                                              "alpha": float(alpha), "beta": float(beta), "k": float(k), "nchw": bool(nchw)}))

    def AddGatherLayer(self, axis=0, name=None):
        """armnn::GatherDescriptor: input 0 the tensor, input 1 the Signed32 indices."""
        return self._add(Layer("Gather", name, 2, 1, {"axis": int(axis)}))

    def AddScatterNdLayer(self, function=0, input_enabled=True, name=None):
        """armnn::ScatterNdDescriptor (no axis): inputs are (input, or a Signed32 shape when input_enabled is False), indices
        [n, nd] and updates; function 0 Update, 1 Add, 2 Sub, 3 Max, 4 Min, 5 Mul."""
        if int(function) not in range(6):
            raise InvalidArgumentException("ScatterNd: unknown function %d" % function)
        return self._add(Layer("ScatterNd", name, 3, 1, {"function": int(function), "input_enabled": bool(input_enabled)}))

    def AddReverseV2Layer(self, name=None):
        """armnn::INetwork::AddReverseV2Layer: input 0 the tensor, input 1 the Signed32 axes to mirror."""
        return self._add(Layer("ReverseV2", name, 2, 1, {}))

    def AddGatherNdLayer(self, name=None):
        """armnn::INetwork::AddGatherNdLayer (no batch dimensions): input 0 the tensor, input 1 Signed32 index tuples
        [..., nd]."""
        return self._add(Layer("GatherNd", name, 2, 1, {}))

    def AddBatchNormalizationLayer(self, eps, mean, variance, beta, gamma, nchw=False, name=None):
        """armnn::INetwork::AddBatchNormalizationLayer: mean, variance, beta, gamma are (ndarray, TensorInfo) pairs of one
        value per channel."""
        layer = self._add(Layer("BatchNormalization", name, 1, 1, {"eps": float(eps), "nchw": bool(nchw)}))
        layer.bn_params = {"mean": mean, "variance": variance, "beta": beta, "gamma": gamma}
        return layer

    def AddInstanceNormalizationLayer(self, gamma=1.0, beta=0.0, eps=1e-12, nchw=False, name=None):
        return self._add(Layer("InstanceNormalization", name, 1, 1, {"gamma": float(gamma), "beta": float(beta), "eps": float(eps),
                                                                      "nchw": bool(nchw)}))

    def AddLstmLayer(self, descriptor, params, name=None):
        """armnn::INetwork::AddLstmLayer on Float32 tensors.  descriptor: dict of armnn::LstmDescriptor fields
        (ActivationFunc, ClippingThresCell, ClippingThresProj, CifgEnabled, PeepholeEnabled, ProjectionEnabled,
        LayerNormEnabled); params: dict name -> (ndarray, TensorInfo) of the LstmInputParams members.  Inputs: input,
        outputStateIn, cellStateIn.  Outputs: scratchBuffer, outputStateOut, cellStateOut, output."""
        layer = self._add(Layer("Lstm", name, 3, 4, dict(descriptor)))
        layer.qlstm_params = params
        return layer

    def AddUnidirectionalSequenceLstmLayer(self, descriptor, params, name=None):
        """armnn::INetwork::AddUnidirectionalSequenceLstmLayer on Float32 tensors: the LstmDescriptor fields plus TimeMajor;
        input [batch, time, input] (or [time, batch, input]).  Outputs: outputStateOut, cellStateOut, output."""
        layer = self._add(Layer("UnidirectionalSequenceLstm", name, 3, 3, dict(descriptor)))
        layer.qlstm_params = params
        return layer

    def AddQLstmLayer(self, descriptor, params, name=None):
        """descriptor: dict of armnn::QLstmDescriptor fields; params: dict name -> (ndarray, TensorInfo) of the
        LstmInputParams members.  Inputs: input, outputStateIn, cellStateIn.  Outputs: outputStateOut,
        cellStateOut, output (include/armnn/INetwork.hpp AddQLstmLayer)."""
        layer = self._add(Layer("QLstm", name, 3, 3, dict(descriptor)))
        layer.qlstm_params = params
        return layer


# ---------------------------------------------------------------------------------------------------
# Layer support (what B200LayerSupport::IsLayerSupported answers) and Optimize
# ---------------------------------------------------------------------------------------------------

_Q8 = (DataType.QAsymmU8, DataType.QAsymmS8, DataType.QSymmS8)


def _infos(layer):
    ins = [s.source.info if s.source is not None else None for s in layer.inputs]
    outs = [s.info for s in layer.outputs]
    return ins, outs


def IsLayerSupported(layer):
    """(supported, reason) for the B200Acc backend: 8-bit quantised NHWC hot path only."""
    ins, outs = _infos(layer)
    if any(i is None for i in ins):
        return False, "unconnected input slot"
    if any(o is None for o in outs):
        return False, "output TensorInfo not set"
    t = layer.type
    if t in ("Input", "Output", "Constant", "Reshape"):
        return True, ""
    if t in ("Convolution2d", "DepthwiseConvolution2d", "Pooling2d", "TransposeConvolution2d") and layer.desc.get("nchw"):
        return False, "%s: this runtime executes NHWC graphs only (the plugin re-lays NCHW layers out)" % t
    if t in ("Convolution2d", "DepthwiseConvolution2d", "FullyConnected"):
        x, w, y = ins[0], ins[1], outs[0]
        if not w.constant:
            return False, "%s: non-constant weights are not supported" % t
        if all(i.dtype == DataType.Float32 for i in list(ins) + list(outs)):
            return True, ""                                  # the fp32 variant (b200k_*_f32)
        if x.dtype not in _Q8 or y.dtype not in _Q8 or w.dtype not in _Q8:
            return False, "%s: input, weights and output must be 8-bit quantised or all Float32" % t
        if len(ins) > 2 and ins[2].dtype != DataType.Signed32:
            return False, "%s: bias must be Signed32" % t
        if w.HasPerAxisQuantization():
            want = {"Convolution2d": 0, "DepthwiseConvolution2d": 3}.get(t)
            if t == "FullyConnected":
                want = 0 if layer.desc["transpose"] else 1
            if w.quant_dim != want:
                return False, "%s: per-axis quantisation must be along the output-channel dimension" % t
        return True, ""
    if t == "BatchMatMul":
        if layer.desc["ax"] or layer.desc["ay"]:
            return False, "BatchMatMul: adjoint inputs are not supported"
        if all(i.dtype == DataType.Float32 for i in list(ins) + list(outs)):
            return True, ""                                  # the fp32 variant (b200k_batch_matmul_f32)
        if any(i.dtype not in _Q8 for i in ins) or outs[0].dtype not in _Q8:
            return False, "BatchMatMul: 8-bit quantised tensors, or Float32 throughout"
        return True, ""
    if t in ("Pooling2d", "Mean", "Reduce", "ElementwiseBinary", "Prelu", "Activation", "Softmax"):
        ok = (DataType.QAsymmU8, DataType.QAsymmS8, DataType.QSymmS16, DataType.Float32)
        if any(i.dtype not in ok for i in ins) or outs[0].dtype not in ok:
            return False, "%s: unsupported data type" % t
        if t in ("ElementwiseBinary", "Prelu") and len(outs[0].shape) > 4:
            return False, "%s: rank > 4" % t
        return True, ""
    if t in ("LogSoftmax", "L2Normalization"):
        ok = (DataType.QAsymmU8, DataType.QAsymmS8, DataType.Float32) + ((DataType.QSymmS16,) if t == "L2Normalization" else ())
        if ins[0].dtype not in ok or outs[0].dtype != ins[0].dtype:
            return False, "%s: unsupported or mismatched data types" % t
        if t == "L2Normalization" and len(ins[0].shape) > 4:
            return False, "L2Normalization: rank > 4"
        return True, ""
    if t in ("Comparison", "LogicalBinary"):
        ok = ((DataType.QAsymmU8, DataType.QAsymmS8, DataType.QSymmS16, DataType.Float32, DataType.Boolean) if t == "Comparison"
              else (DataType.Boolean,))
        if any(i.dtype not in ok for i in ins) or ins[0].dtype != ins[1].dtype or outs[0].dtype != DataType.Boolean:
            return False, "%s: inputs of one supported type and a Boolean output" % t
        if len(outs[0].shape) > 4 or any(len(i.shape) != len(outs[0].shape) for i in ins):
            return False, "%s: operands of one rank <= 4" % t
        return True, ""
    if t == "Gather":
        ok = (DataType.QAsymmU8, DataType.QAsymmS8, DataType.QSymmS16, DataType.Float32, DataType.Signed32)
        if ins[0].dtype not in ok or outs[0].dtype != ins[0].dtype or ins[1].dtype != DataType.Signed32:
            return False, "Gather: one supported element type for input and output, Signed32 indices"
        return True, ""
    if t == "ScatterNd":
        ok = (DataType.QAsymmU8, DataType.QAsymmS8, DataType.QSymmS16, DataType.Float32)
        first_ok = ins[0].dtype == outs[0].dtype if layer.desc["input_enabled"] else ins[0].dtype == DataType.Signed32
        if outs[0].dtype not in ok or ins[2].dtype != outs[0].dtype or ins[1].dtype != DataType.Signed32 or not first_ok:
            return False, "ScatterNd: one supported element type, Signed32 indices (and shape)"
        if len(ins[1].shape) != 2 or not (1 <= ins[1].shape[1] <= min(8, len(outs[0].shape))):
            return False, "ScatterNd: indices must be [n, nd] with nd within the output's rank (and 8)"
        return True, ""
    if t == "ReverseV2":
        ok = (DataType.QAsymmU8, DataType.QAsymmS8, DataType.QSymmS16, DataType.Float32, DataType.Signed32)
        if ins[0].dtype not in ok or outs[0].dtype != ins[0].dtype or ins[1].dtype != DataType.Signed32 or len(ins[0].shape) > 6:
            return False, "ReverseV2: one supported element type, Signed32 axes, rank <= 6"
        return True, ""
    if t == "GatherNd":
        ok = (DataType.QAsymmU8, DataType.QAsymmS8, DataType.QSymmS16, DataType.Float32, DataType.Signed32)
        if ins[0].dtype not in ok or outs[0].dtype != ins[0].dtype or ins[1].dtype != DataType.Signed32:
            return False, "GatherNd: one supported element type for input and output, Signed32 indices"
        if not (1 <= ins[1].shape[-1] <= min(8, len(ins[0].shape))):
            return False, "GatherNd: index tuples longer than the tensor's rank (or than 8)"
        return True, ""
    if t == "BatchNormalization":
        ok = (DataType.QAsymmU8, DataType.QAsymmS8, DataType.QSymmS16, DataType.Float32)
        if ins[0].dtype not in ok or outs[0].dtype not in ok or len(ins[0].shape) != 4:
            return False, "BatchNormalization: 4-D tensors of a supported data type only"
        if any(info.dtype not in ok for _, info in layer.bn_params.values()):
            return False, "BatchNormalization: unsupported parameter data type"
        return True, ""
    if t == "Normalization":
        ok = (DataType.QAsymmU8, DataType.QAsymmS8, DataType.QSymmS16, DataType.Float32)
        if ins[0].dtype not in ok or outs[0].dtype != ins[0].dtype or len(ins[0].shape) != 4:
            return False, "Normalization: 4-D tensors of one supported data type only"
        return True, ""
    if t == "InstanceNormalization":
        if ins[0].dtype != DataType.Float32 or outs[0].dtype != DataType.Float32 or len(ins[0].shape) != 4:
            return False, "InstanceNormalization: 4-D Float32 tensors only (as in the reference)"
        return True, ""
    if t == "ArgMinMax":
        if ins[0].dtype not in (DataType.QAsymmU8, DataType.QAsymmS8, DataType.QSymmS16, DataType.Float32):
            return False, "ArgMinMax: unsupported input data type"
        if outs[0].dtype != DataType.Signed32:
            return False, "ArgMinMax: the output must be Signed32"
        return True, ""
    if t in ("Quantize", "Dequantize"):
        return True, ""
    if t == "Pad":
        if len(ins[0].shape) > 4:
            return False, "Pad: rank > 4"
        mode = layer.desc.get("mode", 0)
        if mode not in (0, 1, 2):
            return False, "Pad: unknown padding mode"
        if mode and any(max(a, b) + (mode == 1) > n for (a, b), n in zip(layer.desc["pads"], ins[0].shape)):
            return False, "Pad: mirrored padding wider than the tensor"
        return True, ""
    if t == "Convolution3d":
        q8 = (DataType.QAsymmU8, DataType.QAsymmS8)
        if len(ins[0].shape) != 5 or len(ins[1].shape) != 5:
            return False, "Convolution3d: 5-D input and weights"
        if ins[0].dtype == DataType.Float32:
            if any(i.dtype != DataType.Float32 for i in list(ins) + list(outs)):
                return False, "Convolution3d: a Float32 input needs Float32 weights, bias and output"
            return True, ""
        if ins[0].dtype not in q8 or outs[0].dtype not in q8 or ins[1].dtype not in q8 + (DataType.QSymmS8,):
            return False, "Convolution3d: 8-bit quantised tensors or Float32 only"
        if len(ins) > 2 and ins[2].dtype != DataType.Signed32:
            return False, "Convolution3d: bias must be Signed32"
        if ins[1].scales is not None and ins[1].quant_dim != 4:
            return False, "Convolution3d: per-axis weights must be quantised along the output channels"
        return True, ""
    if t == "Pooling3d":
        ok = (DataType.QAsymmU8, DataType.QAsymmS8, DataType.QSymmS16, DataType.Float32)
        if len(ins[0].shape) != 5 or ins[0].dtype not in ok or outs[0].dtype != ins[0].dtype:
            return False, "Pooling3d: 5-D tensors of one supported data type"
        return True, ""
    if t in ("Shape", "Rank"):
        want = len(ins[0].shape) if t == "Shape" else 1
        if outs[0].dtype != DataType.Signed32 or outs[0].GetNumElements() != want:
            return False, "%s: the output must hold %d Signed32 element(s)" % (t, want)
        return True, ""
    if t == "FakeQuantization":
        if ins[0].dtype != DataType.Float32 or outs[0].dtype != DataType.Float32 or not layer.desc["max"] > layer.desc["min"]:
            return False, "FakeQuantization: Float32 tensors and min < max"
        return True, ""
    if t in ("ConvertFp16ToFp32", "ConvertFp32ToFp16"):
        a, b = (DataType.Float16, DataType.Float32) if t == "ConvertFp16ToFp32" else (DataType.Float32, DataType.Float16)
        if ins[0].dtype != a or outs[0].dtype != b or ins[0].GetNumElements() != outs[0].GetNumElements():
            return False, "%s: %s input and %s output of one size" % (t, a.name, b.name)
        return True, ""
    if t == "Cast":
        ok = (DataType.QAsymmU8, DataType.QAsymmS8, DataType.QSymmS8, DataType.QSymmS16, DataType.Signed32, DataType.Float32)
        if ins[0].dtype not in ok or outs[0].dtype not in ok or ins[0].GetNumElements() != outs[0].GetNumElements():
            return False, "Cast: unsupported data type or mismatched sizes"
        return True, ""
    if t == "Fill":
        if outs[0].dtype not in (DataType.Float32, DataType.Signed32):
            return False, "Fill: Float32 or Signed32 output only (as in the reference)"
        return True, ""
    if t == "Floor":
        if ins[0].dtype != DataType.Float32 or outs[0].dtype != DataType.Float32:
            return False, "Floor: Float32 only"
        return True, ""
    if t == "ElementwiseUnary":
        ok = (DataType.QAsymmU8, DataType.QAsymmS8, DataType.QSymmS16, DataType.Float32)
        if layer.desc["op"] == 5:
            ok = (DataType.Boolean,)                      # LogicalNot
        elif layer.desc["op"] not in (0, 1, 2, 3, 4, 6, 7, 8):
            return False, "ElementwiseUnary: operation %d is not supported" % layer.desc["op"]
        if ins[0].dtype not in ok or outs[0].dtype != ins[0].dtype:
            return False, "ElementwiseUnary: unsupported or mismatched data types"
        return True, ""
    if t == "TransposeConvolution2d":
        if ins[0].dtype not in _Q8 or outs[0].dtype not in _Q8 or ins[1].dtype not in _Q8:
            return False, "TransposeConvolution2d: 8-bit quantised tensors only"
        if any(s.source.layer.type != "Constant" for s in layer.inputs[1:]):
            return False, "TransposeConvolution2d: weights and bias must be constant"
        return True, ""
    if t == "Resize":
        ok = (DataType.QAsymmU8, DataType.QAsymmS8, DataType.QSymmS16, DataType.Float32)
        if ins[0].dtype not in ok or outs[0].dtype != ins[0].dtype or len(ins[0].shape) != 4:
            return False, "Resize: 4-D tensors of one supported data type only"
        if layer.desc["align_corners"] and layer.desc["half_pixel_centers"]:
            return False, "Resize: align_corners and half_pixel_centers cannot both be set"
        return True, ""
    if t in ("Concat", "Splitter"):
        # RefLayerSupport.cpp:949-979, 2597-2630: one element type for every tensor; quantisation may differ
        if len(ins[0].shape) > 6 or any(i.dtype != ins[0].dtype for i in list(ins) + list(outs)):
            return False, "%s: rank > 6 or mismatched data types" % t
        return True, ""
    if t in ("Tile", "BroadcastTo"):
        if any(i.dtype != outs[0].dtype for i in ins):
            return False, "%s: mismatched data types" % t
        try:
            v = (views.tile_view(ins[0].shape, layer.desc["multiples"])[1] if t == "Tile"
                 else views.broadcast_to_view(ins[0].shape, outs[0].shape))
            views.merge_dims(v)
        except ValueError as e:
            return False, "%s: %s" % (t, e)
        return True, ""
    if t in ("SpaceToDepth", "ChannelShuffle", "Stack", "BatchToSpaceNd", "SpaceToBatchNd"):
        # through Decoder / Encoder in the reference: one element type, quantisation may differ
        if len(outs[0].shape) > 6 or any(i.dtype != outs[0].dtype for i in ins):
            return False, "%s: rank > 6 or mismatched data types" % t
        if t in ("BatchToSpaceNd", "SpaceToBatchNd") and len(ins[0].shape) not in (3, 4):
            return False, "%s: 3 or 4 dimensions only" % t
        return True, ""
    if t in ("Permute", "Transpose", "StridedSlice", "Slice", "DepthToSpace"):
        if len(ins[0].shape) > (4 if t == "StridedSlice" else 6):
            return False, "%s: rank not supported" % t
        if t == "StridedSlice" and (layer.desc.get("ellipsis_mask", 0) or layer.desc.get("new_axis_mask", 0)):
            return False, "StridedSlice: ellipsis and new-axis masks are not supported"
        if ins[0].dtype != outs[0].dtype or not outs[0].same_quantization(ins[0]):
            return False, "%s: input and output must share type and quantisation (the reference copies raw elements)" % t
        return True, ""
    if t in ("Lstm", "UnidirectionalSequenceLstm"):
        if any(i.dtype != DataType.Float32 for i in list(ins) + list(outs)):
            return False, "%s: Float32 tensors only" % t
        if any(info.dtype != DataType.Float32 for item in layer.qlstm_params.values() if item is not None for info in [item[1]]):
            return False, "%s: Float32 weights only" % t
        if layer.desc.get("ActivationFunc", 4) not in (0, 1, 3, 4, 6):
            return False, "%s: unsupported activation function" % t
        return True, ""
    if t == "QLstm":
        if ins[0].dtype != DataType.QAsymmS8 or ins[2].dtype != DataType.QSymmS16:
            return False, "QLstm: input must be QAsymmS8 and cell state QSymmS16"
        return True, ""
    return False, "layer type %s is not on the B200Acc hot path" % t


_FUSABLE_PRODUCERS = ("Convolution2d", "DepthwiseConvolution2d", "FullyConnected", "ElementwiseBinary", "TransposeConvolution2d")


class OptimizedNetwork:
    def __init__(self, layers, model_options):
        self.layers, self.model_options = layers, model_options


def Optimize(network, backend_preferences=("B200Acc",), model_options=None):
    """Checks that B200Acc supports every layer (there is no fallback backend), fuses ReLu / BoundedReLu
    activations into their producer, orders the graph.  Mirrors armnn::Optimize + OptimizeSubgraphView."""
    if "B200Acc" not in tuple(backend_preferences):
        raise InvalidArgumentException("this runtime only provides the B200Acc backend")
    for layer in network.layers:
        ok, reason = IsLayerSupported(layer)
        if not ok:
            raise InvalidArgumentException("Layer of type %s (%s) is not supported on requested backend B200Acc: %s"
                                           % (layer.type, layer.name, reason))
    # activation fusion
    removed = set()
    for act in network.layers:
        if act.type != "Activation" or act.desc["function"] not in (ActivationFunction.ReLu, ActivationFunction.BoundedReLu):
            continue
        src = act.inputs[0].source
        prod = src.layer
        if prod.type not in _FUSABLE_PRODUCERS or prod.fused_activation is not None or len(src.connections) != 1:
            continue
        if prod.type == "ElementwiseBinary" and prod.desc["op"] not in (BinaryOperation.Add, BinaryOperation.Mul, BinaryOperation.Sub):
            continue
        if not src.info.same_quantization(act.outputs[0].info) or src.info.dtype == DataType.Float32:
            continue
        prod.fused_activation = (act.desc["function"], act.desc["a"], act.desc["b"])
        # re-route the activation's consumers to the producer
        src.connections = []
        for consumer in act.outputs[0].connections:
            consumer.source = src
            src.connections.append(consumer)
        removed.add(id(act))
    # residual-add fusion: Convolution2d -> Add(other) [-> ReLu already folded into the Add] becomes one
    # convolution workload whose epilogue adds the other operand (b200k_conv2d_params.add_operand)
    for add in network.layers:
        if add.type != "ElementwiseBinary" or add.desc["op"] != BinaryOperation.Add or id(add) in removed:
            continue
        out_info = add.outputs[0].info
        if out_info.dtype not in _Q8:
            continue
        for side in (0, 1):
            src, other = add.inputs[side].source, add.inputs[1 - side].source
            conv = src.layer
            if (conv.type != "Convolution2d" or conv.fused_activation is not None or len(src.connections) != 1 or
                    getattr(conv, "fused_add", None) is not None or src.info.shape != out_info.shape or
                    other.info.shape != out_info.shape or other.info.dtype not in _Q8 or other.layer is conv):
                continue
            if out_info.shape[-1] % 16 != 0:
                # such a convolution runs on channel-padded copies (b200k_conv2d_scratch_bytes), which has no fused
                # Add: the Add stays a workload of its own
                continue
            conv.fused_add = {"conv_out_info": src.info}
            conv.fused_activation = add.fused_activation
            # the other operand becomes an extra input of the convolution layer (after data, weights, bias)
            extra = InputSlot(conv, len(conv.inputs))
            conv.inputs.append(extra)
            other.connections = [c for c in other.connections if c is not add.inputs[1 - side]]
            extra.source = other
            other.connections.append(extra)
            # the convolution now produces the Add's output
            src.info = out_info
            src.connections = []
            for consumer in add.outputs[0].connections:
                consumer.source = src
                src.connections.append(consumer)
            removed.add(id(add))
            break
    layers = [l for l in network.layers if id(l) not in removed]
    # topological order (layers may have been added in any order)
    order, done = [], set()

    def visit(l):
        if id(l) in done:
            return
        for s in l.inputs:
            visit(s.source.layer)
        done.add(id(l))
        order.append(l)
    for l in layers:
        visit(l)
    return OptimizedNetwork(order, dict(model_options or {}))


# ---------------------------------------------------------------------------------------------------
# Runtime
# ---------------------------------------------------------------------------------------------------

def _qt(info, ptr, scales_ptr=None):
    t = _abi.QTensor()
    t.data = ptr
    t.dtype = _ABI_DTYPE[info.dtype]
    t.scale, t.zero_point = (1.0, 0) if info.dtype == DataType.Boolean else (info.scale, info.offset)
    t.scales = scales_ptr
    return t


def _clamp(layer, info):
    lo, hi = ctypes.c_int32(), ctypes.c_int32()
    kind, a, b = 0, 0.0, 0.0
    if layer.fused_activation is not None:
        fn, a, b = layer.fused_activation
        kind = 1 if fn == ActivationFunction.ReLu else 2
    lib.check(lib.load_library().b200k_activation_clamp(kind, a, b, info.scale, info.offset, _ABI_DTYPE[info.dtype],
                                                        ctypes.byref(lo), ctypes.byref(hi)))
    return lo.value, hi.value


class IRuntime:
    """armnn::IRuntime for one device.  Raises BackendUnavailableException when the device cannot be opened."""

    def __init__(self, device_id=0):
        import torch
        self.torch = torch
        if not torch.cuda.is_available():
            raise BackendUnavailableException("B200Acc: no CUDA device visible")
        rc = lib.load_library().b200k_device_open(device_id)
        if rc != 0:
            raise BackendUnavailableException("B200Acc: " + lib.load_library().b200k_last_error().decode())
        self.device = torch.device("cuda", device_id)
        self.networks = {}

    @staticmethod
    def Create(device_id=0):
        return IRuntime(device_id)

    def LoadNetwork(self, optimized):
        net = LoadedNetwork(self, optimized)
        net_id = len(self.networks)
        self.networks[net_id] = net
        return net_id

    def GetLoadedNetwork(self, net_id):
        return self.networks[net_id]

    def EnqueueWorkload(self, net_id, input_tensors, output_tensors):
        return self.networks[net_id].EnqueueWorkload(input_tensors, output_tensors)

    def UnloadNetwork(self, net_id):
        del self.networks[net_id]


class GraphProgram:
    """Memory-agnostic part of a loaded network: one tensor per output slot and one prepared C-ABI parameter
    struct per layer.  Subclasses say where tensors live (`_alloc`, `_upload`, `_ptr`, `_view`)."""

    def __init__(self, optimized):
        self.layers = optimized.layers
        self.tensors = {}          # id(OutputSlot) -> tensor object of the memory space
        self.aux = []              # per-axis scale arrays, QLstm weight copies: kept alive
        self.workloads = []        # (layer, entry name, params struct)
        self.inputs, self.outputs = {}, {}

    # -- memory (overridden per memory space) ---------------------------------------------------------
    def _alloc(self, info):
        raise NotImplementedError

    def _upload(self, array):
        raise NotImplementedError

    def _ptr(self, tensor):
        raise NotImplementedError

    def _view(self, tensor, shape):
        raise NotImplementedError

    def _dev(self, slot):
        return self.tensors[id(slot)]

    def _scales(self, info):
        if info.scales is None:
            return None
        t = self._upload(info.scales.copy())
        self.aux.append(t)
        return self._ptr(t)

    def _operand(self, slot):
        return _qt(slot.info, self._ptr(self._dev(slot)), self._scales(slot.info))

    def _pack_weights(self, conv_params):
        """Load-time weight preparation (b200k_conv2d_pack); returns a pointer or None.  Only the CUDA
        runtime overrides this."""
        return None

    def _attach_scratch(self, conv_params):
        """Per-call scratch of a convolution workload (b200k_conv2d_scratch_bytes); CUDA runtime only."""

    # -- workload construction -------------------------------------------------------------------------
    def _build(self):
        for layer in self.layers:
            t = layer.type
            if t == "Input":
                self.tensors[id(layer.outputs[0])] = self._alloc(layer.outputs[0].info)
                self.inputs[layer.desc["id"]] = layer.outputs[0]
                continue
            if t == "Constant":
                # RefConstantWorkload: one copy of the layer blob into its output handle, at load time
                self.tensors[id(layer.outputs[0])] = self._upload(layer.const_data)
                continue
            if t == "Output":
                self.outputs[layer.desc["id"]] = layer.inputs[0].source
                continue
            if t == "Reshape":
                # aliasing view, no kernel (RefReshapeWorkload is a memcpy)
                src = self._dev(layer.inputs[0].source)
                self.tensors[id(layer.outputs[0])] = self._view(src, layer.outputs[0].info.shape)
                continue
            for o in layer.outputs:
                self.tensors[id(o)] = self._alloc(o.info)
            made = getattr(self, "_make_" + t)(layer)
            for entry_and_params in (made if isinstance(made, list) else [made]):
                self.workloads.append((layer,) + entry_and_params)

    def _conv_params(self, layer, depthwise):
        x, w = layer.inputs[0].source, layer.inputs[1].source
        y = layer.outputs[0]
        p = _abi.Conv2dParams()
        p.x, p.w, p.y = self._operand(x), self._operand(w), self._operand(y)
        if layer.desc["bias"]:
            p.bias = self._operand(layer.inputs[2].source)
        n, h, wd, c = x.info.shape
        _, oh, ow, oc = y.info.shape
        kh, kw = w.info.shape[1], w.info.shape[2]
        p.n, p.h, p.wd, p.c, p.oh, p.ow, p.oc, p.kh, p.kw = n, h, wd, c, oh, ow, oc, kh, kw
        p.stride_h, p.stride_w = layer.desc["stride"]
        p.pad_top, p.pad_left = layer.desc["pad"][0], layer.desc["pad"][2]
        p.dil_h, p.dil_w = layer.desc["dilation"]
        if y.info.dtype == DataType.Float32:
            return p                                         # the fp32 variant: no clamp, no tables
        p.clamp_lo, p.clamp_hi = _clamp(layer, y.info)
        fused = getattr(layer, "fused_add", None)
        if fused is not None:
            # y carries the convolution's own quantisation only; the stored tensor is the Add's output
            p.add_out = p.y
            p.y = _qt(fused["conv_out_info"], None)
            p.add_operand = self._operand(layer.inputs[-1].source)
        if not depthwise:
            p.packed = self._pack_weights(p)
            self._attach_scratch(p)
        return p

    def _make_Convolution3d(self, layer):
        x, w, y, d = layer.inputs[0].source, layer.inputs[1].source, layer.outputs[0], layer.desc
        p = _abi.Conv3dParams()
        p.x, p.w, p.y = self._operand(x), self._operand(w), self._operand(y)
        if d["bias"]:
            p.bias = self._operand(layer.inputs[2].source)
        p.n, p.d, p.h, p.wd, p.c = x.info.shape
        _, p.od, p.oh, p.ow, p.oc = y.info.shape
        p.kd, p.kh, p.kw = w.info.shape[:3]
        if tuple(w.info.shape[3:]) != (p.c, p.oc):
            raise InvalidArgumentException("Convolution3d: weights %s do not match %d input and %d output channels" % (w.info.shape, p.c, p.oc))
        p.stride_d, p.stride_h, p.stride_w = d["stride"]
        p.pad_front, p.pad_top, p.pad_left = d["pad"][0], d["pad"][2], d["pad"][4]
        p.dil_d, p.dil_h, p.dil_w = d["dilation"]
        if y.info.dtype != DataType.Float32:
            p.clamp_lo, p.clamp_hi = _clamp(layer, y.info)
        return "conv3d_q", p

    def _make_Pooling3d(self, layer):
        x, y, d = layer.inputs[0].source, layer.outputs[0], layer.desc
        p = _abi.Pool3dParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.n, p.d, p.h, p.wd, p.c = x.info.shape
        _, p.od, p.oh, p.ow, _ = y.info.shape
        p.pool_d, p.pool_h, p.pool_w = d["pool"]
        p.stride_d, p.stride_h, p.stride_w = d["stride"]
        p.pad_front, p.pad_back, p.pad_top, p.pad_bottom, p.pad_left, p.pad_right = d["pad"]
        p.pool_type, p.padding_method = int(d["type"]), int(d["method"])
        return "pool3d_q", p

    def _make_Convolution2d(self, layer):
        if layer.outputs[0].info.dtype == DataType.Float32:
            return "conv2d_f32", self._conv_params(layer, False)
        return "conv2d_q8", self._conv_params(layer, False)

    def _make_DepthwiseConvolution2d(self, layer):
        if layer.outputs[0].info.dtype == DataType.Float32:
            return "dwconv2d_f32", self._conv_params(layer, True)
        return "dwconv2d_q8", self._conv_params(layer, True)

    def _make_FullyConnected(self, layer):
        x, w, y = layer.inputs[0].source, layer.inputs[1].source, layer.outputs[0]
        p = _abi.FcParams()
        p.x, p.w, p.y = self._operand(x), self._operand(w), self._operand(y)
        if layer.desc["bias"]:
            p.bias = self._operand(layer.inputs[2].source)
        p.m = x.info.shape[0]
        p.k = int(np.prod(x.info.shape[1:]))                 # 4-D inputs are flattened (FullyConnected.cpp:16-24)
        p.n = y.info.shape[-1]
        p.transpose_w = int(layer.desc["transpose"])
        if y.info.dtype == DataType.Float32:
            return "fully_connected_f32", p
        p.clamp_lo, p.clamp_hi = _clamp(layer, y.info)
        if p.transpose_w:
            c = _abi.Conv2dParams()
            c.w, c.oc, c.kh, c.kw, c.c = p.w, p.n, 1, 1, p.k
            p.packed = self._pack_weights(c)
        return "fully_connected_q8", p

    def _make_BatchMatMul(self, layer):
        x, yv, o = layer.inputs[0].source, layer.inputs[1].source, layer.outputs[0]
        p = _abi.BmmParams()
        p.x, p.y, p.out = self._operand(x), self._operand(yv), self._operand(o)
        xs, ys, os_ = x.info.shape, yv.info.shape, o.info.shape
        p.m, p.n = os_[-2], os_[-1]
        p.k = xs[-2] if layer.desc["tx"] else xs[-1]
        p.batch = int(np.prod(os_[:-2])) if len(os_) > 2 else 1
        bx = int(np.prod(xs[:-2])) if len(xs) > 2 else 1
        by = int(np.prod(ys[:-2])) if len(ys) > 2 else 1
        if bx not in (1, p.batch) or by not in (1, p.batch):
            raise InvalidArgumentException("BatchMatMul: partial batch broadcast is not supported")
        p.batch_stride_x = xs[-1] * xs[-2] if bx == p.batch and p.batch > 1 else 0
        p.batch_stride_y = ys[-1] * ys[-2] if by == p.batch and p.batch > 1 else 0
        p.transpose_x, p.transpose_y = int(layer.desc["tx"]), int(layer.desc["ty"])
        return ("batch_matmul_f32" if o.info.dtype == DataType.Float32 else "batch_matmul_q8"), p

    def _make_Pooling2d(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        p = _abi.Pool2dParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.n, p.h, p.wd, p.c = x.info.shape
        p.oh, p.ow = y.info.shape[1], y.info.shape[2]
        p.pool_h, p.pool_w = layer.desc["pool"]
        p.stride_h, p.stride_w = layer.desc["stride"]
        p.pad_top, p.pad_bottom, p.pad_left, p.pad_right = layer.desc["pad"]
        p.pool_type, p.padding_method = int(layer.desc["type"]), int(layer.desc["method"])
        return "pool2d_q8", p

    def _make_TransposeConvolution2d(self, layer):
        x, w, y = layer.inputs[0].source, layer.inputs[1].source, layer.outputs[0]
        p = _abi.Conv2dParams()
        p.x, p.w, p.y = self._operand(x), self._operand(w), self._operand(y)
        if layer.desc["bias"]:
            p.bias = self._operand(layer.inputs[2].source)
        p.n, p.h, p.wd, p.c = x.info.shape
        _, p.oh, p.ow, p.oc = y.info.shape
        oc, p.kh, p.kw, c = w.info.shape
        if oc != p.oc or c != p.c:
            raise InvalidArgumentException("TransposeConvolution2d: weights %s do not match %d -> %d channels" % (w.info.shape, p.c, p.oc))
        p.stride_h, p.stride_w = layer.desc["stride"]
        p.pad_top, p.pad_left = layer.desc["pad"][0], layer.desc["pad"][2]
        p.dil_h = p.dil_w = 1
        p.clamp_lo, p.clamp_hi = _clamp(layer, y.info)
        return "transpose_conv2d_q8", p

    def _make_ElementwiseUnary(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        p = _abi.UnaryParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.count, p.operation = x.info.GetNumElements(), layer.desc["op"]
        return "unary_q", p

    def _reduce(self, layer, axes, op):
        x, y = layer.inputs[0].source, layer.outputs[0]
        p = _abi.ReduceParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.rank = len(x.info.shape)
        for i, n in enumerate(x.info.shape):
            p.shape[i] = n
        p.axis_mask = sum(1 << int(a) for a in axes)
        p.op = int(op)
        return "reduce_q", p

    def _make_Reduce(self, layer):
        return self._reduce(layer, layer.desc["axis"], layer.desc["op"])

    def _make_Mean(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        if len(x.info.shape) != 4 or tuple(layer.desc["axis"]) != (1, 2):
            return self._reduce(layer, layer.desc["axis"], 2)        # RefMeanWorkload: armnn::Reduce with Mean
        p = _abi.MeanParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.n, p.h, p.wd, p.c = x.info.shape
        return "mean_hw_q8", p

    def _make_ElementwiseBinary(self, layer):
        a, b, o = layer.inputs[0].source, layer.inputs[1].source, layer.outputs[0]
        p = _abi.EltwiseParams()
        p.a, p.b, p.out = self._operand(a), self._operand(b), self._operand(o)
        rank = len(o.info.shape)
        prelu = layer.type == "Prelu"
        if (len(a.info.shape) != rank or len(b.info.shape) != rank) and not prelu:
            raise InvalidArgumentException("ElementwiseBinary: inputs and output must have the same rank")
        if len(a.info.shape) > rank or len(b.info.shape) > rank:
            raise InvalidArgumentException("Prelu: an operand has more dimensions than the output")
        sa = (1,) * (rank - len(a.info.shape)) + tuple(a.info.shape)
        sb = (1,) * (rank - len(b.info.shape)) + tuple(b.info.shape)
        p.rank = rank
        for i in range(rank):
            p.shape_a[i], p.shape_b[i], p.shape_out[i] = sa[i], sb[i], o.info.shape[i]
        p.op = 100 if prelu else int(layer.desc["op"]) + {"Comparison": 200, "LogicalBinary": 210}.get(layer.type, 0)
        if o.info.dtype == DataType.Boolean:
            p.clamp_lo, p.clamp_hi = 0, 255
        else:
            p.clamp_lo, p.clamp_hi = _clamp(layer, o.info) if o.info.dtype != DataType.Float32 else (0, 0)
        return "eltwise_q8", p

    _make_Prelu = _make_ElementwiseBinary
    _make_Comparison = _make_ElementwiseBinary
    _make_LogicalBinary = _make_ElementwiseBinary

    def _make_Activation(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        p = _abi.ActivationParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.count = x.info.GetNumElements()
        p.function, p.a, p.b = int(layer.desc["function"]), layer.desc["a"], layer.desc["b"]
        return "activation_q8", p

    def _make_Softmax(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        shape = x.info.shape
        axis = layer.desc["axis"] % len(shape)
        p = _abi.SoftmaxParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.outer = int(np.prod(shape[:axis])) if axis > 0 else 1
        p.axis_size = shape[axis]
        p.inner = int(np.prod(shape[axis + 1:])) if axis + 1 < len(shape) else 1
        p.beta = layer.desc["beta"]
        return "softmax_q8", p

    def _rows(self, x, axis):
        shape = x.info.shape
        axis = axis % len(shape)
        outer = int(np.prod(shape[:axis])) if axis > 0 else 1
        inner = int(np.prod(shape[axis + 1:])) if axis + 1 < len(shape) else 1
        return outer, int(shape[axis]), inner

    def _make_LogSoftmax(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        p = _abi.SoftmaxParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.outer, p.axis_size, p.inner = self._rows(x, layer.desc["axis"])
        p.beta = layer.desc["beta"]
        return "log_softmax_q", p

    def _make_L2Normalization(self, layer):
        """The channel dimension of the tensor padded to 4 dimensions with leading 1s
        (RefL2NormalizationWorkload.cpp:41-71): the last one for NHWC, the second of four for NCHW."""
        x, y = layer.inputs[0].source, layer.outputs[0]
        rank = len(x.info.shape)
        p = _abi.SoftmaxParams()
        p.x, p.y = self._operand(x), self._operand(y)
        axis = (1 if layer.desc["nchw"] else 3) - (4 - rank)
        if axis < 0:
            # no channel dimension: one channel per element
            p.outer, p.axis_size, p.inner = x.info.GetNumElements(), 1, 1
        else:
            p.outer, p.axis_size, p.inner = self._rows(x, axis)
        p.beta = layer.desc["eps"]
        return "l2_normalization_q", p

    def _make_ArgMinMax(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        p = _abi.ArgMinMaxParams()
        p.x = self._operand(x)
        p.y = self._ptr(self._dev(y))
        p.outer, p.axis_size, p.inner = self._rows(x, layer.desc["axis"])
        if y.info.GetNumElements() != p.outer * p.inner:
            raise InvalidArgumentException("ArgMinMax: output shape %s does not drop the axis of %s" % (y.info.shape, x.info.shape))
        p.function, p.out_int64 = layer.desc["function"], 0
        return "arg_min_max_q", p

    def _make_Gather(self, layer):
        x, idx, y = layer.inputs[0].source, layer.inputs[1].source, layer.outputs[0]
        p = _abi.GatherParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.indices = self._ptr(self._dev(idx))
        p.outer, p.axis_size, p.inner = self._rows(x, layer.desc["axis"])
        p.n_indices = idx.info.GetNumElements()
        if y.info.GetNumElements() != p.outer * p.n_indices * p.inner:
            raise InvalidArgumentException("Gather: output shape %s does not match input %s gathered with %s indices"
                                           % (y.info.shape, x.info.shape, idx.info.shape))
        return "gather_q", p

    def _make_ScatterNd(self, layer):
        first, idx, upd = (s.source for s in layer.inputs)
        y = layer.outputs[0]
        p = _abi.ScatterNdParams()
        if layer.desc["input_enabled"]:
            p.x = self._operand(first)
        p.updates, p.y = self._operand(upd), self._operand(y)
        p.indices = self._ptr(self._dev(idx))
        p.n_indices, p.nd = idx.info.shape
        p.inner = int(np.prod(y.info.shape[p.nd:])) if p.nd < len(y.info.shape) else 1
        for i in range(p.nd):
            p.dims[i] = y.info.shape[i]
        if upd.info.GetNumElements() != p.n_indices * p.inner:
            raise InvalidArgumentException("ScatterNd: updates %s do not hold %d slices of %d elements" % (upd.info.shape, p.n_indices, p.inner))
        p.function = layer.desc["function"]
        return "scatter_nd_q", p

    def _make_ReverseV2(self, layer):
        x, axes, y = layer.inputs[0].source, layer.inputs[1].source, layer.outputs[0]
        p = _abi.ReverseParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.axes, p.n_axes = self._ptr(self._dev(axes)), axes.info.GetNumElements()
        p.rank = len(x.info.shape)
        for i, n in enumerate(x.info.shape):
            p.shape[i] = n
        return "reverse_q", p

    def _make_GatherNd(self, layer):
        x, idx, y = layer.inputs[0].source, layer.inputs[1].source, layer.outputs[0]
        p = _abi.GatherNdParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.indices = self._ptr(self._dev(idx))
        p.nd = idx.info.shape[-1]
        p.n_indices = idx.info.GetNumElements() // p.nd
        p.inner = int(np.prod(x.info.shape[p.nd:])) if p.nd < len(x.info.shape) else 1
        for i in range(p.nd):
            p.dims[i] = x.info.shape[i]
        if y.info.GetNumElements() != p.n_indices * p.inner:
            raise InvalidArgumentException("GatherNd: output shape %s does not match %d tuples of %d elements" % (y.info.shape, p.n_indices, p.inner))
        return "gather_nd_q", p

    @staticmethod
    def _planes(info, nchw):
        n, a, b, c = info.shape
        return (n, a, b * c) if nchw else (n, c, a * b)          # (batch, channels, pixels per plane)

    def _make_BatchNormalization(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        p = _abi.BatchNormParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.n, p.c, p.hw = self._planes(x.info, layer.desc["nchw"])
        p.nchw, p.eps = int(layer.desc["nchw"]), layer.desc["eps"]
        for key in ("mean", "variance", "beta", "gamma"):
            data, info = layer.bn_params[key]
            if info.GetNumElements() != p.c:
                raise InvalidArgumentException("BatchNormalization: %s must hold one value per channel" % key)
            dev = self._upload(np.ascontiguousarray(np.asarray(data).astype(_NP_DTYPE[info.dtype])))
            self.aux.append(dev)
            setattr(p, key, _qt(info, self._ptr(dev), None))
        scratch = self._upload(np.zeros(2 * p.c, np.float32))
        self.aux.append(scratch)
        p.scratch = self._ptr(scratch)
        return "batch_norm_q", p

    def _make_Normalization(self, layer):
        """The reference encodes the output with the input's quantisation (RefNormalizationWorkload.cpp:176-177) and its
        Within variant indexes the tensor as NCHW whatever the layout says (lines 25-28): both kept."""
        x, y, d = layer.inputs[0].source, layer.outputs[0], layer.desc
        p = _abi.NormalizationParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.y.scale, p.y.zero_point = p.x.scale, p.x.zero_point
        shape = x.info.shape
        if d["channel_type"] == 1 or d["nchw"]:
            p.n, p.c, p.h, p.w, p.nchw = shape[0], shape[1], shape[2], shape[3], 1
        else:
            p.n, p.h, p.w, p.c, p.nchw = shape[0], shape[1], shape[2], shape[3], 0
        p.channel_type, p.norm_size = d["channel_type"], d["norm_size"]
        p.alpha, p.beta, p.kappa = d["alpha"], d["beta"], d["k"]
        return "normalization_q", p

    def _make_InstanceNormalization(self, layer):
        x, y, d = layer.inputs[0].source, layer.outputs[0], layer.desc
        p = _abi.InstanceNormParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.n, p.c, p.hw = self._planes(x.info, d["nchw"])
        p.nchw, p.gamma, p.beta, p.eps = int(d["nchw"]), d["gamma"], d["beta"], d["eps"]
        return "instance_norm_q", p

    def _make_convert(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        p = _abi.ConvertParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.count = x.info.GetNumElements()
        return "convert_q", p

    _make_Quantize = _make_convert
    _make_Dequantize = _make_convert

    def _make_Pad(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        p = _abi.PadParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.rank = len(x.info.shape)
        for i, (before, after) in enumerate(layer.desc["pads"]):
            p.shape[i], p.pad_before[i], p.pad_after[i] = x.info.shape[i], before, after
        p.pad_value = layer.desc["value"]
        p.mode = layer.desc.get("mode", 0)
        return "pad_q", p

    def _make_Shape(self, layer):
        """The shape is known when the network is loaded (RefShapeWorkload.hpp, RefRankWorkload.hpp write it at every
        execution): a device constant copied into the output tensor."""
        x, y = layer.inputs[0].source, layer.outputs[0]
        values = np.array(x.info.shape if layer.type == "Shape" else [len(x.info.shape)], np.int32)
        dev = self._upload(values)
        self.aux.append(dev)
        name, p = self._view_copy(y, y, ((len(values),), 0, [1], 0, [1]))
        p.x.data = self._ptr(dev)
        return name, p

    _make_Rank = _make_Shape

    def _make_FakeQuantization(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        p = _abi.ActivationParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.count, p.function, p.a, p.b = x.info.GetNumElements(), 50, layer.desc["min"], layer.desc["max"]
        return "activation_q8", p

    def _make_ConvertFp16ToFp32(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        p = _abi.ConvertFp16Params()
        p.x, p.y = self._ptr(self._dev(x)), self._ptr(self._dev(y))
        p.count, p.to_half = x.info.GetNumElements(), int(layer.type == "ConvertFp32ToFp16")
        return "convert_fp16", p

    _make_ConvertFp32ToFp16 = _make_ConvertFp16ToFp32

    def _make_Cast(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        p = _abi.ConvertParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.count = x.info.GetNumElements()
        return "cast_q", p

    def _make_Fill(self, layer):
        """One element holding the value in the output's type, read with stride 0 over the whole output
        (workloads/Fill.cpp:13-23; Signed32: the value truncated)."""
        y = layer.outputs[0]
        value = np.array([layer.desc["value"]], np.float32).astype(_NP_DTYPE[y.info.dtype])
        dev = self._upload(value)
        self.aux.append(dev)
        name, p = self._view_copy(y, y, views.fill_view(y.info.shape))
        p.x.data = self._ptr(dev)
        return name, p

    def _make_Floor(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        p = _abi.UnaryParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.count, p.operation = x.info.GetNumElements(), 9
        return "unary_q", p

    def _make_Resize(self, layer):
        x, y, d = layer.inputs[0].source, layer.outputs[0], layer.desc
        p = _abi.ResizeParams()
        p.x, p.y = self._operand(x), self._operand(y)
        if d["nchw"]:
            p.n, p.c, p.in_h, p.in_w = x.info.shape
            oh, ow = y.info.shape[2], y.info.shape[3]
        else:
            p.n, p.in_h, p.in_w, p.c = x.info.shape
            oh, ow = y.info.shape[1], y.info.shape[2]
        if (oh, ow) != (d["height"], d["width"]):
            raise InvalidArgumentException("Resize: output shape %s does not match the target size %dx%d" % (y.info.shape, d["height"], d["width"]))
        p.out_h, p.out_w = oh, ow
        p.method, p.align_corners, p.half_pixel_centers, p.nchw = d["method"], int(d["align_corners"]), int(d["half_pixel_centers"]), int(d["nchw"])
        return "resize_q", p

    # -- Concat, Splitter, Permute, Transpose, StridedSlice, Slice: rectangular view copies (armnn_b200/views.py) --
    def _view_copy(self, x, y, view):
        shape, so, ss, do, ds = views.merge_dims(view)
        p = _abi.ViewCopyParams()
        p.x, p.y = self._operand(x), self._operand(y)
        p.rank = len(shape)
        for i in range(len(shape)):
            p.shape[i], p.src_strides[i], p.dst_strides[i] = shape[i], ss[i], ds[i]
        p.src_offset, p.dst_offset = so, do
        return "view_copy_q", p

    def _make_Concat(self, layer):
        y = layer.outputs[0]
        srcs = [s.source for s in layer.inputs]
        vs = views.concat_views(y.info.shape, [x.info.shape for x in srcs], layer.desc["origins"])
        return [self._view_copy(x, y, v) for x, v in zip(reversed(srcs), vs)]

    def _make_Splitter(self, layer):
        x = layer.inputs[0].source
        vs = views.splitter_views(x.info.shape, [o.info.shape for o in layer.outputs], layer.desc["origins"])
        return [self._view_copy(x, o, v) for o, v in zip(layer.outputs, vs)]

    def _make_permute(self, layer, transpose):
        x, y = layer.inputs[0].source, layer.outputs[0]
        out_shape, v = views.permute_view(x.info.shape, layer.desc["mappings"], transpose)
        if tuple(out_shape) != tuple(y.info.shape):
            raise InvalidArgumentException("%s: output shape %s is not the permuted input shape %s" % (layer.type, y.info.shape, out_shape))
        return self._view_copy(x, y, v)

    def _make_Permute(self, layer):
        return self._make_permute(layer, False)

    def _make_Transpose(self, layer):
        return self._make_permute(layer, True)

    def _make_StridedSlice(self, layer):
        x, y, d = layer.inputs[0].source, layer.outputs[0], layer.desc
        walk, out_shape, v = views.strided_slice_view(x.info.shape, d["begin"], d["end"], d["stride"], d["begin_mask"], d["end_mask"],
                                                      d["shrink_axis_mask"])
        if y.info.GetNumElements() != int(np.prod(walk)):
            raise InvalidArgumentException("StridedSlice: output shape %s does not hold the slice %s" % (y.info.shape, walk))
        return self._view_copy(x, y, v)

    def _make_DepthToSpace(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        out_shape, v = views.depth_to_space_view(x.info.shape, layer.desc["block"], layer.desc["nchw"])
        if tuple(out_shape) != tuple(y.info.shape):
            raise InvalidArgumentException("DepthToSpace: output shape %s, expected %s" % (y.info.shape, out_shape))
        return self._view_copy(x, y, v)

    def _make_Tile(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        out_shape, v = views.tile_view(x.info.shape, layer.desc["multiples"])
        if tuple(out_shape) != tuple(y.info.shape):
            raise InvalidArgumentException("Tile: output shape %s, expected %s" % (y.info.shape, out_shape))
        return self._view_copy(x, y, v)

    def _make_BroadcastTo(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        if tuple(layer.desc["shape"]) != tuple(y.info.shape):
            raise InvalidArgumentException("BroadcastTo: output shape %s is not the descriptor's %s" % (y.info.shape, layer.desc["shape"]))
        return self._view_copy(x, y, views.broadcast_to_view(x.info.shape, y.info.shape))

    def _make_BatchToSpaceNd(self, layer):
        x, y, d = layer.inputs[0].source, layer.outputs[0], layer.desc
        out_shape, vs = views.batch_to_space_views(x.info.shape, d["block"], d["edges"], d["nchw"])
        if tuple(out_shape) != tuple(y.info.shape):
            raise InvalidArgumentException("BatchToSpaceNd: output shape %s, expected %s" % (y.info.shape, out_shape))
        return [self._view_copy(x, y, v) for v in vs]

    def _make_SpaceToBatchNd(self, layer):
        x, y, d = layer.inputs[0].source, layer.outputs[0], layer.desc
        out_shape, vs, padded = views.space_to_batch_views(x.info.shape, d["block"], d["edges"], d["nchw"])
        if tuple(out_shape) != tuple(y.info.shape):
            raise InvalidArgumentException("SpaceToBatchNd: output shape %s, expected %s" % (y.info.shape, out_shape))
        work = []
        if padded:
            # the padding holds the output's encoding of 0.0 (workloads/SpaceToBatchNd.cpp:98-101): one element of it,
            # read with stride 0 over the whole output, before the blocks of the input are copied in
            info = y.info
            if info.dtype == DataType.Float32:
                zero = np.zeros(1, np.float32)
            else:
                lo, hi = _TYPE_RANGE[info.dtype]
                zero = np.array([min(max(info.offset, lo), hi)], _NP_DTYPE[info.dtype])
            dev = self._upload(zero)
            self.aux.append(dev)
            name, p = self._view_copy(y, y, views.fill_view(out_shape))
            p.x.data = self._ptr(dev)
            work.append((name, p))
        return work + [self._view_copy(x, y, v) for v in vs]

    def _make_SpaceToDepth(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        out_shape, v = views.space_to_depth_view(x.info.shape, layer.desc["block"], layer.desc["nchw"])
        if tuple(out_shape) != tuple(y.info.shape):
            raise InvalidArgumentException("SpaceToDepth: output shape %s, expected %s" % (y.info.shape, out_shape))
        return self._view_copy(x, y, v)

    def _make_ChannelShuffle(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        if tuple(x.info.shape) != tuple(y.info.shape):
            raise InvalidArgumentException("ChannelShuffle: input and output shapes differ")
        return self._view_copy(x, y, views.channel_shuffle_view(x.info.shape, layer.desc["axis"], layer.desc["groups"]))

    def _make_Stack(self, layer):
        y = layer.outputs[0]
        srcs = [s.source for s in layer.inputs]
        out_shape, vs = views.stack_views(srcs[0].info.shape, len(srcs), layer.desc["axis"])
        if tuple(out_shape) != tuple(y.info.shape) or any(tuple(x.info.shape) != tuple(srcs[0].info.shape) for x in srcs):
            raise InvalidArgumentException("Stack: inputs must share one shape and the output must be %s" % (out_shape,))
        return [self._view_copy(x, y, v) for x, v in zip(srcs, vs)]

    def _make_Slice(self, layer):
        x, y = layer.inputs[0].source, layer.outputs[0]
        out_shape, v = views.slice_view(x.info.shape, layer.desc["begin"], layer.desc["size"])
        if tuple(out_shape) != tuple(y.info.shape):
            raise InvalidArgumentException("Slice: output shape %s is not the block %s" % (y.info.shape, out_shape))
        return self._view_copy(x, y, v)

    _LSTM_FIELDS = {"InputToInputWeights": "w_i2i", "InputToForgetWeights": "w_i2f", "InputToCellWeights": "w_i2c",
                    "InputToOutputWeights": "w_i2o", "RecurrentToInputWeights": "w_r2i", "RecurrentToForgetWeights": "w_r2f",
                    "RecurrentToCellWeights": "w_r2c", "RecurrentToOutputWeights": "w_r2o", "CellToInputWeights": "w_c2i",
                    "CellToForgetWeights": "w_c2f", "CellToOutputWeights": "w_c2o", "InputGateBias": "b_i", "ForgetGateBias": "b_f",
                    "CellBias": "b_c", "OutputGateBias": "b_o", "InputLayerNormWeights": "ln_i", "ForgetLayerNormWeights": "ln_f",
                    "CellLayerNormWeights": "ln_c", "OutputLayerNormWeights": "ln_o", "ProjectionWeights": "w_proj",
                    "ProjectionBias": "b_proj"}

    def _lstm_weights(self, layer, p):
        """Device copies of the weights (the descriptor's handles die after workload creation) and the option switches."""
        d = layer.desc
        for key, field in self._LSTM_FIELDS.items():
            item = layer.qlstm_params.get(key)
            if item is None:
                continue
            dev = self._upload(np.ascontiguousarray(np.asarray(item[0], np.float32)))
            self.aux.append(dev)
            setattr(p, field, self._ptr(dev))
        if d.get("CifgEnabled"):
            p.w_i2i = p.w_r2i = p.w_c2i = p.b_i = p.ln_i = None
        if not d.get("PeepholeEnabled"):
            p.w_c2i = p.w_c2f = p.w_c2o = None
        if not d.get("LayerNormEnabled"):
            p.ln_i = p.ln_f = p.ln_c = p.ln_o = None
        if not d.get("ProjectionEnabled"):
            p.w_proj = p.b_proj = None
        p.activation = int(d.get("ActivationFunc", 4))
        p.cell_clip, p.projection_clip = float(d.get("ClippingThresCell", 0.0)), float(d.get("ClippingThresProj", 0.0))
        p.layer_norm_eps = 1e-8                                     # RefLstmWorkload.hpp: m_LayerNormEpsilon

    def _make_Lstm(self, layer):
        x, h, c = (s.source for s in layer.inputs)
        _, hout, cout, out = layer.outputs
        p = _abi.LstmParams()
        p.batch, p.input_size = x.info.shape
        p.output_size, p.num_units = h.info.shape[1], c.info.shape[1]
        p.input, p.input_stride = self._ptr(self._dev(x)), p.input_size
        p.output_state_in, p.cell_state_in = self._ptr(self._dev(h)), self._ptr(self._dev(c))
        p.output_state_out, p.cell_state_out = self._ptr(self._dev(hout)), self._ptr(self._dev(cout))
        p.output, p.output_stride = self._ptr(self._dev(out)), p.output_size
        self._lstm_weights(layer, p)
        return "lstm_step_f32", p

    def _make_UnidirectionalSequenceLstm(self, layer):
        """One step per time index (RefUnidirectionalSequenceLstmWorkload.cpp:160-293): the first reads the state inputs,
        the others update the state outputs in place; a step's rows are `input_stride` apart in the sequence tensor, so
        neither layout needs a transposed copy."""
        x, h, c = (s.source for s in layer.inputs)
        hout, cout, out = layer.outputs
        time_major = bool(layer.desc.get("TimeMajor", False))
        steps, batch = (x.info.shape[0], x.info.shape[1]) if time_major else (x.info.shape[1], x.info.shape[0])
        n_in, n_out, units = x.info.shape[2], h.info.shape[1], c.info.shape[1]
        work = []
        for t in range(steps):
            p = _abi.LstmParams()
            p.batch, p.input_size, p.num_units, p.output_size = batch, n_in, units, n_out
            p.input = self._ptr(self._dev(x)) + 4 * (t * batch * n_in if time_major else t * n_in)
            p.input_stride = n_in if time_major else steps * n_in
            p.output = self._ptr(self._dev(out)) + 4 * (t * batch * n_out if time_major else t * n_out)
            p.output_stride = n_out if time_major else steps * n_out
            p.output_state_in = self._ptr(self._dev(h if t == 0 else hout))
            p.cell_state_in = self._ptr(self._dev(c if t == 0 else cout))
            p.output_state_out, p.cell_state_out = self._ptr(self._dev(hout)), self._ptr(self._dev(cout))
            if t == 0:
                self._lstm_weights(layer, p)
                first = p
            else:
                for field in list(self._LSTM_FIELDS.values()) + ["activation", "cell_clip", "projection_clip", "layer_norm_eps"]:
                    setattr(p, field, getattr(first, field))
            work.append(("lstm_step_f32", p))
        return work

    def _make_QLstm(self, layer):
        x, h, c = (s.source for s in layer.inputs)
        hout, cout, out = layer.outputs
        d = layer.desc
        p = _abi.QLstmParams()
        p.batch, p.input_size = x.info.shape
        p.output_size, p.num_units = h.info.shape[1], c.info.shape[1]
        p.input, p.input_scale, p.input_zp = self._ptr(self._dev(x)), x.info.scale, x.info.offset
        p.output_state_in, p.output_state_scale, p.output_state_zp = self._ptr(self._dev(h)), h.info.scale, h.info.offset
        p.cell_state_in, p.cell_state_scale = self._ptr(self._dev(c)), c.info.scale
        if not (hout.info.same_quantization(h.info) and cout.info.same_quantization(c.info)):
            raise InvalidArgumentException("QLstm: state outputs must share the state inputs' quantisation")
        p.output_state_out, p.cell_state_out = self._ptr(self._dev(hout)), self._ptr(self._dev(cout))
        p.output, p.output_scale, p.output_zp = self._ptr(self._dev(out)), out.info.scale, out.info.offset
        names = {"InputToInputWeights": ("w_i2i", "s_i2i"), "InputToForgetWeights": ("w_i2f", "s_i2f"),
                 "InputToCellWeights": ("w_i2c", "s_i2c"), "InputToOutputWeights": ("w_i2o", "s_i2o"),
                 "RecurrentToInputWeights": ("w_r2i", "s_r2i"), "RecurrentToForgetWeights": ("w_r2f", "s_r2f"),
                 "RecurrentToCellWeights": ("w_r2c", "s_r2c"), "RecurrentToOutputWeights": ("w_r2o", "s_r2o"),
                 "CellToInputWeights": ("w_c2i", "s_c2i"), "CellToForgetWeights": ("w_c2f", "s_c2f"),
                 "CellToOutputWeights": ("w_c2o", "s_c2o"),
                 "InputGateBias": ("b_i", None), "ForgetGateBias": ("b_f", None), "CellBias": ("b_c", None),
                 "OutputGateBias": ("b_o", None),
                 "InputLayerNormWeights": ("ln_i", "s_lni"), "ForgetLayerNormWeights": ("ln_f", "s_lnf"),
                 "CellLayerNormWeights": ("ln_c", "s_lnc"), "OutputLayerNormWeights": ("ln_o", "s_lno"),
                 "ProjectionWeights": ("w_proj", "s_proj"), "ProjectionBias": ("b_proj", "s_bproj")}
        # The descriptor's ConstTensorHandles are only valid during workload creation
        # (src/armnn/LoadedNetwork.cpp:396), so the workload owns device copies.
        for key, (wf, sf) in names.items():
            if key not in layer.qlstm_params or layer.qlstm_params[key] is None:
                continue
            data, info = layer.qlstm_params[key]
            dev = self._upload(np.ascontiguousarray(np.asarray(data).astype(_NP_DTYPE[info.dtype])))
            self.aux.append(dev)
            setattr(p, wf, self._ptr(dev))
            if sf:
                setattr(p, sf, info.scale)
        if d.get("LayerNormEnabled"):
            # bias scale = layer-norm weight scale / 1024 (RefQLstmWorkload.cpp:261-287)
            for g, key in (("i", "InputLayerNormWeights"), ("f", "ForgetLayerNormWeights"),
                           ("c", "CellLayerNormWeights"), ("o", "OutputLayerNormWeights")):
                if layer.qlstm_params.get(key) is not None:
                    setattr(p, "s_b" + g, float(np.float32(layer.qlstm_params[key][1].scale) / np.float32(1024)))
        else:
            p.ln_i = p.ln_f = p.ln_c = p.ln_o = None
        if d.get("CifgEnabled"):
            p.w_i2i = p.w_r2i = None
        if not d.get("PeepholeEnabled"):
            p.w_c2i = p.w_c2f = p.w_c2o = None
        if not d.get("ProjectionEnabled"):
            p.w_proj = p.b_proj = None
        p.cell_clip, p.projection_clip = d.get("CellClip", 0.0), d.get("ProjectionClip", 0.0)
        p.input_intermediate_scale = d["InputIntermediateScale"]
        p.forget_intermediate_scale = d["ForgetIntermediateScale"]
        p.cell_intermediate_scale = d["CellIntermediateScale"]
        p.output_intermediate_scale = d["OutputIntermediateScale"]
        p.hidden_state_scale, p.hidden_state_zp = d["HiddenStateScale"], d["HiddenStateZeroPoint"]
        return "qlstm_step", p



class LoadedNetwork(GraphProgram):
    """Device tensors + one workload (a prepared C-ABI call) per layer, enqueued in order on one stream."""

    def __init__(self, runtime, optimized):
        super().__init__(optimized)
        torch = runtime.torch
        self.rt, self.torch = runtime, torch
        self.stream = torch.cuda.Stream(device=runtime.device)
        self.graph = None
        with torch.cuda.device(runtime.device):
            self._build()
            # constant uploads and weight packing ran on the current stream; the workloads run on self.stream
            torch.cuda.synchronize(runtime.device)

    def _alloc(self, info):
        tdt = getattr(self.torch, np.dtype(_NP_DTYPE[info.dtype]).name)
        return self.torch.empty(info.shape if info.shape else (1,), dtype=tdt, device=self.rt.device)

    def _upload(self, array):
        return self.torch.from_numpy(np.ascontiguousarray(array)).to(self.rt.device)

    def _ptr(self, tensor):
        return tensor.data_ptr()

    def _view(self, tensor, shape):
        return tensor.view(shape)

    def _pack_weights(self, conv_params):
        l = lib.load_library()
        nbytes = l.b200k_conv2d_pack_bytes(conv_params.oc, conv_params.kh, conv_params.kw, conv_params.c)
        table = self.torch.empty(nbytes // 4, dtype=self.torch.int32, device=self.rt.device)
        self.aux.append(table)
        lib.check(l.b200k_conv2d_pack(ctypes.byref(conv_params), ctypes.c_void_p(table.data_ptr()),
                                      ctypes.c_void_p(self.torch.cuda.current_stream().cuda_stream)))
        return table.data_ptr()

    def _attach_scratch(self, conv_params):
        nbytes = lib.load_library().b200k_conv2d_scratch_bytes(ctypes.byref(conv_params))
        if nbytes:
            buf = self.torch.empty(nbytes, dtype=self.torch.uint8, device=self.rt.device)
            self.aux.append(buf)
            conv_params.scratch, conv_params.scratch_bytes = buf.data_ptr(), nbytes

    # -- execution ---------------------------------------------------------------------------------
    def launch_all(self, stream_handle):
        """Enqueue every workload on the given CUDA stream; returns the number of kernels launched."""
        l = lib.load_library()
        before = l.b200k_kernel_launches()
        for layer, entry, params in self.workloads:
            rc = getattr(l, "b200k_" + entry)(ctypes.byref(params), ctypes.c_void_p(stream_handle))
            if rc != 0:
                raise RuntimeError("workload %s (%s) failed: %s" % (layer.name, entry, l.b200k_last_error().decode()))
        return int(l.b200k_kernel_launches() - before)

    def Execute(self):
        """The workload queue only (inputs and outputs stay in device memory)."""
        if self.graph is not None:
            with self.torch.cuda.stream(self.stream):
                self.graph.replay()
            return self.graph_kernels
        return self.launch_all(self.stream.cuda_stream)

    def CaptureGraph(self):
        """Capture the workload queue into a CUDA graph: removes the per-workload host launches."""
        torch = self.torch
        self.Execute()
        self.stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=self.stream):
            self.graph_kernels = self.launch_all(torch.cuda.current_stream().cuda_stream)    # kernel nodes of the graph
        self.graph = g

    def EnqueueWorkload(self, input_tensors, output_tensors):
        """input_tensors / output_tensors: {binding id: host torch tensor or numpy array}.  Host -> device
        copies, the workload queue and device -> host copies all go to this network's stream; returns after
        the outputs are in host memory (the Map(blocking) of the reference's output copy)."""
        torch = self.torch
        with torch.cuda.stream(self.stream):
            for bid, host in input_tensors.items():
                dst = self._dev(self.inputs[bid])
                src = host if torch.is_tensor(host) else torch.from_numpy(host)
                dst.view(-1).copy_(src.view(-1).view(dst.dtype), non_blocking=True)
            self.Execute()
            for bid, host in output_tensors.items():
                src = self._dev(self.outputs[bid])
                dst = host if torch.is_tensor(host) else torch.from_numpy(host)
                dst.view(-1).view(src.dtype).copy_(src.view(-1), non_blocking=True)
        self.stream.synchronize()
        return 0

    # -- pipelined execution: the next request's input copy overlaps this request's compute ---------------
    def _input_consumers_end(self):
        """Workloads [0, k) include every workload that reads a network input directly."""
        input_ids = {id(slot) for slot in self.inputs.values()}
        k = 0
        for i, (layer, entry, params) in enumerate(self.workloads):
            if any(id(s.source) in input_ids for s in layer.inputs):
                k = i + 1
        return k

    def CapturePipelined(self):
        """Prepare EnqueueAsync / WaitOutputs: the workload queue as two CUDA graphs (the workloads that read the
        network inputs, then the rest), a copy stream, and two sets of pinned output staging buffers."""
        torch = self.torch
        l = lib.load_library()
        self.launch_all(self.stream.cuda_stream)
        self.stream.synchronize()
        k = self._input_consumers_end()

        def capture(lo, hi):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.stream):
                h = torch.cuda.current_stream().cuda_stream
                for layer, entry, params in self.workloads[lo:hi]:
                    rc = getattr(l, "b200k_" + entry)(ctypes.byref(params), ctypes.c_void_p(h))
                    if rc != 0:
                        raise RuntimeError("workload %s (%s) failed: %s" % (layer.name, entry, l.b200k_last_error().decode()))
            return g
        self._head, self._tail = capture(0, k), (capture(k, len(self.workloads)) if k < len(self.workloads) else None)
        self._copy_stream = torch.cuda.Stream(device=self.rt.device)
        self._input_free = None
        self._staging = [{bid: torch.empty(tuple(self._dev(slot).shape), dtype=self._dev(slot).dtype).pin_memory()
                          for bid, slot in self.outputs.items()} for _ in range(2)]
        self._tickets = 0

    def EnqueueAsync(self, input_tensors):
        """Host -> device copy of the inputs on the copy stream (as soon as the previous request's input has been
        consumed), then the workload queue and the device -> host copy of every output into pinned staging on the
        network's stream.  Returns a ticket for WaitOutputs; at most two requests may be in flight.  Host inputs
        should be pinned, otherwise the copy is synchronous."""
        torch = self.torch
        cs = self._copy_stream
        with torch.cuda.stream(cs):
            if self._input_free is not None:
                cs.wait_event(self._input_free)
            for bid, host in input_tensors.items():
                dst = self._dev(self.inputs[bid])
                src = host if torch.is_tensor(host) else torch.from_numpy(host)
                dst.view(-1).copy_(src.view(-1).view(dst.dtype), non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(cs)
        slot = self._tickets % 2
        self._tickets += 1
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ready)
            self._head.replay()
            self._input_free = torch.cuda.Event()
            self._input_free.record(self.stream)
            if self._tail is not None:
                self._tail.replay()
            for bid, out in self.outputs.items():
                self._staging[slot][bid].copy_(self._dev(out), non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.stream)
        return slot, done

    def WaitOutputs(self, ticket, output_tensors):
        """Blocks until the request of `ticket` has finished and copies its outputs to the given host tensors."""
        torch = self.torch
        slot, done = ticket
        done.synchronize()
        for bid, host in output_tensors.items():
            dst = host if torch.is_tensor(host) else torch.from_numpy(host)
            src = self._staging[slot][bid]
            dst.view(-1).view(src.dtype).copy_(src.view(-1))
        return 0

    def input_tensor(self, binding_id):
        return self._dev(self.inputs[binding_id])

    def output_tensor(self, binding_id):
        return self._dev(self.outputs[binding_id])

    def tensor_of(self, slot):
        return self._dev(slot)
