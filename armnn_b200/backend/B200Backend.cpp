// The B200Acc backend object: IBackendInternal, layer support, graph-level optimisation (Pad folding, activation and
// residual-Add fusion), the per-network model context (DeviceId) and, in B200DynamicBackend.cpp, the three extern "C"
// entry points of a dynamic backend (include/armnn/backends/DynamicBackend.hpp:41-43 of the Arm NN tree).  Structure follows RefBackend (src/backends/reference/RefBackend.cpp:22-208) and the sample dynamic backend
// (src/dynamic/sample/SampleDynamicBackend.cpp); the fusion pass restates what the Neon / CL backends do
// (src/backends/cl/ClBackend.cpp:326-390, src/backends/aclCommon/ArmComputeSubgraphUtils.hpp:52-70), whose helper
// header cannot be included because it pulls in the un-vendored Arm Compute Library.
#include "B200Workloads.hpp"

#include <armnn/BackendOptions.hpp>
#include <armnn/backends/IBackendContext.hpp>
#include <armnn/backends/IBackendInternal.hpp>
#include <armnn/backends/OptimizationViews.hpp>
#include <armnn/backends/SubgraphView.hpp>
#include <armnn/utility/PolymorphicDowncast.hpp>
#include <backendsCommon/LayerSupportBase.hpp>
#include <backendsCommon/SubgraphUtils.hpp>
#include <backendsCommon/TensorHandleFactoryRegistry.hpp>

#include <Layer.hpp>
#include <layers/ActivationLayer.hpp>
#include <layers/Convolution2dLayer.hpp>
#include <layers/DepthwiseConvolution2dLayer.hpp>
#include <layers/ElementwiseBinaryLayer.hpp>
#include <layers/FullyConnectedLayer.hpp>
#include <layers/PadLayer.hpp>
#include <layers/Pooling2dLayer.hpp>

#include "B200Backend.hpp"

#include "b200k.h"

namespace armnn
{

namespace
{

bool Is8Bit(const TensorInfo& t)
{
    return t.GetDataType() == DataType::QAsymmU8 || t.GetDataType() == DataType::QAsymmS8 || t.GetDataType() == DataType::QSymmS8;
}

bool IsActType(const TensorInfo& t)
{
    return t.GetDataType() == DataType::QAsymmU8 || t.GetDataType() == DataType::QAsymmS8 ||
           t.GetDataType() == DataType::QSymmS16 || t.GetDataType() == DataType::Float32;
}

// element types the view copies move (Concat ... Slice): the activation types and Signed32
bool IsMoveType(const TensorInfo& t)
{
    return IsActType(t) || t.GetDataType() == DataType::Signed32;
}

// every tensor of the layer is Float32 (an absent bias is an empty TensorInfo)
bool AllFloat32(const std::vector<TensorInfo>& infos)
{
    for (const TensorInfo& t : infos)
    {
        if (t != TensorInfo() && t.GetDataType() != DataType::Float32) { return false; }
    }
    return !infos.empty();
}

bool No(Optional<std::string&> reason, const char* why)
{
    if (reason.has_value()) { reason.value() += std::string("B200Acc: ") + why + " "; }
    return false;
}

}  // namespace

/// Which (layer, data type) combinations the optimizer may assign to B200Acc: the 8-bit quantised NHWC hot path.
/// Same rules as RefLayerSupport for those layers (src/backends/reference/RefLayerSupport.cpp:560-2595) restricted to
/// the quantised types, plus one relaxation: FullyConnected accepts QAsymmS8 input with per-axis QSymmS8 weights,
/// which RefLayerSupport.cpp:1569 refuses although the arithmetic supports it.
class B200LayerSupport : public LayerSupportBase
{
public:
    bool IsLayerSupported(const LayerType& type, const std::vector<TensorInfo>& infos, const BaseDescriptor& descriptor,
                          const Optional<LstmInputParamsInfo>& lstmParamsInfo, const Optional<QuantizedLstmInputParamsInfo>&,
                          Optional<std::string&> reason) const override
    {
        switch (type)
        {
            case LayerType::Input:
            case LayerType::Output:
            case LayerType::Constant:
            case LayerType::MemCopy:
            case LayerType::MemImport:
            case LayerType::Reshape:
                return true;
            case LayerType::Convolution2d:
            case LayerType::DepthwiseConvolution2d:
            {
                // infos = {input, output, weights, biases-or-empty} (src/armnn/BackendHelper.cpp:378-379)
                const DataLayout layout = type == LayerType::Convolution2d
                    ? PolymorphicDowncast<const Convolution2dDescriptor*>(&descriptor)->m_DataLayout
                    : PolymorphicDowncast<const DepthwiseConvolution2dDescriptor*>(&descriptor)->m_DataLayout;
                // NCHW layers run through a re-layout around the NHWC kernels (B200Workloads.cpp: MakeConv); their per-axis
                // weights are quantised along dimension 0 ([O, I, H, W]) like the NHWC ones ([O, H, W, I])
                if (layout != DataLayout::NHWC && layout != DataLayout::NCHW) { return No(reason, "NHWC or NCHW only"); }
                if (!infos[2].IsConstant()) { return No(reason, "non-constant weights are not supported"); }
                if (AllFloat32(infos)) { return true; }                 // the fp32 variant (b200k_conv2d_f32 / b200k_dwconv2d_f32)
                if (!Is8Bit(infos[0]) || !Is8Bit(infos[1]) || !Is8Bit(infos[2])) { return No(reason, "input, output and weights must be 8-bit quantised or all Float32"); }
                if (infos[3] != TensorInfo() && infos[3].GetDataType() != DataType::Signed32) { return No(reason, "bias must be Signed32"); }
                if (infos[2].HasPerAxisQuantization())
                {
                    const unsigned want = type == LayerType::Convolution2d ? 0u : 3u;
                    if (infos[2].GetQuantizationDim().value() != want) { return No(reason, "per-axis quantisation must follow the output channels"); }
                }
                return true;
            }
            case LayerType::FullyConnected:
            {
                if (!infos[2].IsConstant()) { return No(reason, "non-constant weights are not supported"); }
                if (AllFloat32(infos)) { return true; }                 // the fp32 variant (b200k_fully_connected_f32)
                if (!Is8Bit(infos[0]) || !Is8Bit(infos[1]) || !Is8Bit(infos[2])) { return No(reason, "input, output and weights must be 8-bit quantised or all Float32"); }
                const auto& d = *PolymorphicDowncast<const FullyConnectedDescriptor*>(&descriptor);
                if (d.m_BiasEnabled && infos[3].GetDataType() != DataType::Signed32) { return No(reason, "bias must be Signed32"); }
                return true;
            }
            case LayerType::BatchMatMul:
            {
                const auto& d = *PolymorphicDowncast<const BatchMatMulDescriptor*>(&descriptor);
                if (d.m_AdjointX || d.m_AdjointY) { return No(reason, "adjoint inputs are not supported"); }
                if (d.m_DataLayoutX != DataLayout::NCHW || d.m_DataLayoutY != DataLayout::NCHW) { return No(reason, "only the default axis choice is supported"); }
                if (AllFloat32(infos)) { return true; }
                if (!Is8Bit(infos[0]) || !Is8Bit(infos[1]) || !Is8Bit(infos[2])) { return No(reason, "8-bit quantised tensors, or Float32 throughout"); }
                return true;
            }
            case LayerType::Pooling2d:
                return (IsActType(infos[0]) && IsActType(infos[1])) || No(reason, "unsupported data type");
            case LayerType::Pad:
            {
                // Pad layers in front of a convolution or pooling layer are folded into it by OptimizeSubgraphView (the
                // TfLite parser emits them for explicit padding, src/armnnTfLiteParser/TfLiteParser.cpp:829-830); the
                // others run as a workload of their own
                const auto& d = *PolymorphicDowncast<const PadDescriptor*>(&descriptor);
                if (d.m_PaddingMode != PaddingMode::Constant)
                {
                    // MirrorPad.cpp:66-74: a mirrored border is at most as wide as the tensor (less the edge for Reflect)
                    const unsigned int edge = d.m_PaddingMode == PaddingMode::Reflect ? 1u : 0u;
                    for (unsigned int i = 0; i < d.m_PadList.size() && i < infos[0].GetNumDimensions(); ++i)
                    {
                        if (d.m_PadList[i].first + edge > infos[0].GetShape()[i] || d.m_PadList[i].second + edge > infos[0].GetShape()[i])
                        {
                            return No(reason, "mirrored padding wider than the tensor");
                        }
                    }
                }
                if (infos[0].GetNumDimensions() > 4) { return No(reason, "rank > 4"); }
                return (IsActType(infos[0]) && IsActType(infos[1])) || No(reason, "unsupported data type");
            }
            case LayerType::TransposeConvolution2d:
            {
                // infos: input, output, weights[, bias] (RefLayerSupport.cpp: IsTransposeConvolution2dSupported)
                const auto& d = *PolymorphicDowncast<const TransposeConvolution2dDescriptor*>(&descriptor);
                if (d.m_DataLayout != DataLayout::NHWC && d.m_DataLayout != DataLayout::NCHW) { return No(reason, "NHWC or NCHW only"); }
                if (infos.size() < 3 || !Is8Bit(infos[0]) || !Is8Bit(infos[1]) || !Is8Bit(infos[2])) { return No(reason, "8-bit quantised tensors only"); }
                if (d.m_BiasEnabled && (infos.size() < 4 || infos[3].GetDataType() != DataType::Signed32)) { return No(reason, "bias must be Signed32"); }
                return true;
            }
            case LayerType::ElementwiseUnary:
            {
                const auto op = PolymorphicDowncast<const ElementwiseUnaryDescriptor*>(&descriptor)->m_Operation;
                if (op == UnaryOperation::LogicalNot)
                {
                    return (infos[0].GetDataType() == DataType::Boolean && infos[1].GetDataType() == DataType::Boolean) || No(reason, "LogicalNot takes Boolean tensors");
                }
                if (!IsActType(infos[0]) || infos[0].GetDataType() != infos[1].GetDataType()) { return No(reason, "unsupported or mismatched data types"); }
                return true;
            }
            case LayerType::Resize:
            {
                const auto& d = *PolymorphicDowncast<const ResizeDescriptor*>(&descriptor);
                if (d.m_AlignCorners && d.m_HalfPixelCenters) { return No(reason, "align corners and half pixel centres cannot both be set"); }
                if (infos[0].GetNumDimensions() != 4 || infos[1].GetNumDimensions() != 4) { return No(reason, "Resize needs 4-D tensors"); }
                if (!IsActType(infos[0]) || infos[0].GetDataType() != infos[1].GetDataType()) { return No(reason, "unsupported or mismatched data types"); }
                return true;
            }
            case LayerType::Concat:
            case LayerType::Splitter:
            {
                // RefLayerSupport.cpp:949-979 (Concat), :2597-2630 (Splitter): every tensor of the layer has one type;
                // the quantisation parameters may differ (the copy re-quantises)
                if (infos.empty() || infos[0].GetNumDimensions() > 6) { return No(reason, "rank > 6"); }
                for (const TensorInfo& t : infos)
                {
                    if (!IsMoveType(t)) { return No(reason, "unsupported data type"); }
                    if (t.GetDataType() != infos[0].GetDataType()) { return No(reason, "input and output types differ"); }
                }
                return true;
            }
            case LayerType::Tile:
            case LayerType::BroadcastTo:
            {
                // a Tile of a tensor of rank r walks up to 2 r dimensions; dimensions of extent or multiple 1 drop out
                unsigned int dims = 0;
                if (type == LayerType::Tile)
                {
                    const auto& m = PolymorphicDowncast<const TileDescriptor*>(&descriptor)->m_Multiples;
                    if (m.size() != infos[0].GetNumDimensions()) { return No(reason, "one multiple per dimension"); }
                    for (unsigned int i = 0; i < m.size(); ++i) { dims += (m[i] > 1 ? 1u : 0u) + (infos[0].GetShape()[i] > 1 ? 1u : 0u); }
                }
                else { dims = infos[1].GetNumDimensions(); }
                if (dims > 6) { return No(reason, "more than six dimensions to walk"); }
                return (IsMoveType(infos[0]) && infos[1].GetDataType() == infos[0].GetDataType()) || No(reason, "unsupported or mismatched data types");
            }
            case LayerType::BatchToSpaceNd:
            case LayerType::SpaceToBatchNd:
                if (infos[0].GetNumDimensions() != 3 && infos[0].GetNumDimensions() != 4) { return No(reason, "3 or 4 dimensions only"); }
                ARMNN_FALLTHROUGH;
            case LayerType::SpaceToDepth:
            case LayerType::ChannelShuffle:
            case LayerType::Stack:
            {
                // through Decoder / Encoder in the reference: one element type, the quantisation may differ
                for (const TensorInfo& t : infos)
                {
                    if (!IsMoveType(t) || t.GetDataType() != infos[0].GetDataType() || t.GetNumDimensions() > 6) { return No(reason, "unsupported or mismatched data types, or rank > 6"); }
                }
                return true;
            }
            case LayerType::Permute:
            case LayerType::Transpose:
            case LayerType::Slice:
            case LayerType::StridedSlice:
            case LayerType::DepthToSpace:
            {
                if (infos[0].GetNumDimensions() > 6) { return No(reason, "rank > 6"); }
                if (!IsMoveType(infos[0]) || infos[0].GetDataType() != infos[1].GetDataType()) { return No(reason, "unsupported or mismatched data types"); }
                if (infos[0].GetQuantizationScale() != infos[1].GetQuantizationScale() ||
                    infos[0].GetQuantizationOffset() != infos[1].GetQuantizationOffset()) { return No(reason, "input and output quantisation differ (the reference copies raw elements)"); }
                if (type == LayerType::StridedSlice)
                {
                    const auto& d = *PolymorphicDowncast<const StridedSliceDescriptor*>(&descriptor);
                    if (d.m_EllipsisMask != 0 || d.m_NewAxisMask != 0) { return No(reason, "ellipsis and new-axis masks are not supported"); }
                    if (infos[0].GetNumDimensions() > 4) { return No(reason, "rank > 4"); }
                }
                return true;
            }
            case LayerType::Mean:
            case LayerType::Reduce:
            {
                // Mean over H and W of an NHWC tensor has its own kernel; every other choice of axes, and Reduce, runs
                // on the general one (armnn::Reduce, src/backends/reference/workloads/Reduce.cpp:63-175)
                if (infos[0].GetNumDimensions() > 6) { return No(reason, "rank > 6"); }
                return (IsActType(infos[0]) && IsActType(infos[1])) || No(reason, "unsupported data type");
            }
            case LayerType::Comparison:
            case LayerType::LogicalBinary:
            {
                const bool logical = type == LayerType::LogicalBinary;
                if (infos[2].GetDataType() != DataType::Boolean) { return No(reason, "the output must be Boolean"); }
                if (infos[2].GetNumDimensions() > 4 || infos[0].GetNumDimensions() != infos[2].GetNumDimensions() ||
                    infos[1].GetNumDimensions() != infos[2].GetNumDimensions()) { return No(reason, "operands of one rank <= 4"); }
                if (infos[0].GetDataType() != infos[1].GetDataType()) { return No(reason, "input types differ"); }
                if (logical) { return infos[0].GetDataType() == DataType::Boolean || No(reason, "LogicalBinary takes Boolean tensors"); }
                return (IsActType(infos[0]) || infos[0].GetDataType() == DataType::Boolean) || No(reason, "unsupported data type");
            }
            case LayerType::Addition:
            case LayerType::Multiplication:
            case LayerType::Subtraction:
            case LayerType::Division:
            case LayerType::Maximum:
            case LayerType::Minimum:
            case LayerType::Prelu:
            case LayerType::ElementwiseBinary:
            {
                if (infos[2].GetNumDimensions() > 4) { return No(reason, "rank > 4"); }
                if (type != LayerType::Prelu && (infos[0].GetNumDimensions() != infos[2].GetNumDimensions() ||
                                                 infos[1].GetNumDimensions() != infos[2].GetNumDimensions()))
                {
                    return No(reason, "operands of different rank");
                }
                return (IsActType(infos[0]) && IsActType(infos[1]) && IsActType(infos[2])) || No(reason, "unsupported data type");
            }
            case LayerType::Activation:
            {
                const auto fn = PolymorphicDowncast<const ActivationDescriptor*>(&descriptor)->m_Function;
                return (IsActType(infos[0]) && IsActType(infos[1])) || No(reason, "unsupported data type");
            }
            case LayerType::Softmax:
                return (IsActType(infos[0]) && IsActType(infos[1])) || No(reason, "unsupported data type");
            case LayerType::Convolution3d:
            {
                // infos: input, output, weights[, bias]
                const auto& d = *PolymorphicDowncast<const Convolution3dDescriptor*>(&descriptor);
                if (d.m_DataLayout != DataLayout::NDHWC) { return No(reason, "NDHWC only"); }
                if (infos[0].GetNumDimensions() != 5 || infos[1].GetNumDimensions() != 5 || infos[2].GetNumDimensions() != 5) { return No(reason, "5-D tensors only"); }
                if (AllFloat32(infos)) { return true; }
                auto q8 = [](const TensorInfo& t) { return t.GetDataType() == DataType::QAsymmU8 || t.GetDataType() == DataType::QAsymmS8; };
                if (!q8(infos[0]) || !q8(infos[1]) || !(q8(infos[2]) || infos[2].GetDataType() == DataType::QSymmS8)) { return No(reason, "8-bit quantised tensors or Float32 throughout"); }
                if (infos.size() > 3 && infos[3].GetNumElements() > 0 && infos[3].GetDataType() != DataType::Signed32) { return No(reason, "bias must be Signed32"); }
                if (infos[2].HasPerAxisQuantization() && infos[2].GetQuantizationDim().value() != 4) { return No(reason, "per-axis weights must be quantised along the output channels"); }
                return true;
            }
            case LayerType::Pooling3d:
            {
                const auto& d = *PolymorphicDowncast<const Pooling3dDescriptor*>(&descriptor);
                if (d.m_DataLayout != DataLayout::NDHWC) { return No(reason, "NDHWC only"); }
                return (infos[0].GetNumDimensions() == 5 && IsActType(infos[0]) && infos[1].GetDataType() == infos[0].GetDataType()) ||
                       No(reason, "5-D tensors of one supported data type");
            }
            case LayerType::Shape:
            case LayerType::Rank:
                return infos[1].GetDataType() == DataType::Signed32 || No(reason, "the output must be Signed32");
            case LayerType::FakeQuantization:
            {
                const auto& d = *PolymorphicDowncast<const FakeQuantizationDescriptor*>(&descriptor);
                if (!(d.m_Max > d.m_Min)) { return No(reason, "min must be below max"); }
                return (infos[0].GetDataType() == DataType::Float32 && infos[1].GetDataType() == DataType::Float32) || No(reason, "Float32 only");
            }
            case LayerType::ConvertFp16ToFp32:
                return (infos[0].GetDataType() == DataType::Float16 && infos[1].GetDataType() == DataType::Float32) || No(reason, "Float16 -> Float32 only");
            case LayerType::ConvertFp32ToFp16:
                return (infos[0].GetDataType() == DataType::Float32 && infos[1].GetDataType() == DataType::Float16) || No(reason, "Float32 -> Float16 only");
            case LayerType::Cast:
                return (IsMoveType(infos[0]) && IsMoveType(infos[1]) && infos[0].GetNumElements() == infos[1].GetNumElements()) ||
                       No(reason, "unsupported data type or mismatched sizes");
            case LayerType::Fill:
                return ((infos[1].GetDataType() == DataType::Float32 || infos[1].GetDataType() == DataType::Signed32) &&
                        infos[1].GetNumDimensions() >= 1 && infos[1].GetNumDimensions() <= 6) || No(reason, "Float32 or Signed32 output of 1 to 6 dimensions");
            case LayerType::Floor:
                return (infos[0].GetDataType() == DataType::Float32 && infos[1].GetDataType() == DataType::Float32) || No(reason, "Float32 only");
            case LayerType::LogSoftmax:
            case LayerType::L2Normalization:
                if (infos[0].GetDataType() == DataType::QSymmS16 && type == LayerType::LogSoftmax) { return No(reason, "QSymmS16 is not supported"); }
                if (type == LayerType::L2Normalization && infos[0].GetNumDimensions() > 4) { return No(reason, "rank > 4"); }
                return (IsActType(infos[0]) && infos[1].GetDataType() == infos[0].GetDataType()) || No(reason, "unsupported or mismatched data types");
            case LayerType::Gather:
                if (infos[1].GetDataType() != DataType::Signed32) { return No(reason, "indices must be Signed32"); }
                return (IsMoveType(infos[0]) && infos[2].GetDataType() == infos[0].GetDataType()) || No(reason, "unsupported or mismatched data types");
            case LayerType::ScatterNd:
            {
                // infos: input (or shape), indices, updates, output
                const auto& d = *PolymorphicDowncast<const ScatterNdDescriptor*>(&descriptor);
                if (d.m_AxisEnabled) { return No(reason, "the axis option is not supported"); }
                if (infos[1].GetDataType() != DataType::Signed32 || infos[1].GetNumDimensions() != 2) { return No(reason, "indices must be Signed32 [n, nd]"); }
                const unsigned int nd = infos[1].GetShape()[1];
                if (nd < 1 || nd > 8 || nd > infos[3].GetNumDimensions()) { return No(reason, "index tuples longer than the output's rank (or than 8)"); }
                if (!IsActType(infos[3]) || infos[2].GetDataType() != infos[3].GetDataType()) { return No(reason, "unsupported or mismatched data types"); }
                if (d.m_InputEnabled ? infos[0].GetDataType() != infos[3].GetDataType() : infos[0].GetDataType() != DataType::Signed32) { return No(reason, "first input: the tensor, or a Signed32 shape"); }
                return true;
            }
            case LayerType::ReverseV2:
                if (infos[1].GetDataType() != DataType::Signed32 || infos[0].GetNumDimensions() > 6) { return No(reason, "Signed32 axes and rank <= 6"); }
                return (IsMoveType(infos[0]) && infos[2].GetDataType() == infos[0].GetDataType()) || No(reason, "unsupported or mismatched data types");
            case LayerType::GatherNd:
            {
                if (infos[1].GetDataType() != DataType::Signed32 || infos[1].GetNumDimensions() < 1) { return No(reason, "indices must be Signed32"); }
                const unsigned int nd = infos[1].GetShape()[infos[1].GetNumDimensions() - 1];
                if (nd < 1 || nd > 8 || nd > infos[0].GetNumDimensions()) { return No(reason, "index tuples longer than the tensor's rank (or than 8)"); }
                return (IsMoveType(infos[0]) && infos[2].GetDataType() == infos[0].GetDataType()) || No(reason, "unsupported or mismatched data types");
            }
            case LayerType::BatchNormalization:
                if (infos[0].GetNumDimensions() != 4) { return No(reason, "4-D tensors only"); }
                for (const TensorInfo& t : infos) { if (!IsActType(t)) { return No(reason, "unsupported data type"); } }
                return true;
            case LayerType::Normalization:
                if (PolymorphicDowncast<const NormalizationDescriptor*>(&descriptor)->m_NormMethodType != NormalizationAlgorithmMethod::LocalBrightness)
                {
                    return No(reason, "LocalContrast is not supported");
                }
                return (infos[0].GetNumDimensions() == 4 && IsActType(infos[0]) && infos[1].GetDataType() == infos[0].GetDataType()) ||
                       No(reason, "4-D tensors of one supported data type only");
            case LayerType::InstanceNormalization:
                return (infos[0].GetNumDimensions() == 4 && infos[0].GetDataType() == DataType::Float32 && infos[1].GetDataType() == DataType::Float32) ||
                       No(reason, "4-D Float32 tensors only");
            case LayerType::ArgMinMax:
                if (infos[1].GetDataType() != DataType::Signed32 && infos[1].GetDataType() != DataType::Signed64) { return No(reason, "the output must be Signed32 or Signed64"); }
                return IsActType(infos[0]) || No(reason, "unsupported input data type");
            case LayerType::Quantize:
            case LayerType::Dequantize:
                if (infos[0].HasPerAxisQuantization()) { return No(reason, "per-axis input is not supported"); }
                return (IsActType(infos[0]) && IsActType(infos[1])) || No(reason, "unsupported data type");
            case LayerType::Lstm:
            case LayerType::UnidirectionalSequenceLstm:
            {
                // infos: input, outputStateIn, cellStateIn, then the outputs; the weights travel in lstmParamsInfo
                for (const TensorInfo& t : infos) { if (t.GetDataType() != DataType::Float32) { return No(reason, "Float32 tensors only"); } }
                const auto& d = *PolymorphicDowncast<const LstmDescriptor*>(&descriptor);
                const uint32_t f = d.m_ActivationFunc;
                if (f != 0 && f != 1 && f != 3 && f != 4 && f != 6) { return No(reason, "unsupported activation function"); }
                if (lstmParamsInfo.has_value() && lstmParamsInfo.value().m_InputToForgetWeights &&
                    lstmParamsInfo.value().m_InputToForgetWeights->GetDataType() != DataType::Float32) { return No(reason, "Float32 weights only"); }
                return true;
            }
            case LayerType::QLstm:
                if (infos[0].GetDataType() != DataType::QAsymmS8 || infos[2].GetDataType() != DataType::QSymmS16) { return No(reason, "QLstm needs QAsymmS8 input and QSymmS16 cell state"); }
                return true;
            default:
                return No(reason, "layer type is not on the B200Acc hot path");
        }
    }
};

/// Runtime-level state: BackendOptions("B200Acc", {...}) given to IRuntime::Create —
///   "DeviceId"        default GPU of networks that carry no DeviceId ModelOption (else B200ACC_DEVICE_ID, else 0)
///   "GraphReplay"     false: never replay workload queues as CUDA graphs (default true)
///   "WaitSelfTestUs"  > 0: every convolution runs the bounded-wait self-test of b200k_conv2d_params.selftest_us
/// Modelled on ClBackendContext (src/backends/cl/ClBackendContext.cpp:61-215).
class B200BackendContext : public IBackendContext
{
public:
    explicit B200BackendContext(const IRuntime::CreationOptions& options) : IBackendContext(options)
    {
        int device = -1, selfTest = 0;
        bool graph = true;
        for (const auto& bo : options.m_BackendOptions)
        {
            if (bo.GetBackendId() != BackendId(B200BackendId())) { continue; }
            for (size_t i = 0; i < bo.GetOptionCount(); ++i)
            {
                const auto& opt = bo.GetOption(i);
                if (opt.GetName() == "DeviceId" && opt.GetValue().IsInt()) { device = opt.GetValue().AsInt(); }
                if (opt.GetName() == "WaitSelfTestUs" && opt.GetValue().IsInt()) { selfTest = opt.GetValue().AsInt(); }
                if (opt.GetName() == "GraphReplay" && opt.GetValue().IsBool()) { graph = opt.GetValue().AsBool(); }
            }
        }
        B200Context::SetDefaultDevice(device);
        B200Context::SetDefaultSelfTestUs(selfTest);
        B200Context::SetGraphReplayEnabled(graph);
        if (b200k_device_open(B200Context::DefaultDevice()) != B200K_OK)
        {
            throw BackendUnavailableException(std::string("B200Acc: ") + b200k_last_error());
        }
    }
    bool BeforeLoadNetwork(NetworkId) override { return true; }
    bool AfterLoadNetwork(NetworkId) override { return true; }
    bool BeforeUnloadNetwork(NetworkId) override
    {
        B200Context::SynchronizeAll();
        return true;
    }
    bool AfterUnloadNetwork(NetworkId) override { return true; }
    bool AfterEnqueueWorkload(NetworkId) override
    {
        // the contexts this thread has just run workloads on: wait, report device-side failures, next epoch (imported
        // inputs are uploaded afresh by the next inference)
        return B200Context::EndInferenceAll();
    }
};

namespace
{

bool SameQuantisation(const TensorInfo& a, const TensorInfo& b)
{
    return a.GetDataType() == b.GetDataType() && IsQuantizedType(a.GetDataType()) &&
           a.GetQuantizationScale() == b.GetQuantizationScale() && a.GetQuantizationOffset() == b.GetQuantizationOffset();
}

/// [Pad ->] base -> Activation becomes `replacement` (same kind as base, padding already added to its descriptor when
/// there is a Pad) carrying the activation as additional information.
template <typename LayerT>
void Fuse(OptimizationViews& views, LayerT* base, LayerT* replacement, ActivationLayer* act, Layer* pad = nullptr)
{
    replacement->SetAdditionalInfoForObject(std::make_shared<ActivationDescriptor>(act->GetParameters()));
    if (!pad)
    {
        SubgraphView substitution({base, act}, CreateIInputsFrom({base}), CreateIOutputsFrom({act}));
        SubgraphView replacementView(replacement);
        views.AddSubstitution({substitution, replacementView});
        return;
    }
    // the data input is the Pad's, the weights and the bias stay the base layer's
    SubgraphView::IInputSlots inputs{&pad->GetInputSlot(0)};
    for (unsigned int i = 1; i < base->GetNumInputSlots(); ++i) { inputs.push_back(&base->GetInputSlot(i)); }
    SubgraphView substitution({pad, base, act}, std::move(inputs), CreateIOutputsFrom({act}));
    SubgraphView replacementView(replacement);
    views.AddSubstitution({substitution, replacementView});
}

}  // namespace

const BackendId& B200Backend::GetIdStatic()
{
    static const BackendId s_Id{B200BackendId()};
    return s_Id;
}

IBackendInternal::IMemoryManagerUniquePtr B200Backend::CreateMemoryManager() const
{
    return std::make_unique<B200MemoryManager>();
}

IBackendInternal::IWorkloadFactoryPtr B200Backend::CreateWorkloadFactory(const IMemoryManagerSharedPtr& memoryManager) const
{
    return std::make_unique<B200WorkloadFactory>(B200Context::Shared(), PolymorphicPointerDowncast<B200MemoryManager>(memoryManager));
}

namespace
{
/// DeviceId of a network: its ModelOption, else the runtime's default.
int DeviceOf(const ModelOptions& modelOptions)
{
    B200BackendModelContext ctx(modelOptions);
    return ctx.DeviceId() >= 0 ? ctx.DeviceId() : B200Context::DefaultDevice();
}

/// One context (GPU, stream, workload queue), one memory manager and one handle factory per network.
IBackendInternal::IWorkloadFactoryPtr MakeFactories(TensorHandleFactoryRegistry& registry, int device)
{
    auto ctx = std::make_shared<B200Context>(device);
    auto memoryManager = std::make_shared<B200MemoryManager>(ctx);
    registry.RegisterMemoryManager(memoryManager);
    auto factory = std::make_unique<B200TensorHandleFactory>(ctx, memoryManager);
    registry.RegisterCopyAndImportFactoryPair(factory->GetId(), factory->GetId());
    registry.RegisterFactory(std::move(factory));
    return std::make_unique<B200WorkloadFactory>(ctx, memoryManager);
}
}  // namespace

IBackendInternal::IWorkloadFactoryPtr B200Backend::CreateWorkloadFactory(TensorHandleFactoryRegistry& registry) const
{
    return MakeFactories(registry, B200Context::DefaultDevice());
}

// LoadedNetwork hands the network's ModelOptions over here (src/armnn/LoadedNetwork.cpp:264-279): the pattern of
// ClBackend (src/backends/cl/ClBackend.cpp:62-71, 246-250), with the GPU chosen per network
IBackendInternal::IWorkloadFactoryPtr B200Backend::CreateWorkloadFactory(TensorHandleFactoryRegistry& registry,
                                                                         const ModelOptions& modelOptions) const
{
    return MakeFactories(registry, DeviceOf(modelOptions));
}

IBackendInternal::IWorkloadFactoryPtr B200Backend::CreateWorkloadFactory(TensorHandleFactoryRegistry& registry,
                                                                         const ModelOptions& modelOptions,
                                                                         MemorySourceFlags, MemorySourceFlags) const
{
    return MakeFactories(registry, DeviceOf(modelOptions));
}

IBackendInternal::IBackendSpecificModelContextPtr B200Backend::CreateBackendSpecificModelContext(const ModelOptions& modelOptions) const
{
    return IBackendSpecificModelContextPtr{new B200BackendModelContext(modelOptions)};
}

IBackendInternal::IBackendContextPtr B200Backend::CreateBackendContext(const IRuntime::CreationOptions& options) const
{
    return IBackendContextPtr{new B200BackendContext(options)};
}

IBackendInternal::IBackendProfilingContextPtr B200Backend::CreateBackendProfilingContext(const IRuntime::CreationOptions&,
                                                                                         IBackendProfilingPtr&)
{
    return IBackendProfilingContextPtr{};
}

IBackendInternal::ILayerSupportSharedPtr B200Backend::GetLayerSupport() const
{
    static ILayerSupportSharedPtr layerSupport{new B200LayerSupport};
    return layerSupport;
}

IBackendInternal::ILayerSupportSharedPtr B200Backend::GetLayerSupport(const ModelOptions&) const
{
    return GetLayerSupport();
}

std::vector<ITensorHandleFactory::FactoryId> B200Backend::GetHandleFactoryPreferences() const
{
    return {B200TensorHandleFactory::GetIdStatic()};
}

// Called by the optimizer (handle-strategy selection) and by LoadedNetwork for backends that do not own the network's
// factories: no device is touched until a handle is created.
void B200Backend::RegisterTensorHandleFactories(TensorHandleFactoryRegistry& registry)
{
    auto memoryManager = std::make_shared<B200MemoryManager>();
    registry.RegisterMemoryManager(memoryManager);
    auto factory = std::make_unique<B200TensorHandleFactory>(nullptr, memoryManager);
    registry.RegisterCopyAndImportFactoryPair(factory->GetId(), factory->GetId());
    registry.RegisterFactory(std::move(factory));
}

void B200Backend::RegisterTensorHandleFactories(TensorHandleFactoryRegistry& registry, MemorySourceFlags, MemorySourceFlags)
{
    RegisterTensorHandleFactories(registry);
}

BackendCapabilities B200Backend::GetCapabilities() const
{
        // NonConstWeights:true makes the core ask B200LayerSupport (which then refuses non-constant weights with a
        // reason) instead of refusing in LayerSupportHandle (src/armnn/BackendHelper.cpp:371-423)
        return BackendCapabilities("B200Acc", {{"NonConstWeights", true},
                                               {"ProtectedContentAllocation", false},
                                               {"ConstantTensorsAsInputs", true},
                                               {"PreImportIOTensors", false},
                                               {"ExternallyManagedMemory", false},
                                               {"MultiAxisPacking", false},
                                               {"SingleAxisPacking", false},
                                               {"HasFp16", false},
                                               {"AllOrNothing", false}});
}

namespace
{

    /// Convolution2d -> ElementwiseBinary(Add, other) [-> Activation{ReLu, BoundedReLu}] becomes one PreCompiled layer
    /// (inputs: data, weights[, bias], other) whose workload adds the other operand in the convolution's epilogue:
    /// the residual connections of ResNet-style graphs then cost no pass over memory of their own.  The result is what
    /// the three CpuRef workloads in a row produce (the convolution's own 8-bit result is formed, not stored).
    void FuseResidualAdds(const BackendId& backendId, const SubgraphView& subgraph, OptimizationViews& views, std::map<LayerGuid, Layer*>& untouched)
    {
        for (auto it = subgraph.begin(); it != subgraph.end(); ++it)
        {
            Layer& l = *PolymorphicDowncast<Layer*>(*it);
            if (l.GetType() != LayerType::ElementwiseBinary || untouched.find(l.GetGuid()) == untouched.end()) { continue; }
            auto* add = PolymorphicDowncast<ElementwiseBinaryLayer*>(&l);
            if (add->GetParameters().m_Operation != BinaryOperation::Add) { continue; }
            if (add->GetAdditionalInformation<ActivationDescriptor>() != nullptr) { continue; }
            const TensorInfo& addOut = add->GetOutputSlot(0).GetTensorInfo();
            if (!Is8Bit(addOut) || addOut.GetNumDimensions() != 4 || addOut.GetShape()[3] % 16 != 0) { continue; }
            for (unsigned int side = 0; side < 2; ++side)
            {
                OutputSlot* src = add->GetInputSlot(side).GetConnectedOutputSlot();
                OutputSlot* other = add->GetInputSlot(1 - side).GetConnectedOutputSlot();
                if (!src || !other) { continue; }
                Layer& producer = src->GetOwningLayer();
                if (producer.GetType() != LayerType::Convolution2d || untouched.find(producer.GetGuid()) == untouched.end() ||
                    &other->GetOwningLayer() == &producer || src->GetNumConnections() != 1) { continue; }
                auto* conv = PolymorphicDowncast<Convolution2dLayer*>(&producer);
                if (conv->GetAdditionalInformation<ActivationDescriptor>() != nullptr ||
                    conv->GetParameters().m_DataLayout != DataLayout::NHWC) { continue; }
                const TensorInfo& convOut = src->GetTensorInfo();
                const TensorInfo& otherInfo = other->GetTensorInfo();
                if (!Is8Bit(convOut) || convOut.HasMultipleQuantizationScales() || !Is8Bit(otherInfo) ||
                    convOut.GetShape() != addOut.GetShape() || otherInfo.GetShape() != addOut.GetShape()) { continue; }

                ActivationLayer* act = nullptr;
                if (add->GetOutputSlot(0).GetNumConnections() == 1)
                {
                    Layer& child = add->GetOutputSlot(0).GetConnection(0)->GetOwningLayer();
                    if (child.GetType() == LayerType::Activation && untouched.find(child.GetGuid()) != untouched.end())
                    {
                        auto* a = PolymorphicDowncast<ActivationLayer*>(&child);
                        const ActivationFunction fn = a->GetParameters().m_Function;
                        if ((fn == ActivationFunction::ReLu || fn == ActivationFunction::BoundedReLu) &&
                            SameQuantisation(addOut, a->GetOutputSlot(0).GetTensorInfo())) { act = a; }
                    }
                }

                auto* blob = new B200FusedConvAdd;
                blob->m_Convolution = conv->GetParameters();
                blob->m_ConvolutionOutput = convOut;
                if (act) { blob->m_HasActivation = true; blob->m_Activation = act->GetParameters(); }
                CompiledBlobPtr blobPtr(blob, [](const void* p) { delete static_cast<const B200FusedConvAdd*>(p); });
                const unsigned int convInputs = conv->GetNumInputSlots();
                const std::string name = std::string("fused-") + add->GetName() + "-into-" + conv->GetName();
                IConnectableLayer* fused = views.GetINetwork()->AddPrecompiledLayer(
                    PreCompiledDescriptor(convInputs + 1, 1), std::move(blobPtr), Optional<BackendId>(backendId), name.c_str());
                Layer* last = act ? static_cast<Layer*>(act) : static_cast<Layer*>(add);
                fused->GetOutputSlot(0).SetTensorInfo(last->GetOutputSlot(0).GetTensorInfo());

                SubgraphView::IConnectableLayers layers{conv, add};
                if (act) { layers.push_back(act); }
                SubgraphView::IInputSlots inputs;
                for (unsigned int i = 0; i < convInputs; ++i) { inputs.push_back(&conv->GetInputSlot(i)); }
                inputs.push_back(&add->GetInputSlot(1 - side));
                SubgraphView::IOutputSlots outputs{&last->GetOutputSlot(0)};
                views.AddSubstitution({SubgraphView(std::move(layers), std::move(inputs), std::move(outputs)), SubgraphView(fused)});
                untouched.erase(conv->GetGuid());
                untouched.erase(add->GetGuid());
                if (act) { untouched.erase(act->GetGuid()); }
                break;
            }
        }
    }

    /// Pad -> Convolution2d / DepthwiseConvolution2d / Pooling2d becomes the layer itself with the padding added to its
    /// descriptor, when the pad value is the tensor's zero point and only H and W are padded.  The core does this for
    /// the backends named CpuAcc / GpuAcc only (src/armnn/Network.cpp:1394-1401), every other backend folds by itself
    /// as RefBackend does (src/backends/reference/RefBackend.cpp:93-164), with the same shared helpers.
    /// The Pad layer in front of `baseLayer` when it can be folded; `descriptor` then has its padding added.
    template <typename LayerT, typename DescriptorT>
    PadLayer* FoldablePad(LayerT* baseLayer, DescriptorT& descriptor, const std::map<LayerGuid, Layer*>& untouched, bool isPooling)
    {
        OutputSlot* src = baseLayer->GetInputSlot(0).GetConnectedOutputSlot();
        if (!src || src->GetOwningLayer().GetType() != LayerType::Pad) { return nullptr; }
        auto* padLayer = PolymorphicDowncast<PadLayer*>(&src->GetOwningLayer());
        if (untouched.find(padLayer->GetGuid()) == untouched.end() || padLayer->GetOutputSlot(0).GetNumConnections() != 1) { return nullptr; }
        if (padLayer->GetParameters().m_PaddingMode != PaddingMode::Constant) { return nullptr; }      // a mirrored border is no padding value
        bool ok;
        if constexpr (std::is_same<DescriptorT, Pooling2dDescriptor>::value)
        {
            ok = optimizations::pad_fold::TryFoldPadIntoLayer2d(padLayer->GetParameters(), descriptor,
                                                                padLayer->GetOutputSlot().GetTensorInfo(), isPooling);
        }
        else
        {
            ok = optimizations::pad_fold::TryFoldPadIntoLayer2d<DescriptorT>(padLayer->GetParameters(), descriptor,
                                                                             padLayer->GetOutputSlot().GetTensorInfo());
        }
        return ok ? padLayer : nullptr;
    }

    template <typename LayerT, typename DescriptorT>
    void TryFoldPad(Layer& base, OptimizationViews& views, std::map<LayerGuid, Layer*>& untouched, bool isPooling)
    {
        auto* baseLayer = PolymorphicDowncast<LayerT*>(&base);
        if (untouched.find(baseLayer->GetGuid()) == untouched.end()) { return; }
        DescriptorT descriptor = baseLayer->GetParameters();
        PadLayer* padLayer = FoldablePad<LayerT, DescriptorT>(baseLayer, descriptor, untouched, isPooling);
        if (!padLayer) { return; }
        FoldPadLayer2d<LayerT, DescriptorT>(views, baseLayer, descriptor, padLayer);
        untouched.erase(baseLayer->GetGuid());
        untouched.erase(padLayer->GetGuid());
    }

}  // namespace

    /// Fold Activation{ReLu, BoundedReLu} into the producing Convolution2d / DepthwiseConvolution2d / FullyConnected /
    /// ElementwiseBinary when both tensors carry the same quantisation: the workload then clamps in the quantised
    /// domain, which is exactly what the separate CpuRef Activation workload would compute.
OptimizationViews B200Backend::OptimizeSubgraphView(const SubgraphView& subgraph, const ModelOptions& modelOptions) const
{
        OptimizationViews views(modelOptions);
        std::map<LayerGuid, Layer*> untouched;
        for (auto it = subgraph.begin(); it != subgraph.end(); ++it)
        {
            Layer& l = *PolymorphicDowncast<Layer*>(*it);
            untouched.insert({l.GetGuid(), &l});
        }
        FuseResidualAdds(GetId(), subgraph, views, untouched);
        for (auto it = subgraph.begin(); it != subgraph.end(); ++it)
        {
            Layer& base = *PolymorphicDowncast<Layer*>(*it);
            if (untouched.find(base.GetGuid()) == untouched.end()) { continue; }
            const LayerType t = base.GetType();
            if (t != LayerType::Convolution2d && t != LayerType::DepthwiseConvolution2d && t != LayerType::FullyConnected &&
                t != LayerType::ElementwiseBinary) { continue; }
            if (base.GetAdditionalInformation<ActivationDescriptor>() != nullptr) { continue; }
            OutputSlot& out = base.GetOutputSlot(0);
            if (out.GetNumConnections() != 1) { continue; }
            // the fp32 contractions have no fused clamp: their activations stay layers of their own
            if (t != LayerType::ElementwiseBinary && out.GetTensorInfo().GetDataType() == DataType::Float32) { continue; }
            Layer& child = out.GetConnection(0)->GetOwningLayer();
            if (child.GetType() != LayerType::Activation || untouched.find(child.GetGuid()) == untouched.end()) { continue; }
            auto* act = PolymorphicDowncast<ActivationLayer*>(&child);
            const ActivationFunction fn = act->GetParameters().m_Function;
            if (fn != ActivationFunction::ReLu && fn != ActivationFunction::BoundedReLu) { continue; }
            if (!SameQuantisation(out.GetTensorInfo(), act->GetOutputSlot(0).GetTensorInfo())) { continue; }
            const std::string name = std::string("fused-") + child.GetName() + "-into-" + base.GetName();
            INetwork* net = views.GetINetwork();
            if (t == LayerType::Convolution2d)
            {
                // a Pad in front of the convolution goes into the same substitution
                auto* b = PolymorphicDowncast<Convolution2dLayer*>(&base);
                Convolution2dDescriptor desc = b->GetParameters();
                PadLayer* pad = FoldablePad<Convolution2dLayer, Convolution2dDescriptor>(b, desc, untouched, false);
                auto* r = PolymorphicDowncast<Convolution2dLayer*>(net->AddConvolution2dLayer(desc, name.c_str()));
                Fuse(views, b, r, act, pad);
                if (pad) { untouched.erase(pad->GetGuid()); }
            }
            else if (t == LayerType::DepthwiseConvolution2d)
            {
                auto* b = PolymorphicDowncast<DepthwiseConvolution2dLayer*>(&base);
                DepthwiseConvolution2dDescriptor desc = b->GetParameters();
                PadLayer* pad = FoldablePad<DepthwiseConvolution2dLayer, DepthwiseConvolution2dDescriptor>(b, desc, untouched, false);
                auto* r = PolymorphicDowncast<DepthwiseConvolution2dLayer*>(net->AddDepthwiseConvolution2dLayer(desc, name.c_str()));
                Fuse(views, b, r, act, pad);
                if (pad) { untouched.erase(pad->GetGuid()); }
            }
            else if (t == LayerType::FullyConnected)
            {
                auto* b = PolymorphicDowncast<FullyConnectedLayer*>(&base);
                auto* r = PolymorphicDowncast<FullyConnectedLayer*>(net->AddFullyConnectedLayer(b->GetParameters(), name.c_str()));
                Fuse(views, b, r, act);
            }
            else
            {
                auto* b = PolymorphicDowncast<ElementwiseBinaryLayer*>(&base);
                const BinaryOperation op = b->GetParameters().m_Operation;
                if (op != BinaryOperation::Add && op != BinaryOperation::Mul && op != BinaryOperation::Sub) { continue; }
                auto* r = PolymorphicDowncast<ElementwiseBinaryLayer*>(net->AddElementwiseBinaryLayer(b->GetParameters(), name.c_str()));
                Fuse(views, b, r, act);
            }
            untouched.erase(base.GetGuid());
            untouched.erase(child.GetGuid());
        }
        // explicit padding in front of layers the fusions above have left alone
        for (auto it = subgraph.begin(); it != subgraph.end(); ++it)
        {
            Layer& base = *PolymorphicDowncast<Layer*>(*it);
            if (base.GetType() == LayerType::Convolution2d) { TryFoldPad<Convolution2dLayer, Convolution2dDescriptor>(base, views, untouched, false); }
            else if (base.GetType() == LayerType::DepthwiseConvolution2d) { TryFoldPad<DepthwiseConvolution2dLayer, DepthwiseConvolution2dDescriptor>(base, views, untouched, false); }
            else if (base.GetType() == LayerType::Pooling2d) { TryFoldPad<Pooling2dLayer, Pooling2dDescriptor>(base, views, untouched, true); }
        }
        if (views.GetSubstitutions().empty())
        {
            views.AddUntouchedSubgraph(SubgraphView(subgraph));
        }
        else
        {
            ReportUntouchedLayers(views, untouched);
        }
        return views;
}

}  // namespace armnn

