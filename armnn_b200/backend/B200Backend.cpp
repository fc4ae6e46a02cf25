// The B200Acc backend object: IBackendInternal, layer support, graph-level optimisation (activation fusion), and the
// three extern "C" entry points of a dynamic backend (include/armnn/backends/DynamicBackend.hpp:41-43 of the Arm NN
// tree).  Structure follows RefBackend (src/backends/reference/RefBackend.cpp:22-208) and the sample dynamic backend
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
                          const Optional<LstmInputParamsInfo>&, const Optional<QuantizedLstmInputParamsInfo>&,
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
                if (layout != DataLayout::NHWC) { return No(reason, "only NHWC is supported"); }
                if (!Is8Bit(infos[0]) || !Is8Bit(infos[1]) || !Is8Bit(infos[2])) { return No(reason, "input, output and weights must be 8-bit quantised"); }
                if (!infos[2].IsConstant()) { return No(reason, "non-constant weights are not supported"); }
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
                if (!Is8Bit(infos[0]) || !Is8Bit(infos[1]) || !Is8Bit(infos[2])) { return No(reason, "input, output and weights must be 8-bit quantised"); }
                if (!infos[2].IsConstant()) { return No(reason, "non-constant weights are not supported"); }
                const auto& d = *PolymorphicDowncast<const FullyConnectedDescriptor*>(&descriptor);
                if (d.m_BiasEnabled && infos[3].GetDataType() != DataType::Signed32) { return No(reason, "bias must be Signed32"); }
                return true;
            }
            case LayerType::BatchMatMul:
            {
                const auto& d = *PolymorphicDowncast<const BatchMatMulDescriptor*>(&descriptor);
                if (d.m_AdjointX || d.m_AdjointY) { return No(reason, "adjoint inputs are not supported"); }
                if (d.m_DataLayoutX != DataLayout::NCHW || d.m_DataLayoutY != DataLayout::NCHW) { return No(reason, "only the default axis choice is supported"); }
                if (!Is8Bit(infos[0]) || !Is8Bit(infos[1]) || !Is8Bit(infos[2])) { return No(reason, "8-bit quantised tensors only"); }
                return true;
            }
            case LayerType::Pooling2d:
                if (PolymorphicDowncast<const Pooling2dDescriptor*>(&descriptor)->m_DataLayout != DataLayout::NHWC) { return No(reason, "only NHWC is supported"); }
                return (IsActType(infos[0]) && IsActType(infos[1])) || No(reason, "unsupported data type");
            case LayerType::Mean:
            {
                const auto& d = *PolymorphicDowncast<const MeanDescriptor*>(&descriptor);
                if (infos[0].GetNumDimensions() != 4 || d.m_Axis != std::vector<unsigned int>{1, 2}) { return No(reason, "Mean only over H and W of an NHWC tensor"); }
                return (IsActType(infos[0]) && IsActType(infos[1])) || No(reason, "unsupported data type");
            }
            case LayerType::Addition:
            case LayerType::Multiplication:
            case LayerType::ElementwiseBinary:
            {
                if (type == LayerType::ElementwiseBinary)
                {
                    const auto op = PolymorphicDowncast<const ElementwiseBinaryDescriptor*>(&descriptor)->m_Operation;
                    if (op == BinaryOperation::Power || op == BinaryOperation::FloorDiv) { return No(reason, "Power / FloorDiv are not supported"); }
                }
                if (infos[2].GetNumDimensions() > 4) { return No(reason, "rank > 4"); }
                return (IsActType(infos[0]) && IsActType(infos[1]) && IsActType(infos[2])) || No(reason, "unsupported data type");
            }
            case LayerType::Activation:
            {
                const auto fn = PolymorphicDowncast<const ActivationDescriptor*>(&descriptor)->m_Function;
                if (fn == ActivationFunction::Gelu) { return No(reason, "Gelu is not supported"); }
                return (IsActType(infos[0]) && IsActType(infos[1])) || No(reason, "unsupported data type");
            }
            case LayerType::Softmax:
                return (IsActType(infos[0]) && IsActType(infos[1])) || No(reason, "unsupported data type");
            case LayerType::Quantize:
            case LayerType::Dequantize:
                if (infos[0].HasPerAxisQuantization()) { return No(reason, "per-axis input is not supported"); }
                return (IsActType(infos[0]) && IsActType(infos[1])) || No(reason, "unsupported data type");
            case LayerType::QLstm:
                if (infos[0].GetDataType() != DataType::QAsymmS8 || infos[2].GetDataType() != DataType::QSymmS16) { return No(reason, "QLstm needs QAsymmS8 input and QSymmS16 cell state"); }
                return true;
            default:
                return No(reason, "layer type is not on the B200Acc hot path");
        }
    }
};

class B200BackendContext : public IBackendContext
{
public:
    explicit B200BackendContext(const IRuntime::CreationOptions& options) : IBackendContext(options)
    {
        int device = -1;
        for (const auto& bo : options.m_BackendOptions)
        {
            if (bo.GetBackendId() != BackendId(B200BackendId())) { continue; }
            for (size_t i = 0; i < bo.GetOptionCount(); ++i)
            {
                const auto& opt = bo.GetOption(i);
                if (opt.GetName() == "DeviceId" && opt.GetValue().IsInt()) { device = opt.GetValue().AsInt(); }
            }
        }
        B200Device::Configure(device);                   // throws BackendUnavailableException without an sm_100 device
    }
    bool BeforeLoadNetwork(NetworkId) override { return true; }
    bool AfterLoadNetwork(NetworkId) override { return true; }
    bool BeforeUnloadNetwork(NetworkId) override
    {
        cudaStreamSynchronize(B200Device::Get().Stream());
        return true;
    }
    bool AfterUnloadNetwork(NetworkId) override { return true; }
    bool AfterEnqueueWorkload(NetworkId) override
    {
        B200Device::NextEpoch();                          // imported inputs are uploaded afresh by the next inference
        return cudaStreamSynchronize(B200Device::Get().Stream()) == cudaSuccess && b200k_poll_status() == B200K_OK;
    }
};

namespace
{

bool SameQuantisation(const TensorInfo& a, const TensorInfo& b)
{
    return a.GetDataType() == b.GetDataType() && IsQuantizedType(a.GetDataType()) &&
           a.GetQuantizationScale() == b.GetQuantizationScale() && a.GetQuantizationOffset() == b.GetQuantizationOffset();
}

template <typename LayerT>
void Fuse(OptimizationViews& views, LayerT* base, LayerT* replacement, ActivationLayer* act)
{
    replacement->SetAdditionalInfoForObject(std::make_shared<ActivationDescriptor>(act->GetParameters()));
    SubgraphView substitution({base, act}, CreateIInputsFrom({base}), CreateIOutputsFrom({act}));
    SubgraphView replacementView(replacement);
    views.AddSubstitution({substitution, replacementView});
}

}  // namespace

class B200Backend : public IBackendInternal
{
public:
    static const BackendId& GetIdStatic()
    {
        static const BackendId s_Id{B200BackendId()};
        return s_Id;
    }
    const BackendId& GetId() const override { return GetIdStatic(); }

    IMemoryManagerUniquePtr CreateMemoryManager() const override { return std::make_unique<B200MemoryManager>(); }

    IWorkloadFactoryPtr CreateWorkloadFactory(const IMemoryManagerSharedPtr& memoryManager) const override
    {
        return std::make_unique<B200WorkloadFactory>(PolymorphicPointerDowncast<B200MemoryManager>(memoryManager));
    }

    IWorkloadFactoryPtr CreateWorkloadFactory(TensorHandleFactoryRegistry& registry) const override
    {
        auto memoryManager = std::make_shared<B200MemoryManager>();
        registry.RegisterMemoryManager(memoryManager);
        auto factory = std::make_unique<B200TensorHandleFactory>(memoryManager);
        registry.RegisterCopyAndImportFactoryPair(factory->GetId(), factory->GetId());
        registry.RegisterFactory(std::move(factory));
        return std::make_unique<B200WorkloadFactory>(memoryManager);
    }

    IBackendContextPtr CreateBackendContext(const IRuntime::CreationOptions& options) const override
    {
        return IBackendContextPtr{new B200BackendContext(options)};
    }

    IBackendProfilingContextPtr CreateBackendProfilingContext(const IRuntime::CreationOptions&, IBackendProfilingPtr&) override
    {
        return IBackendProfilingContextPtr{};
    }

    ILayerSupportSharedPtr GetLayerSupport() const override
    {
        static ILayerSupportSharedPtr layerSupport{new B200LayerSupport};
        return layerSupport;
    }

    std::vector<ITensorHandleFactory::FactoryId> GetHandleFactoryPreferences() const override
    {
        return {B200TensorHandleFactory::GetIdStatic()};
    }

    void RegisterTensorHandleFactories(TensorHandleFactoryRegistry& registry) override
    {
        auto memoryManager = std::make_shared<B200MemoryManager>();
        registry.RegisterMemoryManager(memoryManager);
        auto factory = std::make_unique<B200TensorHandleFactory>(memoryManager);
        registry.RegisterCopyAndImportFactoryPair(factory->GetId(), factory->GetId());
        registry.RegisterFactory(std::move(factory));
    }

    BackendCapabilities GetCapabilities() const override
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

    /// Convolution2d -> ElementwiseBinary(Add, other) [-> Activation{ReLu, BoundedReLu}] becomes one PreCompiled layer
    /// (inputs: data, weights[, bias], other) whose workload adds the other operand in the convolution's epilogue:
    /// the residual connections of ResNet-style graphs then cost no pass over memory of their own.  The result is what
    /// the three CpuRef workloads in a row produce (the convolution's own 8-bit result is formed, not stored).
    void FuseResidualAdds(const SubgraphView& subgraph, OptimizationViews& views, std::map<LayerGuid, Layer*>& untouched) const
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
                    PreCompiledDescriptor(convInputs + 1, 1), std::move(blobPtr), Optional<BackendId>(GetId()), name.c_str());
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

    /// Fold Activation{ReLu, BoundedReLu} into the producing Convolution2d / DepthwiseConvolution2d / FullyConnected /
    /// ElementwiseBinary when both tensors carry the same quantisation: the workload then clamps in the quantised
    /// domain, which is exactly what the separate CpuRef Activation workload would compute.
    OptimizationViews OptimizeSubgraphView(const SubgraphView& subgraph, const ModelOptions& modelOptions) const override
    {
        OptimizationViews views(modelOptions);
        std::map<LayerGuid, Layer*> untouched;
        for (auto it = subgraph.begin(); it != subgraph.end(); ++it)
        {
            Layer& l = *PolymorphicDowncast<Layer*>(*it);
            untouched.insert({l.GetGuid(), &l});
        }
        FuseResidualAdds(subgraph, views, untouched);
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
                auto* b = PolymorphicDowncast<Convolution2dLayer*>(&base);
                auto* r = PolymorphicDowncast<Convolution2dLayer*>(net->AddConvolution2dLayer(b->GetParameters(), name.c_str()));
                Fuse(views, b, r, act);
            }
            else if (t == LayerType::DepthwiseConvolution2d)
            {
                auto* b = PolymorphicDowncast<DepthwiseConvolution2dLayer*>(&base);
                auto* r = PolymorphicDowncast<DepthwiseConvolution2dLayer*>(net->AddDepthwiseConvolution2dLayer(b->GetParameters(), name.c_str()));
                Fuse(views, b, r, act);
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
};

}  // namespace armnn

extern "C" __attribute__((visibility("default"))) const char* GetBackendId()
{
    return armnn::B200Backend::GetIdStatic().Get().c_str();
}

extern "C" __attribute__((visibility("default"))) void GetVersion(uint32_t* outMajor, uint32_t* outMinor)
{
    if (!outMajor || !outMinor) { return; }
    armnn::BackendVersion v = armnn::IBackendInternal::GetApiVersion();
    *outMajor = v.m_Major;
    *outMinor = v.m_Minor;
}

extern "C" __attribute__((visibility("default"))) void* BackendFactory()
{
    return new armnn::B200Backend();
}
