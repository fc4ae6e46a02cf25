// Workload factory of the B200Acc backend (the counterpart of RefWorkloadFactory,
// src/backends/reference/RefWorkloadFactory.cpp:146-676 of the Arm NN tree).
#pragma once

#include <armnn/Descriptors.hpp>
#include <armnn/Optional.hpp>
#include <armnn/Tensor.hpp>
#include <armnn/backends/WorkloadFactory.hpp>
#include <armnn/backends/Workload.hpp>
#include <armnn/backends/WorkloadData.hpp>

#include "B200TensorHandle.hpp"

namespace armnn
{

/// What B200Backend::OptimizeSubgraphView stores in the PreCompiled layer that replaces
/// Convolution2d -> ElementwiseBinary(Add) [-> Activation{ReLu, BoundedReLu}]: the layer's inputs are the
/// convolution's (data, weights[, bias]) followed by the Add's other operand, its output is the Add's (or the
/// Activation's) output.  The workload is one b200k_conv2d_q8 call with add_operand / add_out set.
struct B200FusedConvAdd
{
    static constexpr uint32_t Magic = 0xB200ADD1u;
    uint32_t                m_Magic = Magic;
    Convolution2dDescriptor m_Convolution;
    TensorInfo              m_ConvolutionOutput;     ///< quantisation of the convolution's own (never stored) result
    bool                    m_HasActivation = false;
    ActivationDescriptor    m_Activation;            ///< applied to the Add's output
};

class B200WorkloadFactory : public IWorkloadFactory
{
public:
    B200WorkloadFactory(const std::shared_ptr<B200Context>& ctx, const std::shared_ptr<B200MemoryManager>& memoryManager);

    const BackendId& GetBackendId() const override;

    static bool IsLayerSupported(const IConnectableLayer& layer, Optional<DataType> dataType, std::string& outReasonIfUnsupported);

    bool SupportsSubTensors() const override { return false; }

    std::unique_ptr<ITensorHandle> CreateSubTensorHandle(ITensorHandle&, TensorShape const&, unsigned int const*) const override
    { return nullptr; }

    std::unique_ptr<ITensorHandle> CreateTensorHandle(const TensorInfo& tensorInfo, const bool IsMemoryManaged = true) const override;
    std::unique_ptr<ITensorHandle> CreateTensorHandle(const TensorInfo& tensorInfo, DataLayout dataLayout,
                                                      const bool IsMemoryManaged = true) const override;

    std::unique_ptr<IWorkload> CreateWorkload(LayerType type, const QueueDescriptor& descriptor,
                                              const WorkloadInfo& info) const override;

private:
    std::shared_ptr<B200Context> m_Ctx;                  ///< the network's GPU, stream and workload queue
    std::shared_ptr<B200MemoryManager> m_MemoryManager;
};

}  // namespace armnn
