// Workload factory of the B200Acc backend (the counterpart of RefWorkloadFactory,
// src/backends/reference/RefWorkloadFactory.cpp:146-676 of the Arm NN tree).
#pragma once

#include <armnn/Optional.hpp>
#include <armnn/backends/WorkloadFactory.hpp>
#include <armnn/backends/Workload.hpp>
#include <armnn/backends/WorkloadData.hpp>

#include "B200TensorHandle.hpp"

namespace armnn
{

class B200WorkloadFactory : public IWorkloadFactory
{
public:
    explicit B200WorkloadFactory(const std::shared_ptr<B200MemoryManager>& memoryManager);

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
    std::shared_ptr<B200MemoryManager> m_MemoryManager;
};

}  // namespace armnn
