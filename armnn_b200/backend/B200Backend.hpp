// B200Acc: an Arm NN compute backend for NVIDIA B200 GPUs (sm_100a), covering the 8-bit quantised operator hot path.
// IBackendInternal implementation in the layout of the in-tree backends (src/backends/reference/RefBackend.hpp,
// src/backends/cl/ClBackend.hpp of the Arm NN tree).  The same sources build two ways:
//   * as a dynamic backend, Nv_B200Acc_backend.so (B200DynamicBackend.cpp adds the three extern "C" entry points of
//     include/armnn/backends/DynamicBackend.hpp:41-43), found through IRuntime::CreationOptions::m_DynamicBackendsPath;
//   * inside the Arm NN tree as src/backends/b200/ (backend.cmake, CMakeLists.txt, B200RegistryInitializer.cpp register
//     it statically in BackendRegistry, as src/backends/reference/RefRegistryInitializer.cpp:15-23 does for CpuRef).
#pragma once

#include <armnn/backends/IBackendInternal.hpp>

#include "B200TensorHandle.hpp"

namespace armnn
{

/// Per-network options: BackendOptions("B200Acc", {{"DeviceId", n}}) in OptimizerOptions::m_ModelOptions selects the GPU
/// the network is loaded on (the multi-GPU mechanism: one LoadedNetwork per GPU, one host thread each).  The pattern is
/// ClBackendModelContext (src/backends/cl/ClBackendModelContext.cpp).
class B200BackendModelContext : public IBackendModelContext
{
public:
    explicit B200BackendModelContext(const ModelOptions& modelOptions)
    {
        for (const auto& bo : modelOptions)
        {
            if (bo.GetBackendId() != BackendId(B200BackendId())) { continue; }
            for (size_t i = 0; i < bo.GetOptionCount(); ++i)
            {
                const auto& opt = bo.GetOption(i);
                if (opt.GetName() == "DeviceId" && opt.GetValue().IsInt()) { m_DeviceId = opt.GetValue().AsInt(); }
            }
        }
    }
    int DeviceId() const { return m_DeviceId; }      ///< -1: not given
private:
    int m_DeviceId = -1;
};

class B200Backend : public IBackendInternal
{
public:
    B200Backend() = default;
    ~B200Backend() override = default;

    static const BackendId& GetIdStatic();
    const BackendId& GetId() const override { return GetIdStatic(); }

    IMemoryManagerUniquePtr CreateMemoryManager() const override;

    IWorkloadFactoryPtr CreateWorkloadFactory(const IMemoryManagerSharedPtr& memoryManager = nullptr) const override;
    IWorkloadFactoryPtr CreateWorkloadFactory(TensorHandleFactoryRegistry& registry) const override;
    IWorkloadFactoryPtr CreateWorkloadFactory(TensorHandleFactoryRegistry& registry, const ModelOptions& modelOptions) const override;
    IWorkloadFactoryPtr CreateWorkloadFactory(TensorHandleFactoryRegistry& registry, const ModelOptions& modelOptions,
                                              MemorySourceFlags inputFlags, MemorySourceFlags outputFlags) const override;

    IBackendContextPtr CreateBackendContext(const IRuntime::CreationOptions& options) const override;
    IBackendProfilingContextPtr CreateBackendProfilingContext(const IRuntime::CreationOptions& creationOptions,
                                                              IBackendProfilingPtr& backendProfiling) override;
    IBackendSpecificModelContextPtr CreateBackendSpecificModelContext(const ModelOptions& modelOptions) const override;

    ILayerSupportSharedPtr GetLayerSupport() const override;
    ILayerSupportSharedPtr GetLayerSupport(const ModelOptions& modelOptions) const override;

    OptimizationViews OptimizeSubgraphView(const SubgraphView& subgraph, const ModelOptions& modelOptions) const override;

    std::vector<ITensorHandleFactory::FactoryId> GetHandleFactoryPreferences() const override;
    void RegisterTensorHandleFactories(TensorHandleFactoryRegistry& registry) override;
    void RegisterTensorHandleFactories(TensorHandleFactoryRegistry& registry, MemorySourceFlags inputFlags,
                                       MemorySourceFlags outputFlags) override;

    BackendCapabilities GetCapabilities() const override;
};

}  // namespace armnn
