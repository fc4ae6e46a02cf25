// The shared-object interface of a dynamic Arm NN backend (include/armnn/backends/DynamicBackend.hpp:41-43 of the
// Arm NN tree; example: src/backends/dynamic/reference/RefDynamicBackend.cpp:12-33).  Only built into
// Nv_B200Acc_backend.so; an in-tree build registers the backend through B200RegistryInitializer.cpp instead.
#include "B200Backend.hpp"

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

/// Not part of the dynamic-backend interface: how many CUDA-graph launches the backend's networks have made in this
/// process and how many kernel nodes those launches contained (for benchmarks that report the kernels a timed region ran).
extern "C" __attribute__((visibility("default"))) void B200AccGraphStats(uint64_t* graphLaunches, uint64_t* graphKernels)
{
    uint64_t l = 0, k = 0;
    armnn::B200Context::Stats(l, k);
    if (graphLaunches) { *graphLaunches = l; }
    if (graphKernels) { *graphKernels = k; }
}

extern "C" __attribute__((visibility("default"))) void* BackendFactory()
{
    return new armnn::B200Backend();
}
