// Static registration for an in-tree build (the backend compiled into libarmnn as src/backends/b200/): the pattern
// of src/backends/reference/RefRegistryInitializer.cpp:15-23 of the Arm NN tree.  Not part of the dynamic backend
// Nv_B200Acc_backend.so, which the runtime registers itself after loading it (a second registration of the same id
// throws, src/armnn/BackendRegistry.cpp:21-29).
#include "B200Backend.hpp"

#include <armnn/BackendRegistry.hpp>

namespace
{

using namespace armnn;

static BackendRegistry::StaticRegistryInitializer g_RegisterHelper
{
    BackendRegistryInstance(),
    B200Backend::GetIdStatic(),
    []()
    {
        return IBackendInternalUniquePtr(new B200Backend);
    }
};

}  // anonymous namespace
